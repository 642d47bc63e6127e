"""Grouped-query attention over the paged cache.

One fused QKV product (rows ``[q; k; v]``), optional per-head RMSNorm of q and k, the
position encoding, the write of k and v into the layer's pages, causal (optionally
windowed) attention over the pages, and the output product.  Order of operations as in
raun6k/Pylon's ``GroupedQueryAttention`` (src/pylon/model/layers.py:81-138) with its cache
write before attention (src/pylon/kv/cache.py:457-476).

Options beyond that: values of another width than the keys (``value_dim``); a soft cap on the
scaled scores, ``s -> c * tanh(s / c)`` (``softcap``); attention in chunks of positions, where a
token sees the keys ``j <= i`` with ``j // chunk == i // chunk`` only, chunks counted from position
0 of the request (``chunk``); and value mixing (``value_mix``): the layer that says ``"source"``
leaves its values in the step under ``value_mix_key``, a layer that says ``"mix"`` replaces its own
values by ``(1 - w) v + w v_source`` of the same token, with w a learnt scalar, before they are cached.

Without rotation, further: the norm of q and of k over their whole rows, all heads at once, with a weight as long as the row
(``qk_norm="whole"``); a window that never hides the first ``keep_first`` positions; a learnt bias by distance (``distance_bias``:
``{"rows": B, "far": D}``; the tensor ``[B, heads]`` holds a row per distance below ``B / 2`` and rows that grow logarithmically
up to the distance ``D``, where the last is reached: ``row(n) = n`` for ``n < B/2``, else
``min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) * (B - B/2)))``; it is added to the scaled score); and a learnt sink per
head in the softmax's denominator (``sink``).

And around the rotation: biases on the three projections (``bias``; the tensors' names are the weights' with ``bias_suffix``),
the per-head norm of q and k behind the rotation instead of before it (``qk_norm="after"``) and without a weight
(``qk_norm_weight=False``), an encoding that rotates only part of a head or pairs neighbouring elements, and any of these
together with values of their own width, chunks or a soft cap: one kernel for bias, rotation, norm and cache write
(``ops.qkv_rotate_write``) then stands between the product and the attention.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import (
    MIXERS, POSITION_ENCODINGS, CacheNeed, KVNeed, LayerCache, Mixer, StepView, TensorDecl,
)
from pylon_b200.parts.spec import PartSpec


def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of a bias table of ``rows`` rows for a key ``n`` positions back (see the module's text).  A quotient of logarithms
    that is an integer but for rounding counts as that integer."""
    half = rows // 2
    if n < half:
        return n
    steps = math.log(n / half) / math.log(far / half) * (rows - half)
    nearest = round(steps)
    return min(rows - 1, half + (nearest if abs(steps - nearest) < 1e-9 else math.floor(steps)))


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens

    def __init__(
        self,
        width: int,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        position: Optional[PartSpec] = None,
        qk_norm_eps: Optional[float] = None,
        window: Optional[int] = None,
        scale: Optional[float] = None,
        names: Optional[Mapping[str, str]] = None,
        value_dim: Optional[int] = None,
        chunk: Optional[int] = None,
        softcap: Optional[float] = None,
        value_mix: Optional[str] = None,
        value_mix_key: str = "values",
        bias: bool = False,
        bias_suffix: str = ".b",
        qk_norm: str = "before",
        qk_norm_weight: bool = True,
        keep_first: int = 0,
        distance_bias: Optional[Mapping[str, float]] = None,
        sink: bool = False,
    ) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads cannot be grouped over {n_kv_heads} KV heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        self.q_size, self.kv_size = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.v_size, self.out_size = self.n_kv_heads * self.value_dim, self.n_heads * self.value_dim
        self.chunk = None if chunk is None else int(chunk)
        self.softcap = None if softcap is None else float(softcap)
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix is 'source', 'mix' or None, not {value_mix!r}")
        if (self.chunk is not None and self.chunk < 1) or (self.softcap is not None and not self.softcap > 0) or self.value_dim < 1:
            raise ValueError(f"chunk {chunk!r}, softcap {softcap!r}, value_dim {value_dim!r}: positive numbers are needed")
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        # the kernels that fuse rotation and cache write take values as wide as the keys and plain causal scores
        self.keep_first, self.has_sink = int(keep_first), bool(sink)
        self.bias_rows, self.bias_far = (None, None) if distance_bias is None else (int(distance_bias["rows"]), float(distance_bias["far"]))
        if self.keep_first < 0 or (self.keep_first and (window is None or chunk is not None)):
            raise ValueError("kept first positions go with a window, and not with chunks")
        if self.bias_rows is not None and (self.bias_rows < 2 or not self.bias_far > self.bias_rows // 2):
            raise ValueError(f"a bias table of {self.bias_rows} rows that ends at distance {self.bias_far}")
        plain_scores = self.plain_scores = self.keep_first > 0 or self.bias_rows is not None or self.has_sink or qk_norm == "whole"
        self.general = self.value_dim != self.head_dim or self.chunk is not None or self.softcap is not None or value_mix is not None or plain_scores
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        if qk_norm not in ("before", "after", "whole"):
            raise ValueError(f"the q/k norm stands 'before' or 'after' the rotation or runs over the 'whole' rows, not {qk_norm!r}")
        if plain_scores and (position is not None or value_mix is not None or bias):
            raise NotImplementedError("whole-row norms, kept first positions, a bias by distance and a sink: without rotation, value mixing and projection biases")
        self.bias, self.bias_suffix, self.qk_norm_place, self.qk_norm_weight = bool(bias), bias_suffix, qk_norm, bool(qk_norm_weight)
        self.window = None if window is None else int(window)
        self.scale = 1.0 / math.sqrt(self.head_dim) if scale is None else float(scale)
        self.position = POSITION_ENCODINGS.build(position) if position is not None else None
        self.names = {
            "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
            "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "value_mix": "vmix", "distance_bias": "distance_bias", "sink": "sink",
            **(names or {}),
        }
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.mix_weight = self.b_qkv = self.bias_table = self.sink = None
        self.kept_value_dim = self.value_dim   # the width values have in the cache: wider than value_dim when they are kept padded
        # what the kernels that fuse norm, rotation and cache write do not take goes through the kernel that takes everything
        self.rotary_general = self.bias or self.qk_norm_place == "after" or (self.qk_norm_eps is not None and not self.qk_norm_weight) \
            or (self.position is not None and (self.general or getattr(self.position, "layout", "halves") != "halves"))
        if self.rotary_general and (value_mix is not None or (self.position is not None and not hasattr(self.position, "tables"))):
            raise NotImplementedError("biases, a norm behind the rotation or a rotation beside values of their own width: not with value mixing, and "
                                      "only with an encoding that rotates by tables of cos and sin")

    # -- weights -------------------------------------------------------------------------
    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        decls = [
            TensorDecl(n["q"], (self.q_size, self.width)),
            TensorDecl(n["k"], (self.kv_size, self.width)),
            TensorDecl(n["v"], (self.v_size, self.width)),
            TensorDecl(n["o"], (self.width, self.out_size)),
        ]
        if self.value_mix is not None:   # the source layer's weight is in the checkpoint too, and is not used
            decls.append(TensorDecl(n["value_mix"], (), "vector", (0.5, 0.1)))
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            sizes = (self.q_size, self.kv_size) if self.qk_norm_place == "whole" else (self.head_dim, self.head_dim)
            decls += [TensorDecl(n["q_norm"], (sizes[0],), "vector"), TensorDecl(n["k_norm"], (sizes[1],), "vector")]
        if self.bias_rows is not None:
            decls.append(TensorDecl(n["distance_bias"], (self.bias_rows, self.n_heads), "vector", (0.0, 0.5)))
        if self.has_sink:
            decls.append(TensorDecl(n["sink"], (self.n_heads,), "vector", (0.0, 1.0)))
        if self.bias:
            decls += [TensorDecl(n[key] + self.bias_suffix, (size,), "vector", (0.0, 0.02))
                      for key, size in (("q", self.q_size), ("k", self.kv_size), ("v", self.v_size))]
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        w_v, w_o = tensors[n["v"]], tensors[n["o"]]
        b_v = tensors[n["v"] + self.bias_suffix] if self.bias else None
        # The tensor-core attention kernels take values as wide as the keys.  Narrower values are kept padded to the keys'
        # width in bfloat16: zero rows in the value projection, zero columns in the output projection; the padding is zero
        # from the product to the cache and meets zeros in the output product, so nothing else needs to know.
        self.kept_value_dim = self.value_dim
        if dtype == torch.bfloat16 and self.value_dim < self.head_dim and self.head_dim % 16 == 0 and self.head_dim <= 256 and not self.plain_scores:
            self.kept_value_dim = self.head_dim
            padded_v = w_v.new_zeros((self.n_kv_heads, self.head_dim, self.width))
            padded_v[:, : self.value_dim] = w_v.view(self.n_kv_heads, self.value_dim, self.width)
            padded_o = w_o.new_zeros((self.width, self.n_heads, self.head_dim))
            padded_o[:, :, : self.value_dim] = w_o.view(self.width, self.n_heads, self.value_dim)
            w_v, w_o = padded_v.view(-1, self.width), padded_o.view(self.width, -1)
            if b_v is not None:
                padded_b = b_v.new_zeros((self.n_kv_heads, self.head_dim))
                padded_b[:, : self.value_dim] = b_v.view(self.n_kv_heads, self.value_dim)
                b_v = padded_b.view(-1)
        # q, k and v share one product: their matrices are stacked by rows at load.
        self.w_qkv = torch.cat((tensors[n["q"]], tensors[n["k"]], w_v), dim=0).contiguous()
        self.w_o = w_o.contiguous()
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm, self.k_norm = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
        if self.bias:
            self.b_qkv = torch.cat((tensors[n["q"] + self.bias_suffix], tensors[n["k"] + self.bias_suffix], b_v)).contiguous()
        if self.value_mix == "mix":
            self.mix_weight = tensors[n["value_mix"]].reshape(1).contiguous()
        if self.bias_rows is not None:
            # one row per distance up to the one where the last bucket is reached: the kernels look a distance up, not its bucket
            rows = torch.tensor([distance_bucket(n, self.bias_rows, self.bias_far) for n in range(int(math.ceil(self.bias_far)) + 1)], device=device)
            self.bias_table = tensors[n["distance_bias"]].index_select(0, rows).contiguous()
        if self.has_sink:
            self.sink = tensors[n["sink"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size() + (0 if self.q_norm is None else 8 * self.head_dim)

    # -- cache ---------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        value_dim = None if self.kept_value_dim == self.head_dim else self.kept_value_dim   # as kept: known once the weights are loaded
        return CacheNeed(kv=KVNeed(self.n_kv_heads, self.head_dim, self.window, value_dim, self.chunk, self.keep_first))

    # -- run -----------------------------------------------------------------------------
    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        if self.rotary_general:
            return self._forward_rotary_general(h, step, cache)
        if self.general:
            return self._forward_general(h, step, cache)
        table = self.position.rotary_table(h.device) if self.position is not None else None
        cos, sin, rotary_dim = table if table is not None else (None, None, 0)
        q_norm, k_norm = self.q_norm, self.k_norm
        if self.position is not None and table is None:
            # An encoding that is not a rotation by a table runs as a step of its own, on normalised q and k and
            # before k goes into the cache; the fused kernel below is left with the cache write.
            qkv = ops.linear(h, self.w_qkv)
            if q_norm is not None:
                ops.qk_norm(qkv, q_norm, k_norm, self.qk_norm_eps, self.n_heads, self.n_kv_heads, self.head_dim)
                q_norm = k_norm = None
            self.position.apply(qkv[:, : self.q_size], qkv[:, self.q_size : self.q_size + self.kv_size], step)
        elif cos is not None and ops.qkv_rotation_fuses(h, self.w_qkv, self.head_dim, rotary_dim, cache.k_pages):
            qkv = None   # a long prompt portion: norms, rotation and cache write in the product's epilogue
        else:
            qkv = ops.linear_for_rotation(h, self.w_qkv, self.head_dim, rotary_dim)   # may be partial sums: the next kernel adds them
        if qkv is None:
            q = ops.linear_qkv_rotated(
                h, self.w_qkv, q_norm, k_norm, self.qk_norm_eps or 0.0, cos, sin, step.positions, step.token_row,
                cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, self.n_heads, self.n_kv_heads, self.head_dim,
            )
        else:
            q = ops.qk_norm_rope_kv_write(
                qkv, q_norm, k_norm, self.qk_norm_eps or 0.0, cos, sin, rotary_dim, step.positions, step.token_row,
                cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, self.n_heads, self.n_kv_heads, self.head_dim,
            )
        context = ops.paged_attention(
            q, cache.k_pages, cache.v_pages, step.positions, step.token_row, step.q_start, step.kv_len, cache.block_table,
            self.n_heads, step.max_q, step.max_kv, window=self.window, scale=self.scale, row_tokens=step.row_tokens,
            rows_alike=step.rows_alike,
        )
        return ops.linear_for_residual(context, self.w_o)

    def _forward_general(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        """Values of their own width, value mixing, chunks or a soft cap: the product, one kernel for norms, mixing and
        cache write, attention, the output product."""
        if self.position is not None:
            raise NotImplementedError("a position encoding together with value_dim, chunk, softcap or value_mix is not built")
        qkv = ops.linear(h, self.w_qkv)
        other, other_width = step.carry.get(self.value_mix_key, (None, None)) if self.value_mix == "mix" else (None, None)
        if self.value_mix == "mix" and other is None:
            raise RuntimeError(f"no earlier layer of this step left values under {self.value_mix_key!r}")
        ops.qk_norm_mix_kv_write(
            qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, step.positions, step.token_row, cache.block_table, cache.page_size,
            cache.k_pages, cache.v_pages, self.n_heads, self.n_kv_heads, self.head_dim, self.kept_value_dim,
            other_values=other, mix_weight=self.mix_weight if other is not None else None, other_head_width=other_width,
            whole_rows=self.qk_norm_place == "whole",
        )
        if self.value_mix == "source":
            step.carry[self.value_mix_key] = (qkv[:, self.q_size + self.kv_size:], self.kept_value_dim)
        context = ops.paged_attention(
            qkv, cache.k_pages, cache.v_pages, step.positions, step.token_row, step.q_start, step.kv_len, cache.block_table,
            self.n_heads, step.max_q, step.max_kv, window=self.window, scale=self.scale, row_tokens=step.row_tokens,
            rows_alike=step.rows_alike, chunk=self.chunk, softcap=self.softcap, sinks=self.sink, keep_first=self.keep_first,
            distance_bias=self.bias_table,
        )
        return ops.linear_for_residual(context, self.w_o)

    def _forward_rotary_general(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        """Biases, any rotation by tables, the norm on either side of it, values of any width: the product, one kernel for all of
        that and the cache write, attention, the output product."""
        cos, sin, rotary_dim, layout = self.position.tables(h.device) if self.position is not None else (None, None, 0, "halves")
        qkv = ops.linear(h, self.w_qkv)
        ops.qkv_rotate_write(
            qkv, self.b_qkv, cos, sin, rotary_dim, layout, None if self.qk_norm_eps is None else self.qk_norm_place, self.q_norm, self.k_norm,
            self.qk_norm_eps or 0.0, step.positions, step.token_row, cache.block_table, cache.page_size, cache.k_pages, cache.v_pages,
            self.n_heads, self.n_kv_heads, self.head_dim, self.kept_value_dim,
        )
        context = ops.paged_attention(
            qkv, cache.k_pages, cache.v_pages, step.positions, step.token_row, step.q_start, step.kv_len, cache.block_table,
            self.n_heads, step.max_q, step.max_kv, window=self.window, scale=self.scale, row_tokens=step.row_tokens,
            rows_alike=step.rows_alike, chunk=self.chunk, softcap=self.softcap,
        )
        return ops.linear_for_residual(context, self.w_o)
