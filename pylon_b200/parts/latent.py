"""Latent attention: keys and values of all heads come out of one small row per token.

Per token, with h the layer's normalised input:

* the query goes through a latent: ``c_q = RMSnorm(W_dq h)`` (a weight), ``q = W_uq c_q`` in ``heads`` heads of
  ``[dim not rotated | rot_dim rotated]``;
* ``W_dkv h`` has ``kv_rank + rot_dim`` numbers: the first ``kv_rank``, RMS-normed (a weight), are the latent ``c``; the last
  ``rot_dim``, rotated by the position (not normed), are a key part that all heads share;
* per head the key's other part is ``W_uk c`` and the value ``W_uv c``; a score is
  ``(q_plain . W_uk c + q_rotated . k_rotated) * scale``; attention is causal inside an optional window, and the softmax's
  denominator may hold ``exp(sink_h)``, a learnt number per head without key or value.

With ``q_rank=None`` the query has no latent of its own: ``q = W_q h`` (tensor ``q``), laid out in heads in the same way.

Only ``[c | k_rotated]`` is kept per token: one cache row of ``kv_rank + rot_dim`` numbers, no value rows.  The per-head
matrices are applied on the query's side and behind the attention instead of on every cached row:
``q_plain . (W_uk c) = (W_uk^T q_plain) . c`` and ``sum_j p_j W_uv c_j = W_uv (sum_j p_j c_j)``, so the attention runs
over the cached rows as they are, every head reading the same row, its values being the row's first ``kv_rank`` columns.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, POSITION_ENCODINGS, CacheNeed, KVNeed, LayerCache, Mixer, StepView, TensorDecl
from pylon_b200.parts.spec import PartSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    takes_padding = True   # the kernels skip tokens without a row; rows without tokens have no query

    def __init__(self, width: int, n_heads: int, head_dim: int, rot_dim: int, value_dim: int, q_rank: Optional[int], kv_rank: int, norm_eps: float,
                 scale: float, position: Optional[PartSpec] = None, window: Optional[int] = None, sink: bool = False,
                 names: Optional[Mapping[str, str]] = None, split_weights: bool = False) -> None:
        self.width, self.n_heads, self.head_dim, self.rot_dim = int(width), int(n_heads), int(head_dim), int(rot_dim)
        self.value_dim, self.q_rank, self.kv_rank = int(value_dim), (None if q_rank is None else int(q_rank)), int(kv_rank)
        if min(self.n_heads, self.head_dim, self.value_dim, self.q_rank or 1, self.kv_rank) < 1 or self.rot_dim < 0:
            raise ValueError("latent attention needs positive sizes")
        self.norm_eps, self.scale = float(norm_eps), float(scale)
        self.window = None if window is None else int(window)
        self.has_sink = bool(sink)
        self.split_weights = bool(split_weights)   # the tensor-core kernel takes the softmax weights with 16 bits instead of 8 (twice the products over the values)
        self.position = POSITION_ENCODINGS.build(position) if position is not None and self.rot_dim else None
        if self.position is not None and not hasattr(self.position, "tables"):
            raise ValueError("latent attention rotates its shared key part by tables of cos and sin")
        self.row = self.kv_rank + self.rot_dim          # what is cached per token
        self.q_head = self.head_dim + self.rot_dim
        self.names = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                      "sink": "sink", "o": "o", **(names or {})}
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.q_norm = self.kv_norm = self.sink = None

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        if self.q_rank is None:
            decls = [TensorDecl(n["q"], (self.n_heads * self.q_head, self.width))]
        else:
            decls = [TensorDecl(n["dq"], (self.q_rank, self.width)), TensorDecl(n["dq_norm"], (self.q_rank,), "vector"),
                     TensorDecl(n["uq"], (self.n_heads * self.q_head, self.q_rank))]
        decls += [
            TensorDecl(n["dkv"], (self.row, self.width)), TensorDecl(n["dkv_norm"], (self.kv_rank,), "vector"),
            TensorDecl(n["uk"], (self.n_heads * self.head_dim, self.kv_rank)), TensorDecl(n["uv"], (self.n_heads * self.value_dim, self.kv_rank)),
            TensorDecl(n["o"], (self.width, self.n_heads * self.value_dim)),
        ]
        if self.has_sink:
            decls.append(TensorDecl(n["sink"], (self.n_heads,), "vector", (0.0, 1.0)))
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # both down projections read the same input: one product, columns [query latent | key/value latent | rotated key part]
        # (without a query latent: [queries of all heads | key/value latent | rotated key part])
        self.w_down = torch.cat((tensors[n["q"] if self.q_rank is None else n["dq"]], tensors[n["dkv"]]), dim=0).contiguous()
        self.w_uq = None if self.q_rank is None else tensors[n["uq"]].contiguous()
        # [heads, kv_rank, dim]: the key matrix of a head, transposed, takes the head's query into the latent's space
        self.w_uk_t = tensors[n["uk"]].view(self.n_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(self.n_heads, self.value_dim, self.kv_rank).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.q_norm, self.kv_norm = (None if self.q_rank is None else tensors[n["dq_norm"]].contiguous()), tensors[n["dkv_norm"]].contiguous()
        self.sink = tensors[n["sink"]].contiguous() if self.has_sink else None

    def weight_bytes(self) -> int:
        matrices = (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.w_o)
        return sum(m.numel() for m in matrices if m is not None) * self.w_o.element_size() + 4 * ((self.q_rank or 0) + self.kv_rank + self.n_heads)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv=KVNeed(1, self.row, self.window, value_dim=0))

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        tokens = h.shape[0]
        cos, sin, rotary_dim, layout = self.position.tables(h.device) if self.position is not None else (None, None, 0, "halves")
        down = ops.linear(h, self.w_down)
        if self.q_rank is None:   # the queries are the product's first columns as they are; the rest is the token's cache row
            q_size = self.n_heads * self.q_head
            ops.latent_norm_rotate_write(
                down[:, q_size:], None, self.kv_norm, self.norm_eps, cos, sin, rotary_dim, layout, step.positions, step.token_row, cache.block_table,
                cache.page_size, cache.k_pages, 0, self.kv_rank, self.rot_dim,
            )
            q = down[:, :q_size].view(tokens, self.n_heads, self.q_head)
        else:
            cq = ops.latent_norm_rotate_write(
                down, self.q_norm, self.kv_norm, self.norm_eps, cos, sin, rotary_dim, layout, step.positions, step.token_row, cache.block_table,
                cache.page_size, cache.k_pages, self.q_rank, self.kv_rank, self.rot_dim,
            )
            q = ops.linear(cq, self.w_uq).view(tokens, self.n_heads, self.q_head)
        query = torch.empty((tokens, self.n_heads, self.row), dtype=h.dtype, device=h.device)
        ops.linear_heads(q[:, :, : self.head_dim], self.w_uk_t, out=query[:, :, : self.kv_rank])
        if self.rot_dim:
            ops.rotate_heads(q[:, :, self.head_dim:], query[:, :, self.kv_rank:], cos, sin, rotary_dim, layout, step.positions)
        context = ops.paged_attention(
            query.view(tokens, self.n_heads * self.row), cache.k_pages, None, step.positions, step.token_row, step.q_start, step.kv_len,
            cache.block_table, self.n_heads, step.max_q, step.max_kv, window=self.window, scale=self.scale, row_tokens=step.row_tokens,
            sinks=self.sink, values_in_keys=self.kv_rank, split_weights=self.split_weights,
        )
        values = ops.linear_heads(context.view(tokens, self.n_heads, self.kv_rank), self.w_uv)
        return ops.linear_for_residual(values.view(tokens, self.n_heads * self.value_dim), self.w_o)
