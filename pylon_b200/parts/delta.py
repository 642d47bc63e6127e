"""The gated delta rule: a recurrent mixer with one matrix of state per head.

Per token, with h the layer's normalised input (no biases anywhere):

* ``q = W_q h`` and ``k = W_k h`` in ``kv_heads`` heads of ``dim``, ``v = W_v h`` in ``heads`` heads of ``vdim``; value
  head i uses query/key head ``i // (heads / kv_heads)``;
* each of q, k, v goes through a short causal convolution over time per channel (``taps`` wide, the last tap on the
  current token, zeros before the sequence starts) and then silu;
* q and k become unit vectors per head, ``x / sqrt(sum x^2 + unit_eps)``, q also times ``dim ** -0.5``;
* per head ``beta = sigmoid(W_b h)`` and the decay ``g = exp(-exp(A_log) * softplus(W_a h + dt_bias))``;
* the state S ``[dim, vdim]`` of a head: ``S = g S``; ``w = beta (v - S^T k)``; ``S = S + k w^T``; ``o = S^T q`` (the
  read-out sees the current token's write);
* ``o`` is divided by its root mean square over ``vdim`` (``norm_eps``), times a weight ``[vdim]`` shared by the heads,
  times ``silu(W_g h)``; then the output projection.

Options: ``decay="channel"`` gives every head a decay per key channel, ``g [dim] = exp(-exp(A_log) * softplus(W_a h + dt_bias))`` with
``dt_bias [heads * dim]``, each factor on its row of S; ``decay_rank`` / ``gate_rank`` put a narrow middle into the decay's / the gate's
projection (``W_a = W_a2 W_a1``: the first factors ride in the one big product, the second are products of their own, float32 out);
``gate_activation="sigmoid"`` gates with ``sigmoid(W_g h)``.

What a request carries from token to token is one float32 state slot: the heads' matrices and the convolution's last
``taps - 1`` inputs.  The six projections are one product; everything behind it that enters the recurrence is float32
(``csrc/delta_rule.cu``).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens: a padded step leaves no state touched that it should not

    def __init__(
        self,
        width: int,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        value_dim: int,
        conv_taps: int,
        norm_eps: float,
        unit_eps: float = 1e-6,
        names: Optional[Mapping[str, str]] = None,
        decay: str = "head",
        decay_rank: Optional[int] = None,
        gate_rank: Optional[int] = None,
        gate_activation: str = "silu",
    ) -> None:
        if decay not in ("head", "channel") or gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"decay {decay!r} (head, channel), gate_activation {gate_activation!r} (silu, sigmoid)")
        self.channel_decay, self.sigmoid_gate = decay == "channel", gate_activation == "sigmoid"
        self.decay_rank, self.gate_rank = (None if rank is None else int(rank) for rank in (decay_rank, gate_rank))
        if (self.decay_rank is not None and self.decay_rank < 1) or (self.gate_rank is not None and self.gate_rank < 1):
            raise ValueError("the middle of a two-factor projection is at least one wide")
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} value heads cannot share {n_kv_heads} query/key heads")
        if conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.value_dim, self.conv_taps = int(head_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.qk_size, self.v_size = self.n_kv_heads * self.head_dim, self.n_heads * self.value_dim
        self.channels = 2 * self.qk_size + self.v_size
        self.names = {
            "q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "decay": "a",
            "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o", "decay_in": "a.in", "gate_in": "g.in", **(names or {}),
        }
        self.w_in = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm = self.w_decay = self.w_gate = None
        self.decay_size = self.n_heads * (self.head_dim if self.channel_decay else 1)
        # the one big product's rows, in the kernel's order of columns: q, k, v, then what is there of gate, a, and b - then the first
        # factors of two-factor projections, which the kernel does not read
        self.own_gate = self.sigmoid_gate or self.gate_rank is not None     # the gate comes as a float32 tensor of its own
        self.own_decay = self.channel_decay or self.decay_rank is not None  # so does the decay's input
        if self.own_decay and not self.channel_decay:
            raise NotImplementedError("a two-factor projection of a decay per head is not built")
        if self.own_gate and not self.sigmoid_gate:
            raise NotImplementedError("a gate of its own goes through a sigmoid; silu with a narrow middle is not built")

    # -- weights -------------------------------------------------------------------------
    def tensors(self) -> Sequence[TensorDecl]:
        n, taps = self.names, self.conv_taps
        return [
            TensorDecl(n["q"], (self.qk_size, self.width)), TensorDecl(n["k"], (self.qk_size, self.width)),
            TensorDecl(n["v"], (self.v_size, self.width)),
            *([TensorDecl(n["gate"], (self.v_size, self.width))] if self.gate_rank is None else
              [TensorDecl(n["gate_in"], (self.gate_rank, self.width)), TensorDecl(n["gate"], (self.v_size, self.gate_rank), "matrix", (0.0, self.gate_rank ** -0.5))]),
            *([TensorDecl(n["decay"], (self.decay_size, self.width))] if self.decay_rank is None else
              [TensorDecl(n["decay_in"], (self.decay_rank, self.width)), TensorDecl(n["decay"], (self.decay_size, self.decay_rank), "matrix", (0.0, self.decay_rank ** -0.5))]),
            TensorDecl(n["beta"], (self.n_heads, self.width)),
            TensorDecl(n["o"], (self.width, self.v_size)),
            TensorDecl(n["q_conv"], (self.qk_size, taps), "vector", (0.0, 0.5)), TensorDecl(n["k_conv"], (self.qk_size, taps), "vector", (0.0, 0.5)),
            TensorDecl(n["v_conv"], (self.v_size, taps), "vector", (0.0, 0.5)),
            TensorDecl(n["a_log"], (self.n_heads,), "vector", (-1.0, 0.5)), TensorDecl(n["dt_bias"], (self.decay_size,), "vector", (0.0, 0.5)),
            TensorDecl(n["norm"], (self.value_dim,), "vector"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # one product for all projections of the layer's input: columns [q | k | v | gate | a | b] of its result, gate and a only where
        # the kernel reads them from there; behind b the first factors of the two-factor projections
        rows = [tensors[n[key]] for key in ("q", "k", "v")]
        if not self.own_gate:
            rows.append(tensors[n["gate"]])
        if not self.own_decay:
            rows.append(tensors[n["decay"]])
        rows.append(tensors[n["beta"]])
        self.kernel_columns = sum(w.shape[0] for w in rows)
        self.extra_columns = {}
        for key, rank, own in (("gate", self.gate_rank, self.own_gate), ("decay", self.decay_rank, self.own_decay)):
            if own:
                first = tensors[n[key + "_in"]] if rank is not None else tensors[n[key]]   # without a middle the whole projection rides along
                at = sum(w.shape[0] for w in rows)
                self.extra_columns[key] = (at, at + first.shape[0])
                rows.append(first)
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_gate = tensors[n["gate"]].contiguous() if self.gate_rank is not None else None
        self.w_decay = tensors[n["decay"]].contiguous() if self.decay_rank is not None else None
        self.w_o = tensors[n["o"]].contiguous()
        self.conv = torch.cat([tensors[n[key]] for key in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()   # [taps, channels]
        self.a_log, self.dt_bias, self.norm = (tensors[n[key]].contiguous() for key in ("a_log", "dt_bias", "norm"))

    def weight_bytes(self) -> int:
        second = sum(w.numel() for w in (self.w_gate, self.w_decay) if w is not None)
        return (self.w_in.numel() + self.w_o.numel() + second) * self.w_in.element_size() + self.conv.numel() * 4

    # -- state ---------------------------------------------------------------------------
    def state_floats(self) -> int:
        return self.n_heads * self.head_dim * self.value_dim + (self.conv_taps - 1) * self.channels

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.state_floats(),), torch.float32))

    # -- run -----------------------------------------------------------------------------
    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        own = {}
        for key, second in (("gate", self.w_gate), ("decay", self.w_decay)):
            if key in self.extra_columns:
                first, last = self.extra_columns[key]
                part = proj[:, first:last]
                # what enters the decay and the gate is float32 from here on: the second factor's product keeps its 32-bit sums
                own[key] = ops.linear(part, second, out_dtype=torch.float32) if second is not None else part.to(torch.float32)
        mixed = ops.gated_delta_rule(
            proj, self.conv, cache.state, step.token_row, step.q_start, step.slots, self.a_log, self.dt_bias, self.norm,
            self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, step.num_rows, self.norm_eps, self.unit_eps,
            decay_in=own.get("decay"), gate_in=own.get("gate"),
        )
        return ops.linear_for_residual(mixed, self.w_o)
