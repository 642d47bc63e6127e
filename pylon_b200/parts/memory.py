"""A matrix of memory per head with exponential gates: the mLSTM layer of xLSTM.

Per token, with h the layer's normalised input:

* ``q = W_q h * dim^-1/2`` and ``k = W_k h`` in ``heads`` heads of ``dim``, ``v = W_v h`` in heads of ``vdim``;
* per head the logarithms of an input gate ``i = cap * tanh((W_i h + b_i) / cap)`` and of a forget gate
  ``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``;
* with a running maximum m that starts at 0: ``m' = max(f + m, i)``; the matrix ``S = exp(f + m - m') S + exp(i - m') k v^T`` and the
  normaliser ``n`` likewise with k alone, both from zero; the read-out ``o = S^T q / (max(|n . q|, exp(-m')) + read_eps)``;
* each head's o divided by its root mean square (``norm_eps``), the heads side by side times a weight, times ``sigmoid(W_g h)``, then
  the output projection.

What a request carries from token to token is one float32 state slot: per head S, n and m.  q, k, v and g are one product, the
gates' logits a second whose 32-bit sums are kept; everything behind them is float32 (``csrc/matrix_memory.cu``).  Tensors: ``q``,
``k`` ``[heads * dim, width]``; ``v``, ``g`` ``[heads * vdim, width]``; ``i``, ``f`` ``[heads, width]`` with ``i.b``, ``f.b``; ``norm
[heads * vdim]``; ``o [width, heads * vdim]``.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("matrix_memory")
class MatrixMemory(Mixer):
    takes_padding = True   # the kernels skip rows without tokens; what they compute for a token without a row is never read

    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, gate_cap: float, norm_eps: float, read_eps: float = 1e-6,
                 names: Optional[Mapping[str, str]] = None) -> None:
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        if min(self.width, self.n_heads, self.head_dim, self.value_dim) < 1 or self.head_dim > 256 or not gate_cap > 0:
            raise ValueError(f"{n_heads} heads of {head_dim} (at most 256) x {value_dim}, gate cap {gate_cap}")
        self.gate_cap, self.norm_eps, self.read_eps = float(gate_cap), float(norm_eps), float(read_eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "i": "i", "f": "f", "norm": "norm", "o": "o", "bias_suffix": ".b", **(names or {})}
        self.w_in = self.w_gates = self.w_o = self.gate_bias = self.norm_weight = None

    def tensors(self) -> Sequence[TensorDecl]:
        n, b = self.names, self.names["bias_suffix"]
        keys, values = self.n_heads * self.head_dim, self.n_heads * self.value_dim
        return [
            TensorDecl(n["q"], (keys, self.width)), TensorDecl(n["k"], (keys, self.width)), TensorDecl(n["v"], (values, self.width)),
            TensorDecl(n["g"], (values, self.width)), TensorDecl(n["o"], (self.width, values)), TensorDecl(n["norm"], (values,), "vector"),
            TensorDecl(n["i"], (self.n_heads, self.width), "matrix", (0.0, 0.1)), TensorDecl(n["i"] + b, (self.n_heads,), "vector", (0.0, 0.5)),
            TensorDecl(n["f"], (self.n_heads, self.width), "matrix", (0.0, 0.1)), TensorDecl(n["f"] + b, (self.n_heads,), "vector", (3.0, 1.0)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n, b = self.names, self.names["bias_suffix"]
        self.w_in = torch.cat((tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]), dim=0).contiguous()   # one product: [q | k | v | g]
        self.w_gates = torch.cat((tensors[n["i"]], tensors[n["f"]]), dim=0).contiguous()                                  # and one whose float32 sums are kept
        self.gate_bias = torch.stack((tensors[n["i"] + b], tensors[n["f"] + b])).contiguous()
        self.norm_weight = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_gates.numel() + self.w_o.numel()) * self.w_o.element_size() + 4 * (2 * self.n_heads + self.n_heads * self.value_dim)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.n_heads * (self.head_dim * self.value_dim + self.head_dim + 1),)))

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        logits = ops.linear(h, self.w_gates, out_dtype=torch.float32)
        out = ops.matrix_memory(proj, logits, self.gate_bias, self.norm_weight, cache.state, step.q_start, step.slots, self.n_heads, self.head_dim,
                                self.value_dim, self.gate_cap, self.norm_eps, self.read_eps, step.num_rows)
        return ops.linear_for_residual(out, self.w_o)
