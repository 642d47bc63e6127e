"""A state-space mixer with one decay per head and step, and a matrix of state per head.

Per token, with h the layer's normalised input, ``inner = heads * vdim``, N the state's rows per head and G groups of heads
that share their input and output maps:

* one projection of h (no bias) with columns ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``;
* x, B and C together go through a short causal convolution over time per channel (``taps`` wide, the last tap on the
  current token, zeros before the sequence starts, a bias) and then silu;
* per head ``dt = softplus(dt + dt_bias)`` (no clamp) and the decay ``a = exp(-exp(A_log) dt)``;
* the state S ``[N, vdim]`` of a head in group g: ``S = a S + dt B_g x^T``; ``y = S^T C_g + D x`` (the read-out sees the
  current token's write);
* the heads' y side by side times ``silu(z)``, then divided by the root mean square of each of ``norm_groups`` equal
  parts (``norm_eps``), times a weight ``[inner]``; then the output projection.

What a request carries from token to token is one float32 state slot: the heads' matrices and the convolution's last
``taps - 1`` inputs.  Everything behind the projection is float32 (``csrc/state_space.cu``).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("state_space")
class StateSpace(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens

    def __init__(self, width: int, n_heads: int, value_dim: int, state_dim: int, groups: int, norm_groups: int, conv_taps: int,
                 norm_eps: float, names: Optional[Mapping[str, str]] = None) -> None:
        self.width, self.n_heads, self.value_dim, self.state_dim = int(width), int(n_heads), int(value_dim), int(state_dim)
        self.groups, self.norm_groups, self.conv_taps, self.norm_eps = int(groups), int(norm_groups), int(conv_taps), float(norm_eps)
        if self.n_heads % self.groups:
            raise ValueError(f"{n_heads} heads cannot share {groups} groups of input and output maps")
        self.inner = self.n_heads * self.value_dim
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels cannot be normed in {norm_groups} equal parts")
        if self.conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.channels = self.inner + 2 * self.groups * self.state_dim
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
                      "norm": "norm", "o": "o", **(names or {})}
        self.w_in = self.w_o = self.conv = self.conv_bias = self.a_log = self.dt_bias = self.skip = self.norm = None

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        return [
            TensorDecl(n["in"], (self.inner + self.channels + self.n_heads, self.width)), TensorDecl(n["o"], (self.width, self.inner)),
            TensorDecl(n["conv"], (self.channels, self.conv_taps), "vector", (0.0, 0.5)), TensorDecl(n["conv_bias"], (self.channels,), "vector", (0.0, 0.1)),
            TensorDecl(n["dt_bias"], (self.n_heads,), "vector", (0.0, 0.5)), TensorDecl(n["a_log"], (self.n_heads,), "vector", (-1.0, 0.5)),
            TensorDecl(n["skip"], (self.n_heads,), "vector"), TensorDecl(n["norm"], (self.inner,), "vector"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        self.w_in, self.w_o = tensors[n["in"]].contiguous(), tensors[n["o"]].contiguous()
        self.conv = tensors[n["conv"]].t().contiguous()   # [taps, channels]
        self.conv_bias, self.dt_bias, self.a_log, self.skip, self.norm = (
            tensors[n[key]].contiguous() for key in ("conv_bias", "dt_bias", "a_log", "skip", "norm"))

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + (self.conv.numel() + self.channels + self.inner) * 4

    def state_floats(self) -> int:
        return self.n_heads * self.state_dim * self.value_dim + (self.conv_taps - 1) * self.channels

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.state_floats(),), torch.float32))

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        mixed = ops.state_space(
            proj, self.conv, self.conv_bias, cache.state, step.token_row, step.q_start, step.slots, self.a_log, self.dt_bias, self.skip,
            self.norm, self.n_heads, self.groups, self.state_dim, self.value_dim, self.norm_groups, step.num_rows, self.norm_eps,
        )
        return ops.linear_for_residual(mixed, self.w_o)
