"""A gated linear recurrence over channels: the recurrent block of Griffin with its real-gated linear recurrent unit.

Per token, with h the layer's normalised input and C channels:

* two branches: ``gate = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal convolution per channel over time (``taps``
  wide, the last tap on the current token, zeros before the sequence starts, a bias, no activation);
* u is cut into ``blocks`` equal parts; in part b ``r = sigmoid(R_b u_b + b_r)`` and ``i = sigmoid(I_b u_b + b_i)`` with square maps;
* ``log a = -decay_factor * r * softplus(lam)``, ``a = exp(log a)``, and the state ``S = a S + sqrt(1 - a^2) * i * u`` from ``S = 0``, the
  first token treated like every other;
* the output projection of ``S * gate``.

What a request carries from token to token is one float32 state slot: S and the convolution's last ``taps - 1`` inputs.  The two
branches are one product and the two gates' maps one product per block; everything behind them that enters the recurrence is float32
(``csrc/linear_recurrence.cu``).  Tensors: ``y``, ``x`` ``[C, width]`` with ``y.b``, ``x.b``; ``conv [C, taps]``, ``conv.b``; ``ra``,
``ri`` ``[blocks, C / blocks, C / blocks]`` (``[out, in]``) with ``ra.b``, ``ri.b`` ``[blocks, C / blocks]``; ``lam [C]``; ``o [width, C]``.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StateNeed, StepView, TensorDecl


@MIXERS.register("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens

    def __init__(self, width: int, channels: int, blocks: int, conv_taps: int, decay_factor: float = 8.0, names: Optional[Mapping[str, str]] = None) -> None:
        self.width, self.channels, self.blocks, self.taps = int(width), int(channels), int(blocks), int(conv_taps)
        if min(self.width, self.channels, self.blocks, self.taps) < 1 or self.channels % self.blocks or self.taps > 16:
            raise ValueError(f"{channels} channels in {blocks} equal parts, a convolution of {conv_taps} taps (1 to 16)")
        self.decay_factor = float(decay_factor)
        self.names = {"y": "y", "x": "x", "conv": "conv", "gate_a": "ra", "gate_i": "ri", "lam": "lam", "o": "o", "bias_suffix": ".b", **(names or {})}
        self.w_in = self.w_gates = self.w_o = self.bias = self.conv_weight = self.conv_bias = self.gate_bias = self.lam = None

    def tensors(self) -> Sequence[TensorDecl]:
        n, b = self.names, self.names["bias_suffix"]
        part = self.channels // self.blocks
        return [
            TensorDecl(n["y"], (self.channels, self.width)), TensorDecl(n["y"] + b, (self.channels,), "vector", (0.0, 0.02)),
            TensorDecl(n["x"], (self.channels, self.width)), TensorDecl(n["x"] + b, (self.channels,), "vector", (0.0, 0.02)),
            TensorDecl(n["conv"], (self.channels, self.taps), "vector", (0.0, 0.3)), TensorDecl(n["conv"] + b, (self.channels,), "vector", (0.0, 0.02)),
            TensorDecl(n["gate_a"], (self.blocks, part, part)), TensorDecl(n["gate_a"] + b, (self.blocks, part), "vector", (0.0, 0.5)),
            TensorDecl(n["gate_i"], (self.blocks, part, part)), TensorDecl(n["gate_i"] + b, (self.blocks, part), "vector", (0.0, 0.5)),
            TensorDecl(n["lam"], (self.channels,), "vector", (-2.0, 1.0)),
            TensorDecl(n["o"], (self.width, self.channels)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n, b = self.names, self.names["bias_suffix"]
        self.w_in = torch.cat((tensors[n["y"]], tensors[n["x"]]), dim=0).contiguous()                      # one product: columns [y | x]
        self.bias = torch.cat((tensors[n["y"] + b], tensors[n["x"] + b])).contiguous()
        self.w_gates = torch.cat((tensors[n["gate_a"]], tensors[n["gate_i"]]), dim=1).contiguous()         # per block: the recurrence gate's rows, then the input gate's
        self.gate_bias = torch.stack((tensors[n["gate_a"] + b].reshape(-1), tensors[n["gate_i"] + b].reshape(-1))).contiguous()
        self.conv_weight, self.conv_bias = tensors[n["conv"]].contiguous(), tensors[n["conv"] + b].contiguous()
        self.lam = tensors[n["lam"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_gates.numel() + self.w_o.numel()) * self.w_o.element_size() + 4 * self.channels * (6 + self.taps)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state=StateNeed((self.channels * self.taps,)))

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        proj = ops.linear(h, self.w_in)
        out = ops.linear_recurrence(proj, self.bias, self.conv_weight, self.conv_bias, self.w_gates, self.gate_bias, self.lam, self.decay_factor,
                                    cache.state, step.token_row, step.q_start, step.slots, step.num_rows, step.max_q)
        return ops.linear_for_residual(out, self.w_o)
