"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up as one product.

raun6k/Pylon's ``FeedForward`` (src/pylon/model/layers.py:13-27); the stacked ``[gate; up]``
layout is the one its loader builds (src/pylon/model/weights.py:65-67).

``clamped_glu`` is the same arrangement with another gated unit: ``g = min(gate(x), limit)``,
``u = clamp(up(x), -limit, limit)``, ``down(g * sigmoid(alpha * g) * (u + 1))``.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import FEED_FORWARDS, FeedForward, StepView, TensorDecl


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, width: int, intermediate: int, names: Optional[Mapping[str, str]] = None,
                 limit: Optional[float] = None, alpha: float = 1.0) -> None:
        self.width, self.intermediate = int(width), int(intermediate)
        self.limit, self.alpha = (None if limit is None else float(limit)), float(alpha)
        if self.limit is not None and not self.limit > 0:
            raise ValueError(f"the limit of a clamped gated unit must be positive, got {limit!r}")
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **(names or {})}
        self.w_gate_up = self.w_down = None
        self.interleaved = False

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        return (
            TensorDecl(n["gate"], (self.intermediate, self.width)),
            TensorDecl(n["up"], (self.intermediate, self.width)),
            TensorDecl(n["down"], (self.width, self.intermediate)),
        )

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # gate and up share one product.  In bfloat16 their rows alternate in groups of 8, so that
        # the product's kernel can apply silu(gate) * up itself; otherwise they lie in two halves.
        self.interleaved = dtype == torch.bfloat16 and self.intermediate % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(tensors[n["gate"]], tensors[n["up"]])
        else:
            self.w_gate_up = torch.cat((tensors[n["gate"]], tensors[n["up"]]), dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        if self.interleaved:
            activation = ops.linear_swiglu(h, self.w_gate_up, limit=self.limit, alpha=self.alpha)
        else:
            activation = ops.swiglu(ops.linear(h, self.w_gate_up), limit=self.limit, alpha=self.alpha)
        return ops.linear_for_residual(activation, self.w_down)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(SwiGLU):
    """``down(g * sigmoid(alpha * g) * (u + 1))`` with ``g = min(gate(x), limit)`` and ``u = clamp(up(x), -limit, limit)``."""

    def __init__(self, width: int, intermediate: int, limit: float, alpha: float = 1.702, names: Optional[Mapping[str, str]] = None) -> None:
        super().__init__(width, intermediate, names, limit=limit, alpha=alpha)


@FEED_FORWARDS.register("gated_unit")
class GatedUnit(FeedForward):
    """``down(act(gate(x)) * up(x))`` with a named activation (``silu``, ``relu``, ``gelu_tanh``) and optional biases on all three
    projections (their tensors are the weights' names with ``bias_suffix``).  Gate and up are one product; biases, activation and
    the product of the two halves are one float32 kernel behind it; the down projection's bias joins its 32-bit result."""

    def __init__(self, width: int, intermediate: int, activation: str = "silu", bias: bool = False, bias_suffix: str = ".b",
                 names: Optional[Mapping[str, str]] = None) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (known: {', '.join(ops.ACTIVATIONS)})")
        self.width, self.intermediate, self.activation = int(width), int(intermediate), activation
        self.bias, self.bias_suffix = bool(bias), bias_suffix
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **(names or {})}
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None
        self.fused = False

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        decls = [TensorDecl(n["gate"], (self.intermediate, self.width)), TensorDecl(n["up"], (self.intermediate, self.width)),
                 TensorDecl(n["down"], (self.width, self.intermediate))]
        if self.bias:
            decls += [TensorDecl(n[key] + self.bias_suffix, (size,), "vector", (0.0, 0.02))
                      for key, size in (("gate", self.intermediate), ("up", self.intermediate), ("down", self.width))]
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # silu without biases is the unit the products' own epilogues apply (rows of gate and up in turn, in groups of 8)
        self.fused = self.activation == "silu" and not self.bias and dtype == torch.bfloat16 and self.intermediate % 8 == 0
        if self.fused:
            self.w_gate_up = ops.interleave_gate_up(tensors[n["gate"]], tensors[n["up"]])
        else:
            self.w_gate_up = torch.cat((tensors[n["gate"]], tensors[n["up"]]), dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()
        if self.bias:
            self.b_gate_up = torch.cat((tensors[n["gate"] + self.bias_suffix], tensors[n["up"] + self.bias_suffix])).contiguous()
            self.b_down = tensors[n["down"] + self.bias_suffix].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size() + (4 * (2 * self.intermediate + self.width) if self.bias else 0)

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        if self.fused:
            return ops.linear_for_residual(ops.linear_swiglu(h, self.w_gate_up), self.w_down)
        activation = ops.gated_unit(ops.linear(h, self.w_gate_up), self.b_gate_up, self.activation)
        if not self.bias:
            return ops.linear_for_residual(activation, self.w_down)
        out = ops.linear(activation, self.w_down, out_dtype=torch.float32)
        return ops.add_bias(out, self.b_down).unsqueeze(0)   # float32, in the form of partial sums: the stream takes it in 32-bit


@FEED_FORWARDS.register("expert_mixture")
class ExpertMixture(FeedForward):
    """A mixture of experts: ``experts`` gated units ``down_e(act(gate_e(x)) * up_e(x))`` without biases, of which every token
    goes through the ``top`` whose router logits ``W_r x (+ b_r)`` are largest, weighted by the softmax over just those logits.
    The router's weights stay float32 and its logits are float32 sums whatever the compute dtype.  An expert's tensors are
    ``e<i>.gate`` / ``.up`` / ``.down``; they are stacked at load, and the tokens of a step are sorted by expert on the device
    (``csrc/experts.cu``), so a step is the same sequence of launches whatever the routing.

    Other forms.  ``gated=False``: an expert is ``down_e(act(up_e(x)))`` and has no gate tensor.  ``routing="sigmoid"``: the scores
    are ``sigmoid(W_r x)``; the ``top`` experts are chosen by score plus a learnt correction (``correction=True``: tensor
    ``correction [experts]``), with ``groups`` only among the experts of the ``groups_keep`` groups of neighbours whose two largest
    choice scores add up to most; the weights are the chosen experts' scores, without the correction, divided by their sum plus
    ``share_eps``.  ``shared_intermediate`` F: one more ungated expert ``shared.up [F, width]`` / ``shared.down`` that every token goes
    through, added times ``sigmoid(w x)``, ``w`` the tensor ``shared.sg [1, width]`` (it rides in the router's product)."""

    def __init__(self, width: int, intermediate: int, experts: int, top: int, activation: str = "silu", router_bias: bool = False,
                 names: Optional[Mapping[str, str]] = None, gated: bool = True, routing: str = "softmax", correction: bool = False,
                 groups: Optional[int] = None, groups_keep: Optional[int] = None, share_eps: float = 0.0,
                 shared_intermediate: Optional[int] = None) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (known: {', '.join(ops.ACTIVATIONS)})")
        self.width, self.intermediate, self.experts, self.top = int(width), int(intermediate), int(experts), int(top)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"a token cannot use {top} of {experts} experts")
        if routing not in ("softmax", "sigmoid"):
            raise ValueError(f"routing is 'softmax' or 'sigmoid', not {routing!r}")
        self.activation, self.router_bias, self.gated, self.routing = activation, bool(router_bias), bool(gated), routing
        self.correction_used = bool(correction)
        self.groups, self.groups_keep = (0, 0) if groups is None else (int(groups), int(groups_keep or groups))
        self.share_eps = float(share_eps)
        self.shared_intermediate = None if shared_intermediate is None else int(shared_intermediate)
        if routing != "sigmoid" and (self.correction_used or self.groups or self.shared_intermediate is not None):
            raise ValueError("a correction, groups of experts and a shared expert go with sigmoid routing")
        if self.groups and (self.experts % self.groups or not 1 <= self.groups_keep <= self.groups or self.top > self.groups_keep * (self.experts // self.groups)):
            raise ValueError(f"{experts} experts in {groups} groups of which {groups_keep} are kept, {top} experts a token")
        self.names = {"router": "router", "router_bias": "router.b", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down",
                      "correction": "correction", "shared_up": "shared.up", "shared_down": "shared.down", "shared_gate": "shared.sg", **(names or {})}
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.correction = self.w_shared_up = self.w_shared_down = None
        self.interleaved = False

    def _expert(self, index: int, key: str) -> str:
        return self.names["expert"].format(index) + self.names[key]

    def tensors(self) -> Sequence[TensorDecl]:
        decls = []
        for e in range(self.experts):
            if self.gated:
                decls.append(TensorDecl(self._expert(e, "gate"), (self.intermediate, self.width)))
            decls += [TensorDecl(self._expert(e, "up"), (self.intermediate, self.width)), TensorDecl(self._expert(e, "down"), (self.width, self.intermediate))]
        decls.append(TensorDecl(self.names["router"], (self.experts, self.width), "vector", (0.0, 0.5)))
        if self.router_bias:
            decls.append(TensorDecl(self.names["router_bias"], (self.experts,), "vector", (0.0, 0.1)))
        if self.correction_used:
            decls.append(TensorDecl(self.names["correction"], (self.experts,), "vector", (0.0, 0.1)))
        if self.shared_intermediate is not None:
            decls += [TensorDecl(self.names["shared_up"], (self.shared_intermediate, self.width)), TensorDecl(self.names["shared_down"], (self.width, self.shared_intermediate)),
                      TensorDecl(self.names["shared_gate"], (1, self.width), "vector", (0.0, 0.5))]
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        # In bfloat16 with silu an expert's gate and up rows alternate in groups of 8, the layout the tcgen05 product's gated epilogue
        # takes (the products for few tokens read either layout); otherwise the two halves lie one after the other.
        self.interleaved = self.gated and dtype == torch.bfloat16 and self.activation == "silu" and self.intermediate % 8 == 0
        if self.gated:
            pair = ops.interleave_gate_up if self.interleaved else (lambda gate, up: torch.cat((gate, up), dim=0))
            self.w_gate_up = torch.stack([pair(tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]) for e in range(self.experts)]).contiguous()
        else:
            self.w_gate_up = torch.stack([tensors[self._expert(e, "up")] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)]).contiguous()
        self.w_router = tensors[self.names["router"]].contiguous()
        self.b_router = tensors[self.names["router_bias"]].contiguous() if self.router_bias else None
        self.correction = tensors[self.names["correction"]].contiguous() if self.correction_used else None
        if self.shared_intermediate is not None:
            self.w_router = torch.cat((self.w_router, tensors[self.names["shared_gate"]]), dim=0).contiguous()   # the gate's row behind the experts' rows
            self.w_shared_up, self.w_shared_down = tensors[self.names["shared_up"]].contiguous(), tensors[self.names["shared_down"]].contiguous()

    def weight_bytes(self) -> int:
        """What a step of many tokens reads: every expert (a step of few tokens reads ``top`` experts a token at most)."""
        shared = 0 if self.w_shared_up is None else self.w_shared_up.numel() + self.w_shared_down.numel()
        return (self.w_gate_up.numel() + self.w_down.numel() + shared) * self.w_down.element_size() + self.w_router.numel() * 4

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        return ops.expert_mixture(h, self.w_router, self.b_router, self.w_gate_up, self.w_down, self.top, self.activation, self.interleaved,
                                  gated=self.gated, routing=self.routing, correction=self.correction, groups=self.groups, groups_keep=self.groups_keep,
                                  share_eps=self.share_eps, common_up=self.w_shared_up, common_down=self.w_shared_down)
