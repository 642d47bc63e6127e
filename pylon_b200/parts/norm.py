"""RMSNorm over the residual stream.

``y = x / sqrt(mean(x^2) + eps) * weight`` in float32, as raun6k/Pylon's ``RMSNorm``
(src/pylon/model/layers.py:30-40).  The norm is where a pending delta joins the 32-bit
residual sum, so add and norm are one kernel.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import NORMS, Norm, ResidualStream, TensorDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """``offset``: the checkpoint stores the weight less this number (a checkpoint that holds the weight's difference from one has ``offset=1``:
    ``y = x / rms(x) * (1 + w)``); the sum is formed once at load, in float32."""

    def __init__(self, width: int, eps: float, weight_name: str = "weight", offset: float = 0.0) -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None

    def tensors(self) -> Sequence[TensorDecl]:
        init = None if self.offset == 0.0 else (1.0 - self.offset, 0.02)
        return (TensorDecl(self.weight_name, (self.width,), "vector", init),)

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        weight = tensors[self.weight_name]
        self.weight = (weight if self.offset == 0.0 else weight + self.offset).contiguous()
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return self.width * 4

    def apply(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not stream.plain:
            return _apply_to_streams(self, "rmsnorm", stream, rows, read)
        delta, stream.pending = stream.pending, None
        # With a row selection the residual stays untouched and the delta is added on the fly.
        return ops.add_rmsnorm(stream.residual, delta, self.weight, self.eps, self.dtype, rows=rows)


def _apply_to_streams(norm, kind: str, stream: ResidualStream, rows: Optional[torch.Tensor], read: Optional[torch.Tensor]) -> torch.Tensor:
    """The general form: one or several copies of the stream, a factor on the pending delta, a route by which it enters
    the copies, the combination of copies that is read, layer norm or RMS norm - one kernel."""
    if rows is None:
        delta, scale, route = stream.take_pending()
    else:   # the stream stays as it is: what is pending stays pending
        delta, scale, route = stream.pending, stream.pending_scale, stream.pending_route
    return ops.streams_update_norm(
        stream.residual, delta, scale, None if route is None else route.mix, None if route is None else route.out, read,
        norm.weight, norm.eps, kind, norm.dtype, rows=rows,
    )


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight`` in float32, the variance being the mean of the squared deviations;
    a weight and no bias.  Like :class:`RMSNorm` it is where a pending delta joins the residual stream."""

    def __init__(self, width: int, eps: float, weight_name: str = "weight") -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None

    def tensors(self) -> Sequence[TensorDecl]:
        return (TensorDecl(self.weight_name, (self.width,), "vector"),)

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return self.width * 4

    def apply(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None) -> torch.Tensor:
        return _apply_to_streams(self, "layernorm", stream, rows, read)


@NORMS.register("dynamic_tanh")
class DynamicTanh(Norm):
    """A norm without statistics: ``tanh(alpha * x) * weight + bias`` in float32, ``alpha`` one learnt number, ``weight`` and ``bias``
    vectors of the width.  Nothing is summed over the row, so there is no eps.  Like the other norms it is where a pending delta
    joins the residual stream.  The three tensors are the part's prefix plus ``weight_name``, ``alpha_name`` and ``bias_name``."""

    def __init__(self, width: int, weight_name: str = "weight", alpha_name: str = "alpha", bias_name: str = "bias") -> None:
        self.width = int(width)
        self.weight_name, self.alpha_name, self.bias_name = weight_name, alpha_name, bias_name
        self.eps = 0.0
        self.weight = self.alpha = self.bias = None
        self.dtype: Optional[torch.dtype] = None

    def tensors(self) -> Sequence[TensorDecl]:
        return (TensorDecl(self.weight_name, (self.width,), "vector"), TensorDecl(self.alpha_name, (), "vector", (0.5, 0.05)),
                TensorDecl(self.bias_name, (self.width,), "vector", (0.0, 0.02)))

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        self.weight, self.bias = tensors[self.weight_name].contiguous(), tensors[self.bias_name].contiguous()
        self.alpha = tensors[self.alpha_name].reshape(1).contiguous()
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return self.width * 8 + 4

    def apply(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is None:
            delta, scale, route = stream.take_pending()
        else:   # the stream stays as it is: what is pending stays pending
            delta, scale, route = stream.pending, stream.pending_scale, stream.pending_route
        return ops.streams_update_norm(
            stream.residual, delta, scale, None if route is None else route.mix, None if route is None else route.out, read,
            self.weight, 0.0, "dynamic_tanh", self.dtype, rows=rows, norm_bias=self.bias, norm_alpha=self.alpha,
        )
