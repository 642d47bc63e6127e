"""Mixers side by side: several mixers read the same normalised input, and the layer's mixer output is the mean of their
outputs, each first RMS-normed over the model width with a weight of its own:

    y = (1 / n) * sum_i  rmsnorm(mixer_i(h)) * w_i

The mixers are any registered kinds (attention beside a recurrent layer, say).  What they keep between steps is kept side
by side as well: at most one of them may ask for paged keys and values and at most one for a state slot, since a layer run
has one of each.  Norms and mean are one float32 kernel, and the result enters the residual sum in 32-bit.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import MIXERS, CacheNeed, LayerCache, Mixer, StepView, TensorDecl
from pylon_b200.parts.spec import PartSpec


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, width: int, mixers: Sequence[PartSpec], prefixes: Sequence[str], norm_names: Sequence[str], norm_eps: float) -> None:
        if not 1 <= len(mixers) <= 4 or len(prefixes) != len(mixers) or len(norm_names) != len(mixers):
            raise ValueError("one to four mixers side by side, each with a prefix for its tensors and the name of its norm's weight")
        self.width, self.norm_eps = int(width), float(norm_eps)
        self.mixers = [MIXERS.build(spec) for spec in mixers]
        self.prefixes, self.norm_names = tuple(prefixes), tuple(norm_names)
        self.norm_weights: list = [None] * len(self.mixers)
        self.dtype = None

    @property
    def takes_padding(self) -> bool:
        return all(mixer.takes_padding for mixer in self.mixers)

    def tensors(self) -> Sequence[TensorDecl]:
        decls = [TensorDecl(prefix + d.name, d.shape, d.role, d.init) for prefix, mixer in zip(self.prefixes, self.mixers) for d in mixer.tensors()]
        return decls + [TensorDecl(name, (self.width,), "vector") for name in self.norm_names]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, mixer in zip(self.prefixes, self.mixers):
            mixer.load({name[len(prefix):]: tensor for name, tensor in tensors.items() if name.startswith(prefix) and name not in self.norm_names},
                       dtype, device)
        self.norm_weights = [tensors[name].contiguous() for name in self.norm_names]
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return sum(mixer.weight_bytes() for mixer in self.mixers) + 4 * self.width * len(self.mixers)

    def cache_need(self) -> CacheNeed:
        needs = [mixer.cache_need() for mixer in self.mixers]
        pages = [need.kv for need in needs if need.kv is not None]
        states = [need.state for need in needs if need.state is not None]
        if len(pages) > 1 or len(states) > 1:
            raise NotImplementedError("of mixers side by side, one may keep paged keys and values and one a state slot")
        return CacheNeed(kv=pages[0] if pages else None, state=states[0] if states else None)

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        outputs = [mixer.forward(h, step, cache) for mixer in self.mixers]   # each takes from the layer's cache what it asked for
        return ops.mean_of_normed(outputs, self.norm_weights, self.norm_eps, self.dtype)


@MIXERS.register("weighted_mixers")
class WeightedMixers(ParallelMixers):
    """Mixers side by side whose outputs are added, each times a fixed factor: ``y = sum_i scale_i * mixer_i(h)``, one float32
    kernel whose result enters the residual sum in 32-bit.  No norms, so no tensors beyond the mixers' own."""

    def __init__(self, mixers: Sequence[PartSpec], prefixes: Sequence[str], scales: Sequence[float]) -> None:
        if not 1 <= len(mixers) <= 4 or len(prefixes) != len(mixers) or len(scales) != len(mixers):
            raise ValueError("one to four mixers side by side, each with a prefix for its tensors and a factor")
        self.mixers = [MIXERS.build(spec) for spec in mixers]
        self.prefixes, self.norm_names = tuple(prefixes), ()
        self.scales = tuple(float(scale) for scale in scales)

    def tensors(self) -> Sequence[TensorDecl]:
        return [TensorDecl(prefix + d.name, d.shape, d.role, d.init) for prefix, mixer in zip(self.prefixes, self.mixers) for d in mixer.tensors()]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, mixer in zip(self.prefixes, self.mixers):
            mixer.load({name[len(prefix):]: tensor for name, tensor in tensors.items() if name.startswith(prefix)}, dtype, device)
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return sum(mixer.weight_bytes() for mixer in self.mixers)

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        outputs = [mixer.forward(h, step, cache) for mixer in self.mixers]
        return ops.weighted_sum(outputs, self.scales, self.dtype)
