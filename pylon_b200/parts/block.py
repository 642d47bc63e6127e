"""Block arrangements: how a mixer, a feed-forward and their norms sit on the residual stream.

``prenorm`` is raun6k/Pylon's ``TransformerBlock`` (src/pylon/model/layers.py:168-200):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.  The adds are deferred to the next norm
(see :class:`~pylon_b200.parts.base.ResidualStream`).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.parts.base import (
    BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, LayerCache, ResidualStream, StepView, StreamRoute, TensorDecl,
)
from pylon_b200.parts.spec import PartSpec


def _prefixed(prefix: str, decls: Sequence[TensorDecl]) -> list[TensorDecl]:
    return [TensorDecl(prefix + d.name, d.shape, d.role, d.init) for d in decls]


def _strip(prefix: str, tensors: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {name[len(prefix):]: tensor for name, tensor in tensors.items() if name.startswith(prefix)}


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """Sub-parts keep their tensors under the given sub-prefixes of the layer's prefix."""

    def __init__(
        self,
        mixer: PartSpec,
        feed_forward: PartSpec,
        mixer_norm: PartSpec,
        ffn_norm: PartSpec,
        mixer_prefix: str = "self_attn.",
        ffn_prefix: str = "mlp.",
        mixer_norm_prefix: str = "input_layernorm.",
        ffn_norm_prefix: str = "post_attention_layernorm.",
    ) -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.ffn_norm = NORMS.build(ffn_norm)
        self._children = (
            (mixer_prefix, self.mixer), (ffn_prefix, self.feed_forward),
            (mixer_norm_prefix, self.mixer_norm), (ffn_norm_prefix, self.ffn_norm),
        )

    def tensors(self) -> Sequence[TensorDecl]:
        return [decl for prefix, part in self._children for decl in _prefixed(prefix, part.tensors())]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, part in self._children:
            part.load(_strip(prefix, tensors), dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for _, part in self._children)

    def forward(self, stream: ResidualStream, step: StepView, cache: LayerCache) -> None:
        stream.add(self.mixer.forward(self.mixer_norm.apply(stream), step, cache))
        stream.add(self.feed_forward.forward(self.ffn_norm.apply(stream), step))


@BLOCKS.register("hyper_prenorm")
class HyperPreNormBlock(Block):
    """A pre-norm layer over a residual stream of one or several copies, the sublayers' outputs times a factor.

    With ``streams`` copies x_1 .. x_S (hyper-connections), sublayer q (1: the mixer, 2: the feed-forward) reads
    ``u = sum_s in_q[s] x_s`` through its norm and its output y goes back into all copies at once, from the old ones:
    ``x_t = sum_s mix_q[s, t] x_s + residual_mult * out_q[t] * y`` (``mix`` is indexed [from, to]).  The three small
    tensors of sublayer q are ``<route_prefix><q>.in`` / ``.out`` / ``.mix``.  With ``streams=None`` there is the one
    residual sum and no such tensors: ``x = x + residual_mult * y``.  ``feed_forward=None`` leaves the second sublayer
    (and its norm) out.  Update and next read are one kernel, as add and norm are in :class:`PreNormBlock`.
    """

    def __init__(
        self,
        mixer: PartSpec,
        feed_forward: Optional[PartSpec],
        mixer_norm: PartSpec,
        ffn_norm: Optional[PartSpec],
        streams: Optional[int] = None,
        residual_mult: float = 1.0,
        mixer_prefix: str = "mix.",
        ffn_prefix: str = "mlp.",
        mixer_norm_prefix: str = "norm1",
        ffn_norm_prefix: str = "norm2",
        route_prefix: str = "hc",
    ) -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.mixer_norm = NORMS.build(mixer_norm)
        self.ffn_norm = NORMS.build(ffn_norm) if feed_forward is not None else None
        self.streams = None if streams is None else int(streams)
        if self.streams is not None and self.streams < 1:
            raise ValueError("a residual stream has at least one copy")
        self.residual_mult = float(residual_mult)
        self.route_prefix = route_prefix
        self._children = [(mixer_prefix, self.mixer), (mixer_norm_prefix, self.mixer_norm)]
        if self.feed_forward is not None:
            self._children += [(ffn_prefix, self.feed_forward), (ffn_norm_prefix, self.ffn_norm)]
        self._sublayers = (1, 2) if self.feed_forward is not None else (1,)
        self.read: dict[int, Optional[torch.Tensor]] = {q: None for q in self._sublayers}
        self.route: dict[int, Optional[StreamRoute]] = {q: None for q in self._sublayers}

    @property
    def takes_padding(self) -> bool:
        return bool(self.mixer.takes_padding and (self.feed_forward is None or self.feed_forward.takes_padding))

    def tensors(self) -> Sequence[TensorDecl]:
        decls = [decl for prefix, part in self._children for decl in _prefixed(prefix, part.tensors())]
        if self.streams is not None:
            for q in self._sublayers:
                decls += [
                    TensorDecl(f"{self.route_prefix}{q}.in", (self.streams,), "vector", (1.0 / self.streams, 0.1)),
                    TensorDecl(f"{self.route_prefix}{q}.out", (self.streams,), "vector", (1.0, 0.1)),
                    TensorDecl(f"{self.route_prefix}{q}.mix", (self.streams, self.streams), "vector", (1.0 / self.streams, 0.1)),
                ]
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, part in self._children:
            part.load(_strip(prefix, tensors), dtype, device)
        if self.streams is not None:
            for q in self._sublayers:
                name = f"{self.route_prefix}{q}."
                self.read[q] = tensors[name + "in"].contiguous()
                self.route[q] = StreamRoute(tensors[name + "mix"].contiguous(), tensors[name + "out"].contiguous())

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for _, part in self._children)

    def forward(self, stream: ResidualStream, step: StepView, cache: LayerCache) -> None:
        copies = 1 if stream.residual.dim() == 2 else stream.residual.shape[1]
        if copies != (self.streams or 1):
            raise ValueError(f"the layer is built for {self.streams or 1} copies of the residual stream, the model runs {copies}")
        stream.add(self.mixer.forward(self.mixer_norm.apply(stream, read=self.read[1]), step, cache), self.residual_mult, self.route[1])
        if self.feed_forward is not None:
            stream.add(self.feed_forward.forward(self.ffn_norm.apply(stream, read=self.read[2]), step), self.residual_mult, self.route[2])


@BLOCKS.register("parallel_sublayers")
class ParallelSublayers(Block):
    """One norm, two readers: with ``h = norm(x)`` the layer is ``x = x + (mixer(h) + feed_forward(h))``.  Both outputs join the
    32-bit residual sum (the mixer's first, the feed-forward's at the next norm); ``feed_forward=None`` leaves the second out.
    The tensors: the mixer's under ``mixer_prefix``, the feed-forward's under ``ffn_prefix``, the norm's under ``norm_prefix``."""

    def __init__(self, mixer: PartSpec, feed_forward: Optional[PartSpec], norm: PartSpec, mixer_prefix: str = "mix.", ffn_prefix: str = "mlp.",
                 norm_prefix: str = "norm1") -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.norm = NORMS.build(norm)
        self._children = [(mixer_prefix, self.mixer), (norm_prefix, self.norm)]
        if self.feed_forward is not None:
            self._children.append((ffn_prefix, self.feed_forward))

    @property
    def takes_padding(self) -> bool:
        return bool(self.mixer.takes_padding and (self.feed_forward is None or self.feed_forward.takes_padding))

    def tensors(self) -> Sequence[TensorDecl]:
        return [decl for prefix, part in self._children for decl in _prefixed(prefix, part.tensors())]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, part in self._children:
            # the norm's own tensor is the bare prefix: it must not take the mixer's or the feed-forward's for its own
            mine = {name: tensor for name, tensor in _strip(prefix, tensors).items() if name in {decl.name for decl in part.tensors()}}
            part.load(mine, dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for _, part in self._children)

    def forward(self, stream: ResidualStream, step: StepView, cache: LayerCache) -> None:
        h = self.norm.apply(stream)
        stream.add(self.mixer.forward(h, step, cache))
        if self.feed_forward is not None:
            stream.add(self.feed_forward.forward(h, step))
