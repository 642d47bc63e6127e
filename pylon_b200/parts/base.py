"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~pylon_b200.parts.spec.PartSpec` (its sizes and constants),
declares the checkpoint tensors it needs by name, receives them in ``load`` and then runs
on the device.  No part knows which model it is in: everything it needs at run time comes
through its constructor parameters, the :class:`StepView` of the current batch and the
:class:`LayerCache` the cache manager hands it.

Kinds of part and the interface each must have:

* **norm** (:class:`Norm`): ``apply(stream, rows=None) -> Tensor`` — fold the stream's
  pending delta into the residual and return the normalised activations.
* **position encoding** (:class:`PositionEncoding`): either ``rotary_table(device)``
  for encodings that are a per-position rotation of (query, key) pairs — the attention
  mixer then fuses them into its own kernel — or ``apply(q, k, step)`` for anything else.
* **mixer** (:class:`Mixer`): ``cache_need()`` says what it keeps between steps (paged keys
  and values, a fixed-size state, both or nothing); ``forward(h, step, cache) -> delta``.
* **feed-forward** (:class:`FeedForward`): ``forward(h, step) -> delta``.
* **block** (:class:`Block`): arranges a mixer, a feed-forward and its norms around the
  residual stream: ``forward(stream, step, cache)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from pylon_b200.parts.spec import PartSpec


# ---------------------------------------------------------------------------------------
# tensors a part asks the loader for
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor a part needs.  ``name`` is relative to the part's prefix.

    ``role`` decides how it is held on the device: ``matrix`` in the compute dtype
    (bfloat16 or float32), ``vector`` (norm weights and the like, used in 32-bit math)
    always in float32, ``table`` (integer tables) in int32.  ``init``: (mean, standard deviation)
    for the random-weights mode where the role's default (matrices N(0, 0.02), vectors
    1 + N(0, 0.02)) would make a degenerate model, e.g. a mixing weight that must lie inside (0, 1).
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: Optional[tuple[float, float]] = None


# ---------------------------------------------------------------------------------------
# what a mixer keeps between steps
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class KVNeed:
    """Paged rows per token: for each of ``n_kv_heads`` heads a key row of ``head_dim`` numbers and a
    value row of ``value_dim`` numbers (``None``: as wide as the key; ``0``: no value rows at all -
    a mixer that keeps one row per token, such as a compressed latent, asks for one head of
    that width and no values).

    ``window``: a query at position p reads keys at positions (p - window, p]; ``None``
    reads all of them.  ``chunk``: a query at position p reads only keys of its own chunk of
    positions, ``[p - p % chunk, p]``.  Either lets the manager give pages back that no later
    token can read.  ``keep_first``: the keys at positions below it stay readable whatever the window says,
    so the pages that hold them are never given back early.  Layers whose KVNeed is equal share a page pool (a cache group).
    """

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None
    chunk: Optional[int] = None
    keep_first: int = 0

    @property
    def bounded(self) -> bool:
        """Whether a token reads only a bounded span of positions before it, however long the request."""
        return self.window is not None or self.chunk is not None

    @property
    def reach(self) -> Optional[int]:
        """The most positions a token reads, itself included (``None``: all of them)."""
        spans = [span for span in (self.window, self.chunk) if span is not None]
        return min(spans) if spans else None

    def first_needed(self, length: int) -> int:
        """The oldest position that the token at position ``length``, or any later one, can read."""
        first = 0
        if self.window is not None:
            first = max(first, length - self.window + 1)
        if self.chunk is not None:
            first = max(first, length - length % self.chunk)
        return first

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per request (``shape`` without the request dimension)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class LayerCache:
    """What the cache manager hands a mixer for one layer and one step.

    ``k_pages``: ``[num_pages, n_kv_heads, page_size, head_dim]`` of this layer; ``v_pages``
    likewise with the value rows' width, or ``None`` if the mixer asked for no value rows.  ``block_table``: int32 ``[rows, width]``, logical page of a row -> physical page
    (-1 where the row holds none, e.g. behind a window).  ``state``: ``[slots, *shape]``;
    a row's state is ``state[step.slots[row]]``.
    """

    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None


class StepView:
    """The batch of one step as the parts see it (all tensors on the device).

    token_ids   int32 [T]     the step's tokens, rows concatenated
    positions   int32 [T]     position of each token in its request
    token_row   int32 [T]     row (request of this step) of each token
    q_start     int32 [R+1]   first token of each row; q_start[R] == T
    kv_len      int32 [R]     tokens the request holds after this step
    slots       int32 [R]     state slot of each row's request
    logit_rows  int32 [L]     tokens whose logits are wanted
    num_tokens, num_rows, num_logits, max_q, max_kv: host integers (upper bounds when the
    step is replayed from a CUDA graph).
    row_tokens: the number of tokens each row brings, as host integers, for parts that plan
    their launches on the host; ``None`` when the step is replayed from a CUDA graph.
    rows_alike: the requests of the step hold about equally many tokens (within an eighth of the
    longest), so that work dealt out evenly by row is dealt out evenly; a hint, never needed for
    a right result.
    padded: the step was padded to the size of a captured CUDA graph.  It may then hold rows
    without tokens (``q_start[r + 1] == q_start[r]``, ``kv_len[r] == 0``, no pages) and, after
    the last row's tokens, padding tokens that belong to no row: ``token_row[t] == -1``, position
    0.  Whatever a part computes for a padding token is never read; it must keep nothing of it
    (no cache write, no state update).  Only models whose parts all say ``takes_padding`` get
    such steps.
    carry: what a part leaves for later parts of the same step, by a name the model's description chooses (the values
    of one layer that later layers mix into their own, say).  Empty at the start of every step.
    """

    token_ids: torch.Tensor
    positions: torch.Tensor
    token_row: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    num_tokens: int
    num_rows: int
    num_logits: int
    max_q: int
    max_kv: int
    dtype: torch.dtype
    device: torch.device
    row_tokens: Optional[tuple] = None
    rows_alike: bool = False
    padded: bool = False

    def __init__(self) -> None:
        self.carry: dict = {}


# ---------------------------------------------------------------------------------------
# base classes
# ---------------------------------------------------------------------------------------
class Part:
    """Common life cycle: construct from parameters, declare tensors, load, run."""

    def tensors(self) -> Sequence[TensorDecl]:
        return ()

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """``tensors``: name (as declared) -> tensor on the device, already in the dtype
        its role asks for."""

    def weight_bytes(self) -> int:
        """Bytes of device memory a step reads from this part's weights."""
        return 0


class Norm(Part):
    def apply(self, stream: "ResidualStream", rows: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Fold what is pending into the stream and return the normalised activations of all tokens, or of ``rows``
        only.  ``read``: for a stream of several copies, the float32 weights ``[copies]`` of the combination that is
        normalised (``None``: their plain sum)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self, device: torch.device) -> Optional[tuple[torch.Tensor, torch.Tensor, int]]:
        """(cos, sin, rotary_dim): float32 ``[positions, rotary_dim // 2]`` tables for
        encodings that rotate pairs ``(j, j + rotary_dim // 2)``; ``None`` otherwise."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, step: StepView) -> None:
        """For encodings without such a table: change ``q [T, heads * d]`` and ``k [T, kv_heads * d]``
        (views with a row stride; already normalised if the mixer has q/k norms) in place, before
        ``k`` is written into the cache."""
        raise NotImplementedError


class Mixer(Part):
    # True if ``forward`` is right for a padded step (see :class:`StepView`): rows without tokens, tokens without a
    # row.  A mixer that indexes its cache or state by ``token_row`` has to look at this; so the default is False, and
    # a model with such a mixer is never padded.
    takes_padding = False

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        """Returns the delta for the residual stream (see :class:`ResidualStream`)."""
        raise NotImplementedError


class FeedForward(Part):
    # A feed-forward works token by token, so padding tokens are usually no concern; one that looks across tokens (a
    # router that balances its load over the batch, say) sets this to False.
    takes_padding = True

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        """Returns the delta for the residual stream (see :class:`ResidualStream`)."""
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    feed_forward: FeedForward

    @property
    def takes_padding(self) -> bool:
        return bool(self.mixer.takes_padding and self.feed_forward.takes_padding)

    def forward(self, stream: "ResidualStream", step: StepView, cache: LayerCache) -> None:
        raise NotImplementedError


@dataclass(frozen=True)
class StreamRoute:
    """How a sublayer's output goes back into a residual stream of several copies, all copies at once from the old ones:
    ``x_t = sum_s mix[s, t] * x_s + scale * out[t] * y``.  ``mix`` float32 ``[copies, copies]`` indexed [from, to],
    ``out`` float32 ``[copies]``, both on the device."""

    mix: torch.Tensor
    out: torch.Tensor


class ResidualStream:
    """The residual sum in float32 plus the delta not yet added to it.

    ``residual`` is ``[T, width]``, or ``[T, copies, width]`` for a model that keeps several copies of the stream
    (hyper-connections).  Parts hand their output to ``add``; the next norm folds it in (one fused kernel reads the
    delta once, updates the 32-bit sum and writes the normalised activations).  A delta is ``[T, width]`` in the
    activation dtype, or float32 partial sums ``[parts, T, width]`` whose sum is the delta (what
    :func:`pylon_b200.kernels.ops.linear_for_residual` may return).  ``add`` may name a factor on the delta and, for
    several copies, the :class:`StreamRoute` by which it enters them.
    """

    def __init__(self, residual: torch.Tensor) -> None:
        self.residual = residual
        self.pending: Optional[torch.Tensor] = None
        self.pending_scale = 1.0
        self.pending_route: Optional[StreamRoute] = None

    @property
    def plain(self) -> bool:
        """One copy, and what is pending is added as it is: the case the fused add + RMSNorm kernels are written for."""
        return self.residual.dim() == 2 and self.pending_scale == 1.0 and self.pending_route is None

    def add(self, delta: torch.Tensor, scale: float = 1.0, route: Optional[StreamRoute] = None) -> None:
        if self.pending is not None:
            self.flush()
        self.pending, self.pending_scale, self.pending_route = delta, float(scale), route

    def take_pending(self) -> tuple[Optional[torch.Tensor], float, Optional[StreamRoute]]:
        pending = (self.pending, self.pending_scale, self.pending_route)
        self.pending, self.pending_scale, self.pending_route = None, 1.0, None
        return pending

    def flush(self) -> None:
        if self.pending is None:
            return
        from pylon_b200.kernels import ops

        if self.plain:
            ops.residual_add(self.residual, self.pending)
            self.pending = None
            return
        delta, scale, route = self.take_pending()
        ops.streams_update_norm(self.residual, delta, scale, None if route is None else route.mix, None if route is None else route.out)

    def total(self) -> torch.Tensor:
        """The stream as one ``[T, width]`` tensor: the sum of its copies, with nothing pending."""
        self.flush()
        return self.residual if self.residual.dim() == 2 else self.residual.sum(dim=1)


# ---------------------------------------------------------------------------------------
# registries
# ---------------------------------------------------------------------------------------
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def decorate(factory: Callable[..., Any]) -> Callable[..., Any]:
            if kind in self._kinds and self._kinds[kind] is not factory:
                raise ValueError(f"{self.what} kind '{kind}' is registered already")
            self._kinds[kind] = factory
            return factory

        return decorate

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec: PartSpec, **extra: Any) -> Any:
        if spec.kind not in self._kinds:
            known = ", ".join(sorted(self._kinds)) or "none"
            raise KeyError(f"unknown {self.what} kind '{spec.kind}' (registered: {known})")
        return self._kinds[spec.kind](**dict(spec.params), **extra)

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
