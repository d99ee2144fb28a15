"""What every part is, and the registries that turn a plan's kinds into parts.

A part owns its constants (given as arguments, never read from a model class),
names the tensors it needs, loads them, and runs on the flat rows of one step.
No part knows which model it is in: a mixer sees rows, the step's per-token and
per-sequence tables (:class:`StepContext`) and its own cache line.

Interfaces
----------
``Norm.forward(ctx, x, delta=None, rows=None, want32=False, write_back=True)``
    x is the float32 residual stream [T, width]; ``delta`` (float32) is added to
    it first (and stored back when ``write_back``); returns the normed rows in the
    model dtype and, if ``want32``, in float32 too.
``Mixer.forward(ctx, act, line, writes_cache)`` -> float32 update [T, width]
    ``line`` is the :class:`~fieldrun_b200.cache.LineView` of the run's cache line.
``Mixer.cache_need()`` -> :class:`~fieldrun_b200.cache.CacheNeed`
``FeedForward.forward(ctx, act, act32)`` -> float32 update [T, width]
``Position.tables(num_positions, device)`` -> (cos, sin) float32 [positions, dim/2]
``Block.forward(ctx, x, pending, line, writes_cache)`` -> (x, pending)
    ``pending`` is an update not yet added to x, so that the next norm adds it.
"""
from __future__ import annotations

import json
import weakref
from typing import Any, Callable, Mapping, Optional

import torch

from ..cache import CacheNeed, LineView
from ..config.plan import PartSpec
from ..weights.loader import TensorNeed, TensorSource


class Part:
    """Base of all parts: constants in, tensors by name, rows through.

    ``replayable`` says that the part's ``forward`` reads the step's tables only on the device
    (``ctx.tok_pos`` and the like, never the host lists) and makes every decision from shapes.  A step of
    such parts can be recorded once as a CUDA graph and run again with other positions and slots.  A part
    that leaves it False is always run directly."""

    replayable: bool = False

    def __init__(self, spec: PartSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype

    def tensor_needs(self) -> list[TensorNeed]:
        return []

    def load(self, source: TensorSource) -> None:
        pass

    def name_of(self, local: str) -> str:
        try:
            return self.spec.tensors[local]
        except KeyError:
            raise KeyError(f"part {self.spec.kind!r} was given no checkpoint name for its tensor {local!r}") from None


class DeferredUpdate:
    """An update of the residual stream that its maker has not summed up yet, so that the norm which adds it
    can do the sum while it reads the stream.  ``materialize`` gives the plain float32 tensor [T, width]; any
    norm can take any deferred update that way."""

    def materialize(self, ctx) -> torch.Tensor:
        raise NotImplementedError


class WeightedRows(DeferredUpdate):
    """The one deferred form that norms may sum themselves: update[t] = sum over r < k, in the order of r, of
    ``weights[t, r] * rows[row_map[t * k + r]]`` (float32 ``rows`` [N, width], float32 ``weights`` [T, k],
    int32 ``row_map`` [T * k]).  Any part may make one: routed experts do (a token's experts in rank order,
    src/minimax.rs:121-123), and so may a mixer that blends several candidates per token.  A norm that
    cannot take it, or not with this ``k``, calls ``materialize``."""

    def __init__(self, rows: torch.Tensor, weights: torch.Tensor, row_map: torch.Tensor):
        self.rows, self.weights, self.row_map = rows, weights, row_map

    @property
    def top_k(self) -> int:
        return int(self.weights.shape[-1])

    def materialize(self, ctx) -> torch.Tensor:
        from ..csrc import ops
        out = ctx.buffer("weighted_rows.sum", (self.weights.shape[0], self.rows.shape[1]), torch.float32)
        ops.expert_combine(self.rows, self.weights, self.row_map, out)
        return out


def as_tensor(ctx, update):
    """The update as a float32 tensor, whatever form it came in (None stays None)."""
    return update.materialize(ctx) if isinstance(update, DeferredUpdate) else update


class Norm(Part):
    accepts_deferred: bool = False       # whether ``delta`` may be a DeferredUpdate of a kind this norm knows

    def forward(self, ctx, x: torch.Tensor, *, delta=None,
                rows: Optional[torch.Tensor] = None, want32: bool = False, write_back: bool = True):
        raise NotImplementedError


class Position:
    """A position encoding handed to a mixer: it fills the tables the mixer's kernel rotates with.
    ``build_position`` gives mixers whose position arguments are equal one and the same object, and
    ``shared_tables`` makes that object's tables once per (length, device): the layers of a model read one
    pair of tables, not one pair each."""

    rotary_dim: int = 0
    interleaved: bool = False

    def tables(self, num_positions: int, device) -> tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        raise NotImplementedError

    def shared_tables(self, num_positions: int, device) -> tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        made = self.__dict__.setdefault("_tables_made", {})
        key = (int(num_positions), str(torch.device(device)))
        if key not in made:
            made.clear()                      # one length at a time: a model's cache is sized once
            made[key] = self.tables(num_positions, device)
        return made[key]


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def prepare(self, num_positions: int, device) -> None:
        """Called once the cache's size is known (tables over positions are made here)."""

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    wants_float32_input: bool = False

    def forward(self, ctx, act: torch.Tensor, act32: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def forward_deferred(self, ctx, act: torch.Tensor, act32: Optional[torch.Tensor]):
        """Like ``forward``, but may return a :class:`DeferredUpdate`."""
        return self.forward(ctx, act, act32)


class Block:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, ctx, x, pending, line: LineView, writes_cache: bool):
        raise NotImplementedError


_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def register_part(category: str, kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    """Make ``kind`` buildable.  ``factory(spec, dtype)`` for parts with tensors, ``factory(args)`` for a
    position encoding, ``factory(mixer, feed_forward, mixer_norm, feed_forward_norm)`` for a block."""
    table = _REGISTRIES[category]
    if kind in table and not replace:
        raise ValueError(f"{category} {kind!r} is already registered")
    table[kind] = factory


def registered(category: str) -> list[str]:
    return sorted(_REGISTRIES[category])


def _factory(category: str, kind: str):
    try:
        return _REGISTRIES[category][kind]
    except KeyError:
        raise KeyError(f"no {category} of kind {kind!r} is registered; registered: {registered(category)}") from None


def build_part(category: str, spec: PartSpec, dtype: torch.dtype):
    return _factory(category, spec.kind)(spec, dtype)


_POSITIONS: "weakref.WeakValueDictionary[str, Position]" = weakref.WeakValueDictionary()


def build_position(args: Optional[Mapping[str, Any]]) -> Optional[Position]:
    """The position encoding of ``args``; equal arguments give the same object while a mixer still holds it."""
    if not args:
        return None
    factory = _factory("position", args["kind"])
    try:
        key = f"{id(factory)}:" + json.dumps(dict(args), sort_keys=True, default=repr)
    except (TypeError, ValueError):
        return factory(args)
    position = _POSITIONS.get(key)
    if position is None:
        position = factory(args)
        try:
            _POSITIONS[key] = position
        except TypeError:                     # an object that cannot be weakly referenced is simply not shared
            pass
    return position


def build_block(kind: str, mixer, feed_forward, mixer_norm, feed_forward_norm) -> Block:
    return _factory("block", kind)(mixer, feed_forward, mixer_norm, feed_forward_norm)
