"""Interfaces of the parts and the registries that map a spec's `kind` to a class.

A part is built from its spec, its tensors and the kernel set (`ops`); it never sees
the model it sits in.  A mixer tells the cache manager what it has to remember
through `cache_need`: keys and values per token in pages (`PagedNeed`), a record of
fixed size per request (`StateNeed`), or nothing.

Buffers for activation rows that a matrix product will read (`[tokens, width]` outputs of
a norm, an activation, a mixer's inner stage) come from `ops.new_rows(n, width, dtype,
device)` rather than `torch.empty`: the kernel set may leave room behind them so that the
matrix library is shown row counts it has met before.  Any tensor still works as a
product's input; it is then copied once.

Adding a part: subclass the interface, give `params` and (for a mixer) `cache_need`,
and call the matching `register_*` with the `kind` string its spec carries.  Nothing
else in the package has to change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

from .spec import ParamDecl


@dataclass(frozen=True)
class PagedNeed:
    """Keys and values of every token (or of the last `window` tokens), in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A float32 record of this shape per live request.  The cache manager hands a request
    its slot with the record cleared to zero, so the state before position 0 is zero
    without the mixer's doing."""
    shape: Tuple[int, ...]


class Mixer:
    """mixer(normed[N, hidden], ctx, cache) -> [N, hidden]

    `ctx` is the step's `StepContext` (token positions, request boundaries, the
    kernels); `cache` is the `CacheView` of this call in the run order or None.
    """

    @staticmethod
    def params(spec, owns_cache: bool = True) -> Dict[str, ParamDecl]:
        """Tensors by local name.  `owns_cache` is false when every call of the block
        reads another call's cache, so tensors that only fill a cache are not needed."""
        raise NotImplementedError

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def workspace_bytes(spec, ops, max_requests: int, max_context: int) -> int:
        """Bytes of kernel scratch the mixer's launches can need at most with
        `max_requests` requests of up to `max_context` cached tokens in a step.  The
        runner reserves the largest answer once, before it captures any launch sequence."""
        return 0

    def __init__(self, spec, tensors, ops, dtype):
        raise NotImplementedError

    def forward(self, normed, ctx, cache):
        raise NotImplementedError


class FeedForward:
    """feed_forward(normed[N, hidden], ctx) -> [N, hidden]"""

    @staticmethod
    def params(spec) -> Dict[str, ParamDecl]:
        raise NotImplementedError

    def __init__(self, spec, tensors, ops, dtype):
        raise NotImplementedError

    def forward(self, normed, ctx):
        raise NotImplementedError


class Norm:
    """norm.add_norm(resid, delta, ctx, rows=None) adds `delta` (or nothing) to the
    float32 residual stream in place and returns the normalised rows in the compute
    dtype; with `rows` it reads only those rows and leaves the stream untouched.
    norm.norm(x, ctx) normalises rows that are not part of the stream."""

    @staticmethod
    def params(spec) -> Dict[str, ParamDecl]:
        raise NotImplementedError

    def __init__(self, spec, tensors, ops, dtype):
        raise NotImplementedError

    def add_norm(self, resid, delta, ctx, rows=None):
        raise NotImplementedError

    def norm(self, x, ctx):
        """The normalised rows of `x` (compute dtype), with no residual stream involved:
        what a norm placed after a sub-layer applies to its output."""
        raise NotImplementedError


class PositionEncoding:
    """A position encoding the attention mixer can apply to q and k.

    `rotation_table()` returns (cos, sin), float32 [max_position, head_dim/2], of a
    rotation that pairs dimension i with i + head_dim/2, or None for no encoding.
    """

    def __init__(self, spec, device):
        raise NotImplementedError

    def rotation_table(self):
        raise NotImplementedError


class Arrangement:
    """How a block wires norm, mixer and feed-forward around the residual stream.

    forward(stream, ctx, cache) -> stream, where `stream` is a `Stream`: the float32
    residual plus the last sub-layer's output that is still to be added (so that the
    addition can be fused into the next norm).
    """

    @staticmethod
    def params(spec, owns_cache: bool = True) -> Dict[str, ParamDecl]:
        """Full tensor names -> declarations for one block."""
        raise NotImplementedError

    def __init__(self, spec, tensors, ops, dtype):
        raise NotImplementedError

    def forward(self, stream, ctx, cache):
        raise NotImplementedError


@dataclass
class Stream:
    resid: object                   # float32 [N, hidden]
    pending: Optional[object]       # compute dtype [N, hidden], not yet added


_MIXERS: Dict[str, type] = {}
_FEED_FORWARDS: Dict[str, type] = {}
_NORMS: Dict[str, type] = {}
_POSITIONS: Dict[str, type] = {}
_ARRANGEMENTS: Dict[str, type] = {}


def _register(table: Dict[str, type], what: str) -> Callable:
    def register(kind: str, cls: type, replace: bool = False) -> type:
        if kind in table and table[kind] is not cls and not replace:
            raise ValueError(f"{what} kind {kind!r} is already registered")
        table[kind] = cls
        return cls
    return register


def _lookup(table: Dict[str, type], what: str) -> Callable:
    def lookup(kind: str) -> type:
        if kind not in table:
            raise KeyError(f"unknown {what} kind {kind!r} (registered: {sorted(table)})")
        return table[kind]
    return lookup


register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
register_arrangement = _register(_ARRANGEMENTS, "arrangement")
mixer_class = _lookup(_MIXERS, "mixer")
feed_forward_class = _lookup(_FEED_FORWARDS, "feed-forward")
norm_class = _lookup(_NORMS, "norm")
position_class = _lookup(_POSITIONS, "position encoding")
arrangement_class = _lookup(_ARRANGEMENTS, "arrangement")
