"""Interfaces of the parts a layer is put together from, and their registry.

Five categories, each with one small interface:

``norm``          ``forward(stream, rows=None) -> Tensor``: applies the pending
                  residual delta, returns the normed rows in the model dtype.
``position``      ``encode_and_store(qkv, heads, kv_heads, head_dim, ctx, cache, dtype) -> q``:
                  encodes positions into Q and K of a fused qkv matrix (given in
                  the model dtype or as float32 partial sums [S, N, width]), puts
                  K, V into the layer's cache pages and returns Q [N, heads*head_dim].
``mixer``         ``cache_request() -> PagedKV | SlotState | None`` and
                  ``forward(x, ctx, cache) -> Tensor [N, hidden]``.
``feed_forward``  ``forward(x, ctx) -> Tensor [N, hidden]``.
``block``         ``forward(stream, ctx, cache) -> None``: the arrangement of the
                  four above around the residual stream.  A block kind declares the
                  places it has (``slots``: place name -> category); a layer's
                  ``LayerSpec.parts`` fills exactly those.

Every part is constructed from a ``PartSpec`` (kind + parameters) alone, names
its tensors with ``param_specs()`` and receives them in ``load()``.  A part
never sees the model configuration, the architecture's name or another layer.
New kinds are added with ``register_part(category, kind, cls)``; nothing else in
the package has to change.

A step can be recorded once (a CUDA graph) and replayed: steps in which every
request brings one token share a recording per bucket of requests, other steps
get one at their exact counts when their shape comes again.  A replay runs no
Python, so whatever a part decides on the
host from the step's facts has to be the same for every step that replays one
recording: ``capture_key(host)`` returns a hashable that determines all such
decisions (kernel choice, grid sizes), or ``NOT_CAPTURABLE`` (the default) for a
part whose ``forward`` works on the host per request, synchronises or allocates
by data.  The engine records one step per distinct tuple of keys and sends
steps with a part that cannot be captured to the launched path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Hashable, Mapping, Optional, Tuple

import torch

from yalis_b200.config.spec import PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    ``init`` says what the random-weights mode writes: ``normal`` = N(0, 0.02)
    (the reference's GPT._init_weights, yalis/external/model.py:113-120),
    ``ones`` or ``zeros``.  ``keep_float32``: held in float32 whatever the
    engine's dtype (norm scales).  ``integer``: an integer table, held as int32.
    """

    shape: Tuple[int, ...]
    init: str = "normal"
    keep_float32: bool = False
    integer: bool = False


# ---- what a mixer may ask of the cache manager ---------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values in pages. ``window`` None keeps every key; W keeps, for a
    query at position p, the keys at positions > p - W."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotState:
    """A tensor of fixed shape per request (zeroed when the request is admitted)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class PagedKVCache:
    """What a paged mixer gets for one schedule entry: its two pools
    [pages, kv_heads, page_size, head_dim] and the name of its page group, under
    which the step context holds the block tables.  ``writable`` is False for an
    entry that reads the cache of another entry."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, group: str, writable: bool = True):
        self.k, self.v, self.group, self.writable = k, v, group, writable

    @property
    def page_size(self) -> int:
        return self.k.shape[2]


class SlotStateCache:
    """What a stateful mixer gets: ``state`` [max_slots + 1, *shape]; rows are indexed
    by the step context's ``slots``.  The last row belongs to no request: the padding
    rows of a recorded step point there, so a kernel may update ``state[ctx.slots]``
    for every row of the step without a test."""

    def __init__(self, state: torch.Tensor, writable: bool = True):
        self.state, self.writable = state, writable


# ---- the residual stream ----------------------------------------------------------

class ResidualStream:
    """The float32 residual stream [N, hidden] with one pending delta.

    A sub-layer's output is not added at once: it is parked in ``pending`` and
    the next norm adds it while it reads the stream (one pass instead of two).
    ``pending`` is [N, hidden] in the model dtype, or float32 split partial sums
    [S, N, hidden] that are added in order.
    """

    def __init__(self, x: torch.Tensor, dtype: torch.dtype):
        self.x = x
        self.dtype = dtype
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        self.flush()
        self.pending = delta

    def flush(self) -> None:
        if self.pending is not None:
            from yalis_b200.ops.elementwise import residual_add
            residual_add(self.x, self.pending)
            self.pending = None


# ---- parts ---------------------------------------------------------------------------

class _NotCapturable:
    def __repr__(self) -> str:
        return "NOT_CAPTURABLE"


NOT_CAPTURABLE = _NotCapturable()   # answer of Part.capture_key: run this part's steps launch by launch


class Part:
    category = ""

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by param_specs(), on the device, in the engine's dtype."""

    def capture_key(self, host) -> Hashable:
        """What a recorded step of this part depends on beyond the shapes of its tensors (see the module
        docstring).  ``host`` is the step's ``HostStep``.  Return None when ``forward`` launches the same
        kernels whatever the requests' lengths are."""
        return NOT_CAPTURABLE

    def matrix_flops_per_token(self) -> float:
        """Floating-point operations per token in this part's matrix products (2 per weight of every 2-D tensor)."""
        return float(sum(2 * ps.shape[0] * ps.shape[1] for ps in self.param_specs().values() if len(ps.shape) == 2))


class Norm(Part):
    category = "norm"

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        """The norm of a plain tensor [N, width] in its own dtype (for arrangements that norm a sub-layer's
        output rather than the stream)."""
        raise NotImplementedError


NOT_ROTARY = object()     # answer of PositionEncoding.rotary_frequencies for encodings a mixer's kernel cannot apply itself


class PositionEncoding(Part):
    category = "position"

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        raise NotImplementedError

    def rotary_frequencies(self, head_dim: int, device):
        """For mixers whose kernel can encode positions itself (one launch less): the float32 inverse
        frequencies [head_dim / 2] of a half-split rotary encoding with angle position * frequency, ``None``
        for "store and use Q, K unrotated", or ``NOT_ROTARY`` (the default) for anything else - the mixer
        then calls ``encode_and_store``."""
        return NOT_ROTARY


class Mixer(Part):
    category = "mixer"

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec)
        self.position = position

    def cache_request(self):
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        """Floating-point operations, beyond the matrix products, of ``q_len`` tokens fed after ``ctx_before``
        cached ones (for rooflines; 0 when the mixer has none worth counting)."""
        return 0.0


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of parts around the residual stream.

    ``slots`` names the places of the arrangement and the category of part each takes; the layer's
    ``LayerSpec.parts`` must fill exactly these.  The built parts arrive as a dictionary and are also set as
    attributes (``self.mixer`` ...).  A place of category ``position`` is built first and handed to the
    block's mixers.  A block keeps at most one cache: what its ``cache_request`` returns (by default its
    mixer's request, or nothing when it has no mixer).
    """

    category = "block"
    slots: Mapping[str, str] = {}

    def __init__(self, spec: PartSpec, parts: Dict[str, Part]):
        super().__init__(spec)
        self.parts = dict(parts)
        for name, part in self.parts.items():
            setattr(self, name, part)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        raise NotImplementedError

    def cache_request(self):
        mixers = [p for p in self.parts.values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise NotImplementedError("a block with several mixers must say itself what it caches")
        return mixers[0].cache_request() if mixers else None

    def capture_key(self, host) -> Hashable:
        keys = []
        for part in self.parts.values():
            key = part.capture_key(host)
            if key is NOT_CAPTURABLE:
                return NOT_CAPTURABLE
            keys.append(key)
        return tuple(keys)


def build_block(layer) -> Block:
    """The block of a ``LayerSpec`` with all its parts."""
    _ensure_builtin()
    try:
        factory = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY["block"])) or "none"
        raise ValueError(f"no block of kind {layer.block.kind!r} is registered (known: {known})") from None
    slots = dict(getattr(factory, "slots", {}))
    missing = [n for n in slots if n not in layer.parts]
    unknown = [n for n in layer.parts if n not in slots]
    if missing or unknown:
        raise ValueError(f"block kind {layer.block.kind!r} has the places {sorted(slots)}: "
                         + (f"the layer fills none of {missing}" if missing else "")
                         + ("; " if missing and unknown else "")
                         + (f"the layer names {unknown}, which the block does not have" if unknown else ""))
    built: Dict[str, Part] = {}
    positions = [n for n, c in slots.items() if c == "position"]
    for name in positions:
        built[name] = make_part("position", layer.parts[name])
    position = built[positions[0]] if len(positions) == 1 else None
    for name, category in slots.items():
        if category == "position":
            continue
        extra = {"position": position} if category == "mixer" else {}
        built[name] = make_part(category, layer.parts[name], **extra)
    ordered = {name: built[name] for name in slots}
    return factory(layer.block, ordered)


# ---- registry ---------------------------------------------------------------------------

_REGISTRY: Dict[str, Dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r} (one of {', '.join(CATEGORIES)})")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _REGISTRY[category][kind] = factory


def make_part(category: str, spec: PartSpec, **kwargs: Any) -> Part:
    _ensure_builtin()
    try:
        factory = _REGISTRY[category][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "none"
        raise ValueError(f"no {category} of kind {spec.kind!r} is registered (known: {known})") from None
    return factory(spec, **kwargs)


def registered(category: str) -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_REGISTRY[category]))


def _ensure_builtin() -> None:
    from yalis_b200.parts import attention, block, norm, rotary, swiglu  # noqa: F401
