"""Architecture-neutral description of a model: which parts, in which order.

A model is data.  ``ModelSpec`` lists the layers; each ``LayerSpec`` names, by
kind and parameters, the block arrangement and the parts inside it (mixer,
feed-forward, norms, position encoding; which of them a layer has is decided
by its block kind).  Kinds are looked up in the part
registry (``yalis_b200.parts.base``) when the model is built, so different
layers may use different mixers and feed-forwards, and a kind defined outside
the package works like a built-in one.

``schedule`` is the order in which layers run: a list of entries naming a layer
by index.  A layer may appear more than once (its weights are reused; each
appearance has a cache of its own unless it says otherwise), and an entry may
read the cache that an earlier entry wrote (``cache_of``) instead of writing
one.

An architecture (``yalis_b200.config.registry``) turns its ``config.json`` into
a ``ModelSpec`` and says under which tensor names the weights of each part are
stored.  Nothing in this file knows any architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` with its sizes and constants in ``params``."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the block arrangement and the parts it is made of.

    ``parts`` maps the names of the block's places (for the pre-norm block:
    ``norm_1``, ``mixer``, ``norm_2``, ``feed_forward``, ``position``) to the
    part that fills each.  Which places exist is the block kind's business
    (``Block.slots``): another arrangement may have a norm after the mixer, one
    norm for both branches, or no feed-forward at all.

    ``weight_prefix`` is where this layer's tensors live in the checkpoint
    (for instance ``model.layers.3.``); ``weight_names`` maps
    ``"<place>.<param>"`` to the tensor name under that prefix.
    """

    block: PartSpec
    parts: Mapping[str, PartSpec]
    weight_prefix: str
    weight_names: Mapping[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer``.  ``cache_of`` = index of an earlier schedule entry
    whose cache this entry reads instead of keeping its own (None: own cache)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    embedding_name: str                 # tensor name of the token table [vocab, hidden]
    head_name: Optional[str]            # tensor name of the output matrix; None = tied to the embedding
    final_norm_names: Mapping[str, str]  # "<param>" -> tensor name
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    embedding_scale: Optional[float] = None   # token rows are multiplied by it as they enter the stream (None: not)
    logit_softcap: Optional[float] = None     # logits become cap * tanh(logits / cap) (None: not)

    def __post_init__(self):
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.cache_of is not None and not 0 <= e.cache_of < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(n_layers))
