"""A model built from a ``ModelSpec``: blocks of registered parts run in schedule order.

Nothing here is specific to an architecture.  The class names every tensor it
expects (for the loader and for the random-weights mode), asks every mixer what
cache it wants, and runs embedding -> schedule -> final norm -> output matrix
(yalis/external/model.py:137-197), with the output computed only for the rows
whose logits are wanted (the reference computes all positions, model.py:184).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from yalis_b200.config.spec import ModelSpec
from yalis_b200.ops.elementwise import embedding, softcap_
from yalis_b200.ops.linear import linear
from yalis_b200.parts.base import NOT_CAPTURABLE, Block, ParamSpec, ResidualStream, build_block, make_part


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks: List[Block] = [build_block(layer) for layer in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None

    # ---- tensors ---------------------------------------------------------------------
    def _layer_tensor_names(self, li: int) -> Dict[str, Dict[str, str]]:
        """part slot -> {local parameter name -> tensor name in the checkpoint}."""
        layer, block = self.spec.layers[li], self.blocks[li]
        out: Dict[str, Dict[str, str]] = {}
        for slot, part in block.parts.items():
            names = {}
            for local in part.param_specs():
                key = f"{slot}.{local}"
                if key not in layer.weight_names:
                    raise KeyError(f"layer {li}: the architecture names no tensor for {key}")
                names[local] = layer.weight_prefix + layer.weight_names[key]
            out[slot] = names
        return out

    def expected_tensors(self) -> Dict[str, ParamSpec]:
        """Every tensor of the checkpoint by name, in a fixed order."""
        s = self.spec
        out: Dict[str, ParamSpec] = {s.embedding_name: ParamSpec((s.vocab_size, s.hidden_size))}

        def put(name: str, ps: ParamSpec):
            if name in out and out[name] != ps:
                raise ValueError(f"tensor {name} is expected with two different specs: {out[name]} and {ps}")
            out[name] = ps

        for li, block in enumerate(self.blocks):
            names = self._layer_tensor_names(li)
            for slot, part in block.parts.items():
                for local, ps in part.param_specs().items():
                    put(names[slot][local], ps)
        for local, ps in self.final_norm.param_specs().items():
            put(s.final_norm_names[local], ps)
        if s.head_name is not None:
            put(s.head_name, ParamSpec((s.vocab_size, s.hidden_size)))
        return out

    def load(self, fetch: Callable[[str], torch.Tensor], dtype: torch.dtype) -> None:
        """``fetch(name)`` returns the named tensor on the device in its final dtype."""
        s = self.spec
        self.dtype = dtype
        self.embedding = fetch(s.embedding_name).contiguous()
        for li, block in enumerate(self.blocks):
            names = self._layer_tensor_names(li)
            for slot, part in block.parts.items():
                part.load({local: fetch(name) for local, name in names[slot].items()})
        self.final_norm.load({local: fetch(s.final_norm_names[local]) for local in self.final_norm.param_specs()})
        self.head = self.embedding if s.head_name is None else fetch(s.head_name).contiguous()

    # ---- cache -------------------------------------------------------------------------
    def cache_requests(self) -> List[Optional[object]]:
        """What the block of each schedule entry wants to keep (an entry that reads another
        entry's cache still says what it expects to find there)."""
        return [self.blocks[e.layer].cache_request() for e in self.spec.schedule]

    def capture_key(self, host):
        """The keys of all parts that run in a step, or ``NOT_CAPTURABLE`` if one of them cannot be recorded."""
        keys = []
        for part in [self.blocks[i] for i in sorted({e.layer for e in self.spec.schedule})] + [self.final_norm]:
            key = part.capture_key(host)
            if key is NOT_CAPTURABLE:
                return NOT_CAPTURABLE
            keys.append(key)
        return tuple(keys)

    # ---- forward -----------------------------------------------------------------------
    def forward(self, ctx, caches: List[Optional[object]]) -> ResidualStream:
        x = embedding(self.embedding, ctx.token_ids, bad_flag=ctx.error_flag, scale=self.spec.embedding_scale,
                      from_slot=ctx.token_from_slot, chosen=ctx.chosen if ctx.token_from_slot is not None else None)
        stream = ResidualStream(x, self.dtype)
        for entry, cache in zip(self.spec.schedule, caches):
            self.blocks[entry.layer].forward(stream, ctx, cache)
        return stream

    def logits(self, stream: ResidualStream, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the given token rows."""
        h = self.final_norm.forward(stream, rows=rows)
        out = linear(h, self.head, out_dtype=torch.float32)
        if self.spec.logit_softcap is not None:
            softcap_(out, self.spec.logit_softcap)
        return out

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        add(self.embedding)
        add(self.head)
        for b in self.blocks:
            for part in b.parts.values():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor) and v.is_cuda:
                        add(v)
        add(getattr(self.final_norm, "weight", None))
        return total
