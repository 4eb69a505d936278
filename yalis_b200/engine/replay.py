"""Trace replay on top of ``Engine.step``: no forward pass, cache or loader of its own.

A trace is a sequence of steps; each step lists, per request, its next tokens
and the places whose logits are wanted, plus the requests that end after the
step.  Tokens are given, nothing is sampled and nothing is scheduled: the
replayer only creates requests on first sight, calls the engine's step function
with exactly the step's entries, and finishes the requests named in ``end``.
The reference's nearest hook is ``get_logits=True`` of its generate loop
(yalis/engine.py:519-520, 570-571).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from .engine import Engine, StepEntry


class Replayer:
    """``graphs=True`` sends every step whose entries all bring one token through the recorded
    (CUDA graph) form of the step, the one generation uses for decoding; other steps, and all
    steps without it, are launched kernel by kernel.  Both go through ``Engine.run_step``."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, max_live: int = 4,
                 engine: Optional[Engine] = None, graphs: bool = False):
        if 64 % page_size and page_size % 64:
            raise ValueError("page_size must divide 64 or be a multiple of it")
        # The pool holds max_tokens, with each live request rounded up to whole pages.
        unit = max(page_size, 64)
        pool_tokens = -(-max_tokens // unit) * unit
        self.graphs = graphs
        self.steps_replayed = 0        # steps that ran from a recording
        self.engine = engine or Engine(model_dir, dtype=dtype, page_size=page_size,
                                       num_pages=pool_tokens // page_size, max_slots=max_live)

    def run_step(self, step: Dict) -> Optional[np.ndarray]:
        entries: List[StepEntry] = []
        for e in step.get("entries", []):
            if not self.engine.has_request(e["id"]):
                if self.engine.add_request(e["id"]) is None:
                    raise RuntimeError(f"step {step.get('step')}: no free slot for request {e['id']!r}")
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = None
        if entries:
            out = self.engine.run(entries, graphs=self.graphs)
            self.steps_replayed += out.captured
            if out.logits is not None:
                logits = out.logits.float().cpu().numpy()
            self.engine.check_device_errors()
        for rid in step.get("end", []):
            if self.engine.has_request(rid):
                self.engine.finish_request(rid)
        return logits
