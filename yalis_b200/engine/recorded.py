"""Steps recorded once and replayed: CUDA graphs over buffers of fixed size.

A step in which every request brings one token launches a few hundred small
kernels; launched one by one from Python they cost more than they run.  The
engine records such a step once per (batch bucket, kind of token choice, keys of
the parts) and every later step of that kind is: fill one pinned buffer with
the step's arrays, copy it, launch the graph.  Steps that hold prompt portions
are recorded too, with room for their tokens, requests, wanted rows and longest
portion rounded up, once the same kind of step has come a second time (a small
model's step of a few hundred tokens is otherwise bound by the host's
launches).  The graph holds the whole step:
embedding, all blocks, final norm, output matrix, token choice and the copy of
the error word beside the chosen tokens.

This file only runs what the engine has prepared: validation, page
reservation and commit happen in ``Engine.run_step`` for launched and replayed
steps alike, and the step's arrays are written by the same ``Engine._fill``.
What is particular here is the fixed size: a bucket of 1, 2, 4, ... requests
(and, for steps with portions, of tokens in multiples of 64), padded with rows
that belong to no request and that every kernel skips, and block tables at their full row
width, of which a step copies only the columns in use.

Shapes inside a graph are fixed, so nothing in a recorded step may depend on a
request's length except through the parts' ``capture_key`` (a part whose choice
of kernel or grid depends on lengths answers with what decides it, and each
distinct answer is recorded separately).  The first step of a kind runs once
launch by launch before it is recorded, so that libraries are initialised
outside the recording; per-request state is saved around that trial, because the
replay that follows runs the same step again (keys and values are simply
written twice).

The reference gets the same effect from torch.compile's "reduce-overhead" mode
(yalis/engine.py:44-48, 109).
"""

from __future__ import annotations

import ctypes
import dataclasses
import gc
from typing import Optional

import torch

from yalis_b200.engine.context import HostStep, StepLayout
from yalis_b200.ops import _lib


def bucket_for(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


def _copy_rows_to_device(dst: torch.Tensor, src: torch.Tensor, rows: int, cols: int) -> None:
    """dst[:rows, :cols] <- src[:rows, :cols] (pinned host to device, both int32 with the same row width):
    one strided copy on the current stream."""
    if rows <= 0 or cols <= 0:
        return
    pitch = dst.stride(0) * 4
    status = _lib.lib().yalis_copy_rows_h2d(ctypes.c_void_p(dst.data_ptr()), ctypes.c_size_t(pitch),
                                            ctypes.c_void_p(src.data_ptr()), ctypes.c_size_t(src.stride(0) * 4),
                                            ctypes.c_size_t(cols * 4), ctypes.c_size_t(rows), _lib.stream())
    if status != 0:
        raise _lib.KernelError(f"copy_rows_h2d: status {status}")


class RecordedStep:
    """Static buffers and the graph for one kind of step (see the module docstring)."""

    def __init__(self, engine, n_tokens: int, n_requests: int, n_rows: int, single_tokens: bool, mode: str,
                 keep_logits: bool, key: tuple, longest_portion: Optional[int] = None):
        self.engine, self.mode, self.keep_logits, self.key = engine, mode, keep_logits, key
        self.longest_portion = longest_portion          # the most tokens a request may bring to a replay (None: one)
        self.size, self.n_tokens, self.n_rows, self.single_tokens = n_requests, n_tokens, n_rows, single_tokens
        self.widths = [g.max_pages_per_request for g in engine.groups]
        self.layout = StepLayout(n_tokens, n_requests, n_rows, self.widths, sampling=(mode == "sampled"))
        self.host = torch.zeros(self.layout.total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        self.h = self.layout.views(self.host, as_numpy=True)
        self.host_tables = self.layout.views(self.host, as_numpy=False)["tables"]
        self.dev_tables = self.layout.views(self.dev, as_numpy=False)["tables"]
        for view in self.h["tables"]:
            view[:] = -1
        self.dev.copy_(self.host)
        self.tokens = torch.zeros(max(1, n_rows), dtype=torch.int32, device=engine.device) if mode != "none" else None
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self.replays = 0
        self.last_used = 0          # the engine's count of steps when this recording was last asked for
        self.copy_done: Optional[torch.cuda.Event] = None
        self.ctx = None
        self.d = None

    def _body(self) -> None:
        eng = self.engine
        stream = eng.model.forward(self.ctx, eng.storage.entries)
        if self.n_rows == 0:
            return
        logits = eng.model.logits(stream, self.ctx.logit_rows)
        if self.keep_logits:
            if self.logits is None:
                self.logits = torch.empty_like(logits)
            self.logits.copy_(logits)
        if self.mode != "none":
            eng._choose(logits, self.d, self.mode, out=self.tokens)
            eng.chosen[-1:].copy_(eng._error_word)

    def _record(self, host: HostStep) -> None:
        eng = self.engine
        # The facts of this step stand for every step that will replay the recording (they share the parts' keys),
        # but for the longest portion, which is the recording's bound: launches are sized by it.
        if self.longest_portion is not None:
            host = dataclasses.replace(host, max_q_len=self.longest_portion, memo=dict(host.memo))
        self.ctx, self.d = eng._context(self.layout, self.dev, host, decode_only=self.single_tokens)
        saved_state = eng.storage.snapshot_state()
        saved_chosen = eng.chosen.clone()
        self._body()                                   # the trial: libraries initialise, buffers get their sizes
        eng.storage.restore_state(saved_state)
        eng.chosen.copy_(saved_chosen)
        torch.cuda.synchronize()
        before = _lib.LAUNCHES[0]
        graph = torch.cuda.CUDAGraph()
        # No garbage collection while the stream is capturing: a collected tensor or graph of an engine
        # that is no longer used frees device memory, which is not allowed then and invalidates the capture.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=eng.graph_pool()):
                self._body()
        finally:
            if gc_was_on:
                gc.enable()
        self.launches = _lib.LAUNCHES[0] - before
        self.graph = graph

    def run(self, host: HostStep, entries, q_lens, sampling, draws, n_want):
        from yalis_b200.engine.engine import StepOutput
        eng = self.engine
        n = len(entries)
        if self.copy_done is not None:
            self.copy_done.synchronize()               # the last copy out of the pinned buffer has finished
        used = [min(g.max_pages_per_request, -(-host.max_kv_len // g.page_size)) for g in eng.groups]
        eng._fill(self.h, host.slots, entries, host.ctx_before, q_lens, sampling, draws, used,
                  [eng.manager.table(g.name) for g in eng.groups], eng.null_slot)
        prefix = self.layout.prefix
        self.dev[:prefix].copy_(self.host[:prefix], non_blocking=True)
        copied = prefix
        for dst, src, u in zip(self.dev_tables, self.host_tables, used):
            _copy_rows_to_device(dst, src, n, u)
            copied += n * u
        self.copy_done = torch.cuda.Event()
        self.copy_done.record()
        if self.graph is None:
            self._record(host)
        self.graph.replay()
        self.replays += 1
        logits = self.logits[:n_want] if self.keep_logits and n_want else None
        tokens = self.tokens[:n_want] if self.mode != "none" and n_want else None
        return StepOutput(logits, tokens, True, 4 * copied)
