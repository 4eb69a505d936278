"""Decode steps replayed as CUDA graphs.

A step in which every request brings exactly one token launches a few hundred
small kernels; launched one by one from Python they cost more than they run.
Such a step is captured once per batch bucket (1, 2, 4, ... requests, padded
with rows that every kernel skips) into a CUDA graph over static device
buffers, and every later step of that bucket is: fill one pinned buffer with
the step's positions, lengths and block-table rows, one host->device copy, one
graph launch.  The graph holds the whole step: embedding, all blocks, final
norm, output matrix and token selection; the chosen tokens stay in a device
buffer that the next step reads when the caller does not supply tokens from
the host (the reference gets the same effect from torch.compile's
"reduce-overhead" mode, yalis/engine.py:44-48, 109).

Shapes inside a graph are fixed, so nothing in a captured step may depend on a
request's length: attention grids are sized by the bucket only, and block
tables are uploaded at the full row width.
"""

from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from yalis_b200.engine.context import HostStep, StepContext
from yalis_b200.ops import _lib
from yalis_b200.ops import sampling as sampling_ops
from yalis_b200.sampling.sampler import SamplingParams, _as_int64


def bucket_for(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _Bucket:
    """Static buffers and the captured graph for one batch size."""

    def __init__(self, engine, size: int, greedy: bool, keep_logits: bool, long_context: bool = False,
                 deal_tiles: bool = False):
        self.engine, self.size, self.greedy, self.keep_logits = engine, size, greedy, keep_logits
        self.long_context, self.deal_tiles = long_context, deal_tiles
        dev = engine.device
        self.widths = [g.max_pages_per_request for g in engine.groups]
        r = size
        # int32 layout: positions | req_of_token | q_start | kv_len | slots | logit_rows | top_k | tables... ;
        # then float32 temperature, top_p; then int64 seed, draw (kept 8-byte aligned at the end)
        self.n_i32 = 6 * r + (r + 1) + sum(r * w for w in self.widths)      # six arrays of r, q_start, the tables
        self.n_i32 += (-self.n_i32) % 2
        total = self.n_i32 + 2 * r + 4 * r
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(r, dtype=torch.int32, device=dev)       # input of a step, output of its sampling
        self.tokens_host = torch.zeros(r, dtype=torch.int32).pin_memory()
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self.copy_done: Optional[torch.cuda.Event] = None
        h, d = self.host.numpy(), self.dev
        o = 0

        limit = [self.n_i32]

        def take(n):
            nonlocal o
            if o + n > limit[0]:
                raise AssertionError("the step buffer's regions overlap")
            a, b = h[o:o + n], d[o:o + n]
            o += n
            return a, b

        self.h_pos, d_pos = take(r)
        self.h_req, d_req = take(r)
        self.h_qs, d_qs = take(r + 1)
        self.h_kv, d_kv = take(r)
        self.h_slots, d_slots = take(r)
        self.h_rows, d_rows = take(r)
        self.h_topk, self.d_topk = take(r)
        self.h_tables, d_tables = {}, {}
        for g, w in zip(engine.groups, self.widths):
            a, b = take(r * w)
            self.h_tables[g.name], d_tables[g.name] = a.reshape(r, w), b.view(r, w)
        o, limit[0] = self.n_i32, total
        a, b = take(r)
        self.h_temp, self.d_temp = a.view(np.float32), b.view(torch.float32)
        a, b = take(r)
        self.h_topp, self.d_topp = a.view(np.float32), b.view(torch.float32)
        a, b = take(2 * r)
        self.h_seed, self.d_seed = a.view(np.int64), b.view(torch.int64)
        a, b = take(2 * r)
        self.h_draw, self.d_draw = a.view(np.int64), b.view(torch.int64)
        self.ctx = StepContext(
            n_tokens=r, n_requests=r, token_ids=self.tokens, positions=d_pos, req_of_token=d_req, q_start=d_qs,
            kv_len=d_kv, slots=d_slots, logit_rows=d_rows, block_tables=d_tables,
            # lengths are not part of a captured step; only whether it is of the long-context kind (more key splits)
            host=HostStep(slots=[], q_start=list(range(r + 1)), ctx_before=[], max_q_len=1,
                          max_kv_len=engine.max_context if long_context else 0, deal_tiles=deal_tiles),
            error_flag=engine._error_flag, decode_only=True, settled=True)

    def fill(self, slots: Sequence[int], lengths: Sequence[int], params: Optional[Sequence[SamplingParams]],
             draws: Optional[Sequence[int]]) -> None:
        """Host side of a step: ``lengths[i]`` tokens are cached for slot i before it."""
        n, r = len(slots), self.size
        self.h_pos[:n] = lengths
        self.h_req[:n] = np.arange(n, dtype=np.int32)
        self.h_req[n:] = -1
        self.h_qs[:n + 1] = np.arange(n + 1, dtype=np.int32)
        self.h_qs[n + 1:] = n
        self.h_kv[:n] = np.asarray(lengths, dtype=np.int32) + 1
        self.h_slots[:n] = slots
        self.h_rows[:n] = np.arange(n, dtype=np.int32)
        self.h_rows[n:] = -1
        mgr = self.engine.manager
        for g in self.engine.groups:
            used = min(g.max_pages_per_request, -(-(max(lengths) + 1) // g.page_size))
            tbl, dst = mgr.table(g.name), self.h_tables[g.name]
            for i, s in enumerate(slots):
                dst[i, :used] = tbl[s, :used]
        if not self.greedy:
            for i, (p, d) in enumerate(zip(params, draws)):
                self.h_temp[i], self.h_topk[i], self.h_topp[i] = p.temperature, p.top_k or 0, p.top_p
                self.h_seed[i], self.h_draw[i] = _as_int64(p.seed), int(d)
        self.dev.copy_(self.host, non_blocking=True)
        self.copy_done = torch.cuda.Event()
        self.copy_done.record()

    def _body(self) -> None:
        eng = self.engine
        stream = eng.model.forward(self.ctx, eng.storage.entries)
        logits = eng.model.logits(stream, self.ctx.logit_rows)
        if self.keep_logits:
            if self.logits is None:
                self.logits = torch.empty_like(logits)
            self.logits.copy_(logits)
        if self.greedy:
            sampling_ops.argmax(logits, out=self.tokens)
        else:
            sampling_ops.sample(logits, self.d_temp, self.d_topk, self.d_topp, self.d_seed, self.d_draw, out=self.tokens)

    def run(self) -> None:
        if self.graph is None:
            # The eager run warms up libraries and writes the same cache entries the replay will.
            saved = self.tokens.clone()
            self._body()
            self.tokens.copy_(saved)
            torch.cuda.synchronize()
            l0 = _lib.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            # No garbage collection while the stream is capturing: a collected tensor or graph of an engine
            # that is no longer used frees device memory, which is not allowed then and invalidates the capture.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self.engine.graph_pool()):
                    self._body()
            finally:
                if gc_was_on:
                    gc.enable()
            self.launches = _lib.LAUNCHES[0] - l0
            self.graph = graph
        self.graph.replay()


class GraphedDecoder:
    """Runs decode-only steps of the engine through per-bucket CUDA graphs."""

    def __init__(self, engine):
        self.engine = engine
        self._buckets: Dict[tuple, _Bucket] = {}
        self.last_bucket: Optional[_Bucket] = None

    def step(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None,
             params: Optional[Sequence[SamplingParams]] = None, draws: Optional[Sequence[int]] = None,
             keep_logits: bool = False) -> _Bucket:
        """One decode step for the requests holding ``slots``.  ``tokens`` are this step's
        input ids from the host; None means "what the previous step of this bucket chose",
        which is still on the device.  Returns the bucket, whose ``tokens`` buffer holds
        the chosen ids (rows in the order of ``slots``) once the stream has run."""
        eng = self.engine
        n = len(slots)
        greedy = params is None or all(p.greedy for p in params)
        mgr = eng.manager
        lengths = [mgr.length(s) for s in slots]
        from yalis_b200.ops import attention as attn_ops
        # The kind of step decides how attention kernels divide their work (they cannot look at lengths when a
        # captured step is replayed): dealt tiles for long or uneven batches, more key splits for one long request.
        deal_tiles = attn_ops.deal_tiles_hint([l + 1 for l in lengths])
        long_context = not deal_tiles and max(lengths) + 1 > attn_ops.LONG_CONTEXT
        key = (bucket_for(n), greedy, keep_logits, long_context, deal_tiles)
        b = self._buckets.get(key)
        if b is None:
            b = self._buckets[key] = _Bucket(eng, key[0], greedy, keep_logits, long_context, deal_tiles)
        for s, l in zip(slots, lengths):
            if l + 1 > eng.max_context or not mgr.fits(l + 1):
                from yalis_b200.engine.engine import StepError
                raise StepError(f"a request would hold {l + 1} tokens, more than the limit {eng.max_context}")
            if not mgr.reserve(s, l + 1):
                from yalis_b200.engine.engine import OutOfPages
                raise OutOfPages(f"no pages left for a decode step (free: {eng.free_pages()})")
        if b.copy_done is not None:
            b.copy_done.synchronize()           # the last copies out of the pinned buffers have finished
        if tokens is None and self.last_bucket is not None and self.last_bucket is not b:
            # the same requests moved to another kind of step (e.g. past the long-context mark): their last
            # tokens are in the buffer of the bucket that chose them
            b.tokens[:n].copy_(self.last_bucket.tokens[:n], non_blocking=True)
        if tokens is not None:
            if min(tokens) < 0 or max(tokens) >= eng.vocab_size:
                from yalis_b200.engine.engine import StepError
                raise StepError(f"token id outside [0, {eng.vocab_size})")
            b.tokens_host[:n] = torch.as_tensor(list(tokens), dtype=torch.int32)
            b.tokens[:n].copy_(b.tokens_host[:n], non_blocking=True)
        b.fill(slots, lengths, params, draws)
        b.run()
        for s, l in zip(slots, lengths):
            mgr.commit(s, l + 1)
        eng.steps_run += 1
        eng.last_h2d_bytes = b.host.numel() * 4 + (4 * n if tokens is not None else 0)
        self.last_bucket = b
        return b
