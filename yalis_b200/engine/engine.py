"""The engine core: a model, its cache and the one step function.

``Engine.step`` takes a batch of (request, its next tokens): portions of
prompts beside single decoded tokens, cut anywhere.  It reserves pages for
exactly these tokens, runs them as one flat batch against what earlier steps
left in the cache, and returns float32 logits at the wanted places.  It does
not sample and it does not decide what runs next: the scheduler above it does.

The reference has three homogeneous step functions instead (whole padded
prompts, one token per row, or the same T > 1 per row: yalis/engine.py:63-165).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from yalis_b200 import native
from yalis_b200.cache.manager import CacheManager
from yalis_b200.cache.storage import CacheStorage, plan_groups
from yalis_b200.config.registry import load_config, parse_config
from yalis_b200.engine.context import HostStep, StepContext
from yalis_b200.engine.model import Model
from yalis_b200.ops.attention import deal_tiles_hint
from yalis_b200.weights.loader import init_random, load_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class OutOfPages(RuntimeError):
    """A step needs more pages than are free; nothing was run."""


class StepError(RuntimeError):
    """A step was given something it cannot run (unknown request, bad token id, bad index)."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into
    ``tokens``) whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported: the engine runs in bfloat16 or float32")
        return dtype
    if dtype in ("fp16", "float16"):
        raise ValueError("float16 is not supported: weights are kept in bfloat16 (or float32 on the 32-bit path)")
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not one of {', '.join(DTYPES)}") from None


class Engine:
    """Model + cache manager + cache storage + step().

    Parameters
    ----------
    model_dir / config+seed : a folder with config.json and model.safetensors, or a
        config dictionary with a seed for random weights made on the device.
    dtype       : "bfloat16" (serving precision) or "float32" (true 32-bit path).
    page_size   : tokens per page.
    num_pages   : pages per group (given directly or as ``cache_tokens // page_size``).
    max_slots   : most requests alive at once.
    max_context : most tokens one request may hold (default: the model's limit).
    """

    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[dict] = None, seed: int = 0,
                 dtype="bfloat16", page_size: int = 16, num_pages: Optional[int] = None,
                 cache_tokens: Optional[int] = None, max_slots: int = 64, max_context: Optional[int] = None,
                 device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("yalis_b200 needs a CUDA device: there is no CPU path")
        native.load("cuda")   # fail now, loudly, if the kernels cannot be built or loaded
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(dtype)
        # Float32 products stay float32 (no TF32); bfloat16 products accumulate in float32.
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        if (model_dir is None) == (config is None):
            raise ValueError("give either model_dir or config")
        if model_dir is not None:
            self.arch, self.config = load_config(model_dir)
        else:
            self.arch, self.config = parse_config(config)
        self.spec = self.arch.model_spec(self.config)
        self.model = Model(self.spec)
        with torch.no_grad():
            if model_dir is not None:
                load_weights(self.model, model_dir, self.device, self.dtype)
            else:
                init_random(self.model, seed, self.device, self.dtype)
        self.vocab_size = self.spec.vocab_size
        self.page_size = int(page_size)
        self.max_context = int(max_context or self.spec.max_position)
        if num_pages is None:
            if cache_tokens is None:
                cache_tokens = min(self.max_context * max_slots, 1 << 20)
            num_pages = max(1, -(-int(cache_tokens) // self.page_size))
        self.num_pages = int(num_pages)
        self.max_slots = int(max_slots)
        requests = self.model.cache_requests()
        self.groups = plan_groups(requests, self.page_size, self.num_pages, self.max_context)
        self.manager = CacheManager(self.max_slots, self.groups)
        self.storage = CacheStorage(requests, [e.cache_of for e in self.spec.schedule], self.groups, self.max_slots,
                                    self.device, self.dtype)
        self._slot_of: Dict[Hashable, int] = {}
        self._error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._staging: List[Tuple[torch.Tensor, Optional[torch.cuda.Event]]] = []
        self._staging_next = 0
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self._graph_pool = None
        self._decoder = None

    def graph_pool(self):
        """One memory pool shared by all captured decode graphs."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    @property
    def decoder(self):
        """The CUDA-graph runner of decode-only steps (made on first use)."""
        if self._decoder is None:
            from yalis_b200.engine.decode_graph import GraphedDecoder
            self._decoder = GraphedDecoder(self)
        return self._decoder

    # ---- requests ------------------------------------------------------------------------
    def has_request(self, request: Hashable) -> bool:
        return request in self._slot_of

    def slot_of(self, request: Hashable) -> int:
        return self._slot_of[request]

    def length(self, request: Hashable) -> int:
        """Tokens the request holds in the cache."""
        return self.manager.length(self._slot_of[request])

    def add_request(self, request: Hashable) -> Optional[int]:
        """Give the request a slot (None if every slot is taken)."""
        if request in self._slot_of:
            raise StepError(f"request {request!r} is already live")
        slot = self.manager.acquire()
        if slot is None:
            return None
        self.storage.reset_slot(slot)
        self._slot_of[request] = slot
        return slot

    def finish_request(self, request: Hashable) -> None:
        """Give back everything the request holds."""
        slot = self._slot_of.pop(request)
        self.manager.release(slot)

    def can_run(self, request: Hashable, n_new_tokens: int) -> bool:
        slot = self._slot_of[request]
        return self.manager.can_reserve(slot, self.manager.length(slot) + n_new_tokens)

    def free_pages(self) -> Dict[str, int]:
        return {g.name: self.manager.free_pages(g.name) for g in self.groups}

    # ---- the step ---------------------------------------------------------------------------
    def _staging_buffer(self, n: int) -> Tuple[torch.Tensor, int]:
        """A pinned int32 buffer of at least n elements whose last copy has finished."""
        if not self._staging:
            self._staging = [(None, None), (None, None)]
        i = self._staging_next
        self._staging_next = (i + 1) % len(self._staging)
        buf, ev = self._staging[i]
        if ev is not None:
            ev.synchronize()
        if buf is None or buf.numel() < n:
            size = max(n, 4096, 2 * (buf.numel() if buf is not None else 0))
            buf = torch.empty(size, dtype=torch.int32).pin_memory()
        self._staging[i] = (buf, None)
        return buf, i

    def _build_context(self, slots: Sequence[int], entries: Sequence[StepEntry]) -> StepContext:
        q_lens = [len(e.tokens) for e in entries]
        before = [self.manager.length(s) for s in slots]
        n, r = sum(q_lens), len(entries)
        n_want = sum(len(e.want) for e in entries)
        widths = [g.max_pages_per_request for g in self.groups]
        # Only the columns that some request of this step can touch are copied.
        max_kv = max(b + q for b, q in zip(before, q_lens))
        used = [min(w, -(-max_kv // g.page_size)) for w, g in zip(widths, self.groups)]
        total = 3 * n + (r + 1) + 2 * r + n_want + sum(r * u for u in used)
        pinned, which = self._staging_buffer(total)
        host = pinned.numpy()
        o = 0
        tok = host[o:o + n]; o += n
        pos = host[o:o + n]; o += n
        req = host[o:o + n]; o += n
        qs = host[o:o + r + 1]; o += r + 1
        kv = host[o:o + r]; o += r
        sl = host[o:o + r]; o += r
        rows = host[o:o + n_want]; o += n_want
        t = w = 0
        qs[0] = 0
        for i, e in enumerate(entries):
            q = q_lens[i]
            tok[t:t + q] = np.asarray(e.tokens, dtype=np.int64)
            pos[t:t + q] = np.arange(before[i], before[i] + q, dtype=np.int32)
            req[t:t + q] = i
            for j in e.want:
                rows[w] = t + j
                w += 1
            t += q
            qs[i + 1] = t
            kv[i] = before[i] + q
            sl[i] = slots[i]
        tables_off = []
        for g, u in zip(self.groups, used):
            tbl = self.manager.table(g.name)
            view = host[o:o + r * u].reshape(r, u)
            for i, s in enumerate(slots):
                view[i] = tbl[s, :u]
            tables_off.append((o, u))
            o += r * u
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[:total], non_blocking=True)
        self.last_h2d_bytes = 4 * total
        ev = torch.cuda.Event()
        ev.record()
        self._staging[which] = (pinned, ev)
        o = 0
        d_tok = dev[o:o + n]; o += n
        d_pos = dev[o:o + n]; o += n
        d_req = dev[o:o + n]; o += n
        d_qs = dev[o:o + r + 1]; o += r + 1
        d_kv = dev[o:o + r]; o += r
        d_sl = dev[o:o + r]; o += r
        d_rows = dev[o:o + n_want]; o += n_want
        tables = {g.name: dev[off:off + r * u].view(r, u) for g, (off, u) in zip(self.groups, tables_off)}
        return StepContext(
            n_tokens=n, n_requests=r, token_ids=d_tok, positions=d_pos, req_of_token=d_req, q_start=d_qs, kv_len=d_kv,
            slots=d_sl, logit_rows=d_rows, block_tables=tables,
            host=HostStep(slots=slots, q_start=[int(x) for x in qs], ctx_before=before, max_q_len=max(q_lens),
                          max_kv_len=max_kv,
                          deal_tiles=all(q == 1 for q in q_lens) and deal_tiles_hint([b + 1 for b in before])),
            error_flag=self._error_flag, decode_only=all(q == 1 for q in q_lens), settled=True)

    def _validate(self, slots: Sequence[int], entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(set(slots)) != len(slots):
            raise StepError("a request appears twice in one step")
        for s, e in zip(slots, entries):
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab_size:
                raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab_size})")
            for j in e.want:
                if not 0 <= j < len(e.tokens):
                    raise StepError(f"request {e.request!r}: wanted place {j} is outside its {len(e.tokens)} tokens")
            new_len = self.manager.length(s) + len(e.tokens)
            if new_len > self.max_context or not self.manager.fits(new_len):
                raise StepError(f"request {e.request!r} would hold {new_len} tokens, more than the limit {self.max_context}")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch of live requests (by the ids given to ``add_request``); returns
        float32 logits [wanted, vocab] on the device in the order of the entries and of
        their ``want`` (None if nothing is wanted)."""
        for e in entries:
            if e.request not in self._slot_of:
                raise StepError(f"request {e.request!r} is not live (add_request first)")
        return self.step_slots([self._slot_of[e.request] for e in entries], entries)

    @torch.no_grad()
    def step_slots(self, slots: Sequence[int], entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The step function proper, for callers that manage slots themselves (the
        scheduler): entry i belongs to the request that holds ``slots[i]``."""
        self._validate(slots, entries)
        new_lens = [self.manager.length(s) + len(e.tokens) for s, e in zip(slots, entries)]
        for s, e, nl in zip(slots, entries, new_lens):
            if not self.manager.reserve(s, nl):
                raise OutOfPages(f"no pages left for request {e.request!r} to reach {nl} tokens "
                                 f"(free: {self.free_pages()})")
        ctx = self._build_context(slots, entries)
        stream = self.model.forward(ctx, self.storage.entries)
        logits = self.model.logits(stream, ctx.logit_rows) if ctx.logit_rows.numel() else None
        for s, nl in zip(slots, new_lens):
            self.manager.commit(s, nl)
        self.steps_run += 1
        if os.environ.get("YALIS_B200_CHECK"):
            self.check_device_errors()
        return logits

    def check_device_errors(self) -> None:
        """Synchronise and raise if any kernel flagged a bad id or an unmapped page."""
        if int(self._error_flag.item()):
            self._error_flag.zero_()
            raise StepError("a kernel reported a token id or page outside its range")
