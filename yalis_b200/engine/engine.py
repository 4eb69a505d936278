"""The engine core: a model, its cache and the one step function.

``Engine.run_step`` takes a batch of (request, its next tokens): portions of
prompts beside single decoded tokens, cut anywhere.  It reserves pages for
exactly these tokens (for all requests or for none), runs them as one flat
batch against what earlier steps left in the cache, returns float32 logits at
the wanted places and, if asked, chooses a token at each of them.  It does not
decide what runs next: the scheduler above it does.

There is one step function.  Whether a step is launched kernel by kernel or
replayed from a recording (a CUDA graph over buffers of fixed size: per bucket
of requests for steps in which every request brings one token, at the exact
counts for other steps whose shape comes again) is decided inside it, after the same
validation and reservation, from the same host arrays, and followed by the same
commit; trace replay and generation therefore drive the same code.

A chosen token stays on the device (``Engine.chosen``, one entry per slot): a
later step may name it as a request's input (``StepEntry.tokens = None``)
without the host having read it, which lets the caller run ahead of the tokens.

The reference has three homogeneous step functions instead (whole padded
prompts, one token per row, or the same T > 1 per row: yalis/engine.py:63-165)
and leaves the replay of its decode step to torch.compile (:44-48, 109).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from yalis_b200 import native
from yalis_b200.cache.manager import CacheManager
from yalis_b200.cache.storage import CacheStorage, group_page_bytes, plan_groups
from yalis_b200.config.engine_config import EngineConfig
from yalis_b200.config.registry import load_config, parse_config
from yalis_b200.engine.context import HostStep, StepContext, StepLayout
from yalis_b200.engine.model import Model
from yalis_b200.ops import _lib
from yalis_b200.ops import sampling as sampling_ops
from yalis_b200.parts.base import NOT_CAPTURABLE
from yalis_b200.sampling.sampler import SamplingParams, as_int64
from yalis_b200.weights.loader import init_random, load_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
_ENGINE_OPTIONS = ("dtype", "page_size", "num_pages", "cache_tokens", "memory_fraction", "max_slots",
                   "max_tokens_per_step", "prefill_chunk", "max_context", "use_graphs", "device")


class OutOfPages(RuntimeError):
    """A step needs more pages than are free; nothing was run and nothing was reserved."""


class StepError(RuntimeError):
    """A step was given something it cannot run (unknown request, bad token id, bad index),
    or a kernel of an earlier step reported a fault through the device error word."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into
    ``tokens``) whose logits are wanted.  ``tokens = None`` stands for one token: the one
    an earlier step chose for this request and left on the device."""

    request: Hashable
    tokens: Optional[Sequence[int]]
    want: Sequence[int] = ()


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]     # float32 [wanted, vocab] on the device (None: nothing wanted or not kept)
    tokens: Optional[torch.Tensor]     # int32 [wanted] chosen tokens on the device (None: no choice was asked for)
    captured: bool                     # the step was replayed from a recording
    h2d_bytes: int                     # bytes of step metadata copied to the device


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


class ChosenTokens:
    """A copy of the per-slot chosen tokens (and of the device error word) on its way to the host."""

    def __init__(self, engine: "Engine", host: torch.Tensor, event: torch.cuda.Event, step: int):
        self._engine, self._host, self._event, self.step = engine, host, event, step
        self._values: Optional[np.ndarray] = None

    def wait(self) -> np.ndarray:
        """int32 [max_slots]: the token each slot's request was given last, as of the copy.  Raises
        ``StepError`` if a kernel up to then reported a fault."""
        if self._values is None:
            self._event.synchronize()
            values = self._host.numpy().copy()
            self._engine._recycle(self._host)
            self._host = None
            self._values = values[:-2]
            word = int(values[-1])
            if word:
                self._engine._clear_error_word()
                raise StepError(f"a kernel reported a fault by step {self.step}: {_lib.describe_error_word(word)}")
        return self._values


class Engine:
    """Model + cache manager + cache storage + the step function.

    ``Engine(model_dir)`` reads a folder with config.json and model.safetensors;
    ``Engine(config=dict, seed=s)`` makes random weights on the device.  How it runs is an
    ``EngineConfig`` (``engine_config=``), whose fields may also be given as keywords.
    """

    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[dict] = None, seed: int = 0,
                 engine_config: Optional[EngineConfig] = None, **options):
        unknown = [k for k in options if k not in _ENGINE_OPTIONS]
        if unknown:
            raise TypeError(f"unknown engine option(s): {', '.join(unknown)}")
        if "dtype" in options and isinstance(options["dtype"], torch.dtype):
            options["dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(options["dtype"], str(options["dtype"]))
        ec = engine_config or EngineConfig(**{"page_size": 16, **options})
        if engine_config is not None and options:
            ec = engine_config.with_(**options)
        self.engine_config = ec
        if not torch.cuda.is_available():
            raise RuntimeError("yalis_b200 needs a CUDA device: there is no CPU path")
        native.load("cuda")   # fail now, loudly, if the kernels cannot be built or loaded
        self.device = torch.device(ec.device)
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(ec.dtype)
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
        self.page_size = ec.page_size
        self.max_context = min(ec.max_context or self.spec.max_position, self.spec.max_position)
        self.max_slots = ec.max_slots
        requests = self.model.cache_requests()
        cache_of = [e.cache_of for e in self.spec.schedule]
        element = 2 if self.dtype == torch.bfloat16 else 4
        page_bytes = sum(group_page_bytes(requests, cache_of, self.page_size, element).values())
        free_bytes = torch.cuda.mem_get_info(self.device)[0] if ec.memory_fraction is not None else None
        self.num_pages = ec.pool_pages(self.spec.max_position, free_bytes, page_bytes or None) if page_bytes else 1
        self.groups = plan_groups(requests, self.page_size, self.num_pages, self.max_context, self.max_slots,
                                  ec.max_tokens_per_step)
        self.manager = CacheManager(self.max_slots, self.groups)
        self.storage = CacheStorage(requests, cache_of, self.groups, self.max_slots, self.device, self.dtype)
        self._slot_of: Dict[Hashable, int] = {}
        self._error_word = _lib.error_word(self.device)
        # per slot the token chosen last; then the slot that is nobody's (padding); then a copy of the error word
        self.chosen = torch.zeros(self.max_slots + 2, dtype=torch.int32, device=self.device)
        self.null_slot = self.max_slots
        self._has_choice = [False] * self.max_slots
        self._staging: List[Tuple[Optional[torch.Tensor], Optional[torch.cuda.Event]]] = [(None, None), (None, None)]
        self._staging_next = 0
        self._report_buffers: List[torch.Tensor] = []
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self.last_captured = None           # the recording the last step replayed (None: it was launched)
        self._graph_pool = None
        self._recordings: Dict[tuple, object] = {}
        self._seen_shapes: Dict[tuple, int] = {}
        self._steps_seen = 0

    # ---- requests ------------------------------------------------------------------------
    def has_request(self, request: Hashable) -> bool:
        return request in self._slot_of

    def slot_of(self, request: Hashable) -> int:
        return self._slot_of[request]

    def length(self, request: Hashable) -> int:
        """Tokens the request holds in the cache."""
        return self.manager.length(self._slot_of[request])

    def reset_slot(self, slot: int) -> None:
        """What a newly admitted request's slot starts from: zeroed state, no chosen token."""
        self.storage.reset_slot(slot)
        self._has_choice[slot] = False

    def add_request(self, request: Hashable) -> Optional[int]:
        """Give the request a slot (None if every slot is taken)."""
        if request in self._slot_of:
            raise StepError(f"request {request!r} is already live")
        slot = self.manager.acquire()
        if slot is None:
            return None
        self.reset_slot(slot)
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

    def graph_pool(self):
        """One memory pool shared by all recorded steps."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # ---- device error word and chosen tokens ---------------------------------------------------
    def _clear_error_word(self) -> None:
        self._error_word.zero_()
        self.chosen[-1:].zero_()

    def check_device_errors(self) -> None:
        """Synchronise and raise if any kernel reported a fault (bad token id, unmapped page, a wait that ran out)."""
        word = int(self._error_word.item())
        if word:
            self._clear_error_word()
            raise StepError(f"a kernel reported a fault: {_lib.describe_error_word(word)}")

    def _recycle(self, host: torch.Tensor) -> None:
        self._report_buffers.append(host)

    def fetch_chosen(self) -> ChosenTokens:
        """Start copying the chosen tokens of all slots, and the error word as the last step left it, to
        the host; ``wait()`` on the result gives them."""
        host = self._report_buffers.pop() if self._report_buffers else torch.empty(self.max_slots + 2, dtype=torch.int32).pin_memory()
        host.copy_(self.chosen, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return ChosenTokens(self, host, event, self.steps_run)

    # ---- the step ---------------------------------------------------------------------------
    def _staging_buffer(self, n: int) -> Tuple[torch.Tensor, int]:
        """A pinned int32 buffer of at least n elements whose last copy has finished."""
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

    def _validate(self, slots: Sequence[int], entries: Sequence[StepEntry], sampling, draws) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(slots) != len(entries):
            raise StepError("one slot per entry")
        if len(set(slots)) != len(slots):
            raise StepError("a request appears twice in one step")
        n_want = 0
        for s, e in zip(slots, entries):
            if e.tokens is None:
                if not self._has_choice[s]:
                    raise StepError(f"request {e.request!r}: no token was chosen for it on the device yet")
                count = 1
            else:
                count = len(e.tokens)
                if count == 0:
                    raise StepError(f"request {e.request!r} brings no tokens")
                lo, hi = min(e.tokens), max(e.tokens)
                if lo < 0 or hi >= self.vocab_size:
                    raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab_size})")
            for j in e.want:
                if not 0 <= j < count:
                    raise StepError(f"request {e.request!r}: wanted place {j} is outside its {count} tokens")
            n_want += len(e.want)
            new_len = self.manager.length(s) + count
            if new_len > self.max_context or not self.manager.fits(new_len):
                raise StepError(f"request {e.request!r} would hold {new_len} tokens, more than the limit {self.max_context}")
        if sampling is not None:
            if len(sampling) != n_want or draws is None or len(draws) != n_want:
                raise StepError("choosing tokens needs one SamplingParams and one draw counter per wanted place")

    @staticmethod
    def _fill(views, slots, entries, before, q_lens, sampling, draws, used, tables_of, null_slot) -> None:
        """Write a step's arrays into (views of) a pinned buffer; what the step leaves unused is padding."""
        tok, src, pos, req = views["tok"], views["src"], views["pos"], views["req"]
        qs, kv, sl, rows, row_slot = views["qs"], views["kv"], views["slots"], views["rows"], views["row_slot"]
        t = w = 0
        qs[0] = 0
        single = max(q_lens, default=0) == 1 and min(q_lens) == 1 and all(len(e.want) <= 1 and (not e.want or e.want[0] == 0) for e in entries)
        if single:
            # every request brings one token (a decode step): the same arrays without a loop over numpy scalars
            r = len(entries)
            tok[:r] = [0 if e.tokens is None else e.tokens[0] for e in entries]
            src[:r] = [s if e.tokens is None else -1 for s, e in zip(slots, entries)]
            pos[:r] = before
            req[:r] = np.arange(r, dtype=np.int32)
            qs[:r + 1] = np.arange(r + 1, dtype=np.int32)
            kv[:r] = np.asarray(before, dtype=np.int32) + 1
            sl[:r] = slots
            wanted = [i for i, e in enumerate(entries) if len(e.want)]
            w = len(wanted)
            rows[:w] = wanted
            row_slot[:w] = [slots[i] for i in wanted]
            t = r
        for i, e in enumerate(() if single else entries):
            q = q_lens[i]
            if e.tokens is None:
                tok[t], src[t] = 0, slots[i]
            else:
                tok[t:t + q] = np.asarray(e.tokens, dtype=np.int64)
                src[t:t + q] = -1
            pos[t:t + q] = np.arange(before[i], before[i] + q, dtype=np.int32)
            req[t:t + q] = i
            last = len(e.want) - 1
            for k, j in enumerate(e.want):
                rows[w] = t + j
                # the token chosen at a request's last wanted place is the one kept for it on the device
                row_slot[w] = slots[i] if k == last else -1
                w += 1
            t += q
            qs[i + 1] = t
            kv[i] = before[i] + q
            sl[i] = slots[i]
        r = len(entries)
        tok[t:], src[t:], pos[t:], req[t:] = 0, -1, 0, -1
        qs[r + 1:], kv[r:], sl[r:] = t, 0, null_slot
        rows[w:], row_slot[w:] = -1, -1
        if sampling is not None and "temp" in views:
            temp, topk, topp, seed, draw = views["temp"], views["topk"], views["topp"], views["seed"], views["draw"]
            for i, (p, d) in enumerate(zip(sampling, draws)):
                temp[i], topk[i], topp[i] = p.temperature, p.top_k or 0, p.top_p
                seed[i], draw[i] = as_int64(p.seed), int(d)
            temp[w:], topk[w:], topp[w:], seed[w:], draw[w:] = 0.0, 0, 0.0, 0, 0
        rows_of = np.asarray(slots, dtype=np.int64)
        for view, u, tbl in zip(views["tables"], used, tables_of):
            view[:len(slots), :u] = tbl[rows_of, :u]

    def _context(self, layout: StepLayout, dev: torch.Tensor, host: HostStep, decode_only: bool) -> Tuple[StepContext, dict]:
        d = layout.views(dev, as_numpy=False)
        tables = {g.name: t for g, t in zip(self.groups, d["tables"])}
        ctx = StepContext(
            n_tokens=layout.n, n_requests=layout.r, token_ids=d["tok"], positions=d["pos"], req_of_token=d["req"],
            q_start=d["qs"], kv_len=d["kv"], slots=d["slots"], logit_rows=d["rows"], block_tables=tables, host=host,
            error_flag=self._error_word, decode_only=decode_only, settled=True, token_from_slot=d["src"],
            chosen=self.chosen)
        return ctx, d

    def _choose(self, logits: torch.Tensor, d: dict, mode: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A token for every row of ``logits``; each request's last one also goes to its slot of ``chosen``."""
        if mode == "greedy":
            return sampling_ops.argmax(logits, out=out, scatter_index=d["row_slot"], scatter=self.chosen)
        return sampling_ops.sample(logits, d["temp"], d["topk"], d["topp"], d["seed"], d["draw"], out=out,
                                   scatter_index=d["row_slot"], scatter=self.chosen)

    def step(self, entries: Sequence[StepEntry], **kwargs) -> Optional[torch.Tensor]:
        """Run one batch of live requests (by the ids given to ``add_request``); returns
        float32 logits [wanted, vocab] on the device in the order of the entries and of
        their ``want`` (None if nothing is wanted)."""
        return self.run(entries, **kwargs).logits

    def run(self, entries: Sequence[StepEntry], **kwargs) -> StepOutput:
        """``run_step`` for requests named by the ids given to ``add_request``."""
        for e in entries:
            if e.request not in self._slot_of:
                raise StepError(f"request {e.request!r} is not live (add_request first)")
        return self.run_step([self._slot_of[e.request] for e in entries], entries, **kwargs)

    @torch.no_grad()
    def run_step(self, slots: Sequence[int], entries: Sequence[StepEntry],
                 sampling: Optional[Sequence[SamplingParams]] = None, draws: Optional[Sequence[int]] = None,
                 graphs: Optional[bool] = None, keep_logits: bool = True) -> StepOutput:
        """The step function: entry i belongs to the request that holds ``slots[i]``.

        ``sampling`` / ``draws``: one ``SamplingParams`` and one draw counter per wanted place, in order; a
        token is then chosen at each.  ``graphs``: replay a recording when the step's shape allows it (default:
        the engine configuration's ``use_graphs``).  ``keep_logits=False`` lets a step that chooses tokens drop
        the logits.  Raises ``OutOfPages`` (nothing reserved, nothing run) or ``StepError``.
        """
        slots = [int(s) for s in slots]
        self._validate(slots, entries, sampling, draws)
        q_lens = [1 if e.tokens is None else len(e.tokens) for e in entries]
        before = [self.manager.length(s) for s in slots]
        new_lens = [b + q for b, q in zip(before, q_lens)]
        if not self.manager.reserve_many(slots, new_lens):
            raise OutOfPages(f"no pages left for a step of {sum(q_lens)} tokens of {len(entries)} requests "
                             f"(free: {self.free_pages()})")
        q_start = [0]
        for q in q_lens:
            q_start.append(q_start[-1] + q)
        host = HostStep(slots=slots, q_start=q_start, ctx_before=before, max_q_len=max(q_lens), max_kv_len=max(new_lens))
        n_want = sum(len(e.want) for e in entries)
        mode = "none" if sampling is None else ("greedy" if all(p.greedy for p in sampling) else "sampled")
        keep = keep_logits or mode == "none"
        recording = None
        if self.engine_config.use_graphs if graphs is None else graphs:
            key = self.model.capture_key(host)
            if key is not NOT_CAPTURABLE:
                recording = self._recording(host, n_want, mode, keep, key)
        if recording is not None:
            out = recording.run(host, entries, q_lens, sampling, draws, n_want)
        else:
            out = self._run_launched(host, entries, q_lens, sampling, draws, n_want, mode, keep)
        self.manager.commit_many(slots, new_lens)
        if mode != "none":
            for s, e in zip(slots, entries):
                if len(e.want):
                    self._has_choice[s] = True
        self.steps_run += 1
        self.last_h2d_bytes = out.h2d_bytes
        self.last_captured = recording
        if os.environ.get("YALIS_B200_CHECK"):
            self.check_device_errors()
        return out

    def _run_launched(self, host: HostStep, entries, q_lens, sampling, draws, n_want, mode, keep) -> StepOutput:
        n, r = host.q_start[-1], len(entries)
        used = [min(g.max_pages_per_request, -(-host.max_kv_len // g.page_size)) for g in self.groups]
        layout = StepLayout(n, r, n_want, used, sampling=(mode == "sampled"))
        pinned, which = self._staging_buffer(layout.total)
        self._fill(layout.views(pinned, as_numpy=True), host.slots, entries, host.ctx_before, q_lens, sampling, draws, used,
                   [self.manager.table(g.name) for g in self.groups], self.null_slot)
        dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[:layout.total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._staging[which] = (pinned, ev)
        ctx, d = self._context(layout, dev, host, decode_only=host.max_q_len == 1)
        stream = self.model.forward(ctx, self.storage.entries)
        logits = tokens = None
        if n_want:
            logits = self.model.logits(stream, ctx.logit_rows)
            if mode != "none":
                tokens = self._choose(logits, d, mode)
                self.chosen[-1:].copy_(self._error_word)
        return StepOutput(logits if keep else None, tokens, False, 4 * layout.total)

    MAX_EXACT_RECORDINGS = 256      # recordings of steps other than single tokens kept at a time
    IDLE_STEPS_BEFORE_EVICTION = 2048   # a recording makes room for another only after so many steps without use

    def _recording(self, host: HostStep, n_want: int, mode: str, keep_logits: bool, capture_key):
        """The recording that replays a step with these facts, or None if the step is to be launched.

        Steps of single tokens share a recording per bucket of requests (padded).  Any other step (prompt portions,
        portions beside decoding requests) is recorded with room for its tokens, requests, wanted rows and longest
        portion rounded up (tokens to a multiple of 64, the others to powers of two; the rest is padding: rows of
        no request, requests without tokens), and only when the same kind of step has been seen before: serving
        fills its token budget step after step, one-off shapes are not worth a recording (it costs about three
        launched steps).  When these recordings are full, the least recently used one makes
        room only if it has lain idle for ``IDLE_STEPS_BEFORE_EVICTION`` steps; otherwise the new shape is
        launched.  (Least-recently-used alone records every step anew when more shapes than there is room for
        come in turn: 130 shapes with room for 48 took 7.1 s instead of 4.2.)"""
        from yalis_b200.engine.recorded import RecordedStep, bucket_for
        n, r = host.q_start[-1], len(host.slots)
        self._steps_seen += 1
        if host.max_q_len == 1:
            if n_want == 0:
                return None
            size = bucket_for(r)
            shape = (size, size, size, True)
        else:
            # room for the step: tokens to the next multiple of 64 (a power of two up to 64), requests, wanted
            # rows and the longest portion to the next power of two; what the step leaves unused is padding
            shape = (bucket_for(max(n, 16)) if n <= 64 else -(-n // 64) * 64, bucket_for(r),
                     bucket_for(n_want) if n_want else 0, False, bucket_for(max(host.max_q_len, 16)))
        key = (shape[0], mode, keep_logits, capture_key, shape)
        rec = self._recordings.get(key)
        if rec is not None:
            if not shape[3]:
                self._recordings[key] = self._recordings.pop(key)          # most recently used last
            rec.last_used = self._steps_seen
            return rec
        if not shape[3]:
            seen = self._seen_shapes.get(key, 0)
            self._seen_shapes[key] = seen + 1
            if seen == 0:
                if len(self._seen_shapes) > 4096:
                    self._seen_shapes.clear()
                return None
            exact = [k for k in self._recordings if not k[4][3]]
            if len(exact) >= self.MAX_EXACT_RECORDINGS:
                if self._steps_seen - self._recordings[exact[0]].last_used < self.IDLE_STEPS_BEFORE_EVICTION:
                    return None
                del self._recordings[exact[0]]
        rec = self._recordings[key] = RecordedStep(self, shape[0], shape[1], shape[2], shape[3], mode, keep_logits, key,
                                                   longest_portion=None if shape[3] else shape[4])
        rec.last_used = self._steps_seen
        return rec
