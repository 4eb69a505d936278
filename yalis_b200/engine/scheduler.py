"""The scheduler: which tokens of which requests run in the next step.

The reference has none: a call to generate is one fixed, padded batch that is
prefilled whole and decoded in lock-step (yalis/engine.py:371-573).  Here
requests arrive in a queue and every step is planned anew:

1. **Decodes first.**  Every running request whose cached tokens reach its last
   token but one contributes that last token (one token each).
2. **Then portions of prompts** of the running requests that are still being
   prefilled, oldest first, each at most ``prefill_chunk`` tokens and together
   within what is left of ``max_tokens_per_step``.
3. **Then admissions** from the waiting queue, first come first served, while a
   slot is free, budget is left and the pages of the first portion can be had.

A request is a list of tokens (prompt + what it has generated) and a count of
how many of them the cache holds; a step feeds the next q of them, and when
that reaches the end, the logits of the last fed token are sampled.  Prefill
and decode are the same thing with q > 1 or q = 1.

**When pages run out** the step never faults:

* a decode that cannot get its page preempts the *youngest* running request
  (the one admitted last, possibly itself): its pages and slot are freed and it
  returns to the front of the waiting queue with all its tokens, to be
  recomputed;
* a prompt portion that cannot get its pages is shortened to what fits, or
  waits for a later step;
* if nothing at all can run while requests are live, the youngest is preempted
  to let the others through; a request that cannot run even alone (its tokens
  exceed the whole pool) is finished with the reason ``"out_of_pages"``.

Finishing (``max_new_tokens`` reached, the EOS id drawn, or the context limit)
frees slot and pages within the same update, before the next plan.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from yalis_b200.cache.manager import CacheManager
from yalis_b200.sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass(eq=False)          # a request is itself: membership tests must not compare token lists
class Request:
    id: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_id: Optional[int] = None
    # ---- scheduler state ----
    state: str = WAITING
    output: List[int] = field(default_factory=list)
    slot: Optional[int] = None
    computed: int = 0                 # tokens the cache holds
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1             # admission order (for "youngest")

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def total(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def last_token(self) -> int:
        return self.output[-1] if self.output else self.prompt[-1]


@dataclass
class PlannedEntry:
    request: Request
    start: int        # index of the first token fed (== request.computed)
    count: int        # tokens fed
    samples: bool     # the portion reaches the request's last token: sample after it
    slot: Optional[int] = None    # the request's slot when the step ran (it may finish and lose it in the update)


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, manager: CacheManager, max_tokens_per_step: int = 2048, prefill_chunk: Optional[int] = None,
                 max_context: Optional[int] = None, reset_slot=None):
        if max_tokens_per_step <= 0:
            raise ValueError("max_tokens_per_step must be positive")
        if prefill_chunk is not None and prefill_chunk <= 0:
            raise ValueError("prefill_chunk must be positive")
        self.manager = manager
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk or max_tokens_per_step
        self.max_context = max_context
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._admissions = 0
        self._reset_slot = reset_slot      # called with the slot of a newly admitted request

    # ---- queue -------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.id!r} has an empty prompt")
        if request.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        limit = self.max_context
        if limit is not None:
            if len(request.prompt) > limit:
                # the reference refuses over-long prompts (yalis/engine.py:353-358)
                raise ValueError(f"prompt of {len(request.prompt)} tokens exceeds the context limit {limit}")
            # ... and clamps the number of new tokens to what fits (yalis/engine.py:359-368)
            request.max_new_tokens = min(request.max_new_tokens, limit - len(request.prompt) + 1)
        if not self.manager.fits(len(request.prompt)):
            raise ValueError(f"prompt of {len(request.prompt)} tokens exceeds the block-table width")
        request.state = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- helpers -----------------------------------------------------------------------
    def _release(self, r: Request) -> None:
        if r.slot is not None:
            self.manager.release(r.slot)
            r.slot = None
        r.computed = 0

    def _finish(self, r: Request, reason: str) -> None:
        self._release(r)
        r.state, r.finish_reason = FINISHED, reason
        if r in self.running:
            self.running.remove(r)
        self.finished.append(r)

    def _preempt(self, r: Request, plan: StepPlan) -> None:
        """Free everything the request holds; it goes back to the head of the queue."""
        plan.entries = [e for e in plan.entries if e.request is not r]
        self._release(r)
        self.running.remove(r)
        r.state = WAITING
        r.preemptions += 1
        self.waiting.appendleft(r)
        plan.preempted.append(r)

    def _youngest(self, exclude: Optional[Request] = None) -> Optional[Request]:
        cands = [r for r in self.running if r is not exclude]
        return max(cands, key=lambda r: r.admitted_at) if cands else None

    def _fitting(self, r: Request, want: int) -> int:
        """The largest count <= want whose pages can be reserved now (0 if none)."""
        lo, hi = 0, want
        base = r.computed
        if self.manager.can_reserve(r.slot, base + want):
            return want
        while lo < hi:                      # can_reserve is monotone in the length
            mid = (lo + hi + 1) // 2
            if self.manager.can_reserve(r.slot, base + mid):
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ---- planning ----------------------------------------------------------------------
    def plan(self) -> StepPlan:
        plan = StepPlan()
        while True:
            self._plan_once(plan)
            if plan.entries or not self.running:
                break
            # Live requests, but none can move: make room by preempting the youngest.
            victim = self._youngest()
            if len(self.running) == 1:
                self._finish(victim, "out_of_pages")
                plan.failed.append(victim)
            else:
                self._preempt(victim, plan)
        return plan

    def _plan_once(self, plan: StepPlan) -> None:
        budget = self.max_tokens_per_step - plan.n_tokens
        planned = {id(e.request) for e in plan.entries}
        # 1. decodes, oldest first, so that the youngest is the first to give way
        in_order = sorted(self.running, key=lambda r: r.admitted_at)
        decoding = [r for r in in_order if id(r) not in planned and r.total - r.computed == 1][:max(budget, 0)]
        if decoding and self.manager.reserve_many([r.slot for r in decoding], [r.computed + 1 for r in decoding]):
            # the usual case: every one of them gets its page (or needs none), nobody has to give way
            plan.entries.extend(PlannedEntry(r, r.computed, 1, True) for r in decoding)
            planned.update(id(r) for r in decoding)
            budget -= len(decoding)
            in_order = ()
        for r in in_order:
            if id(r) in planned or r not in self.running or r.total - r.computed != 1:
                continue
            if budget <= 0:
                break
            ok = self.manager.reserve(r.slot, r.computed + 1)
            while not ok:
                victim = self._youngest()
                if victim is r:
                    if len(self.running) == 1:      # alone and still no page: it can never continue
                        self._finish(r, "out_of_pages")
                        plan.failed.append(r)
                    else:
                        self._preempt(r, plan)
                    break
                self._preempt(victim, plan)
                planned.discard(id(victim))
                ok = self.manager.reserve(r.slot, r.computed + 1)
            if ok:
                plan.entries.append(PlannedEntry(r, r.computed, 1, True))
                planned.add(id(r))
                budget -= 1
        budget = self.max_tokens_per_step - plan.n_tokens
        # 2. portions of running prompts
        for r in sorted(self.running, key=lambda r: r.admitted_at):
            if budget <= 0:
                break
            if id(r) in planned:
                continue
            left = r.total - r.computed
            if left <= 1:
                continue
            count = self._fitting(r, min(left, self.prefill_chunk, budget))
            if count == 0:
                continue
            self.manager.reserve(r.slot, r.computed + count)
            plan.entries.append(PlannedEntry(r, r.computed, count, count == left))
            planned.add(id(r))
            budget -= count
        # 3. admissions
        while self.waiting and budget > 0 and self.manager.free_slots() > 0:
            r = self.waiting[0]
            if r in plan.preempted:
                break                      # not in the step that preempted it
            slot = self.manager.acquire()
            r.slot, r.computed = slot, 0
            count = self._fitting(r, min(r.total, self.prefill_chunk, budget))
            if count == 0:
                self.manager.release(slot)
                r.slot = None
                if not self.running and not plan.entries:
                    # nothing else holds pages, yet not one token fits
                    self.waiting.popleft()
                    r.state, r.finish_reason = FINISHED, "out_of_pages"
                    self.finished.append(r)
                    plan.failed.append(r)
                    continue
                break
            self.waiting.popleft()
            if self._reset_slot is not None:
                self._reset_slot(slot)
            self.manager.reserve(slot, count)
            r.state = RUNNING
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            plan.entries.append(PlannedEntry(r, 0, count, count == r.total))
            budget -= count

    # ---- after the step -----------------------------------------------------------------
    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Record what the step computed; ``sampled`` has one token per sampling entry,
        in plan order.  Returns the requests that finished."""
        done: List[Request] = []
        it = iter(sampled)
        for e in plan.entries:
            e.request.computed = e.start + e.count
        self.manager.commit_many([e.request.slot for e in plan.entries], [e.request.computed for e in plan.entries])
        for e in plan.entries:
            r = e.request
            if not e.samples:
                continue
            tok = int(next(it))
            r.output.append(tok)
            if r.eos_id is not None and tok == r.eos_id:
                reason = "eos"
            elif len(r.output) >= r.max_new_tokens:
                reason = "length"
            elif self.max_context is not None and r.total > self.max_context:
                reason = "context"
            else:
                continue
            self._finish(r, reason)
            done.append(r)
        return done
