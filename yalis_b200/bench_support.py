"""Pieces of the benchmark that drive the engine below the scheduler: a batch of requests
prefilled to a given length and then decoded for K steps with the chosen tokens fed back
on the device, a timed prefill, and the byte and flop counts of the model for rooflines."""

from __future__ import annotations

from typing import Callable, Dict, List

import time

import torch

from yalis_b200.engine.engine import Engine, StepEntry
from yalis_b200.parts.base import PagedKV
from yalis_b200.sampling.sampler import GREEDY


def model_numbers(engine: Engine) -> Dict[str, object]:
    """Bytes a decode step must read and flops of a prefill, from the built model."""
    m = engine.model
    elt = 2 if engine.dtype == torch.bfloat16 else 4
    emb_bytes = m.embedding.numel() * m.embedding.element_size()
    tied = m.head.data_ptr() == m.embedding.data_ptr()
    # every weight a step uses once: all layer matrices and norms, the output matrix; of the
    # embedding table only the rows of the step's tokens are read
    weight_bytes = m.weight_bytes() - (0 if tied else emb_bytes)
    kv_per_token = 0
    for req, cache in zip(m.cache_requests(), engine.storage.entries):
        if isinstance(req, PagedKV) and getattr(cache, "writable", False):
            kv_per_token += 2 * req.num_kv_heads * req.head_dim * elt
    matrix_flops = 0.0
    mixers = []
    for entry in engine.spec.schedule:
        b = m.blocks[entry.layer]
        matrix_flops += sum(part.matrix_flops_per_token() for part in b.parts.values())
        mixers += [part for part in b.parts.values() if hasattr(part, "mixing_flops")]
    head_params = m.head.shape[0] * m.head.shape[1]

    def flops_prefill(tokens: int, logit_rows: int = 1) -> float:
        """One prompt of ``tokens`` tokens from an empty cache, logits at ``logit_rows`` places."""
        return tokens * matrix_flops + sum(mx.mixing_flops(tokens, 0) for mx in mixers) + 2.0 * logit_rows * head_params

    return {"weight_bytes_per_step": weight_bytes, "kv_bytes_per_token": kv_per_token, "flops_prefill": flops_prefill,
            "matrix_flops_per_token": matrix_flops}


SETTLE_SECONDS = 1.0     # idle time between the prompt phase and the decode steps of DecodeBench


class DecodeBench:
    """``batch`` requests with ``prompt_len`` cached tokens each, decoded step by step through the engine's
    step function (recorded steps, greedy choice) with the chosen tokens fed back on the device."""

    def __init__(self, engine: Engine, batch: int, prompt_len: int, seed: int = 0, prefill_tokens_per_step: int = 2048,
                 settle_seconds: float = SETTLE_SECONDS):
        self.engine, self.batch, self.prompt_len, self.seed = engine, batch, prompt_len, seed
        self.settle_seconds = settle_seconds
        self.per_step = prefill_tokens_per_step
        self.ids = [("bench", seed, i) for i in range(batch)]
        self.slots: List[int] = []
        self.steps_done = 0
        self.launches_per_step = 0
        self.h2d_bytes_per_step = 0

    def prepare(self) -> None:
        eng = self.engine
        gen = torch.Generator().manual_seed(self.seed)
        for rid in self.ids:
            slot = eng.add_request(rid)
            if slot is None:
                raise RuntimeError("no free slot for the benchmark batch")
            self.slots.append(slot)
        group, group_tokens = [], 0
        prompts = [torch.randint(0, eng.vocab_size, (self.prompt_len,), generator=gen).tolist() for _ in self.ids]

        def flush():
            nonlocal group, group_tokens
            if group:
                eng.run([StepEntry(rid, p, [len(p) - 1]) for rid, p in group], sampling=[GREEDY] * len(group),
                        draws=[0] * len(group), keep_logits=False)
                group, group_tokens = [], 0

        for rid, p in zip(self.ids, prompts):
            if group_tokens + len(p) > self.per_step:
                flush()
            group.append((rid, p))
            group_tokens += len(p)
        flush()
        self._entries = [StepEntry(rid, None, [0]) for rid in self.ids]
        self._greedy = [GREEDY] * self.batch
        self.run(1)
        # The prompt phase draws the full power limit and leaves the SM clock low for the next 0.1 s (measured:
        # 1,297 MHz and 3.96 ms a step right after it, 1,417 MHz and 3.26 ms twenty steps later, 1,965 MHz after
        # that; with this pause 1,965 MHz from the first step).  The steps timed here are to say what the decode
        # kernels do, so they start from a settled clock; the end-to-end figure has no such pause.
        torch.cuda.synchronize()
        time.sleep(self.settle_seconds)

    def run(self, steps: int) -> None:
        eng = self.engine
        for i in range(steps):
            eng.run_step(self.slots, self._entries, sampling=self._greedy, draws=[self.steps_done + i] * self.batch,
                         graphs=True, keep_logits=False)
        self.steps_done += steps
        if steps and eng.last_captured is not None:
            self.launches_per_step = eng.last_captured.launches
            self.h2d_bytes_per_step = eng.last_h2d_bytes

    def run_timed(self, steps: int) -> float:
        """Milliseconds of ``steps`` decode steps on the device (CUDA events, synchronised on both sides)."""
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._timed_from = self.steps_done
        start.record()
        self.run(steps)
        end.record()
        torch.cuda.synchronize()
        self.engine.check_device_errors()
        return start.elapsed_time(end)

    def mean_context(self, steps: int) -> float:
        """Mean number of cached tokens per request that the timed steps attended to."""
        first = self.prompt_len + self._timed_from + 1
        return first + (steps - 1) / 2.0

    def finish(self) -> None:
        for rid in self.ids:
            self.engine.finish_request(rid)
        self.slots = []


def prefill_bench(engine: Engine, tokens: int, warmup: int = 2, iters: int = 3) -> float:
    """Milliseconds (median of ``iters``) of one step that prefills a single ``tokens``-token prompt (logits of
    its last token)."""
    gen = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, engine.vocab_size, (tokens,), generator=gen).tolist()
    times = []
    for i in range(warmup + iters):
        rid = ("prefill", i)
        engine.add_request(rid)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry(rid, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.finish_request(rid)
        if i >= warmup:
            times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]        # the median: single steps vary by a few percent with the clocks
