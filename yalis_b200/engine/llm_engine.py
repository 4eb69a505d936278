"""``LLMEngine``: the Python entry point, in the reference's manner.

    engine = LLMEngine(ModelConfig(...), InferenceConfig(...))
    tokens, metrics = engine.generate(prompts, tokens_to_generate=50)

(yalis/engine.py:168-573).  ``prompts`` are lists of token ids (strings need a
tokenizer in the model folder).  Unlike the reference, whose call is one fixed
batch, the prompts go through the scheduler: any number of them, admitted as
slots and pages allow, prefilled in portions beside the decoding of others.
"""

from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from yalis_b200.config.presets import preset
from yalis_b200.config.runtime import InferenceConfig, ModelConfig
from yalis_b200.engine.engine import Engine, StepEntry
from yalis_b200.engine.scheduler import Request, Scheduler, StepPlan
from yalis_b200.engine.timers import Timers
from yalis_b200.sampling.sampler import Sampler, SamplingParams, request_seed


class _PendingTokens:
    """A decode step whose chosen tokens are on their way to the host."""

    def __init__(self, requests, slots, host, event):
        self.requests, self.slots, self.host, self.event = requests, slots, host, event
        self.positions = None          # index of the placeholder in each request's output

    def read(self) -> List[int]:
        self.event.synchronize()
        return self.host[:len(self.requests)].tolist()


class LLMEngine:
    def __init__(self, model_config: ModelConfig, inference_config: InferenceConfig, device: str = "cuda:0"):
        self.model_config = model_config
        self.inference_config = ic = inference_config
        kwargs = dict(dtype=model_config.precision, page_size=ic.page_size, max_slots=ic.max_batch_size,
                      max_context=None, device=device,
                      cache_tokens=ic.cache_tokens or ic.max_batch_size * ic.max_length)
        if model_config.random_weights:
            cfg = preset(model_config.model_name)
            kwargs["max_context"] = min(ic.max_length, cfg["max_position_embeddings"])
            self.engine = Engine(config=cfg, seed=model_config.seed, **kwargs)
        else:
            from yalis_b200.config.registry import load_config
            _, cfg = load_config(model_config.model_path)
            kwargs["max_context"] = min(ic.max_length, getattr(cfg, "max_position_embeddings", ic.max_length))
            self.engine = Engine(model_config.model_path, **kwargs)
        self.device = self.engine.device
        self.sampler = Sampler(self.device)
        self.tokenizer = None
        self._requests_made = 0
        self.use_graphs = os.environ.get("YALIS_DISABLE_DECODE_CUDAGRAPHS", "0") != "1"
        self.max_steps_in_flight = 2        # decode steps the host may run ahead of the tokens it has read
        self._token_buffers: List[torch.Tensor] = []

    # ---- tokenizer (optional sugar; token ids are the interface) -----------------------
    def _tokenize(self, prompts: Sequence[str]) -> List[List[int]]:
        if self.tokenizer is None:
            path = self.model_config.model_path
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(path)
            except Exception as e:
                raise ValueError(f"string prompts need a tokenizer in {path}: {e}") from None
        return [self.tokenizer(p)["input_ids"] for p in prompts]

    def _eos_id(self) -> Optional[int]:
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            return self.tokenizer.eos_token_id
        return self.engine.spec.eos_token_id

    # ---- generation ------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Union[List[str], List[List[int]]], tokens_to_generate: int = 50,
                 report_throughput: bool = False, ignore_eos: Optional[bool] = True,
                 enable_nvtx: Optional[bool] = False, get_logits: Optional[bool] = False):
        """Generate ``tokens_to_generate`` tokens after each prompt.

        Returns ``(tokens, metrics)`` or ``(tokens, metrics, logits)`` with
        ``get_logits``: ``tokens`` is an int64 tensor [batch, generated] on the device;
        a row that ended early at EOS (``ignore_eos=False``) is filled up with EOS, as in
        the reference (yalis/engine.py:509-519).  ``logits`` is a list, per request, of
        float32 tensors [generated_i, vocab] (the logits each token was drawn from).
        """
        timers = Timers()
        t_tok = time.perf_counter()
        if len(prompts) == 0:
            raise ValueError("no prompts")
        if isinstance(prompts[0], str):
            prompts = self._tokenize(prompts)
        tokenization_ms = (time.perf_counter() - t_tok) * 1e3
        ic = self.inference_config
        eos = None if ignore_eos else self._eos_id()
        sched = Scheduler(self.engine.manager, ic.max_tokens_per_step, ic.prefill_chunk,
                          max_context=self.engine.max_context, reset_slot=self.engine.storage.reset_slot)
        requests = []
        for i, p in enumerate(prompts):
            sp = SamplingParams(temperature=ic.temperature if ic.temperature is not None else 1.0, top_k=ic.top_k,
                                top_p=ic.top_p if ic.top_p is not None else 1.0,
                                seed=request_seed(ic.seed, self._requests_made + i))
            r = Request(i, [int(t) for t in p], tokens_to_generate, sp, eos_id=eos)
            sched.add(r)
            requests.append(r)
        self._requests_made += len(prompts)
        logits_out: Dict[int, List[torch.Tensor]] = {r.id: [] for r in requests}
        nvtx = torch.cuda.nvtx if enable_nvtx else None
        first_token_ms = None
        n_decode_steps = 0
        timers.start("generate")
        t0 = time.perf_counter()
        pending: List[_PendingTokens] = []      # decode steps whose tokens the host has not read yet
        while sched.has_work():
            plan = sched.plan()
            if plan.preempted:
                self._resolve(pending)          # a preempted request is recomputed from its real tokens
            if not plan.entries:
                if plan.failed or plan.preempted:
                    continue
                raise RuntimeError("the scheduler made no progress")
            decode_only = all(e.count == 1 for e in plan.entries)
            name = "decode" if decode_only else "prefill"
            if nvtx:
                nvtx.range_push("Decode" if decode_only else "Prefill")
            timers.start(name)
            if self.use_graphs and all(e.count == 1 and e.samples for e in plan.entries):
                sampled = self._run_decode(plan, pending, logits_out if get_logits else None)
            else:
                self._resolve(pending)
                sampled = self._run_plan(plan, logits_out if get_logits else None)
            timers.stop(name)
            if nvtx:
                nvtx.range_pop()
            if first_token_ms is None and sampled:
                first_token_ms = (time.perf_counter() - t0) * 1e3
            n_decode_steps += decode_only
            sched.update(plan, sampled)
            if pending and pending[-1].positions is None:
                pending[-1].positions = [len(r.output) - 1 for r in pending[-1].requests]
        self._resolve(pending)
        timers.stop("generate")
        times, counts = timers.get_times()
        n_cols = max(len(r.output) for r in requests)
        fill = eos if eos is not None else 0
        out = torch.full((len(requests), n_cols), fill, dtype=torch.int64)
        for i, r in enumerate(requests):
            out[i, :len(r.output)] = torch.tensor(r.output, dtype=torch.int64)
        out = out.to(self.device)
        e2e = times[("generate",)]
        generated = sum(len(r.output) for r in requests)
        reasons = sorted({r.finish_reason for r in requests})
        metrics = {
            "BatchSize": len(requests),
            "PromptLength": max(len(r.prompt) for r in requests),
            "DecodeLength": tokens_to_generate,
            "Throughput": generated / (e2e / 1e3) if e2e > 0 else 0.0,
            "TTFT": first_token_ms if first_token_ms is not None else 0.0,
            "TBT": (times.get(("generate", "decode"), 0.0) / counts[("generate", "decode")])
            if counts.get(("generate", "decode")) else 0.0,
            "E2E": e2e,
            "TokenizationTime": tokenization_ms,
            "FinishedReason": "EOS" if reasons == ["eos"] else ("Max Token Length" if reasons == ["length"] else ",".join(map(str, reasons))),
            "Preemptions": sum(r.preemptions for r in requests),
            "Steps": counts.get(("generate", "decode"), 0) + counts.get(("generate", "prefill"), 0),
        }
        if report_throughput:
            print(f"[Metrics] BatchSize = {metrics['BatchSize']}, PromptLength = {metrics['PromptLength']}, "
                  f"DecodeLength = {tokens_to_generate}, Throughput = {metrics['Throughput']:.2f} tok/s, "
                  f"TTFT = {metrics['TTFT']:.4f} ms, TBT = {metrics['TBT']:.4f} ms, E2E = {e2e:.4f} ms, "
                  f"FinishedReason = {metrics['FinishedReason']}")
        if get_logits:
            return out, metrics, [torch.stack(logits_out[r.id]) if logits_out[r.id] else None for r in requests]
        return out, metrics

    def _run_decode(self, plan: StepPlan, pending: List["_PendingTokens"], logits_out) -> List[int]:
        """A step of single tokens through the captured decode graph (unless
        YALIS_DISABLE_DECODE_CUDAGRAPHS=1, the reference's switch, yalis/engine.py:44-48).

        The host does not wait for the step: the chosen tokens are copied to pinned memory
        asynchronously and read one or two steps later, and the next step of the same batch
        takes its input ids from the device.  That is possible while nothing the host decides
        depends on the token values: requests that stop at an EOS id are read at once.
        Returns the tokens, or -1 placeholders that ``_resolve`` fills in later."""
        reqs = [e.request for e in plan.entries]
        slots = [r.slot for r in reqs]
        n = len(reqs)
        # the same requests as the step before (not merely the same slots: a request that takes over a slot
        # with a one-token prompt starts with that token, not with what the slot's last owner drew)
        same_batch = bool(pending) and len(pending[-1].requests) == n and all(
            a is b for a, b in zip(pending[-1].requests, reqs))
        if pending and not same_batch:
            self._resolve(pending)
        bucket = self.engine.decoder.step(
            slots, tokens=None if same_batch else [r.last_token for r in reqs], params=[r.sampling for r in reqs],
            draws=[len(r.output) for r in reqs], keep_logits=logits_out is not None)
        host = self._token_buffers.pop() if self._token_buffers else torch.empty(self.engine.max_slots, dtype=torch.int32).pin_memory()
        host[:n].copy_(bucket.tokens[:n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        if logits_out is not None:
            for i, r in enumerate(reqs):
                logits_out[r.id].append(bucket.logits[i].clone())
        entry = _PendingTokens(reqs, slots, host, event)
        if any(r.eos_id is not None for r in reqs):
            tokens = entry.read()
            self._token_buffers.append(host)
            return tokens
        pending.append(entry)
        if len(pending) > self.max_steps_in_flight:
            self._resolve(pending, keep=self.max_steps_in_flight)
        return [-1] * n

    def _resolve(self, pending: List["_PendingTokens"], keep: int = 0) -> None:
        """Read the tokens of all but the newest ``keep`` pending steps into the requests' outputs."""
        while len(pending) > keep:
            entry = pending.pop(0)
            for r, pos, tok in zip(entry.requests, entry.positions, entry.read()):
                r.output[pos] = tok
            self._token_buffers.append(entry.host)

    def _run_plan(self, plan: StepPlan, logits_out) -> List[int]:
        """One engine step for the plan, then one draw per entry that reached its last token."""
        entries, slots, samplers = [], [], []
        for e in plan.entries:
            toks = e.request.tokens[e.start:e.start + e.count]
            entries.append(StepEntry(e.request.id, toks, [e.count - 1] if e.samples else []))
            slots.append(e.request.slot)
            if e.samples:
                samplers.append(e.request)
        logits = self.engine.step_slots(slots, entries)
        if not samplers:
            return []
        toks = self.sampler.sample(logits, [r.sampling for r in samplers], [len(r.output) for r in samplers])
        if logits_out is not None:
            for i, r in enumerate(samplers):
                logits_out[r.id].append(logits[i].clone())
        return toks.tolist()

    def reset_kv_cache(self, max_batch_size: Optional[int] = None) -> None:
        """Kept for callers of the reference (yalis/engine.py): the cache needs no reset
        between calls here, every request gives its pages back when it finishes."""


def generate(model: Union[str, LLMEngine], prompts: List[List[int]], max_new_tokens: int = 50,
             temperature: float = 0.0, top_k: Optional[int] = None, top_p: float = 0.0, seed: int = 1234,
             precision: str = "bf16", ignore_eos: bool = True, **inference_options) -> List[List[int]]:
    """Token ids in, token ids out: generate after each prompt with a model folder (or an
    existing ``LLMEngine``).  The defaults (temperature 0, top_p 0) are greedy."""
    if isinstance(model, LLMEngine):
        engine = model
        engine.inference_config.temperature, engine.inference_config.top_k = temperature, top_k
        engine.inference_config.top_p, engine.inference_config.seed = top_p, seed
    else:
        longest = max(len(p) for p in prompts) + max_new_tokens
        ic = InferenceConfig(max_batch_size=inference_options.pop("max_batch_size", min(len(prompts), 64)),
                             max_length_of_generated_sequences=inference_options.pop(
                                 "max_length_of_generated_sequences", longest),
                             temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, **inference_options)
        engine = LLMEngine(ModelConfig(model_name=model, model_path=model, precision=precision), ic)
    tokens, _ = engine.generate(prompts, tokens_to_generate=max_new_tokens, ignore_eos=ignore_eos)
    rows = tokens.tolist()
    return [row[:max_new_tokens] for row in rows]
