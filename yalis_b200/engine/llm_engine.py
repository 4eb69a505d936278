"""``LLMEngine`` and ``generate``: the Python entry points.

    engine = LLMEngine(ModelConfig(...), InferenceConfig(...))
    tokens, metrics = engine.generate(prompts, tokens_to_generate=50)          # the reference's call
    results = generate(model_dir, prompts, max_new_tokens=50, eos_id=2)        # per-request results

``LLMEngine.generate`` keeps the reference's signature and return value
(yalis/engine.py:371-379, 570-573): a padded [batch, generated] tensor and a
metrics dictionary.  ``LLMEngine.run`` and the module-level ``generate`` return
one ``Generation`` per prompt instead: its tokens at their true length, why it
ended, and the logits if asked for; sampling parameters may differ between
the prompts of one call.

``prompts`` are lists of token ids (strings need a tokenizer in the model
folder).  Unlike the reference, whose call is one fixed batch, the prompts go
through the scheduler: any number of them, admitted as slots and pages allow,
prefilled in portions beside the decoding of others.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from yalis_b200.config.presets import preset
from yalis_b200.config.runtime import InferenceConfig, ModelConfig
from yalis_b200.engine.engine import ChosenTokens, Engine, StepEntry
from yalis_b200.engine.scheduler import Request, Scheduler, StepPlan
from yalis_b200.engine.timers import Timers
from yalis_b200.sampling.sampler import SamplingParams, request_seed

PENDING = -1      # placeholder in a request's output for a token that is chosen but not yet read by the host


@dataclass
class Generation:
    """What one prompt led to."""

    tokens: List[int]                         # the generated tokens, at their true number
    finish_reason: str                        # "length", "eos", "context" or "out_of_pages"
    logits: Optional[torch.Tensor] = None     # float32 [len(tokens), vocab]: what each token was drawn from
    preemptions: int = 0


class _Pending:
    """The chosen tokens of one step on their way to the host, and where they go."""

    def __init__(self, report: ChosenTokens, targets):
        self.report, self.targets = report, targets      # targets: (request, index in its output, slot)

    def resolve(self) -> None:
        values = self.report.wait()
        for request, index, slot in self.targets:
            request.output[index] = int(values[slot])


class LLMEngine:
    def __init__(self, model_config: ModelConfig, inference_config: InferenceConfig, device: str = "cuda:0"):
        self.model_config = model_config
        self.inference_config = ic = inference_config
        if model_config.random_weights:
            cfg = preset(model_config.model_name)
            ec = ic.engine_config(model_config.precision, min(ic.max_length, cfg["max_position_embeddings"]), device)
            self.engine = Engine(config=cfg, seed=model_config.seed, engine_config=ec)
        else:
            self.engine = Engine(model_config.model_path, engine_config=ic.engine_config(model_config.precision, None, device))
        self.device = self.engine.device
        self.tokenizer = None
        self._requests_made = 0
        # the reference's switch (yalis/engine.py:44-48) turns recorded decode steps off
        self.use_graphs = ic.use_graphs and os.environ.get("YALIS_DISABLE_DECODE_CUDAGRAPHS", "0") != "1"
        self.max_steps_in_flight = 2        # steps the host may run ahead of the tokens it has read

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
    def run(self, prompts: Union[List[str], List[List[int]]], max_new_tokens: int = 50,
            sampling: Union[None, SamplingParams, Sequence[Optional[SamplingParams]]] = None,
            eos_id: Optional[int] = None, return_logits: bool = False, enable_nvtx: bool = False,
            step_log: Optional[list] = None):
        """Generate after each prompt; returns ``(results, metrics)`` with one ``Generation`` per prompt.

        ``sampling``: one ``SamplingParams`` for all prompts, or a list with one per prompt (None entries take
        the configuration's defaults with a seed of their own).  ``eos_id``: a request ends when it draws this
        token (None: only by length).  ``return_logits``: keep the float32 logits every token was drawn from.
        ``step_log``: a list that receives, per step, a dictionary with its ``tokens``, ``requests``,
        ``decoding`` (requests that brought one token), ``h2d_bytes``, ``captured``, ``replayed_launches``
        (kernels in the recording, if the step replayed one) and the CUDA events ``start`` / ``end`` around it
        (for benchmarks).
        """
        t_tok = time.perf_counter()
        if len(prompts) == 0:
            raise ValueError("no prompts")
        if isinstance(prompts[0], str):
            prompts = self._tokenize(prompts)
        tokenization_ms = (time.perf_counter() - t_tok) * 1e3
        if sampling is None or isinstance(sampling, SamplingParams):
            sampling = [sampling] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError(f"{len(sampling)} sampling parameter sets for {len(prompts)} prompts")
        ic, eng = self.inference_config, self.engine
        sched = Scheduler(eng.manager, ic.max_tokens_per_step, ic.prefill_chunk, max_context=eng.max_context,
                          reset_slot=eng.reset_slot)
        requests = []
        for i, (p, sp) in enumerate(zip(prompts, sampling)):
            if sp is None:
                sp = ic.default_sampling(request_seed(ic.seed, self._requests_made + i))
            r = Request(i, [int(t) for t in p], max_new_tokens, sp, eos_id=eos_id)
            sched.add(r)
            requests.append(r)
        self._requests_made += len(prompts)
        logits_out: Optional[Dict[int, List[torch.Tensor]]] = {r.id: [] for r in requests} if return_logits else None
        nvtx = torch.cuda.nvtx if enable_nvtx else None
        timers = Timers()
        first_token_ms = None
        timers.start("generate")
        t0 = time.perf_counter()
        pending: List[_Pending] = []
        try:
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
                if step_log is not None:
                    entry = {"tokens": plan.n_tokens, "requests": len(plan.entries),
                             "decoding": sum(e.count == 1 for e in plan.entries), "start": torch.cuda.Event(enable_timing=True),
                             "end": torch.cuda.Event(enable_timing=True)}
                    entry["start"].record()
                sampled = self._run_plan(plan, pending, logits_out)
                if step_log is not None:
                    entry["end"].record()
                    entry["h2d_bytes"], entry["captured"] = eng.last_h2d_bytes, eng.last_captured is not None
                    entry["replayed_launches"] = eng.last_captured.launches if eng.last_captured is not None else 0
                    step_log.append(entry)
                timers.stop(name)
                if nvtx:
                    nvtx.range_pop()
                sched.update(plan, sampled)
                if pending and pending[-1].targets is None:
                    # now the placeholders have their places in the outputs
                    pending[-1].targets = [(e.request, len(e.request.output) - 1, e.slot) for e in plan.entries if e.samples]
                if sampled and first_token_ms is None:
                    self._resolve(pending)          # the first token, really there
                    first_token_ms = (time.perf_counter() - t0) * 1e3
                if len(pending) > self.max_steps_in_flight:
                    self._resolve(pending, keep=self.max_steps_in_flight)
            self._resolve(pending)
        except BaseException:
            for r in list(sched.running):       # leave the cache as it was found
                if r.slot is not None:
                    eng.manager.release(r.slot)
                    r.slot = None
            raise
        timers.stop("generate")
        times, counts = timers.get_times()
        e2e = times[("generate",)]
        generated = sum(len(r.output) for r in requests)
        reasons = sorted({str(r.finish_reason) for r in requests})
        metrics = {
            "BatchSize": len(requests),
            "PromptLength": max(len(r.prompt) for r in requests),
            "DecodeLength": max_new_tokens,
            "Throughput": generated / (e2e / 1e3) if e2e > 0 else 0.0,
            "TTFT": first_token_ms if first_token_ms is not None else 0.0,
            "TBT": (times.get(("generate", "decode"), 0.0) / counts[("generate", "decode")])
            if counts.get(("generate", "decode")) else 0.0,
            "E2E": e2e,
            "TokenizationTime": tokenization_ms,
            "FinishedReason": "EOS" if reasons == ["eos"] else ("Max Token Length" if reasons == ["length"] else ",".join(reasons)),
            "Preemptions": sum(r.preemptions for r in requests),
            "Steps": counts.get(("generate", "decode"), 0) + counts.get(("generate", "prefill"), 0),
            "DecodeSteps": counts.get(("generate", "decode"), 0),
            "DecodeTime": times.get(("generate", "decode"), 0.0),
            "GeneratedTokens": generated,
        }
        results = [Generation(list(r.output), str(r.finish_reason),
                              (torch.stack(logits_out[r.id]) if logits_out[r.id] else None) if logits_out is not None else None,
                              r.preemptions) for r in requests]
        return results, metrics

    @torch.no_grad()
    def generate(self, prompts: Union[List[str], List[List[int]]], tokens_to_generate: int = 50,
                 report_throughput: bool = False, ignore_eos: Optional[bool] = True,
                 enable_nvtx: Optional[bool] = False, get_logits: Optional[bool] = False):
        """The reference's call (yalis/engine.py:371-379): generate ``tokens_to_generate`` tokens after each prompt.

        Returns ``(tokens, metrics)`` or ``(tokens, metrics, logits)`` with ``get_logits``: ``tokens`` is an
        int64 tensor [batch, generated] on the device; a row that ended early at EOS (``ignore_eos=False``)
        is filled up with EOS, as in the reference (:509-519).  ``logits`` is a list, per request, of float32
        tensors [generated_i, vocab].  ``run`` gives the rows at their true lengths with their reasons.
        """
        if len(prompts) and isinstance(prompts[0], str):
            prompts = self._tokenize(prompts)
        eos = None if ignore_eos else self._eos_id()
        results, metrics = self.run(prompts, tokens_to_generate, None, eos, bool(get_logits), bool(enable_nvtx))
        n_cols = max(len(g.tokens) for g in results)
        out = torch.full((len(results), n_cols), eos if eos is not None else 0, dtype=torch.int64)
        for i, g in enumerate(results):
            out[i, :len(g.tokens)] = torch.tensor(g.tokens, dtype=torch.int64)
        out = out.to(self.device)
        if report_throughput:
            print(f"[Metrics] BatchSize = {metrics['BatchSize']}, PromptLength = {metrics['PromptLength']}, "
                  f"DecodeLength = {tokens_to_generate}, Throughput = {metrics['Throughput']:.2f} tok/s, "
                  f"TTFT = {metrics['TTFT']:.4f} ms, TBT = {metrics['TBT']:.4f} ms, E2E = {metrics['E2E']:.4f} ms, "
                  f"FinishedReason = {metrics['FinishedReason']}")
        if get_logits:
            return out, metrics, [g.logits for g in results]
        return out, metrics

    def _run_plan(self, plan: StepPlan, pending: List[_Pending], logits_out) -> List[int]:
        """One engine step for the plan, with a token chosen for every entry that reached its request's last
        token.  The host does not wait for the step: the chosen tokens stay on the device, where the next step
        finds them, and are copied to the host behind it; the plan's requests get placeholders that
        ``_resolve`` fills in one or two steps later.  That is possible while nothing the host decides depends on
        the token values: a step with a request that stops at an EOS id is read at once.
        Returns one token or placeholder per sampling entry."""
        entries, slots, params, draws = [], [], [], []
        for e in plan.entries:
            r = e.request
            e.slot = r.slot
            toks = r.tokens[e.start:e.start + e.count]
            if e.count == 1 and toks[0] == PENDING:
                toks = None                         # chosen by an earlier step and still on the device
            elif PENDING in toks:
                self._resolve(pending)
                toks = r.tokens[e.start:e.start + e.count]
            entries.append(StepEntry(r.id, toks, [e.count - 1] if e.samples else []))
            slots.append(r.slot)
            if e.samples:
                params.append(r.sampling)
                draws.append(len(r.output))
        if not params:
            self.engine.run_step(slots, entries, graphs=self.use_graphs)
            return []
        out = self.engine.run_step(slots, entries, sampling=params, draws=draws, graphs=self.use_graphs,
                                   keep_logits=logits_out is not None)
        if logits_out is not None:
            samplers = [e.request for e in plan.entries if e.samples]
            for i, r in enumerate(samplers):
                logits_out[r.id].append(out.logits[i].clone())
        report = self.engine.fetch_chosen()
        if any(e.samples and e.request.eos_id is not None for e in plan.entries):
            self._resolve(pending)
            values = report.wait()
            return [int(values[e.slot]) for e in plan.entries if e.samples]
        pending.append(_Pending(report, None))
        return [PENDING] * len(params)

    def _resolve(self, pending: List[_Pending], keep: int = 0) -> None:
        """Read the tokens of all but the newest ``keep`` pending steps into the requests' outputs."""
        while len(pending) > keep:
            pending.pop(0).resolve()

    def reset_kv_cache(self, max_batch_size: Optional[int] = None) -> None:
        """Kept for callers of the reference (yalis/engine.py): the cache needs no reset
        between calls here, every request gives its pages back when it finishes."""


def generate(model: Union[str, LLMEngine], prompts: List[List[int]], max_new_tokens: int = 50,
             temperature: float = 0.0, top_k: Optional[int] = None, top_p: float = 0.0, seed: int = 1234,
             eos_id: Optional[int] = None, return_logits: bool = False,
             sampling: Optional[Sequence[Optional[SamplingParams]]] = None, precision: str = "bf16",
             **inference_options) -> List[Generation]:
    """Token ids in, token ids out: generate after each prompt with a model folder (or an existing
    ``LLMEngine``) and return one ``Generation`` per prompt (``.tokens`` at their true length, ``.finish_reason``,
    ``.logits`` with ``return_logits``).  ``temperature``, ``top_k``, ``top_p`` and ``seed`` hold for every
    prompt (the defaults, temperature 0 and top_p 0, are greedy) unless ``sampling`` gives a
    ``SamplingParams`` per prompt.  A request ends at ``eos_id`` if one is given."""
    if isinstance(model, LLMEngine):
        engine = model
    else:
        longest = max(len(p) for p in prompts) + max_new_tokens
        ic = InferenceConfig(max_batch_size=inference_options.pop("max_batch_size", min(len(prompts), 64)),
                             max_length_of_generated_sequences=inference_options.pop(
                                 "max_length_of_generated_sequences", longest), **inference_options)
        engine = LLMEngine(ModelConfig(model_name=model, model_path=model, precision=precision), ic)
    if sampling is None:
        sampling = [SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=request_seed(seed, i))
                    for i in range(len(prompts))]
    results, _ = engine.run(prompts, max_new_tokens, sampling, eos_id, return_logits)
    return results
