#!/usr/bin/env python3
"""Serving benchmark of the engine on one B200: decode tokens per second of the
Llama-3-8B shape (random weights, bfloat16, page size 16), batch 8, 1,024-token prompts.

    python bench.py [--gpus 1] [--steps K] [--warmup W]        # prints ONE JSON line
    python bench.py --impl reference                            # the reference arm (baseline/reference_arm.py)
    python bench.py --workload mixed-1b | serve-3b              # the other workloads, one JSON line each

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens per second
with the K steps timed on the device (CUDA events) and the chosen tokens fed back on
the device; ``e2e`` is the same metric through ``LLMEngine.generate`` (host token ids in
and out; every step copies its inputs from pinned host memory and its chosen tokens back):
all prompts are admitted in one step, and the decode steps of the full batch are timed
from the start of the first to the end of the last, host work between them included.
The line also carries a 2,048-token prefill (``prefill``), the decode step's HBM roofline
(``roofline``), decode at batch 1 and 64 (``points``), the SM clocks sampled during the
timed region (``clocks``) and the number of this library's kernels launched in it
(``gpu_launches``).  Between timed iterations nothing is flushed: a decode step streams
all weights (15 GB), far more than the 126 MB L2.  The device-timed steps start one
second after the prompt phase, which draws the power limit and leaves the SM clock low for
a tenth of a second (``config.settle``); ``right_after_prompts`` is the same measurement
without the pause, and ``e2e`` has none either.

``--workload mixed-1b``: Llama-3.2-1B shape, 64 requests decoding beside a 4,096-token
prompt fed in portions of 512 (steps of 576 tokens); ``value`` is tokens per second over
those mixed steps.  ``--workload serve-3b``: Llama-3.2-3B shape, 32 requests with prompts
of 128 to 16,384 tokens, 256 new tokens each at temperature 0.8; ``value`` is generated
tokens per second of the whole call.  For these, ``--warmup`` and ``--steps`` count whole
calls (defaults 2 and 3; the median call is reported).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PRESET = "Llama-3-8B"
PROMPT_LEN = 1024
PREFILL_TOKENS = 2048
PAGE_SIZE = 16          # as the benchmark configuration states it (the engine's own default, 64, is a few percent faster)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            peaks = dict(FALLBACK_PEAKS)
            for k in peaks:
                if isinstance(raw.get(k), (int, float)):
                    peaks[k] = float(raw[k])
            return peaks, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    self.samples.append([c.strip() for c in out[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """Runs the unmodified reference (a copy of its package under baseline/_ref) through its own
    ``LLMEngine.generate`` in a process of its own and passes its JSON line on."""
    script = os.path.join(ROOT, "baseline", "reference_arm.py")
    cmd = [sys.executable, script, "--steps", str(args.steps), "--warmup", str(max(3, args.warmup)), "--batch", str(args.batch),
           "--prompt-len", str(PROMPT_LEN)]
    last_reason = None
    for backend in ("flash", "sdpa"):           # the reference's default first; its other single-GPU backend if that one cannot run here
        try:
            proc = subprocess.run(cmd + ["--backend", backend], capture_output=True, text=True, timeout=1500)
        except subprocess.TimeoutExpired:
            last_reason = f"the reference arm ({backend} backend) did not finish within 1500 s"
            continue
        line = None
        for out_line in reversed(proc.stdout.strip().splitlines()):
            try:
                parsed = json.loads(out_line)
            except ValueError:
                continue
            if isinstance(parsed, dict) and parsed.get("impl") == "reference":
                line = parsed
                break
        if line is not None and "unavailable" not in line:
            print(json.dumps(line))
            return 0
        last_reason = (line or {}).get("unavailable") or \
            f"the reference arm ({backend} backend) ended with code {proc.returncode}: " + \
            " ".join((proc.stderr.strip().splitlines() or ["no output"])[-1].split())[:300]
    print(json.dumps({"impl": "reference", "unavailable": last_reason}))
    return 0


def decode_span(step_log, batch):
    """(steps, milliseconds) of the decode steps of the full batch in a step log: from the start of the first
    to the end of the last, so that whatever the host does between them counts."""
    full = [s for s in step_log if s["decoding"] == batch and s["tokens"] == batch]
    if len(full) < 2:
        return len(full), 0.0, full
    return len(full), full[0]["start"].elapsed_time(full[-1]["end"]), full


def run_workload(args) -> int:
    import random
    import torch
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig, SamplingParams
    from yalis_b200.config.presets import preset
    from yalis_b200.ops import _lib
    from yalis_b200.sampling.sampler import GREEDY

    # two warm-up calls: the first meets the shapes of the steps, the second records those that came again
    calls, warm = (args.steps or 3), (2 if args.warmup is None else args.warmup)
    if args.workload == "mixed-1b":
        name, decoders, short, long_prompt, chunk, new = "Llama-3.2-1B", 64, 256, 4096, 512, 128
        cfg = preset(name)
        llm = LLMEngine(ModelConfig(model_name=name, random_weights=True, seed=0, precision="bf16"),
                        InferenceConfig(max_batch_size=decoders + 1, max_length_of_generated_sequences=long_prompt + new + 64,
                                        cache_tokens=decoders * (short + new + 64) + long_prompt + new + 64,
                                        max_tokens_per_step=decoders + chunk, prefill_chunk=chunk, page_size=args.page_size))
        gen = torch.Generator().manual_seed(0)
        vocab = llm.engine.vocab_size
        prompts = [torch.randint(0, vocab, (short,), generator=gen).tolist() for _ in range(decoders)]
        prompts.append(torch.randint(0, vocab, (long_prompt,), generator=gen).tolist())
        sampling = [GREEDY] * len(prompts)
        metric = (f"tokens/s over steps of {decoders} decoding requests beside a {chunk}-token portion of a "
                  f"{long_prompt}-token prompt (Llama-3.2-1B shape)")
        picked = lambda s: s["decoding"] == decoders and s["tokens"] == decoders + chunk
        sizes = {"decoding_requests": decoders, "decoder_prompt": short, "long_prompt": long_prompt, "prefill_chunk": chunk,
                 "max_tokens_per_step": decoders + chunk, "new_tokens": new}
    else:
        name, n_req, lo, hi, new = "Llama-3.2-3B", 32, 128, 16384, 256
        cfg = preset(name)
        rng = random.Random(1)
        lens = [rng.randint(lo, hi) for _ in range(n_req)]
        llm = LLMEngine(ModelConfig(model_name=name, random_weights=True, seed=0, precision="bf16"),
                        InferenceConfig(max_batch_size=n_req, max_length_of_generated_sequences=hi + new + 64,
                                        cache_tokens=sum(lens) + n_req * (new + 2 * args.page_size),
                                        max_tokens_per_step=2048, page_size=args.page_size))
        gen = torch.Generator().manual_seed(0)
        vocab = llm.engine.vocab_size
        prompts = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lens]
        sampling = [SamplingParams(temperature=0.8, top_p=1.0, seed=100 + i) for i in range(n_req)]
        metric = (f"generated tokens/s, {n_req} requests with prompts of {lo} to {hi} tokens, {new} new tokens each at "
                  f"temperature 0.8 (Llama-3.2-3B shape)")
        picked = None
        sizes = {"requests": n_req, "prompt_tokens_total": sum(lens), "prompt_min": min(lens), "prompt_max": max(lens),
                 "new_tokens": new, "max_tokens_per_step": 2048, "temperature": 0.8}
    for _ in range(warm):
        llm.run(prompts, new, sampling)
    records = []
    with ClockSampler() as cs:
        for _ in range(calls):
            log = []
            l0 = _lib.LAUNCHES[0]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            results, metrics = llm.run(prompts, new, sampling, step_log=log)
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            replayed = sum(s["captured"] for s in log)
            rec = {"wall_s": wall, "generated": sum(len(g.tokens) for g in results), "steps": len(log),
                   "preemptions": metrics["Preemptions"], "decode_ms": metrics["TBT"],
                   "launched": _lib.LAUNCHES[0] - l0 + sum(s["replayed_launches"] for s in log),
                   "replayed_steps": int(replayed), "ttft_ms": metrics["TTFT"]}
            if picked is not None:
                chosen = [s for s in log if picked(s)]
                rec["picked_steps"] = len(chosen)
                rec["picked_ms"] = sum(s["start"].elapsed_time(s["end"]) for s in chosen)
                rec["picked_tokens"] = sum(s["tokens"] for s in chosen)
                rec["picked_span_ms"] = chosen[0]["start"].elapsed_time(chosen[-1]["end"]) if chosen else 0.0
            prefill_steps = [s for s in log if s["decoding"] != s["requests"]]
            rec["prefill_tokens"] = sum(s["tokens"] for s in prefill_steps)
            rec["prefill_ms"] = sum(s["start"].elapsed_time(s["end"]) for s in prefill_steps)
            records.append(rec)
    llm.engine.check_device_errors()
    clocks = cs.summary()
    if picked is not None:
        records.sort(key=lambda r: r["picked_span_ms"])
        mid = records[len(records) // 2]
        value = mid["picked_tokens"] / (mid["picked_span_ms"] / 1e3) if mid["picked_span_ms"] else None
        ms_per_step = mid["picked_span_ms"] / max(1, mid["picked_steps"])
        steps = mid["picked_steps"]
    else:
        records.sort(key=lambda r: r["wall_s"])
        mid = records[len(records) // 2]
        value = mid["generated"] / mid["wall_s"]
        ms_per_step = mid["decode_ms"]
        steps = mid["steps"]
    peaks, peak_source = load_peaks()
    line = {
        "metric": metric, "value": round(value, 1) if value else None, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "calls_timed": calls, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random weights N(0, 0.02)", "impl": "ours", "workload": args.workload,
        "config": dict({"model": name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                        "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                        "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": args.page_size,
                        "parallelism": "none", "peaks": peak_source,
                        "l2": "inputs larger than L2 (2.5 GB and 6.4 GB of weights per step)"}, **sizes),
        "call": {"wall_s": round(mid["wall_s"], 4), "generated_tokens": mid["generated"], "steps": mid["steps"],
                 "whole_call_tok_s": round(mid["generated"] / mid["wall_s"], 1), "decode_step_ms": round(mid["decode_ms"], 4),
                 "prefill_tok_s": round(mid["prefill_tokens"] / (mid["prefill_ms"] / 1e3), 1) if mid["prefill_ms"] else None,
                 "ttft_ms": round(mid["ttft_ms"], 3), "preemptions": mid["preemptions"],
                 "steps_replayed_from_recordings": mid["replayed_steps"]},
        "clocks": clocks, "gpu_launches": int(mid["launched"]),
    }
    if picked is not None:
        line["call"]["mixed_step_device_ms"] = round(mid["picked_ms"] / max(1, mid["picked_steps"]), 4)
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode-8b", choices=["decode-8b", "mixed-1b", "serve-3b"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--page-size", type=int, default=None, help="tokens per cache page (default: 16 as the benchmark "
                    "configuration states for decode-8b, the engine's 64 for the other workloads)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 / 64, prefill and e2e (for profiling)")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: this engine runs on one GPU; --gpus N > 1 is not supported")
        return 2
    if args.workload != "decode-8b":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no scheduler: it cannot run prompt "
                              "portions beside decoding requests, nor requests of unequal lengths without padding"}))
            return 0
        args.page_size = args.page_size or 64
        return run_workload(args)
    args.steps = 256 if args.steps is None else args.steps
    args.warmup = 16 if args.warmup is None else args.warmup
    page_size = args.page_size or PAGE_SIZE
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    from yalis_b200.bench_support import DecodeBench, model_numbers, prefill_bench
    from yalis_b200.config.presets import PRESETS, preset
    from yalis_b200.ops import _lib

    peaks, peak_source = load_peaks()
    cfg = preset(PRESET)
    full_layers = cfg["num_hidden_layers"]
    name = PRESET
    if args.layers is not None and args.layers != full_layers:
        cfg["num_hidden_layers"] = args.layers
        name = f"{PRESET}-L{args.layers}"
        PRESETS[name] = cfg
    batches = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    max_len = PROMPT_LEN + args.steps + args.warmup + 64
    cache_tokens = max(max(batches) * (max_len + page_size), PREFILL_TOKENS + 64)
    llm = LLMEngine(ModelConfig(model_name=name, random_weights=True, seed=0, precision="bf16"),
                    InferenceConfig(max_batch_size=max(batches), max_length_of_generated_sequences=max(max_len, PREFILL_TOKENS + 64),
                                    temperature=0.0, top_p=0.0, page_size=page_size, cache_tokens=cache_tokens,
                                    max_tokens_per_step=max(PREFILL_TOKENS, args.batch * PROMPT_LEN)))
    engine = llm.engine
    numbers = model_numbers(engine)

    results = {}
    launches = 0
    clocks = None
    for b in batches:
        bench = DecodeBench(engine, b, PROMPT_LEN, seed=b)
        bench.prepare()
        bench.run(args.warmup)
        if b == args.batch:
            with ClockSampler() as cs:
                ms = bench.run_timed(args.steps)
            launches = bench.launches_per_step * args.steps
            clocks = cs.summary()
        else:
            ms = bench.run_timed(args.steps)
        results[b] = {"ms_per_step": ms / args.steps, "tok_s": b * args.steps / (ms / 1e3), "kv_tokens": bench.mean_context(args.steps)}
        bench.finish()
        if b == args.batch and not args.skip_points:
            # the same steps right after the prompt phase, without the pause: what the low clock after it costs
            bench = DecodeBench(engine, b, PROMPT_LEN, seed=b + 1000, settle_seconds=0.0)
            bench.prepare()
            bench.run(args.warmup)
            with ClockSampler() as cs:
                ms = bench.run_timed(args.steps)
            unsettled = {"value": round(b * args.steps / (ms / 1e3), 2), "ms_per_step": round(ms / args.steps, 4),
                         "sm_mhz": cs.summary().get("sm_mhz")}
            bench.finish()

    main_r = results[args.batch]
    step_bytes = numbers["weight_bytes_per_step"] + args.batch * main_r["kv_tokens"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main_r["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s (Llama-3-8B shape, batch {args.batch}, {PROMPT_LEN}-token prompts)",
        "value": round(main_r["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": PRESET, "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
            "seq_len": PROMPT_LEN, "context": cfg["max_position_embeddings"], "page_size": page_size, "parallelism": "none",
            "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": peak_source,
            "settle": "1 s idle between the prompt phase and the warm-up steps (the clock recovers from the power cap)",
        },
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if not args.skip_points:
        line["right_after_prompts"] = unsettled
        line["points"] = {f"decode_b{b}": round(r["tok_s"], 2) for b, r in results.items() if b != args.batch}
        pf = prefill_bench(engine, PREFILL_TOKENS, warmup=3, iters=7)
        flops = numbers["flops_prefill"](PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pf / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
                           "frac": round(flops / (pf / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        # end to end through the public entry point: host token ids in, host token ids out
        gen = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, engine.vocab_size, (PROMPT_LEN,), generator=gen).tolist() for _ in range(args.batch)]
        for _ in range(2):          # the second call records the steps whose shapes the first one met
            llm.generate(prompts, tokens_to_generate=args.warmup)
        log = []
        results_e2e, metrics = llm.run(prompts, args.steps + 1, step_log=log)
        tokens_out = [g.tokens for g in results_e2e]
        n_steps, span_ms, full = decode_span(log, args.batch)
        line["e2e"] = {"value": round(args.batch * n_steps / (span_ms / 1e3), 2) if span_ms else None, "unit": "tokens/s",
                       "steps": n_steps, "h2d_bytes_per_step": full[-1]["h2d_bytes"] if full else None,
                       "d2h_bytes_per_step": 4 * (engine.max_slots + 2), "tokens_returned": sum(len(t) for t in tokens_out),
                       "whole_call_tok_s": round(metrics["Throughput"], 2), "ttft_ms": round(metrics["TTFT"], 3)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
