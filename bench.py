#!/usr/bin/env python3
"""Serving benchmark of the engine on one B200: decode tokens per second of the
Llama-3-8B shape (random weights, bfloat16, page size 16), batch 8, 1,024-token prompts.

    python bench.py [--gpus 1] [--steps K] [--warmup W]        # prints ONE JSON line
    python bench.py --impl reference                            # the reference arm

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens per second
with the K steps timed on the device (CUDA events) and the sampled tokens fed back on
the device; ``e2e`` is the same metric through ``LLMEngine.generate`` (host token ids in
and out, a host->device copy of the step's inputs and a device->host read of its tokens
every step).  The line also carries a 2,048-token prefill (``prefill``), the decode
step's HBM roofline (``roofline``), decode at batch 1 and 64 (``points``), the SM clocks
sampled during the timed region (``clocks``) and the number of this library's kernels
launched in it (``gpu_launches``).  Between timed iterations nothing is flushed: a decode
step streams all weights (15 GB), far more than the 126 MB L2.
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
    """Runs the unmodified reference from baseline/_ref, if it can be imported there."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "yalis")):
        why = "baseline/_ref holds no installed reference (pip install of axonn-ai/yalis was not possible offline)"
    else:
        proc = subprocess.run([sys.executable, "-c", "import yalis"], capture_output=True, text=True,
                              env=dict(os.environ, PYTHONPATH=ref))
        if proc.returncode != 0:
            last = (proc.stderr.strip().splitlines() or ["import failed"])[-1]
            why = ("the installed reference cannot be imported: " + last +
                   " (its setup.py leaves out sub-packages, and axonn / litgpt / lightning are not installed; "
                   "it also needs a Hugging Face checkpoint and tokenizer from the network)")
    if why is None:
        why = "the reference needs a converted Hugging Face checkpoint and tokenizer, which cannot be fetched offline"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 / 64, prefill and e2e (for profiling)")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: this engine runs on one GPU; --gpus N > 1 is not supported")
        return 2
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
    cache_tokens = max(max(batches) * (max_len + PAGE_SIZE), PREFILL_TOKENS + 64)
    llm = LLMEngine(ModelConfig(model_name=name, random_weights=True, seed=0, precision="bf16"),
                    InferenceConfig(max_batch_size=max(batches), max_length_of_generated_sequences=max(max_len, PREFILL_TOKENS + 64),
                                    temperature=0.0, top_p=0.0, page_size=PAGE_SIZE, cache_tokens=cache_tokens,
                                    max_tokens_per_step=PREFILL_TOKENS))
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
            l0 = _lib.LAUNCHES[0]
            with ClockSampler() as cs:
                ms = bench.run_timed(args.steps)
            launches = bench.launches_per_step * args.steps if bench.launches_per_step else _lib.LAUNCHES[0] - l0
            clocks = cs.summary()
        else:
            ms = bench.run_timed(args.steps)
        results[b] = {"ms_per_step": ms / args.steps, "tok_s": b * args.steps / (ms / 1e3), "kv_tokens": bench.mean_context(args.steps)}
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
            "seq_len": PROMPT_LEN, "context": cfg["max_position_embeddings"], "page_size": PAGE_SIZE, "parallelism": "none",
            "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": peak_source,
        },
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if not args.skip_points:
        line["points"] = {f"decode_b{b}": round(r["tok_s"], 2) for b, r in results.items() if b != args.batch}
        pf = prefill_bench(engine, PREFILL_TOKENS, warmup=3, iters=7)
        flops = numbers["flops_prefill"](PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pf / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
                           "frac": round(flops / (pf / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        # end to end through the public entry point: host token ids in, host token ids out
        gen = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, engine.vocab_size, (PROMPT_LEN,), generator=gen).tolist() for _ in range(args.batch)]
        llm.generate(prompts, tokens_to_generate=args.warmup)
        tokens, metrics = llm.generate(prompts, tokens_to_generate=args.steps + 1)
        tokens = tokens.cpu()
        tbt = metrics["TBT"]
        line["e2e"] = {"value": round(args.batch / (tbt / 1e3), 2) if tbt else None, "unit": "tokens/s",
                       "h2d_bytes_per_step": llm.engine.last_h2d_bytes, "d2h_bytes_per_step": 4 * args.batch,
                       "whole_call_tok_s": round(metrics["Throughput"], 2), "ttft_ms": round(metrics["TTFT"], 3)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
