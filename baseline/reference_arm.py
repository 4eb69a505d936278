#!/usr/bin/env python3
"""The reference arm of bench.py: axonn-ai/yalis itself, unmodified, on the benchmark's workload.

    python baseline/reference_arm.py --steps K --warmup W [--batch 8] [--prompt-len 1024]

Runs the reference's own ``LLMEngine.generate`` (yalis/engine.py:371-573) on its own
``GPT`` (yalis/external/model.py) built by its own ``get_model`` with
``random_init=True`` from its own registry entry ``Llama-3-8B``
(yalis/external/config.py:757-773), with its default options (``attention_backend=flash``,
contiguous cache, its ``torch.compile`` decorators as shipped), and prints one JSON line
in bench.py's format with ``"impl": "reference"``.  Nothing of ``yalis_b200`` is imported.

The tree under ``baseline/_ref/yalis`` is a plain copy of the reference's ``yalis``
package.  What is stood in for, and why (also named in the JSON line under ``stood_in``):

* ``axonn`` (not installed; its tensor-parallel runtime): group sizes of 1 and identity
  ``Drop`` / ``Gather``, which is what it does on one GPU.
* ``lightning.fabric.seed_everything`` (not installed): ``torch.manual_seed``.
* ``litgpt`` (not installed): ``litgpt.model`` is the reference's own model file, which is
  where its config looks its norm class up (yalis/external/config.py:239-249);
  ``litgpt.utils.lazy_load`` is never called here.
* ``LLMEngine.__init__`` (yalis/engine.py:173-215) is not called, because it needs a converted
  Hugging Face checkpoint and a tokenizer from the network: its body is restated below with
  ``random_init=True`` and without the tokenizer (prompts are token ids; the reference
  accepts those, :311-336).  Everything after construction, the timed loop included, is the
  reference's code.
* torch's own CUDA libraries are loaded with global symbol visibility before the import,
  because the reference's compiled extension ``vllm_ops`` (built by its setup.py without
  linking them) is imported by its package although the dense path never calls it.
"""

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

STOOD_IN = ["axonn (group size 1, identity Drop/Gather)", "lightning.fabric.seed_everything (torch.manual_seed)",
            "litgpt (alias of the reference's own model file)",
            "LLMEngine.__init__ (restated with random_init=True, no tokenizer, no checkpoint)"]


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
    return 0


def install_stand_ins():
    import torch

    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    for name in ("libc10_cuda.so", "libtorch_cuda.so"):
        ctypes.CDLL(os.path.join(libdir, name), mode=ctypes.RTLD_GLOBAL)

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []
        for k, v in attrs.items():
            setattr(m, k, v)
        sys.modules[name] = m
        return m

    class Identity:
        @staticmethod
        def apply(x, *a, **k):
            return x

    cfg = types.SimpleNamespace(G_intra_r=1, G_intra_c=1, G_intra_d=1)

    def init(G_intra_r=1, G_intra_c=1, G_intra_d=1, **_):
        if (G_intra_r, G_intra_c, G_intra_d) != (1, 1, 1):
            raise RuntimeError("the stand-in for axonn runs on one GPU only")

    ax = module("axonn.axonn", config=cfg, init=init,
                comm_handle=types.SimpleNamespace(inner_intra_layer_parallel_group=None))
    module("axonn", axonn=ax)
    comm = module("axonn.intra_layer.communication", Drop=Identity, Gather=Identity)
    module("axonn.intra_layer", communication=comm)
    module("lightning")
    module("lightning.fabric", seed_everything=lambda seed, **k: torch.manual_seed(seed))
    module("litgpt")
    module("litgpt.utils", lazy_load=None)
    sys.path.insert(0, REF)
    import yalis  # noqa: F401  (the reference's package, from the copy)
    import yalis.external.model as ref_model
    sys.modules["litgpt"].model = ref_model
    sys.modules["litgpt.model"] = ref_model


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self._stop, self._thread = [], threading.Event(), None

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
        for s in self.samples:
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_engine(batch: int, max_length: int, backend: str):
    """What ``LLMEngine.__init__`` does (yalis/engine.py:173-215), with random weights and no tokenizer."""
    import torch
    import yaml
    from yalis.attention.kv_cache import KVSlotsManager
    from yalis.config import InferenceConfig
    from yalis.engine import NUM_BLOCKS, PAGE_BLOCK_SIZE, LLMEngine, precision_to_dtype
    from yalis.external.config import name_to_config
    from yalis.initialize import init_distributed
    from yalis.model import get_model

    inference_config = InferenceConfig(max_batch_size=batch, max_length_of_generated_sequences=max_length,
                                       top_k=None, top_p=0.0, temperature=0.0, attention_backend=backend)
    engine = object.__new__(LLMEngine)
    engine.device = "cuda"
    engine.dtype = precision_to_dtype["bf16"]
    init_distributed(tp_dims=inference_config.tp_dims)
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "model_config.yaml"), "w") as f:
            yaml.safe_dump(dict(name_to_config["Llama-3-8B"]), f)
        model = get_model(d, engine.dtype, max_sequence_length=inference_config.max_length, random_init=True,
                          use_intra_head_parallelism=inference_config.use_intra_head_parallelism,
                          attention_backend=inference_config.attention_backend,
                          use_paged_kv_caching=inference_config.use_paged_kv_caching,
                          prestore_kv_cache=inference_config.prestore_kv_cache, disable_tp=False)
    model = engine._make_params_contiguous(model)
    model.set_kv_cache(max_batch_size=batch, device=engine.device, dtype=engine.dtype)
    engine.model = model
    engine.tokenizer = types.SimpleNamespace(pad_token=0, eos_token_id=None, padding_side="right")
    engine.model_config = types.SimpleNamespace(model_name="Llama-3-8B", precision="bf16")
    engine.inference_config = inference_config
    engine.kv_slots_manager = KVSlotsManager(batch, inference_config.use_paged_kv_caching, 16384 // PAGE_BLOCK_SIZE,
                                             NUM_BLOCKS, PAGE_BLOCK_SIZE)
    torch.cuda.empty_cache()
    return engine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--backend", default="flash", choices=["flash", "sdpa"], help="the reference's default is flash")
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "yalis")):
        return unavailable("baseline/_ref holds no copy of the reference's yalis package")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        install_stand_ins()
    except Exception as e:                                   # the exact import error, as the line's reason
        return unavailable(f"the reference cannot be imported: {type(e).__name__}: {e}")
    try:
        max_length = args.prompt_len + args.steps + args.warmup + 8
        engine = build_engine(args.batch, max_length, args.backend)
    except Exception as e:
        return unavailable(f"the reference's model could not be built ({args.backend} backend): {type(e).__name__}: {e}")

    gen = torch.Generator().manual_seed(1)
    vocab = engine.model.config.padded_vocab_size
    prompts = [torch.randint(0, vocab, (args.prompt_len,), generator=gen).tolist() for _ in range(args.batch)]
    try:
        # warm-up: compiles both step functions and records the decode graph; W decode steps each
        for _ in range(2):
            engine.generate(prompts, tokens_to_generate=max(3, args.warmup) + 1)
        torch.cuda.synchronize()
        with ClockSampler() as cs:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            tokens, metrics = engine.generate(prompts, tokens_to_generate=args.steps + 1)
            host_tokens = tokens.cpu()
            end.record()
            torch.cuda.synchronize()
        clocks = cs.summary()
    except Exception as e:
        return unavailable(f"the reference's generate failed ({args.backend} backend): {type(e).__name__}: {e}")
    tbt = float(metrics["TBT"])                              # its own CUDA-event time per decode step
    decode_tok_s = args.batch / (tbt / 1e3) if tbt else None
    # end to end: the decode phase of the call as a whole (everything after its prefill step, host work included)
    decode_phase_ms = float(metrics["E2E"]) - float(metrics["TTFT"])
    e2e_tok_s = args.batch * args.steps / (decode_phase_ms / 1e3) if decode_phase_ms > 0 else None
    cfg = engine.model.config
    line = {
        "metric": f"decode tok/s (Llama-3-8B shape, batch {args.batch}, {args.prompt_len}-token prompts)",
        "value": round(decode_tok_s, 2) if decode_tok_s else None, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(tbt, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights (the reference's default init)",
        "impl": "reference",
        "config": {"model": "Llama-3-8B", "layers": cfg.n_layer, "hidden": cfg.n_embd, "heads": cfg.n_head,
                   "kv_heads": cfg.n_query_groups, "head_dim": cfg.head_size, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.padded_vocab_size, "global_batch": args.batch, "seq_len": args.prompt_len,
                   "attention_backend": args.backend, "paged": False, "torch_compile": "as shipped (decode: reduce-overhead)",
                   "parallelism": "none", "l2": "inputs larger than L2 (15 GB of weights per step)"},
        "e2e": {"value": round(e2e_tok_s, 2) if e2e_tok_s else None, "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "LLMEngine.generate with host token ids in and host tokens out; the reference keeps the "
                        "tokens on the device between steps and copies all of them back once at the end",
                "whole_call_tok_s": round(float(metrics["Throughput"]), 2), "ttft_ms": round(float(metrics["TTFT"]), 3),
                "whole_call_ms": round(start.elapsed_time(end), 3), "tokens_read_back": int(host_tokens.numel())},
        "clocks": clocks, "stood_in": STOOD_IN,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    code = main()
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    sys.exit(code)
