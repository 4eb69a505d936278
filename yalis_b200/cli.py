"""Command line in the manner of the reference's ``examples/infer.py``: build an
engine from a ``ModelConfig`` and an ``InferenceConfig``, generate for a batch of
prompts a number of times, report throughput, print the outputs.  The reference
script has its values as constants (examples/infer.py:15-88: model id, 16 prompts,
tokens_to_gen=512, MAX_BATCH_SIZE=32, precision "bf16", top_p=0.80,
temperature=1.0, 10 iterations); here they are options with those names.

Examples
    python -m yalis_b200.cli --model DIR --prompt-ids 1,2,3 --prompt-ids 4,5 --tokens-to-gen 16
    python -m yalis_b200.cli --preset tiny-A --random-weights --random-prompts 4 --prompt-len 33 \\
        --temperature 0 --top-p 0
    python -m yalis_b200.cli --preset tiny-B --write-random-model /tmp/tinyB --seed 1

Greedy decoding is ``--temperature 0 --top-p 0`` (the reference's rule,
yalis/external/sampling.py:64).
"""

from __future__ import annotations

import argparse
import sys
from typing import List

import torch


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(" ", "").split(",") if t]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="yalis_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    m = ap.add_argument_group("model (ModelConfig)")
    m.add_argument("--model", "--model-path", dest="model_path", help="folder with config.json and model.safetensors")
    m.add_argument("--preset", "--model-name", dest="model_name", help="a preset name, e.g. Llama-3-8B, tiny-A")
    m.add_argument("--random-weights", action="store_true", help="seeded random weights for --preset, made on the GPU")
    m.add_argument("--write-random-model", metavar="DIR", help="write config.json + model.safetensors for --preset and exit")
    m.add_argument("--precision", "--dtype", dest="precision", default="bf16", choices=["bf16", "fp32"])
    m.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    g = ap.add_argument_group("generation (InferenceConfig)")
    g.add_argument("--max-batch-size", type=int, default=32)
    g.add_argument("--max-length", type=int, default=1024, help="max_length_of_generated_sequences: most tokens per request")
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=0.80)
    g.add_argument("--sampling-seed", type=int, default=1234)
    g.add_argument("--tokens-to-gen", "--max-new-tokens", dest="tokens_to_gen", type=int, default=512)
    g.add_argument("--no-ignore-eos", action="store_true", help="stop a request at its EOS token")
    e = ap.add_argument_group("engine")
    e.add_argument("--page-size", type=int, default=64)
    e.add_argument("--cache-tokens", type=int, default=None, help="size of the page pool in tokens")
    e.add_argument("--num-pages", type=int, default=None, help="size of the page pool in pages")
    e.add_argument("--memory-fraction", type=float, default=None,
                   help="size of the page pool as a share of the device memory free after loading")
    e.add_argument("--no-graphs", action="store_true", help="launch every step kernel by kernel")
    e.add_argument("--max-tokens-per-step", type=int, default=2048)
    e.add_argument("--chunk", "--prefill-chunk", dest="prefill_chunk", type=int, default=None)
    p = ap.add_argument_group("prompts")
    p.add_argument("--prompt-ids", action="append", default=[], metavar="I,J,K", help="one prompt as token ids (repeatable)")
    p.add_argument("--prompt", action="append", default=[], help="one prompt as text (needs a tokenizer in the model folder)")
    p.add_argument("--random-prompts", type=int, default=0, help="this many prompts of uniform random ids")
    p.add_argument("--prompt-len", type=int, default=128)
    r = ap.add_argument_group("run")
    r.add_argument("--iterations", type=int, default=1, help="generate this many times (the reference script does 10)")
    r.add_argument("--report-throughput", action="store_true")
    r.add_argument("--nvtx", action="store_true", help="NVTX ranges Prefill / Decode around the steps")
    r.add_argument("--quiet", action="store_true", help="do not print the generated ids")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from yalis_b200.config.presets import preset

    if args.write_random_model:
        if not args.model_name:
            raise SystemExit("--write-random-model needs --preset")
        from yalis_b200.weights.loader import write_random_model
        print(write_random_model(preset(args.model_name), args.write_random_model, seed=args.seed))
        return 0
    if not args.model_path and not (args.model_name and args.random_weights):
        raise SystemExit("give --model DIR, or --preset NAME --random-weights")

    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig

    model_config = ModelConfig(model_name=args.model_name or args.model_path, model_path=args.model_path,
                               precision=args.precision, random_weights=bool(args.random_weights and not args.model_path),
                               seed=args.seed)
    inference_config = InferenceConfig(
        max_batch_size=args.max_batch_size, max_length_of_generated_sequences=args.max_length, top_k=args.top_k,
        top_p=args.top_p, temperature=args.temperature, page_size=args.page_size, cache_tokens=args.cache_tokens,
        num_pages=args.num_pages, memory_fraction=args.memory_fraction, use_graphs=not args.no_graphs,
        max_tokens_per_step=args.max_tokens_per_step, prefill_chunk=args.prefill_chunk, seed=args.sampling_seed)
    engine = LLMEngine(model_config=model_config, inference_config=inference_config)

    prompts = [_ids(p) for p in args.prompt_ids]
    if args.random_prompts:
        gen = torch.Generator().manual_seed(args.seed)
        vocab = engine.engine.vocab_size
        prompts += [torch.randint(0, vocab, (args.prompt_len,), generator=gen).tolist() for _ in range(args.random_prompts)]
    text_prompts = list(args.prompt)
    if text_prompts and prompts:
        raise SystemExit("give prompts either as text or as ids, not both")
    batch = text_prompts or prompts
    if not batch:
        raise SystemExit("no prompts: use --prompt-ids, --prompt or --random-prompts")
    print(f"Number of prompts = {len(batch)}")
    for _ in range(args.iterations):
        tokens, metrics = engine.generate(batch, tokens_to_generate=args.tokens_to_gen,
                                          report_throughput=args.report_throughput or args.iterations > 1,
                                          ignore_eos=not args.no_ignore_eos, enable_nvtx=args.nvtx)
    rows = tokens.cpu().tolist()
    if not args.quiet:
        for i, row in enumerate(rows):
            print("==========================")
            if text_prompts and engine.tokenizer is not None:
                print(f"prompt = {text_prompts[i]}")
                print(f"output = {engine.tokenizer.decode(row, skip_special_tokens=True)}")
            else:
                print(f"prompt = {batch[i][:16]}{' ...' if len(batch[i]) > 16 else ''}")
                print(f"output = {row}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
