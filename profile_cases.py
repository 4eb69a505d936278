"""Small, self-contained workloads of single kernels, for timing and for profiler captures.

    python profile_cases.py attention_decode --batch 64 --ctx 1040 --launches 8
    python profile_cases.py gemm_wstream --tokens 8 --n 28672 --k 4096 --launches 8

Each case allocates inputs larger than the L2 cache but at most a few GB, launches the
kernel a few times, and prints the mean time per launch measured with CUDA events.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _time(fn, launches: int, graph: bool = True) -> float:
    """Microseconds per launch.  With ``graph`` the launches are captured into one CUDA graph
    and replayed, so that host launch cost does not hide the kernels' own time."""
    fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not graph:
        start.record()
        for _ in range(launches):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / launches * 1e3
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(launches):
            fn()
    g.replay()
    torch.cuda.synchronize()
    reps = 5
    start.record()
    for _ in range(reps):
        g.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (reps * launches) * 1e3


def attention_decode(args) -> None:
    from types import SimpleNamespace
    from yalis_b200.ops.attention import (decode_attention_lean, decode_attention_tma, decode_splits, decode_tma_splits,
                                          paged_attention_mma)
    dev = "cuda:0"
    nh, g, hs, page, b, ctx = args.heads, args.kv_heads, args.head_dim, args.page_size, args.batch, args.ctx
    pages_per = -(-ctx // page)
    num_pages = b * pages_per
    layers = max(2, min(8, int(400e6 // max(1, num_pages * g * page * hs * 4)) + 1))    # rotate pools: > L2 in total
    pools = [(torch.randn(num_pages, g, page, hs, device=dev).to(torch.bfloat16),
              torch.randn(num_pages, g, page, hs, device=dev).to(torch.bfloat16)) for _ in range(layers)]
    table = torch.randperm(num_pages, device=dev).to(torch.int32).view(b, pages_per).contiguous()
    q = torch.randn(b, nh * hs, device=dev).to(torch.bfloat16)
    pos = torch.full((b,), ctx - 1, dtype=torch.int32, device=dev)
    q_start = torch.arange(b + 1, dtype=torch.int32, device=dev)
    req = torch.arange(b, dtype=torch.int32, device=dev)
    splits = args.splits or (decode_tma_splits(b, g, False) if args.kernel == "tma" else decode_splits(b, g))   # as the engine chooses
    state = {"i": 0}

    def fn():
        k, v = pools[state["i"] % layers]
        state["i"] += 1
        if args.kernel == "tma":
            decode_attention_tma(q, k, v, pos, q_start, table, nh, g, hs, n_splits=splits)
        elif args.kernel == "lean":
            decode_attention_lean(q, k, v, pos, q_start, table, nh, g, hs, n_blocks=args.blocks or None)
        else:
            paged_attention_mma(q, k, v, pos, q_start, req, table, 1, nh, g, hs, n_splits=splits)

    us = _time(fn, args.launches, graph=not args.eager)
    kv_bytes = b * ctx * 2 * g * hs * 2
    print(f"attention_decode ({args.kernel}) batch {b} ctx {ctx} splits {splits}: {us:.1f} us per launch, "
          f"{kv_bytes / us / 1e6:.2f} TB/s of K/V")


def attention_prefill(args) -> None:
    """The prompt attention of one step, one layer's worth of heads: requests that bring ``--tokens`` tokens each
    (a list: portions of prompts, 1 for a decoding request) behind ``--before`` cached ones (causal).
    ``--splits 0`` lets the engine's policy choose the key splits."""
    from types import SimpleNamespace
    from yalis_b200.ops.attention import paged_attention_mma, prefill_attention_tcgen05, prefill_kv_splits
    dev = "cuda:0"
    nh, g, hs, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    q_lens = [int(x) for x in str(args.tokens).split(",")]
    before = [int(x) for x in str(args.before).split(",")]
    assert len(q_lens) == len(before), "--tokens and --before list one number per request"
    pages_per = [-(-(b + q) // page) for q, b in zip(q_lens, before)]
    pages = sum(pages_per)
    k_pool = torch.randn(pages, g, page, hs, device=dev).to(torch.bfloat16)
    v_pool = torch.randn(pages, g, page, hs, device=dev).to(torch.bfloat16)
    table = torch.zeros(len(q_lens), max(pages_per), dtype=torch.int32)
    perm, at = torch.randperm(pages).to(torch.int32), 0
    for r, n_pages in enumerate(pages_per):
        table[r, :n_pages] = perm[at:at + n_pages]
        at += n_pages
    table = table.to(dev)
    n = sum(q_lens)
    q = torch.randn(n, nh * hs, device=dev).to(torch.bfloat16)
    pos = torch.cat([torch.arange(b, b + ql, dtype=torch.int32) for ql, b in zip(q_lens, before)]).to(dev)
    starts = [0]
    for ql in q_lens:
        starts.append(starts[-1] + ql)
    q_start = torch.tensor(starts, dtype=torch.int32, device=dev)
    req = torch.cat([torch.full((ql,), r, dtype=torch.int32) for r, ql in enumerate(q_lens)]).to(dev)
    splits, limit = args.splits, args.tiles_per_split
    if splits == 0:
        splits, limit = prefill_kv_splits(SimpleNamespace(q_start=starts, ctx_before=before), nh // g, g, hs)

    if args.kernel == "library":
        # The bar: the library attention that the reference's flash backend calls (yalis/attention/backend_impl/
        # flash.py:52-65), on one request's keys laid out contiguously (its paged form wants pages of 256).
        assert len(q_lens) == 1 and before == [0], "--kernel library times one whole prompt"
        from flash_attn import flash_attn_func
        q4 = q.view(1, n, nh, hs)
        k4 = torch.randn(1, n, g, hs, device=dev).to(torch.bfloat16)
        v4 = torch.randn(1, n, g, hs, device=dev).to(torch.bfloat16)

    def fn():
        if args.kernel == "tcgen05":
            prefill_attention_tcgen05(q, k_pool, v_pool, pos, q_start, table, max(q_lens), nh, g, hs, kv_splits=splits,
                                      tiles_per_split=limit)
        elif args.kernel == "library":
            flash_attn_func(q4, k4, v4, causal=True)
        else:
            paged_attention_mma(q, k_pool, v_pool, pos, q_start, req, table, max(q_lens), nh, g, hs)

    us = _time(fn, args.launches, graph=not args.eager)
    flops = 4.0 * nh * hs * sum(ql * b + ql * (ql + 1) / 2 for ql, b in zip(q_lens, before))
    print(f"attention_prefill ({args.kernel}) tokens {q_lens} after {before} heads {nh}/{g} head_dim {hs} key splits "
          f"{splits} of at least {limit} tiles: {us:.1f} us per launch, {flops / us / 1e6:.1f} TFLOP/s (causal flops)")


def gemm_wstream(args) -> None:
    from yalis_b200.ops.linear import gemm_wstream as gemm, wstream_splits
    dev = "cuda:0"
    m, n, k = args.tokens, args.n, args.k
    copies = max(2, min(8, int(400e6 // (n * k * 2)) + 1))
    ws = [(torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    state = {"i": 0}

    def fn():
        w = ws[state["i"] % copies]
        state["i"] += 1
        if args.library:
            torch.matmul(x, w.t())
        else:
            gemm(x, w, split=args.split)

    us = _time(fn, args.launches, graph=not args.eager)
    print(f"{'library product' if args.library else 'gemm_wstream'} tokens {m} n {n} k {k} splits "
          f"{wstream_splits(n, k) if args.split and not args.library else 1}: "
          f"{us:.1f} us per launch, {n * k * 2 / us / 1e6:.2f} TB/s of weights")


def elementwise(args) -> None:
    """The memory-bound kernels between the products at prefill size: residual add + RMSNorm, SiLU-mul and
    rotary + cache write for ``--tokens`` tokens of the Llama-3-8B shape."""
    from yalis_b200.ops.elementwise import add_rmsnorm, rope_kv_write, silu_mul
    from yalis_b200.parts.rotary import inverse_frequencies
    dev = "cuda:0"
    n, hidden, inter, nh, g, hs, page = args.tokens, 4096, 14336, 32, 8, 128, 64
    bf = torch.bfloat16
    copies = 4                                                  # rotate buffers: more than the L2 holds
    xs = [torch.randn(n, hidden, device=dev) for _ in range(copies)]
    deltas = [torch.randn(n, hidden, device=dev).to(bf) for _ in range(copies)]
    w = torch.ones(hidden, device=dev)
    gus = [torch.randn(n, 2 * inter, device=dev).to(bf) for _ in range(copies)]
    qkvs = [torch.randn(n, (nh + 2 * g) * hs, device=dev).to(bf) for _ in range(copies)]
    pages = -(-n // page)
    k_pool = torch.zeros(pages, g, page, hs, dtype=bf, device=dev)
    v_pool = torch.zeros_like(k_pool)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    pos = torch.arange(n, dtype=torch.int32, device=dev)
    req = torch.zeros(n, dtype=torch.int32, device=dev)
    inv = inverse_frequencies(hs, 500000.0, None).to(dev)
    st = {"i": 0}

    def nxt():
        st["i"] += 1
        return st["i"] % copies

    us = _time(lambda: add_rmsnorm(xs[nxt()], deltas[st["i"] % copies], w, 1e-5, bf), args.launches, graph=not args.eager)
    print(f"add_rmsnorm {n} x {hidden}: {us:.1f} us, {n * hidden * (4 + 4 + 2 + 2) / us / 1e6:.2f} TB/s")
    us = _time(lambda: silu_mul(gus[nxt()]), args.launches, graph=not args.eager)
    print(f"silu_mul {n} x {inter}: {us:.1f} us, {n * inter * 6 / us / 1e6:.2f} TB/s")
    us = _time(lambda: rope_kv_write(qkvs[nxt()], pos, req, inv, k_pool, v_pool, table, nh, g, hs), args.launches,
               graph=not args.eager)
    print(f"rope_kv_write {n} tokens: {us:.1f} us, {n * (nh + 2 * g) * hs * 4 / us / 1e6:.2f} TB/s")


def sampling(args) -> None:
    """Token selection over ``--rows`` rows of 128,256 logits: argmax, and the sampling kernels with top-k / top-p."""
    from yalis_b200.ops.sampling import argmax, sample
    dev = "cuda:0"
    rows, vocab = args.rows, 128256
    logits = torch.randn(rows, vocab, device=dev) * 3.0
    i64 = lambda v: torch.full((rows,), v, dtype=torch.int64, device=dev)
    f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=dev)
    k32 = lambda v: torch.full((rows,), v, dtype=torch.int32, device=dev)
    print(f"argmax {rows} rows: {_time(lambda: argmax(logits), args.launches, graph=not args.eager):.1f} us")
    for name, t, k, p in (("temperature only", 1.0, 0, 1.0), ("top-p 0.8", 1.0, 0, 0.8), ("top-k 50", 1.0, 50, 1.0),
                          ("top-k 50, top-p 0.9, T 0.7", 0.7, 50, 0.9)):
        us = _time(lambda: sample(logits, f32(t), k32(k), f32(p), i64(1), i64(2)), args.launches, graph=not args.eager)
        print(f"sample {rows} rows, {name}: {us:.1f} us")


def prefill(args) -> None:
    """One prompt of ``--tokens`` tokens through the whole engine (Llama-3-8B shape, ``--layers`` layers)."""
    from yalis_b200.bench_support import prefill_bench
    from yalis_b200.config.presets import preset
    from yalis_b200.engine.engine import Engine
    cfg = preset(args.preset)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    engine = Engine(config=cfg, seed=0, dtype=args.dtype, page_size=64, cache_tokens=args.tokens + 64, max_slots=2,
                    max_context=args.tokens + 64)
    ms = prefill_bench(engine, args.tokens, warmup=1, iters=args.launches)
    print(f"prefill {args.preset} layers {cfg['num_hidden_layers']} tokens {args.tokens} {args.dtype}: {ms:.3f} ms, "
          f"{args.tokens / ms * 1e3:.0f} tokens/s")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--eager", action="store_true", help="launch one by one instead of replaying a CUDA graph")
    sub = ap.add_subparsers(dest="case", required=True)
    a = sub.add_parser("attention_decode")
    a.add_argument("--batch", type=int, default=64)
    a.add_argument("--ctx", type=int, default=1040)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--page-size", type=int, default=64)
    a.add_argument("--splits", type=int, default=0)
    a.add_argument("--kernel", default="tma", choices=["tma", "lean", "mma"],
                   help="TMA-fed decode kernel (a block per pair and split), the one that deals tiles to a fixed grid, or the cp.async one")
    a.add_argument("--blocks", type=int, default=0, help="grid of the lean kernel (0: as the engine chooses)")
    a.add_argument("--launches", type=int, default=8)
    a.set_defaults(fn=attention_decode)
    gm = sub.add_parser("gemm_wstream")
    gm.add_argument("--tokens", type=int, default=8)
    gm.add_argument("--n", type=int, default=28672)
    gm.add_argument("--k", type=int, default=4096)
    gm.add_argument("--split", action="store_true")
    gm.add_argument("--library", action="store_true", help="time the library's product on the same operands instead")
    gm.add_argument("--launches", type=int, default=8)
    gm.set_defaults(fn=gemm_wstream)
    ap_ = sub.add_parser("attention_prefill")
    ap_.add_argument("--tokens", default="2048", help="tokens each request brings, comma-separated")
    ap_.add_argument("--before", default="0", help="tokens each request has cached already, comma-separated")
    ap_.add_argument("--splits", type=int, default=1, help="most key splits of a tile of queries (0: the engine's choice)")
    ap_.add_argument("--tiles-per-split", type=int, default=1, help="key tiles from which a tile of queries is divided")
    ap_.add_argument("--heads", type=int, default=32)
    ap_.add_argument("--kv-heads", type=int, default=8)
    ap_.add_argument("--head-dim", type=int, default=128)
    ap_.add_argument("--page-size", type=int, default=64)
    ap_.add_argument("--kernel", default="tcgen05", choices=["tcgen05", "mma", "library"],
                     help="library: flash_attn's kernel on contiguous keys, as the bar")
    ap_.add_argument("--launches", type=int, default=4)
    ap_.set_defaults(fn=attention_prefill)
    ew = sub.add_parser("elementwise")
    ew.add_argument("--tokens", type=int, default=2048)
    ew.add_argument("--launches", type=int, default=4)
    ew.set_defaults(fn=elementwise)
    sm = sub.add_parser("sampling")
    sm.add_argument("--rows", type=int, default=8)
    sm.add_argument("--launches", type=int, default=4)
    sm.set_defaults(fn=sampling)
    pf = sub.add_parser("prefill")
    pf.add_argument("--preset", default="Llama-3-8B")
    pf.add_argument("--layers", type=int, default=4)
    pf.add_argument("--tokens", type=int, default=2048)
    pf.add_argument("--dtype", default="bfloat16")
    pf.add_argument("--launches", type=int, default=2)
    pf.set_defaults(fn=prefill)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
