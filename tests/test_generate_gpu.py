"""Greedy and sampled generation through the Python entry point and the command line."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
from tiny import page_size_of, tiny_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def prompts_for(cfg, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def engine_for(model_dir, precision, **kw):
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    opts = dict(max_batch_size=4, max_length_of_generated_sequences=128, temperature=0.0, top_p=0.0)
    opts.update(kw)
    return LLMEngine(ModelConfig(model_name="tiny", model_path=model_dir, precision=precision), InferenceConfig(**opts))


@pytest.mark.parametrize("which, lengths, new, chunk", [("A", [5, 17, 33], 16, None), ("B", [1, 40, 100], 12, 24)])
def test_greedy_generation_equals_plain_float32(which, lengths, new, chunk):
    d = tiny_model_dir(which, 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, lengths)
    eng = engine_for(d, "fp32", page_size=page_size_of(which), prefill_chunk=chunk, max_tokens_per_step=64)
    tokens, metrics, logits = eng.generate(prompts, tokens_to_generate=new, get_logits=True)
    assert tokens.shape == (len(prompts), new) and tokens.dtype == torch.int64 and tokens.is_cuda
    for p, row, lg in zip(prompts, tokens.tolist(), logits):
        assert row == plain.greedy_generate(p, new, w, cfg)
        ref = plain.forward_logits(p + row[:-1], w, cfg)[len(p) - 1:]
        assert np.abs(lg.cpu().numpy() - ref.numpy()).max() <= 1e-4 * float(ref.abs().max())
    assert metrics["BatchSize"] == len(prompts) and metrics["DecodeLength"] == new and metrics["FinishedReason"] == "Max Token Length"
    assert metrics["Throughput"] > 0 and metrics["E2E"] > 0
    eng.engine.manager.check()
    assert all(eng.engine.manager.free_pages(g.name) == g.num_pages for g in eng.engine.groups)


@pytest.mark.parametrize("which", ["A", "C", "D"])
def test_greedy_generation_bfloat16_follows_the_oracle(which):
    """In bfloat16 every generated token is the oracle's best or within rounding of it
    (the reference's own criterion is top-5 containment: tests/basic_correctness/test_yalis_vs_hf.py:163-185).
    C and D have the head sizes of the TMA / tcgen05 kernels; decode steps run as captured graphs."""
    d = tiny_model_dir(which, 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [5, 17, 33])
    eng = engine_for(d, "bf16", page_size=page_size_of(which))
    tokens, _ = eng.generate(prompts, tokens_to_generate=16)
    for p, row in zip(prompts, tokens.tolist()):
        seq = list(p)
        for tok in row:
            ref = plain.forward_logits(seq, w, cfg)[-1]
            assert tok in torch.topk(ref, 5).indices.tolist()
            assert float(ref.max() - ref[tok]) <= 2e-2 * float(ref.abs().max())
            seq.append(tok)


def test_more_prompts_than_slots_and_few_pages():
    """Nine prompts, three slots, a pool that forces waiting and preemption: the tokens are
    those of each prompt generated alone."""
    d = tiny_model_dir("B", 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [30, 3, 61, 12, 45, 8, 70, 22, 5], seed=4)
    eng = engine_for(d, "fp32", max_batch_size=3, page_size=8, cache_tokens=104, prefill_chunk=16, max_tokens_per_step=40)
    tokens, metrics = eng.generate(prompts, tokens_to_generate=10)
    for p, row in zip(prompts, tokens.tolist()):
        assert row == plain.greedy_generate(p, 10, w, cfg)
    assert metrics["Preemptions"] > 0
    eng.engine.manager.check()


def test_waiting_and_preemption_in_bfloat16_with_the_native_kernels():
    """The same pressure in bfloat16 with head size 64 (tcgen05 / TMA kernels, captured decode steps that
    run ahead of the host): every token is the oracle's best on the row's own prefix, or within rounding."""
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [30, 3, 61, 12, 45, 8, 70, 22, 5], seed=4)
    eng = engine_for(d, "bf16", max_batch_size=3, page_size=16, cache_tokens=112, prefill_chunk=16, max_tokens_per_step=40)
    tokens, metrics = eng.generate(prompts, tokens_to_generate=10)
    assert metrics["Preemptions"] > 0
    for p, row in zip(prompts, tokens.tolist()):
        seq = list(p)
        for tok in row:
            ref = plain.forward_logits(seq, w, cfg)[-1]
            assert float(ref.max() - ref[tok]) <= 2e-2 * float(ref.abs().max())
            seq.append(tok)
    eng.engine.manager.check()
    assert all(eng.engine.manager.free_pages(g.name) == g.num_pages for g in eng.engine.groups)


def test_results_at_their_true_lengths_with_reasons_and_sampling_per_request():
    """``generate`` returns one result per prompt: a row that met its EOS id is shorter and says so, a request that
    can never fit the pool fails alone with ``out_of_pages``, and two requests of one call may sample
    differently (here: one greedy, one at temperature 0.9)."""
    from yalis_b200 import Generation, SamplingParams, generate
    from yalis_b200.sampling.sampler import GREEDY
    d = tiny_model_dir("A", 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [9, 20, 90], seed=2)
    free = [plain.greedy_generate(p, 12, w, cfg) for p in prompts[:2]]
    eos = free[0][4]
    eng = engine_for(d, "fp32", max_batch_size=3, page_size=16, cache_tokens=64)     # 4 pages: the 90-token prompt never fits
    out = generate(eng, prompts, max_new_tokens=12, eos_id=eos, return_logits=True)
    assert all(isinstance(g, Generation) for g in out)
    stop = free[0].index(eos)
    assert out[0].tokens == free[0][:stop + 1] and out[0].finish_reason == "eos" and len(out[0].tokens) < 12
    if eos not in free[1]:
        assert out[1].tokens == free[1] and out[1].finish_reason == "length"
    assert out[2].tokens == [] and out[2].finish_reason == "out_of_pages" and out[2].logits is None
    assert out[0].logits.shape == (stop + 1, cfg["vocab_size"])
    ref = plain.forward_logits(prompts[0] + out[0].tokens[:-1], w, cfg)[len(prompts[0]) - 1:]
    assert np.abs(out[0].logits.cpu().numpy() - ref.numpy()).max() <= 1e-4 * float(ref.abs().max())
    eng.engine.manager.check()
    # sampling per request: the greedy row is the plain model's, the other one draws (and is reproducible)
    hot = SamplingParams(temperature=0.9, top_p=0.95, seed=7)
    a = generate(eng, prompts[:2], max_new_tokens=12, sampling=[GREEDY, hot])
    b = generate(eng, prompts[:2], max_new_tokens=12, sampling=[GREEDY, hot])
    assert a[0].tokens == free[0] and a[1].tokens == b[1].tokens and a[1].tokens != free[1]
    alone = generate(eng, prompts[1:2], max_new_tokens=12, sampling=[hot])
    assert alone[0].tokens == a[1].tokens                      # what it draws does not depend on its neighbours
    with pytest.raises(ValueError):
        generate(eng, prompts[:2], sampling=[GREEDY])


def test_a_fault_reported_by_a_kernel_stops_generation():
    """Kernels never trap: they raise a bit in the device error word.  The host reads the word with every
    batch of tokens it fetches and raises, naming what was reported; nothing is left held.  The word is set
    here by hand between two steps (no kernel is made to fail)."""
    from yalis_b200.engine.engine import StepError
    from yalis_b200.ops import _lib
    d = tiny_model_dir("A", 0.3)
    cfg = plain.read_config(d)
    prompts = prompts_for(cfg, [9, 20], seed=2)
    for precision in ("fp32", "bf16"):
        eng = engine_for(d, precision)
        eng.generate(prompts, tokens_to_generate=4)              # a clean call first
        run_step, calls = eng.engine.run_step, [0]

        def faulty(*args, **kw):
            calls[0] += 1
            if calls[0] == 3:
                _lib.error_word(eng.device).fill_(_lib.FLAG_WAIT_PRODUCT | _lib.FLAG_BAD_PAGE)
            return run_step(*args, **kw)

        eng.engine.run_step = faulty
        with pytest.raises(StepError, match="weight-streaming product.*|block-table"):
            eng.generate(prompts, tokens_to_generate=10)
        eng.engine.run_step = run_step
        assert all(eng.engine.manager.free_pages(g.name) == g.num_pages for g in eng.engine.groups)
        assert eng.engine.manager.free_slots() == eng.engine.max_slots
        tokens, _ = eng.generate(prompts, tokens_to_generate=4)  # the word was cleared: the engine goes on
        assert tokens.shape == (2, 4)
    with pytest.raises(StepError):
        rid = eng.engine.add_request("x")
        _lib.error_word(eng.device).fill_(_lib.FLAG_BAD_ID)
        try:
            eng.engine.check_device_errors()
        finally:
            eng.engine.finish_request("x")


def test_eos_stops_a_row_and_pads_it():
    d = tiny_model_dir("A", 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [9, 20], seed=2)
    free = [plain.greedy_generate(p, 12, w, cfg) for p in prompts]
    eos = free[0][4]                                        # make the 5th token of row 0 the EOS id
    eng = engine_for(d, "fp32")
    eng.engine.spec = type(eng.engine.spec)(**{**{f: getattr(eng.engine.spec, f) for f in eng.engine.spec.__dataclass_fields__},
                                               "eos_token_id": eos})
    tokens, metrics = eng.generate(prompts, tokens_to_generate=12, ignore_eos=False)
    row0 = tokens[0].tolist()
    stop = free[0].index(eos)
    assert row0[:stop + 1] == free[0][:stop + 1] and all(t == eos for t in row0[stop + 1:])
    if eos not in free[1]:
        assert tokens[1].tolist() == free[1]


def test_sampling_is_reproducible_and_independent_of_the_batch():
    d = tiny_model_dir("A", 0.3)
    cfg = plain.read_config(d)
    prompts = prompts_for(cfg, [7, 19, 4], seed=6)
    kw = dict(temperature=0.8, top_p=0.9, top_k=50, seed=99)
    a, _ = engine_for(d, "fp32", **kw).generate(prompts, tokens_to_generate=12)
    b, _ = engine_for(d, "fp32", **kw).generate(prompts, tokens_to_generate=12)
    assert torch.equal(a, b)
    # request 0 alone draws what it drew in the batch (its seed and draw counter are its own)
    alone, _ = engine_for(d, "fp32", **kw).generate(prompts[:1], tokens_to_generate=12)
    assert alone[0].tolist() == a[0].tolist()
    c, _ = engine_for(d, "fp32", **dict(kw, seed=100)).generate(prompts, tokens_to_generate=12)
    assert not torch.equal(a, c)


def test_generate_shortcut_and_command_line():
    from yalis_b200 import generate
    d = tiny_model_dir("A", 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [6, 11], seed=8)
    out = [g.tokens for g in generate(d, prompts, max_new_tokens=5, precision="fp32")]
    assert out == [plain.greedy_generate(p, 5, w, cfg) for p in prompts]
    proc = subprocess.run([sys.executable, "-m", "yalis_b200.cli", "--model", d, "--precision", "fp32", "--temperature", "0",
                           "--top-p", "0", "--tokens-to-gen", "5", "--max-length", "64",
                           "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", ",".join(map(str, prompts[1]))],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("output = ")]
    assert [eval(l[len("output = "):]) for l in lines] == out


def attention_kinds(eng):
    """The (tiles dealt out, long context) pairs among the keys of the engine's recorded steps."""
    found = set()

    def walk(key):
        if isinstance(key, tuple):
            if len(key) == 2 and all(isinstance(v, bool) for v in key):
                found.add(key)
            else:
                for v in key:
                    walk(v)

    for key in eng.engine._recordings:
        walk(key[3])
    return found


def follows_the_oracle(prompts, tokens, w, cfg):
    for p, row in zip(prompts, tokens.tolist()):
        seq = list(p)
        for tok in row:
            ref = plain.forward_logits(seq, w, cfg)[-1]
            assert float(ref.max() - ref[tok]) <= 2e-2 * float(ref.abs().max())
            seq.append(tok)


def test_long_context_kind_of_decode_steps(monkeypatch):
    """Decode steps of one request beyond the long-context mark are captured as a kind of their own, with more
    key splits merged through global memory; with the mark lowered to 48 tokens a tiny model crosses it."""
    from yalis_b200.ops import attention as attn_ops
    monkeypatch.setattr(attn_ops, "LONG_CONTEXT", 48)
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [30])
    eng = engine_for(d, "bf16", page_size=page_size_of("C"))
    tokens, _ = eng.generate(prompts, tokens_to_generate=40)
    assert attention_kinds(eng) == {(False, False), (False, True)}   # it crossed the mark
    follows_the_oracle(prompts, tokens, w, cfg)


def test_long_or_uneven_batches_have_their_key_tiles_dealt_out(monkeypatch):
    """Two or more requests of which one is long (beyond the long-context mark), or much longer than the others,
    make a kind of decode step of their own, in which the attention kernel deals the key tiles of all requests
    to a fixed grid.  With the marks lowered a tiny model gets there: first by the long-context mark while it
    decodes, then (mark out of reach) by one prompt of 100 tokens beside short ones."""
    from yalis_b200.ops import attention as attn_ops
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    monkeypatch.setattr(attn_ops, "LONG_CONTEXT", 48)
    prompts = prompts_for(cfg, [30, 44, 17])
    eng = engine_for(d, "bf16", page_size=page_size_of("C"))
    before = attn_ops.LAUNCHED["decode_lean"]
    tokens, _ = eng.generate(prompts, tokens_to_generate=24)
    assert attention_kinds(eng) == {(False, False), (True, False)}
    assert attn_ops.LAUNCHED["decode_lean"] > before
    follows_the_oracle(prompts, tokens, w, cfg)
    monkeypatch.setattr(attn_ops, "LONG_CONTEXT", 8192)
    monkeypatch.setattr(attn_ops, "DEAL_MIN_LONGEST", 64)
    assert attn_ops.deal_tiles_hint([101, 6, 8]) and not attn_ops.deal_tiles_hint([101, 90, 80]) \
        and not attn_ops.deal_tiles_hint([40, 2, 2]) and not attn_ops.deal_tiles_hint([5000])
    prompts = prompts_for(cfg, [100, 5, 7], seed=3)
    eng = engine_for(d, "bf16", page_size=page_size_of("C"), max_length_of_generated_sequences=192)
    before = attn_ops.LAUNCHED["decode_lean"]
    tokens, _ = eng.generate(prompts, tokens_to_generate=24)
    assert attention_kinds(eng) == {(True, False)}
    assert attn_ops.LAUNCHED["decode_lean"] > before
    follows_the_oracle(prompts, tokens, w, cfg)


def test_decode_steps_with_more_pairs_than_resident_blocks(monkeypatch):
    """A batch with more (request, KV head) pairs than blocks fit the GPU at once goes to the decode kernel that
    deals tiles to a fixed grid; with the GPU taken for two SMs, five requests of a tiny model are such a batch
    (4 blocks for 10 pairs, so block borders cut pairs), through captured steps, lengths growing across tiles."""
    from yalis_b200.ops import attention as attn_ops
    monkeypatch.setattr(attn_ops, "SM_COUNT", 2)
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [30, 61, 3, 100, 17])
    eng = engine_for(d, "bf16", page_size=page_size_of("C"), max_batch_size=5, max_length_of_generated_sequences=192)
    before = attn_ops.LAUNCHED["decode_lean"]
    tokens, _ = eng.generate(prompts, tokens_to_generate=40)
    assert attn_ops.LAUNCHED["decode_lean"] > before
    for p, row in zip(prompts, tokens.tolist()):
        seq = list(p)
        for tok in row:
            ref = plain.forward_logits(seq, w, cfg)[-1]
            assert float(ref.max() - ref[tok]) <= 2e-2 * float(ref.abs().max())
            seq.append(tok)


def test_prompt_portions_with_their_keys_divided_among_blocks(monkeypatch):
    """The policy that divides the keys of a tile of queries among several blocks of the tcgen05 prompt kernel
    only does so for long contexts; here it is made to (up to three shares of one key tile or more) for the
    portions of a tiny model's prompts, and says what it should for shapes measured on the GPU."""
    from types import SimpleNamespace
    from yalis_b200.ops import attention as attn_ops
    choice = lambda q_start, before, per: attn_ops.prefill_kv_splits(SimpleNamespace(q_start=q_start, ctx_before=before), per, 8, 128)
    assert choice([0, 2048], [12000], 3)[0] > 1         # 392 blocks: 1.3 waves
    assert choice([0, 512], [3584], 4)[0] > 1           # 128 blocks: less than half the GPU
    assert choice([0, 2048], [12000], 4)[0] == 1        # 512 blocks of two to an SM are even enough
    assert choice([0, 2048], [0], 4)[0] == 1 and choice([0, 8192], [0], 4)[0] == 1 and choice([0, 300, 301], [0, 500], 4)[0] == 1
    splits, limit = choice([0, 1, 2048], [14012, 816], 3)    # a decoding request with a long context beside a fresh prompt
    assert splits > 2 and limit * splits >= 14012 // 64 + 1 and limit >= 24
    monkeypatch.setattr(attn_ops, "prefill_kv_splits", lambda host, per, g, hs, skip_single=False: (3, 1))
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [150, 61, 100])
    eng = engine_for(d, "bf16", page_size=page_size_of("C"), prefill_chunk=48, max_tokens_per_step=64,
                     max_length_of_generated_sequences=192)
    before = attn_ops.LAUNCHED["prefill_tcgen05"]
    tokens, _ = eng.generate(prompts, tokens_to_generate=6)
    assert attn_ops.LAUNCHED["prefill_tcgen05"] > before
    follows_the_oracle(prompts, tokens, w, cfg)


def test_steps_of_portions_and_decoding_requests_use_two_attention_kernels(monkeypatch):
    """While long prompts are still read in portions, requests with short prompts already decode: in such steps the
    decoding requests go to the decode kernel once they hold enough tokens (here: any), the portions to the
    prompt kernel."""
    from yalis_b200.ops import attention as attn_ops
    monkeypatch.setattr(attn_ops, "MIXED_DECODE_MIN_KEYS", 0)
    d = tiny_model_dir("C", 0.02)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [150, 20, 90, 7])
    eng = engine_for(d, "bf16", page_size=page_size_of("C"), prefill_chunk=32, max_tokens_per_step=40,
                     max_length_of_generated_sequences=192)
    before = attn_ops.LAUNCHED["decode_lean"], attn_ops.LAUNCHED["prefill_tcgen05"]
    tokens, _ = eng.generate(prompts, tokens_to_generate=12)
    assert attn_ops.LAUNCHED["decode_lean"] > before[0] and attn_ops.LAUNCHED["prefill_tcgen05"] > before[1]
    follows_the_oracle(prompts, tokens, w, cfg)
    assert attn_ops.mixed_step_splits_off_decodes(type("H", (), dict(q_start=[0, 1, 2, 50], ctx_before=[5, 9, 100]))()) is True
    monkeypatch.setattr(attn_ops, "MIXED_DECODE_MIN_KEYS", 4096)
    assert not attn_ops.mixed_step_splits_off_decodes(type("H", (), dict(q_start=[0, 1, 2, 50], ctx_before=[5, 9, 100]))())
    assert attn_ops.mixed_step_splits_off_decodes(type("H", (), dict(q_start=[0, 1, 2, 50], ctx_before=[3000, 2000, 100]))())


def test_sampling_with_block_tables_used_to_their_last_entry():
    """Requests that grow into the last page their block-table row can name, decoded with sampling in
    captured steps: the per-row sampling parameters and the tables lie in one buffer and must not overlap
    (a fuzzing run found the last table entries overwritten by the temperatures)."""
    d = tiny_model_dir("B", 0.3)
    cfg = plain.read_config(d)
    prompts = prompts_for(cfg, [18, 7, 2, 43, 52], seed=9)
    new = 19
    longest = max(len(p) for p in prompts) + new
    kw = dict(temperature=0.8, top_p=0.9, seed=5, max_batch_size=4, page_size=8,
              max_length_of_generated_sequences=-(-longest // 8) * 8, cache_tokens=400)
    a, _ = engine_for(d, "fp32", **kw).generate(prompts, tokens_to_generate=new)
    os.environ["YALIS_DISABLE_DECODE_CUDAGRAPHS"] = "1"
    try:
        b, _ = engine_for(d, "fp32", **kw).generate(prompts, tokens_to_generate=new)
    finally:
        del os.environ["YALIS_DISABLE_DECODE_CUDAGRAPHS"]
    assert torch.equal(a, b)            # captured steps draw what step-by-step launches draw


def test_a_one_token_prompt_that_takes_over_a_slot():
    """One slot, requests one after the other, one of them with a single prompt token: its first step is
    a step of one token like a decode step, but its input is its own prompt token (a fuzzing run found it fed
    the token that the slot's last owner drew)."""
    d = tiny_model_dir("A", 0.3)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = prompts_for(cfg, [9, 1, 14, 1], seed=12)
    eng = engine_for(d, "fp32", max_batch_size=1)
    tokens, _ = eng.generate(prompts, tokens_to_generate=6)
    for p, row in zip(prompts, tokens.tolist()):
        assert row == plain.greedy_generate(p, 6, w, cfg)
