"""Random configurations, workloads and engine settings (fixed seeds): the replayer against the plain
model under every cutting, and generation through the scheduler and the captured decode steps against
the plain model's tokens.  A run of this kind found three faults that the hand-made cases had missed
(overlapping regions of a step buffer, a one-token prompt taking over a slot, garbage collection during a
graph capture); a few dozen trials stay here."""

import random
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
import traces
from yalis_b200.config.presets import _llama
from yalis_b200.weights.loader import write_random_model

pytestmark = pytest.mark.gpu


def random_config(rng, head_sizes):
    hs = rng.choice(head_sizes)
    g = rng.choice([1, 2, 3])
    nh = g * rng.choice([1, 2, 4, 5])
    scaling = rng.choice([None, dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=64)])
    cfg = _llama(rng.choice([64, 72, 100, 136, 200, 52]), rng.choice([1, 2]), nh, g, rng.choice([96, 104, 176, 250, 64]), 512,
                 scaling, tied=rng.choice([True, False]), head_dim=hs, vocab=rng.choice([257, 300, 512, 1000]),
                 theta=rng.choice([10000.0, 500000.0]), eps=rng.choice([1e-5, 1e-6]))
    return dict(cfg, bos_token_id=None, eos_token_id=None)


def force_rare_paths(monkeypatch, attn_ops, seed):
    """Choices that the attention wrappers only make for long contexts, made for every step: decoding requests of
    mixed steps in the decode kernel, and the keys of prompt tiles divided among blocks in changing ways."""
    rng = random.Random(seed)
    monkeypatch.setattr(attn_ops, "MIXED_DECODE_MIN_KEYS", 0)
    monkeypatch.setattr(attn_ops, "prefill_kv_splits",
                        lambda host, per, g, hs, skip_single=False: rng.choice([(1, 1), (2, 1), (3, 1), (4, 2), (2, 3)]))


@pytest.mark.parametrize("seed, sms, rare", [(1, None, False), (2, None, False), (5, 1, False), (6, None, True), (7, 1, True)])
def test_replay_of_random_configurations(seed, sms, rare, monkeypatch):
    """``sms``: the number of SMs the attention wrappers plan for; with 1, decode steps of two requests already
    count as large batches and go to the kernel that deals key tiles to a fixed grid (two blocks, or one).
    ``rare``: see ``force_rare_paths``."""
    from yalis_b200.engine.replay import Replayer
    from yalis_b200.ops import attention as attn_ops
    if sms is not None:
        monkeypatch.setattr(attn_ops, "SM_COUNT", sms)
    if rare:
        force_rare_paths(monkeypatch, attn_ops, seed)
    rng = random.Random(seed)
    for trial in range(6):
        cfg = random_config(rng, [16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 224, 256, 24, 40])
        page = rng.choice([8, 16, 32, 64])
        lengths = [rng.randint(1, 40), rng.randint(41, 150), rng.randint(60, 200)]
        with tempfile.TemporaryDirectory() as d:
            for dtype, std, tol in (("float32", 0.2, 1e-4), ("bfloat16", 0.03, 3e-2)):
                write_random_model(cfg, d, seed=trial, std=std)
                pcfg, w = plain.read_config(d), plain.read_weights(d)
                gen = torch.Generator().manual_seed(trial)
                reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for i, n in enumerate(lengths)}
                want = {rid: plain.forward_logits(t, w, pcfg).numpy() for rid, t in reqs.items()}
                for build in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
                    steps = traces.number(build(reqs))
                    rep = Replayer(d, dtype, traces.peak_tokens(steps), page_size=page, graphs=trial % 2 == 1)   # every other trial through recorded steps
                    out = {}
                    for s in steps:
                        r = rep.run_step(s)
                        if r is not None:
                            out[s["step"]] = r
                    got = traces.collect(steps, out, cfg["vocab_size"])
                    err = max(np.abs(got[r] - want[r]).max() / np.abs(want[r]).max() for r in want)
                    assert err < tol, (seed, trial, dtype, build.__name__, err, cfg, page, lengths)


@pytest.mark.parametrize("seed, sms, rare", [(2, None, False), (3, None, False), (4, 1, False), (8, None, True), (9, 1, True)])
def test_generation_with_random_settings(seed, sms, rare, monkeypatch):
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    from yalis_b200.ops import attention as attn_ops
    if sms is not None:
        monkeypatch.setattr(attn_ops, "SM_COUNT", sms)           # see test_replay_of_random_configurations
    if rare:
        force_rare_paths(monkeypatch, attn_ops, seed)
    rng = random.Random(seed)
    for trial in range(12):
        cfg = random_config(rng, [16, 32, 64, 128, 64, 128, 192, 256, 48])
        vocab = cfg["vocab_size"]
        page = rng.choice([8, 16, 32, 64])
        new = rng.randint(4, 20)
        lens = [rng.randint(1, 90) for _ in range(rng.randint(1, 9))]
        slots = rng.randint(1, 4)
        need = max(lens) + new + page
        cache = rng.choice([need + page, 2 * need, slots * need])          # some pools force waiting and preemption
        dtype = rng.choice(["bf16", "bf16", "fp32"])
        temp = rng.choice([0.0, 0.0, 0.8])
        what = (seed, trial, cfg, page, lens, new, slots, cache, dtype, temp)
        with tempfile.TemporaryDirectory() as d:
            write_random_model(cfg, d, seed=trial, std=0.3 if dtype == "fp32" else 0.03)
            pcfg, w = plain.read_config(d), plain.read_weights(d)
            gen = torch.Generator().manual_seed(trial)
            eng = LLMEngine(ModelConfig(model_name="t", model_path=d, precision=dtype),
                            InferenceConfig(max_batch_size=slots, max_length_of_generated_sequences=need, temperature=temp,
                                            top_p=0.0 if temp == 0 else 0.9, page_size=page, cache_tokens=cache,
                                            prefill_chunk=rng.choice([None, 16, 24, 64]),
                                            max_tokens_per_step=rng.choice([32, 48, 128])))
            for call in range(rng.choice([1, 1, 2])):                        # the engine is used again
                prompts = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lens]
                tokens, _ = eng.generate(prompts, tokens_to_generate=new)
                eng.engine.manager.check()
                assert all(eng.engine.manager.free_pages(g.name) == g.num_pages for g in eng.engine.groups), what
                eng.engine.check_device_errors()
                assert tokens.shape == (len(prompts), new) and int(tokens.min()) >= 0 and int(tokens.max()) < vocab, what
                if temp != 0:
                    continue
                for p, row in zip(prompts, tokens.tolist()):
                    if dtype == "fp32":
                        assert row == plain.greedy_generate(p, new, w, pcfg), what
                    else:
                        seq = list(p)
                        for tok in row:
                            ref = plain.forward_logits(seq, w, pcfg)[-1]
                            assert float(ref.max() - ref[tok]) <= 3e-2 * float(ref.abs().max()), what
                            seq.append(tok)
                lens = [rng.randint(1, max(lens)) for _ in range(rng.randint(1, 6))]
