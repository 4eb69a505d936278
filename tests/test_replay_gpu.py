"""Replay of the same requests cut four ways, in float32 and bfloat16, against the plain
implementation: each request whole; most of it in one step and the last 32 tokens one by
one; portions of changing size down to two tokens; and up to four live requests mixed, with
so few pages that they are used again.  One run goes through ``bin/trace_run`` as a
program; the rest use the same replayer in-process."""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
import traces
from tiny import page_size_of, tiny_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# relative to the largest |logit| of the request
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
STD = {"float32": 0.2, "bfloat16": 0.02}     # wide weights in float32 make attention far from uniform


def make_requests(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def lengths_for(which):
    return {"A": [5, 17, 33, 70, 100, 128], "B": [1, 40, 100, 64, 203, 90], "C": [3, 64, 65, 130, 200, 77],
            "D": [16, 63, 129, 250, 34, 100]}[which]


_oracle_cache = {}


def oracle(which, std, requests):
    key = (which, std, tuple(sorted((k, tuple(v)) for k, v in requests.items())))
    if key not in _oracle_cache:
        d = tiny_model_dir(which, std)
        cfg, w = plain.read_config(d), plain.read_weights(d)
        _oracle_cache[key] = {rid: plain.forward_logits(t, w, cfg).numpy() for rid, t in requests.items()}
    return _oracle_cache[key]


def replay_in_process(model_dir, dtype, page_size, steps, max_tokens, graphs=False):
    from yalis_b200.engine.replay import Replayer
    rep = Replayer(model_dir, dtype, max_tokens, page_size=page_size, graphs=graphs)
    out = {}
    for s in steps:
        r = rep.run_step(s)
        if r is not None:
            out[s["step"]] = r
    rep.engine.manager.check()
    for g in rep.engine.groups:
        assert rep.engine.manager.free_pages(g.name) == g.num_pages     # every page came back
    return out, rep


def compare(got, want, tol, what):
    assert set(got) == set(want), what
    worst = 0.0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        scale = np.abs(want[rid]).max()
        err = np.abs(got[rid] - want[rid]).max() / scale
        worst = max(worst, err)
        if err > tol:
            bad = np.argwhere(np.abs(got[rid] - want[rid]).max(axis=1) / scale > tol)
            raise AssertionError(f"{what}: request {rid} differs by {err:.3e} (tolerance {tol}); "
                                 f"first wrong position {int(bad[0])} of {want[rid].shape[0]}")
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions", "mixed", "tail_decoded/recorded", "mixed/recorded",
                                 "portions/recorded"])
def test_cuttings_match_plain(which, dtype, cut):
    cut, _, recorded = cut.partition("/")
    std = STD[dtype]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, lengths_for(which), seed=11)
    want = oracle(which, std, requests)
    build = {"whole": traces.whole, "tail_decoded": traces.tail_decoded, "portions": traces.portions,
             "mixed": traces.mixed}[cut]
    steps = traces.number(build(requests))
    peak = traces.peak_tokens(steps)
    out, rep = replay_in_process(d, dtype, page_size_of(which), steps, peak, graphs=bool(recorded))
    got = traces.collect(steps, out, cfg["vocab_size"])
    compare(got, want, TOL[dtype], f"{which}/{dtype}/{cut}{'/recorded' if recorded else ''}")
    if recorded:
        single = sum(all(len(e["tokens"]) == 1 for e in s["entries"]) for s in steps)
        assert rep.steps_replayed >= single             # and steps with portions whose shape came a second time
        assert rep.steps_replayed > 0
    if cut == "mixed":
        # the pool was smaller than the sum of all requests: pages were used again
        assert peak < sum(traces.round_up(len(t)) for t in requests.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(dtype):
    """The logits at a position do not depend on the cutting beyond rounding: in float32
    every kernel sums in a fixed order, so the four ways agree to the last bit or two."""
    which, std = "B", 0.2
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [3, 61, 130, 77, 18], seed=5)
    results = []
    for build, graphs in ((traces.whole, False), (traces.tail_decoded, False), (traces.portions, False), (traces.mixed, False),
                          (traces.tail_decoded, True), (traces.mixed, True)):
        steps = traces.number(build(requests))
        out, rep = replay_in_process(d, dtype, page_size_of(which), steps, traces.peak_tokens(steps), graphs=graphs)
        assert (rep.steps_replayed > 0) == graphs
        results.append(traces.collect(steps, out, cfg["vocab_size"]))
    tol = 1e-6 if dtype == "float32" else 2e-2
    for other in results[1:]:
        compare(other, results[0], tol, f"cut vs whole ({dtype})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype):
    """The program itself: JSON lines in, ``done <step>`` lines and <step>.f32 files out."""
    which = "A"
    std = STD[dtype]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [9, 64, 65, 120, 30], seed=3)
    steps = traces.number(traces.whole(requests) + traces.tail_decoded(requests) + traces.portions(requests)
                          + traces.mixed(requests))
    # the four phases reuse the ids r0.. one after the other; every phase ends its requests
    peak = traces.peak_tokens(steps)
    with tempfile.TemporaryDirectory() as out_dir:
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(peak), "--page-size", str(page_size_of(which))],
            input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
        assert done == [f"done {s['step']}" for s in steps]
        out = {s["step"]: np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4") for s in steps}
    want = oracle(which, std, requests)
    # split the concatenated trace back into its four phases
    phase_starts = []
    n_whole = len(traces.whole(requests)); n_tail = len(traces.tail_decoded(requests)); n_port = len(traces.portions(requests))
    bounds = [0, n_whole, n_whole + n_tail, n_whole + n_tail + n_port, len(steps)]
    for a, b in zip(bounds[:-1], bounds[1:]):
        got = traces.collect(steps[a:b], out, cfg["vocab_size"])
        compare(got, want, TOL[dtype], f"trace_run/{dtype}/steps {a}-{b}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype):
    """One prompt token, then 250 tokens one by one (positions across many pages); and the
    first tokens of a sequence asked for alone."""
    which, std = "B", STD[dtype]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [251], seed=8)
    steps = traces.number(traces.tail_decoded(requests, tail=250))
    out, _ = replay_in_process(d, dtype, page_size_of(which), steps, traces.peak_tokens(steps))
    got = traces.collect(steps, out, cfg["vocab_size"])
    want = oracle(which, std, requests)
    compare(got, want, TOL[dtype], f"long decoding {dtype}")
    toks = requests["r0"]
    first = traces.number([{"entries": [{"id": "f", "tokens": toks[:1], "want": [0]}], "end": []},
                           {"entries": [{"id": "f", "tokens": toks[1:3], "want": [0, 1]}], "end": ["f"]}])
    out, _ = replay_in_process(d, dtype, page_size_of(which), first, 64)
    got = traces.collect(first, out, cfg["vocab_size"])
    compare(got, {"f": want["r0"][:3]}, TOL[dtype], f"first tokens {dtype}")


def decoding_together(requests, heads, leave_after):
    """A trace in which the requests are fed whole up to ``heads[i]`` tokens and then decode together, one
    token each per step; request i ends (and leaves the batch) ``leave_after[i]`` steps after the decoding began,
    or when its tokens run out."""
    ids = list(requests)
    steps = [{"entries": [{"id": rid, "tokens": requests[rid][:h], "want": list(range(h))} for rid, h in zip(ids, heads)],
              "end": []}]
    at = dict(zip(ids, heads))
    live, k = list(ids), 0
    while live:
        k += 1
        entries, end = [], []
        for i, rid in enumerate(ids):
            if rid not in live:
                continue
            entries.append({"id": rid, "tokens": [requests[rid][at[rid]]], "want": [0]})
            at[rid] += 1
            if at[rid] == len(requests[rid]) or k == leave_after[i]:
                end.append(rid)
        live = [rid for rid in live if rid not in end]
        steps.append({"entries": entries, "end": end})
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "C"])
def test_recorded_steps_with_padding_and_changes_of_kind(which, dtype, monkeypatch):
    """Steps replayed from recordings, where they differ from launched ones: three live requests in a recording
    made for four (a padding row), a request that leaves so that the others move to a smaller recording, and
    requests that grow past the marks by which the attention part keys its recordings (lowered here so that a
    tiny model crosses them): from the plain kind to dealt tiles while three decode, to the long-context kind
    when one is left.  Every logit against the plain model, as for launched steps."""
    from yalis_b200.ops import attention as attn_ops
    monkeypatch.setattr(attn_ops, "LONG_CONTEXT", 60)
    std = STD[dtype]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [70, 30, 52], seed=21)
    want = oracle(which, std, requests)
    steps = traces.number(decoding_together(requests, heads=[40, 6, 20], leave_after=[99, 14, 25]))
    out, rep = replay_in_process(d, dtype, page_size_of(which), steps, traces.peak_tokens(steps), graphs=True)
    got = traces.collect(steps, out, cfg["vocab_size"])
    want = {rid: want[rid][:got[rid].shape[0]] for rid in got}
    compare(got, want, TOL[dtype], f"recorded steps {which}/{dtype}")
    assert rep.steps_replayed == len(steps) - 1
    sizes = {key[0] for key in rep.engine._recordings}
    assert sizes == {4, 2, 1}                                     # 3 live in a recording of 4, then 2, then 1
    if which == "C" and dtype == "bfloat16":                      # the kernels that look at the kind of step
        kinds = set()
        for key in rep.engine._recordings:
            kinds |= {k for block in key[3] if isinstance(block, tuple) for k in block if isinstance(k, tuple)}
        assert kinds == {(False, False), (True, False), (False, True)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_steps_that_take_their_tokens_from_the_device(dtype, graphs):
    """A step may name "the token chosen for this request last" instead of a token id: the choice stays on the
    device and the host need not have read it.  Greedy decoding that way gives the logits of the plain model on
    the sequence it produces, and the same tokens as decoding with the ids passed through the host."""
    from yalis_b200.engine.engine import Engine, StepEntry
    from yalis_b200.sampling.sampler import GREEDY
    which, std = "C", STD[dtype]
    d = tiny_model_dir(which, std)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    prompts = make_requests(cfg, [23, 5, 40], seed=9)
    eng = Engine(d, dtype=dtype, page_size=page_size_of(which), cache_tokens=512, max_slots=4)
    for rid in prompts:
        eng.add_request(rid)
    ids = list(prompts)
    out = eng.run([StepEntry(rid, prompts[rid], [len(prompts[rid]) - 1]) for rid in ids], sampling=[GREEDY] * 3, draws=[0] * 3)
    seqs = {rid: list(prompts[rid]) for rid in ids}
    logits = {rid: [out.logits[i].cpu()] for i, rid in enumerate(ids)}
    reports = [eng.fetch_chosen()]
    for k in range(1, 12):
        if k == 6:
            eng.finish_request(ids.pop(1))               # the batch shrinks: another recording, same slots
        out = eng.run([StepEntry(rid, None, [0]) for rid in ids], sampling=[GREEDY] * len(ids), draws=[k] * len(ids),
                      graphs=graphs)
        assert out.captured == graphs
        for i, rid in enumerate(ids):
            logits[rid].append(out.logits[i].cpu())
        reports.append(eng.fetch_chosen())                # read only after the loop: the host runs ahead
    slot = {rid: eng.slot_of(rid) for rid in ids}
    for rid in prompts:
        s = slot.get(rid, 1)                              # the request that left held slot 1
        for k, rep in enumerate(reports):
            if rid in ids or k < 6:
                seqs[rid].append(int(rep.wait()[s]))
    for rid in prompts:
        ref = plain.forward_logits(seqs[rid][:-1], w, cfg)[len(prompts[rid]) - 1:]
        got = torch.stack(logits[rid])
        assert got.shape == ref.shape
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err <= TOL[dtype], (rid, err)
        if dtype == "float32":
            assert seqs[rid][len(prompts[rid]):] == plain.greedy_generate(prompts[rid], len(seqs[rid]) - len(prompts[rid]), w, cfg)
    with pytest.raises(Exception, match="no token was chosen"):
        eng.add_request("new")
        eng.run([StepEntry("new", None, [0])])
    for rid in ids + ["new"]:
        eng.finish_request(rid)
    eng.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "C"])
def test_steps_with_portions_are_recorded_when_their_shape_repeats(which, dtype):
    """Three requests fed in lockstep, 16 tokens each per step and then single tokens beside one portion: the second
    step of a shape is recorded (a CUDA graph with room for its tokens, requests and wanted rows rounded up, the
    rest padding), the later ones replay it, with other tokens, positions and pages each time.  Every logit
    against the plain model."""
    std = STD[dtype]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [100, 100, 120], seed=31)
    want = oracle(which, std, requests)
    ids = list(requests)
    steps, at = [], {rid: 0 for rid in ids}
    for k in range(5):                                             # five steps of 3 x 16 tokens
        steps.append({"entries": [{"id": rid, "tokens": requests[rid][at[rid]:at[rid] + 16], "want": [3, 15]} for rid in ids], "end": []})
        for rid in ids:
            at[rid] += 16
    for k in range(4):                                             # four steps: two single tokens beside a portion of 10
        entries = [{"id": rid, "tokens": requests[rid][at[rid]:at[rid] + 1], "want": [0]} for rid in ids[:2]]
        entries.append({"id": ids[2], "tokens": requests[ids[2]][at[ids[2]]:at[ids[2]] + 10], "want": [9]})
        steps.append({"entries": entries, "end": []})
        at[ids[0]] += 1; at[ids[1]] += 1; at[ids[2]] += 10
    steps[-1]["end"] = ids
    steps = traces.number(steps)
    out, rep = replay_in_process(d, dtype, page_size_of(which), steps, traces.peak_tokens(steps), graphs=True)
    assert rep.steps_replayed == (5 - 1) + (4 - 1)                 # all but the first of each shape
    exact = [key for key in rep.engine._recordings if not key[4][3]]
    # room for (tokens, requests, wanted rows, longest portion): 12 tokens of 3 requests in 16 and 4, and so on
    assert sorted(key[4][:3] + key[4][4:] for key in exact) == [(16, 4, 4, 16), (64, 4, 8, 16)]
    row = {rid: [] for rid in ids}
    for s in steps:
        arr = out[s["step"]].reshape(-1, cfg["vocab_size"])
        i = 0
        for e in s["entries"]:
            for j in e["want"]:
                pos = (0 if not row[e["id"]] else row[e["id"]][-1][1]) + j
                ref = want[e["id"]][pos]
                err = np.abs(arr[i] - ref).max() / np.abs(want[e["id"]]).max()
                assert err <= TOL[dtype], (s["step"], e["id"], pos, err)
                i += 1
            row[e["id"]].append((None, (0 if not row[e["id"]] else row[e["id"]][-1][1]) + len(e["tokens"])))


def test_shapes_that_turn_over_faster_than_they_repeat_are_launched(monkeypatch):
    """Four shapes of step in turn with room for two recordings: the two that are recorded first stay and replay,
    the others are launched, nothing is recorded over and over; every step gives the logits of the launched
    path.  A recording that has lain idle long enough makes room in the end."""
    from yalis_b200.engine import recorded
    from yalis_b200.engine.engine import Engine, StepEntry
    d = tiny_model_dir("C", STD["float32"])          # float32: a padded step gives the same bits
    made = []
    init = recorded.RecordedStep.__init__
    monkeypatch.setattr(recorded.RecordedStep, "__init__", lambda self, *a, **k: (made.append(a[1]), init(self, *a, **k))[1])
    lengths = [16, 40, 70, 130] * 4 + [16, 40] * 2 + [70] * 8         # in turn; then the recorded two; then one of the others
    outputs = {}
    for graphs in (False, True):
        eng = Engine(d, dtype="float32", page_size=16, num_pages=32, max_slots=2)
        eng.MAX_EXACT_RECORDINGS, eng.IDLE_STEPS_BEFORE_EVICTION = 2, 6
        outputs[graphs] = []
        for k, n in enumerate(lengths):
            eng.add_request(k)
            out = eng.run([StepEntry(k, [(7 * k + i) % 50 for i in range(n)], [n - 1])], graphs=graphs)
            outputs[graphs].append((out.captured, out.logits.float().cpu()))
            eng.finish_request(k)
        eng.manager.check()
    assert made == [16, 64, 128]                                      # room for 70 only once the recording for 16 had lain idle
    captured = [c for c, _ in outputs[True]]
    assert captured == [False] * 4 + [True, True, False, False] * 3 + [True] * 4 + [False] * 4 + [True] * 4
    for (_, a), (_, b) in zip(outputs[False], outputs[True]):
        torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_tensors_stored_in_float32_stay_so_under_bfloat16():
    """A checkpoint whose embedding, one fused projection part, one down projection and the final norm are stored
    in float32: the bfloat16 engine keeps them in float32 (their products run on the exact kernels, bfloat16 rows
    against float32 weights) and its logits still match the plain model, whole and decoded, launched and recorded."""
    from yalis_b200.weights.safetensors_io import Checkpoint, write_safetensors
    which, dtype, std = "C", "bfloat16", STD["bfloat16"]
    src = tiny_model_dir(which, std)
    with tempfile.TemporaryDirectory() as d:
        with Checkpoint(src) as ck:
            tensors = {n: ck.get(n).clone() for n in ck.names()}
        wide = [n for n in tensors if n.endswith(("embed_tokens.weight", "layers.0.self_attn.k_proj.weight",
                                                   "layers.1.mlp.down_proj.weight", "model.norm.weight"))]
        assert len(wide) == 4
        for n in wide:
            tensors[n] = tensors[n].float()
        write_safetensors(os.path.join(d, "model.safetensors"), tensors)
        with open(os.path.join(src, "config.json")) as f, open(os.path.join(d, "config.json"), "w") as g:
            g.write(f.read())
        cfg = plain.read_config(d)
        requests = make_requests(cfg, [40, 70], seed=21)
        w = plain.read_weights(d)
        want = {rid: plain.forward_logits(t, w, cfg).numpy() for rid, t in requests.items()}
        for graphs in (False, True):
            steps = traces.number(traces.tail_decoded(requests))
            out, rep = replay_in_process(d, dtype, page_size_of(which), steps, traces.peak_tokens(steps), graphs=graphs)
            model = rep.engine.model
            assert model.embedding.dtype == torch.float32 and model.blocks[0].mixer.w_qkv.dtype == torch.float32
            assert model.blocks[1].feed_forward.w_down.dtype == torch.float32
            assert model.blocks[1].mixer.w_qkv.dtype == torch.bfloat16
            compare(traces.collect(steps, out, cfg["vocab_size"]), want, TOL[dtype], f"float32-stored tensors, graphs={graphs}")


def test_a_refused_step_reserves_nothing():
    """A step that needs more pages than are free raises before anything runs and keeps no page, whoever calls it."""
    from yalis_b200.engine.engine import Engine, OutOfPages, StepEntry
    d = tiny_model_dir("A", 0.2)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=4, max_slots=3)
    for rid in "abc":
        eng.add_request(rid)
    eng.step([StepEntry("a", [1] * 20, [19])])
    free = eng.free_pages()
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", [2] * 10, []), StepEntry("b", [3] * 16, []), StepEntry("c", [4] * 17, [])])
    assert eng.free_pages() == free and eng.length("b") == 0 and eng.length("a") == 20
    assert eng.step([StepEntry("a", [2] * 10, []), StepEntry("b", [3] * 16, [15])]).shape[0] == 1
    eng.manager.check()


def test_wanted_subset_and_skipped_logits():
    """``want`` may be empty or a subset; rows come back in the order of entries and want."""
    which, dtype, std = "A", "float32", 0.2
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, [20, 12], seed=4)
    want = oracle(which, std, requests)
    a, b = requests["r0"], requests["r1"]
    steps = traces.number([
        {"entries": [{"id": "a", "tokens": a[:10], "want": []}, {"id": "b", "tokens": b[:5], "want": [4, 0]}], "end": []},
        {"entries": [{"id": "b", "tokens": b[5:], "want": [6]}, {"id": "a", "tokens": a[10:], "want": [9, 3]}], "end": ["a", "b"]},
    ])
    out, _ = replay_in_process(d, dtype, 16, steps, 128)
    s0, s1 = out[0].reshape(-1, cfg["vocab_size"]), out[1].reshape(-1, cfg["vocab_size"])
    ref = lambda rid, pos: want[rid][pos]
    for got, exp in ((s0[0], ref("r1", 4)), (s0[1], ref("r1", 0)), (s1[0], ref("r1", 11)), (s1[1], ref("r0", 19)),
                     (s1[2], ref("r0", 13))):
        assert np.abs(got - exp).max() <= 1e-4 * np.abs(exp).max()
    assert s0.shape[0] == 2 and s1.shape[0] == 3


@pytest.mark.parametrize("which", ["C", "D"])
def test_head_sizes_64_and_128_take_the_tma_and_tcgen05_kernels(which):
    """With the head sizes they are built for, bfloat16 steps go to the tcgen05 prompt kernel and to the
    TMA-fed decode kernel that also rotates and stores (and float32 steps to neither)."""
    from yalis_b200.ops import attention as attn_ops
    std = STD["bfloat16"]
    d = tiny_model_dir(which, std)
    cfg = plain.read_config(d)
    requests = make_requests(cfg, lengths_for(which)[2:4], seed=5)
    steps = traces.number(traces.tail_decoded(requests))
    before = dict(attn_ops.LAUNCHED)
    replay_in_process(d, "bfloat16", page_size_of(which), steps, traces.peak_tokens(steps))
    took = {k: attn_ops.LAUNCHED[k] - before.get(k, 0) for k in attn_ops.LAUNCHED}
    layers = cfg["num_hidden_layers"]
    assert took.get("prefill_tcgen05", 0) == layers * len(requests)         # one prompt portion per request
    assert took.get("decode_tma_fused", 0) == layers * 32 * len(requests)     # 32 decoded tokens each, one step each
    assert took.get("generic", 0) == 0 and took.get("mma", 0) == 0
    before = dict(attn_ops.LAUNCHED)
    replay_in_process(d, "float32", page_size_of(which), steps, traces.peak_tokens(steps))
    took = {k: attn_ops.LAUNCHED[k] - before.get(k, 0) for k in attn_ops.LAUNCHED}
    assert took.get("generic", 0) > 0 and sum(v for k, v in took.items() if k != "generic") == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_of_the_8b_shape(dtype):
    """Layer sizes of Llama-3-8B (width 4096, 32 heads over 8 KV heads of 128, inner width 14336) with one
    layer and a small vocabulary, whole and with the tail decoded token by token, against the plain model."""
    from yalis_b200.config.presets import preset
    from yalis_b200.weights.loader import write_random_model
    cfg = preset("Llama-3-8B")
    cfg.update(num_hidden_layers=1, vocab_size=2048, max_position_embeddings=512, bos_token_id=None, eos_token_id=None)
    with tempfile.TemporaryDirectory() as d:
        write_random_model(cfg, d, seed=4, std=0.02)
        pcfg, w = plain.read_config(d), plain.read_weights(d)
        requests = make_requests(pcfg, [150, 40], seed=2)
        want = {rid: plain.forward_logits(t, w, pcfg).numpy() for rid, t in requests.items()}
        del w
        for build, graphs in ((traces.whole, False), (traces.tail_decoded, False), (traces.portions, False), (traces.mixed, False),
                              (traces.tail_decoded, True)):
            steps = traces.number(build(requests))
            out, _ = replay_in_process(d, dtype, 16, steps, traces.peak_tokens(steps), graphs=graphs)
            got = traces.collect(steps, out, pcfg["vocab_size"])
            compare(got, want, TOL[dtype], f"8B layer/{dtype}/{build.__name__}{'/recorded' if graphs else ''}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_of_the_8b_shape_with_its_vocabulary(dtype):
    """Two layers at the full sizes of Llama-3-8B including the vocabulary of 128,256: the output product, the
    two-phase argmax and the sampler at that width run on the engine's path, in both precisions.  A short request
    cut three ways against the plain model, then greedy and sampled tokens through the entry point."""
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig, SamplingParams
    from yalis_b200.config.presets import preset
    from yalis_b200.sampling.sampler import GREEDY
    from yalis_b200.weights.loader import write_random_model
    cfg = preset("Llama-3-8B")
    cfg.update(num_hidden_layers=2, max_position_embeddings=256, bos_token_id=None, eos_token_id=None)
    with tempfile.TemporaryDirectory() as d:
        write_random_model(cfg, d, seed=6, std=0.02)
        pcfg, w = plain.read_config(d), plain.read_weights(d)
        assert pcfg["vocab_size"] == 128256
        requests = make_requests(pcfg, [21, 9], seed=3)
        want = {rid: plain.forward_logits(t, w, pcfg).numpy() for rid, t in requests.items()}
        for build, graphs in ((traces.whole, False), (lambda r: traces.tail_decoded(r, tail=6), True),
                              (lambda r: traces.mixed(r, tail=4), False)):
            steps = traces.number(build(requests))
            out, _ = replay_in_process(d, dtype, 16, steps, traces.peak_tokens(steps), graphs=graphs)
            got = traces.collect(steps, out, pcfg["vocab_size"])
            compare(got, want, TOL[dtype], f"8B two layers/{dtype}")
        eng = LLMEngine(ModelConfig(model_name="two", model_path=d, precision="fp32" if dtype == "float32" else "bf16"),
                        InferenceConfig(max_batch_size=2, max_length_of_generated_sequences=64, page_size=16))
        prompts = list(requests.values())
        hot = SamplingParams(temperature=0.7, top_k=40, top_p=0.9, seed=11)
        results, _ = eng.run(prompts, 5, sampling=[GREEDY, hot], return_logits=True)
        again, _ = eng.run(prompts, 5, sampling=[GREEDY, hot])
        assert [g.tokens for g in results] == [g.tokens for g in again]
        seq = list(prompts[0])
        for k, tok in enumerate(results[0].tokens):          # the greedy row: the plain model's best, or within rounding
            ref = plain.forward_logits(seq, w, pcfg)[-1]
            assert float(ref.max() - ref[tok]) <= (1e-5 if dtype == "float32" else 2e-2) * float(ref.abs().max())
            got = results[0].logits[k].cpu()
            assert float((got - ref).abs().max() / ref.abs().max()) <= TOL[dtype]
            seq.append(tok)
        seq = list(prompts[1])
        near = 48 if dtype == "float32" else 400             # bfloat16 moves ranks among 128,256 close logits
        for tok in results[1].tokens:                        # the sampled row: among the best of the plain model (top_k = 40)
            ref = plain.forward_logits(seq, w, pcfg)[-1]
            assert tok in torch.topk(ref, near).indices.tolist()
            seq.append(tok)
