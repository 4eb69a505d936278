"""Generality of the parts: kinds defined here, outside the package, are registered, built
from a config, given weights, cache and state by the framework, and stepped like built-in
ones, without a change to any file of the package.

* ``running_mean``: a toy mixer with per-request state of its own (a running sum and a
  count), so portions and single tokens must carry state across steps, slots must be
  zeroed on admission and reused slots must not leak.
* a schedule that runs a layer twice, the second time reading the first run's cache.
* ``top1_experts``: a toy feed-forward with routing (float32 router logits, one of three small
  gated MLPs per token).
* ``decay``: a toy position encoding that is no rotation (keys grow and queries shrink by a
  factor per position, so a score decays with distance); the attention part then keeps its
  separate encode-and-store step on every path.
* ``sandwich`` and ``mixer_only``: block arrangements with other places than the built-in one
  (a norm after the mixer; no feed-forward at all), declared by the block kinds themselves.
* ``running_mean_on_device``: the stateful mixer written so that a step of single tokens can
  be recorded and replayed (it reads its slots from the device), run through the entry point
  with recorded steps; the host-loop variant says nothing about recording and is launched.
* an embedding scale and a soft cap on the logits, from the toy architecture's config.
"""

import os
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
import traces
from yalis_b200.config import registry
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from yalis_b200.ops.linear import linear
from yalis_b200.ops.elementwise import rope_kv_write
from yalis_b200.parts.base import (NOT_CAPTURABLE, Block, FeedForward, Mixer, ParamSpec, PositionEncoding, SlotState,
                                   register_part)

pytestmark = pytest.mark.gpu


class RunningMean(Mixer):
    """y_t = W . mean(x_0 .. x_t): keeps [sum (hidden), count] per request."""

    def __init__(self, spec, position=None):
        super().__init__(spec, position)
        self.hidden = spec.params["hidden_size"]
        self.w = None

    def param_specs(self):
        return {"mix": ParamSpec((self.hidden, self.hidden))}

    def load(self, tensors):
        self.w = tensors["mix"].contiguous()

    def cache_request(self):
        return SlotState((self.hidden + 1,), torch.float32)

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        for i, slot in enumerate(ctx.host.slots):
            a, b = ctx.host.q_start[i], ctx.host.q_start[i + 1]
            st = cache.state[slot]
            sums = st[:-1] + torch.cumsum(x[a:b].float(), dim=0)
            counts = st[-1] + torch.arange(1, b - a + 1, device=x.device, dtype=torch.float32)
            out[a:b] = (sums / counts[:, None]).to(x.dtype)
            st[:-1] = sums[-1]
            st[-1] = counts[-1]
        return linear(out, self.w)


class RunningMeanOnDevice(RunningMean):
    """The same mixer, with steps of single tokens done by index operations over the device's slot array,
    so that such a step can be recorded: nothing in it depends on the host's lists."""

    def forward(self, x, ctx, cache):
        if not ctx.decode_only:
            return super().forward(x, ctx, cache)
        slots = ctx.slots.long()                          # padding rows point to the state row that is nobody's
        st = cache.state.index_select(0, slots)
        sums = st[:, :-1] + x.float()
        counts = st[:, -1:] + 1.0
        cache.state.index_copy_(0, slots, torch.cat([sums, counts], dim=1))
        return linear((sums / counts).to(x.dtype), self.w)

    def capture_key(self, host):
        # steps of single tokens launch the same whatever the lengths; steps with portions loop on the host
        return None if host.max_q_len == 1 else NOT_CAPTURABLE


class Sandwich(Block):
    """x += after(mixer(norm_1(x))); x += feed_forward(norm_2(x)): a norm on the mixer's output."""

    slots = {"position": "position", "norm_1": "norm", "mixer": "mixer", "after": "norm", "norm_2": "norm",
             "feed_forward": "feed_forward"}

    def forward(self, stream, ctx, cache):
        y = self.mixer.forward(self.norm_1.forward(stream), ctx, cache)
        if y.dim() == 3:                                  # partial sums of a split product
            y = y.sum(0).to(stream.dtype)
        stream.add(self.after.normalize(y))
        stream.add(self.feed_forward.forward(self.norm_2.forward(stream), ctx))


class MixerOnly(Block):
    """x += mixer(norm_1(x)) and nothing else."""

    slots = {"position": "position", "norm_1": "norm", "mixer": "mixer"}

    def forward(self, stream, ctx, cache):
        stream.add(self.mixer.forward(self.norm_1.forward(stream), ctx, cache))


class Top1Experts(FeedForward):
    """Router logits in float32; every token goes to the expert with the largest one."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.inner, self.n = spec.params["hidden_size"], spec.params["intermediate_size"], spec.params["experts"]

    def param_specs(self):
        specs = {"router": ParamSpec((self.n, self.hidden), keep_float32=True)}
        for j in range(self.n):
            specs[f"gate{j}"] = ParamSpec((self.inner, self.hidden))
            specs[f"up{j}"] = ParamSpec((self.inner, self.hidden))
            specs[f"down{j}"] = ParamSpec((self.hidden, self.inner))
        return specs

    def load(self, tensors):
        self.t = tensors

    def forward(self, x, ctx):
        choice = (x.float() @ self.t["router"].float().T).argmax(dim=-1)
        out = torch.zeros_like(x)
        for j in range(self.n):
            rows = (choice == j).nonzero().flatten()
            if rows.numel():
                h = x[rows]
                a = torch.nn.functional.silu((h @ self.t[f"gate{j}"].T).float()) * (h @ self.t[f"up{j}"].T).float()
                out[rows] = a.to(x.dtype) @ self.t[f"down{j}"].T
        return out


class Decay(PositionEncoding):
    """q_t <- q_t * gamma^(-t), k_t <- k_t * gamma^t: the score of (t, s) is scaled by gamma^(s - t)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.gamma = float(spec.params["gamma"])

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache, dtype=None):
        if qkv.dim() == 3:                       # partial sums of a split product
            qkv = qkv.sum(0)
        qkv = qkv.float()
        nq, nk = num_heads * head_dim, num_kv_heads * head_dim
        grow = torch.pow(torch.tensor(self.gamma, device=qkv.device), ctx.positions.float())[:, None]
        scaled = torch.cat([qkv[:, :nq] / grow, qkv[:, nq:nq + nk] * grow, qkv[:, nq + nk:]], dim=1).to(dtype).contiguous()
        store = cache.writable
        return rope_kv_write(scaled, ctx.positions, ctx.req_of_token, None, cache.k if store else None,
                             cache.v if store else None, ctx.block_tables[cache.group], num_heads, num_kv_heads, head_dim,
                             out_dtype=dtype, bad_flag=ctx.error_flag)


class ToyArchitecture:
    """hidden/heads from its own config.json keys; layer kinds chosen per layer by ``mixers``."""

    @staticmethod
    def parse_config(raw):
        return dict(raw)

    @staticmethod
    def config_to_dict(cfg):
        return dict(cfg)

    @staticmethod
    def model_spec(c):
        h = c["width"]
        norm = PartSpec("rms_norm", {"size": h, "eps": c["eps"]})
        ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": c["inner"]})
        rot = PartSpec("rotary", {"head_dim": c["head_dim"], "theta": 10000.0, "scaling": None})
        attn = PartSpec("paged_attention", {"hidden_size": h, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"],
                                            "head_dim": c["head_dim"]})
        attn_names = {"mixer.q_proj": "attn.q.weight", "mixer.k_proj": "attn.k.weight", "mixer.v_proj": "attn.v.weight",
                      "mixer.o_proj": "attn.o.weight"}
        common = {"feed_forward.gate_proj": "ff.gate.weight", "feed_forward.up_proj": "ff.up.weight",
                  "feed_forward.down_proj": "ff.down.weight", "norm_1.weight": "n1.weight", "norm_2.weight": "n2.weight"}
        routed = PartSpec("top1_experts", {"hidden_size": h, "intermediate_size": c["inner"], "experts": 3})
        routed_names = dict({"feed_forward.router": "ff.router.weight"},
                            **{f"feed_forward.{n}{j}": f"ff.{j}.{n}.weight" for j in range(3) for n in ("gate", "up", "down")})
        decay = PartSpec("decay", {"gamma": 0.98})
        layers = []
        for i, kind in enumerate(c["mixers"]):
            if kind == "attention":
                mixer, names = attn, dict(attn_names, **common)
            elif kind == "window_attention":
                mixer = PartSpec("paged_attention", dict(attn.params, window=c["window"]))
                names = dict(attn_names, **common)
            else:
                mixer, names = PartSpec(kind, {"hidden_size": h}), dict({"mixer.mix": "mean.mix.weight"}, **common)
            ff, pos = ffn, rot
            if c.get("ffs") and c["ffs"][i] == "routed":
                ff = routed
                names = dict({k: v for k, v in names.items() if not k.startswith("feed_forward.")}, **routed_names)
            if c.get("positions") and c["positions"][i] == "decay":
                pos = decay
            parts = {"position": pos, "norm_1": norm, "mixer": mixer, "norm_2": norm, "feed_forward": ff}
            block = c["blocks"][i] if c.get("blocks") else "pre_norm_residual"
            if block == "sandwich":
                parts["after"] = norm
                names = dict(names, **{"after.weight": "after.weight"})
            elif block == "mixer_only":
                parts = {k: parts[k] for k in ("position", "norm_1", "mixer")}
                names = {k: v for k, v in names.items() if k.split(".")[0] in parts}
            layers.append(LayerSpec(PartSpec(block), parts, f"toy.{i}.", names))
        schedule = tuple(ScheduleEntry(l, c) for l, c in c["schedule"])
        return ModelSpec("ToyForCausalLM", h, c["vocab"], c["max_len"], tuple(layers), schedule, norm, "toy.embed.weight",
                         "toy.head.weight", {"weight": "toy.norm.weight"}, embedding_scale=c.get("embed_scale"),
                         logit_softcap=c.get("softcap"))


def setup_module(module):
    register_part("mixer", "running_mean", RunningMean, replace=True)
    register_part("mixer", "running_mean_on_device", RunningMeanOnDevice, replace=True)
    register_part("block", "sandwich", Sandwich, replace=True)
    register_part("block", "mixer_only", MixerOnly, replace=True)
    register_part("feed_forward", "top1_experts", Top1Experts, replace=True)
    register_part("position", "decay", Decay, replace=True)
    registry.register_architecture("ToyForCausalLM", ToyArchitecture, replace=True)


def toy_config(mixers, schedule, window=None, head_dim=8, ffs=None, positions=None, blocks=None, embed_scale=None,
               softcap=None):
    return dict(architectures=["ToyForCausalLM"], width=40, heads=4, kv_heads=2, head_dim=head_dim, inner=56, vocab=97,
                max_len=160, eps=1e-5, mixers=mixers, schedule=schedule, window=window, ffs=ffs, positions=positions,
                blocks=blocks, embed_scale=embed_scale, softcap=softcap, torch_dtype="bfloat16")


def plain_toy(tokens, w, c):
    """Whole-sequence float32 reference of the toy model, written out here."""
    cfg = dict(num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
               rms_norm_eps=c["eps"], rope_theta=10000.0, rope_scaling=None)
    t = len(tokens)
    pos = torch.arange(t)
    x = w["toy.embed.weight"][torch.tensor(tokens)]
    if c.get("embed_scale"):
        x = x * c["embed_scale"]
    kept = {}
    for idx, (layer, cache_of) in enumerate(c["schedule"]):
        p = f"toy.{layer}."
        h = plain.rms_norm(x, w[p + "n1.weight"], c["eps"])
        if c["mixers"][layer] in ("attention", "window_attention"):
            window = c["window"] if c["mixers"][layer] == "window_attention" else None
            nh, g, hs = c["heads"], c["kv_heads"], c["head_dim"]
            if c.get("positions") and c["positions"][layer] == "decay":
                grow = torch.pow(torch.tensor(0.98), pos.float())[:, None, None]
                encode_q, encode_k = (lambda z: z / grow), (lambda z: z * grow)
            else:
                cos, sin = plain.rope_tables(pos, plain.rope_inverse_frequencies(hs, 10000.0, None))
                encode_q = encode_k = lambda z: plain.apply_rope(z, cos, sin)
            q = encode_q((h @ w[p + "attn.q.weight"].T).view(t, nh, hs))
            if cache_of is None:
                k = encode_k((h @ w[p + "attn.k.weight"].T).view(t, g, hs))
                v = (h @ w[p + "attn.v.weight"].T).view(t, g, hs)
                kept[idx] = (k, v)
            else:
                k, v = kept[cache_of]
            y = plain.causal_attention(q, k, v, pos, pos, window=window).reshape(t, nh * hs) @ w[p + "attn.o.weight"].T
        else:
            means = torch.cumsum(h, dim=0) / torch.arange(1, t + 1)[:, None]
            y = means @ w[p + "mean.mix.weight"].T
        block = c["blocks"][layer] if c.get("blocks") else "pre_norm_residual"
        if block == "sandwich":
            y = plain.rms_norm(y, w[p + "after.weight"], c["eps"])
        x = x + y
        if block == "mixer_only":
            continue
        h = plain.rms_norm(x, w[p + "n2.weight"], c["eps"])
        if c.get("ffs") and c["ffs"][layer] == "routed":
            choice = (h @ w[p + "ff.router.weight"].T).argmax(dim=-1)
            y = torch.zeros_like(h)
            for j in range(3):
                rows = (choice == j).nonzero().flatten()
                y[rows] = plain.swiglu(h[rows], w[p + f"ff.{j}.gate.weight"], w[p + f"ff.{j}.up.weight"], w[p + f"ff.{j}.down.weight"])
            x = x + y
        else:
            x = x + plain.swiglu(h, w[p + "ff.gate.weight"], w[p + "ff.up.weight"], w[p + "ff.down.weight"])
    logits = plain.rms_norm(x, w["toy.norm.weight"], c["eps"]) @ w["toy.head.weight"].T
    if c.get("softcap"):
        logits = c["softcap"] * torch.tanh(logits / c["softcap"])
    return logits


def replay_all_cuttings(c, seed, lengths, std, dtype, page_size=16, builds=None, graphs=False):
    """The toy model of config ``c`` cut every way against ``plain_toy``; returns the replayers."""
    from yalis_b200.engine.replay import Replayer
    from yalis_b200.weights.loader import write_random_model
    reps = []
    with tempfile.TemporaryDirectory() as d:
        write_random_model(c, d, seed=seed, std=std)
        w = plain.read_weights(d)
        g = torch.Generator().manual_seed(seed + 1)
        requests = {f"r{i}": torch.randint(0, c["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
        want = {rid: plain_toy(t, w, c).numpy() for rid, t in requests.items()}
        for build in builds or (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = traces.number(build(requests))
            rep = Replayer(d, dtype, traces.peak_tokens(steps), page_size=page_size, max_live=4, graphs=graphs)
            out = {}
            for s in steps:
                r = rep.run_step(s)
                if r is not None:
                    out[s["step"]] = r
            got = traces.collect(steps, out, c["vocab"])
            tol = 1e-4 if dtype == "float32" else 3e-2
            for rid in want:
                err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
                assert err < tol, (build.__name__, rid, err)
            rep.engine.manager.check()
            reps.append(rep)
    return reps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixers, schedule", [
    (["attention", "running_mean", "attention"], [(0, None), (1, None), (2, None)]),
    (["running_mean", "attention"], [(0, None), (1, None), (0, None), (1, 1)]),      # both layers twice; the second
])                                                                                        # attention run reads the first's cache
def test_toy_model_steps_like_a_builtin(dtype, mixers, schedule):
    from yalis_b200.engine.replay import Replayer
    from yalis_b200.weights.loader import write_random_model
    c = toy_config(mixers, schedule)
    std = 0.2 if dtype == "float32" else 0.05
    with tempfile.TemporaryDirectory() as d:
        write_random_model(c, d, seed=2, std=std)
        w = plain.read_weights(d)
        g = torch.Generator().manual_seed(1)
        requests = {f"r{i}": torch.randint(0, c["vocab"], (n,), generator=g).tolist() for i, n in enumerate([50, 7, 90, 33, 64])}
        want = {rid: plain_toy(t, w, c).numpy() for rid, t in requests.items()}
        for build in (traces.whole, traces.portions, traces.mixed):
            steps = traces.number(build(requests))
            rep = Replayer(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4)
            state_entries = [e for e in rep.engine.storage.entries if hasattr(e, "state")]
            assert state_entries and all(e.state.shape[0] == 4 + 1 for e in state_entries)   # a row per slot and nobody's
            out = {}
            for s in steps:
                r = rep.run_step(s)
                if r is not None:
                    out[s["step"]] = r
            got = traces.collect(steps, out, c["vocab"])
            tol = 1e-4 if dtype == "float32" else 3e-2
            for rid in want:
                err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
                assert err < tol, (build.__name__, rid, err)
            rep.engine.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layers_have_pages_of_their_own(dtype):
    """A toy model with one layer over all keys and one over a window of 20: two page groups;
    the window group gives pages back while a request grows, and the logits match the plain
    model at every position (a wrong edge of the window would show at once)."""
    from yalis_b200.engine.replay import Replayer
    from yalis_b200.weights.loader import write_random_model
    c = toy_config(["window_attention", "attention"], [(0, None), (1, None)], window=20, head_dim=16)
    std = 0.2 if dtype == "float32" else 0.05
    with tempfile.TemporaryDirectory() as d:
        write_random_model(c, d, seed=5, std=std)
        w = plain.read_weights(d)
        g = torch.Generator().manual_seed(2)
        requests = {f"r{i}": torch.randint(0, c["vocab"], (n,), generator=g).tolist() for i, n in enumerate([150, 33, 97])}
        want = {rid: plain_toy(t, w, c).numpy() for rid, t in requests.items()}
        for build in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = traces.number(build(requests))
            rep = Replayer(d, dtype, traces.peak_tokens(steps), page_size=8, max_live=4)
            names = sorted(g.name for g in rep.engine.groups)
            assert names == ["kv_all", "kv_window_20"]
            out, low_water = {}, None
            for s in steps:
                r = rep.run_step(s)
                if r is not None:
                    out[s["step"]] = r
                if build is traces.tail_decoded and any(e["id"] == "r0" for e in s["entries"]) and rep.engine.has_request("r0"):
                    slot = rep.engine.slot_of("r0")
                    lo, hi = rep.engine.manager.held_range("kv_window_20", slot)
                    held_all = rep.engine.manager.held_range("kv_all", slot)
                    assert (hi - lo) * 8 <= 20 + 2 * 8 and held_all[0] == 0        # the window group lets go, the other keeps all
                    low_water = lo
            if build is traces.tail_decoded:
                assert low_water and low_water > 10
            got = traces.collect(steps, out, c["vocab"])
            tol = 1e-4 if dtype == "float32" else 3e-2
            for rid in want:
                err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
                assert err < tol, (build.__name__, rid, err)
            rep.engine.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(dtype):
    """A layer with a routed feed-forward and a layer whose position encoding is no rotation (head size
    64: in bfloat16 its decode steps go to the TMA kernel through the separate encode-and-store step),
    cut every way, against the plain model."""
    from yalis_b200.engine.replay import Replayer
    from yalis_b200.ops import attention as attn_ops
    from yalis_b200.weights.loader import write_random_model
    c = toy_config(["attention", "attention"], [(0, None), (1, None)], head_dim=64, ffs=["routed", "dense"],
                   positions=["rotary", "decay"])
    std = 0.2 if dtype == "float32" else 0.05
    with tempfile.TemporaryDirectory() as d:
        write_random_model(c, d, seed=9, std=std)
        w = plain.read_weights(d)
        g = torch.Generator().manual_seed(3)
        requests = {f"r{i}": torch.randint(0, c["vocab"], (n,), generator=g).tolist() for i, n in enumerate([70, 9, 120, 40])}
        want = {rid: plain_toy(t, w, c).numpy() for rid, t in requests.items()}
        before = dict(attn_ops.LAUNCHED)
        for build in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = traces.number(build(requests))
            rep = Replayer(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4)
            out = {}
            for s in steps:
                r = rep.run_step(s)
                if r is not None:
                    out[s["step"]] = r
            got = traces.collect(steps, out, c["vocab"])
            tol = 1e-4 if dtype == "float32" else 3e-2
            for rid in want:
                err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
                assert err < tol, (build.__name__, rid, err)
            rep.engine.manager.check()
        if dtype == "bfloat16":
            took = {k: attn_ops.LAUNCHED[k] - before.get(k, 0) for k in attn_ops.LAUNCHED}
            assert took.get("decode_tma", 0) > 0 and took.get("decode_tma_fused", 0) > 0    # the decay layer, the rotary layer


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_block_arrangements_and_model_hooks(dtype):
    """A layer with a norm after its mixer, a layer without a feed-forward, an embedding scale and a soft cap on
    the logits: block kinds and config keys of this file only, cut every way (the steps of single tokens
    both launched and replayed from recordings), against the plain model."""
    c = toy_config(["attention", "running_mean_on_device", "attention"], [(0, None), (1, None), (2, None)],
                   blocks=["sandwich", "mixer_only", "pre_norm_residual"], embed_scale=3.0, softcap=5.0)
    std = 0.2 if dtype == "float32" else 0.05
    for graphs in (False, True):
        reps = replay_all_cuttings(c, 4, [50, 7, 90, 33, 64], std, dtype, graphs=graphs)
        assert (sum(r.steps_replayed for r in reps) > 0) == graphs
    from yalis_b200.parts.base import build_block
    spec = ToyArchitecture.model_spec(c)
    assert sorted(build_block(spec.layers[1]).parts) == ["mixer", "norm_1", "position"]
    with pytest.raises(ValueError, match="feed_forward"):
        build_block(LayerSpec(PartSpec("pre_norm_residual"), spec.layers[1].parts, "x.", {}))       # a place left empty
    with pytest.raises(ValueError, match="after"):
        build_block(LayerSpec(PartSpec("pre_norm_residual"), spec.layers[0].parts, "x.", {}))       # a place the block lacks


@pytest.mark.parametrize("mixer, recorded", [("running_mean_on_device", True), ("running_mean", False)])
def test_a_stateful_mixer_through_the_entry_point(mixer, recorded):
    """Greedy generation with the toy architecture through ``LLMEngine``: more prompts than slots, so slots are
    reused and their state must start from zero.  The mixer that reads its slots from the device has its decode
    steps recorded and replayed (the first step of a recording runs twice and must not advance the state twice;
    padding rows must not touch a request's state); the one that loops on the host says nothing about recording
    and is launched step by step.  Both must give the plain model's tokens."""
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    from yalis_b200.weights.loader import write_random_model
    c = toy_config(["attention", mixer], [(0, None), (1, None)])
    with tempfile.TemporaryDirectory() as d:
        write_random_model(c, d, seed=6, std=0.3)
        w = plain.read_weights(d)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, c["vocab"], (n,), generator=g).tolist() for n in (9, 30, 4, 17, 1)]
        eng = LLMEngine(ModelConfig(model_name="toy", model_path=d, precision="fp32"),
                        InferenceConfig(max_batch_size=3, max_length_of_generated_sequences=64, temperature=0.0, top_p=0.0,
                                        page_size=16))
        tokens, _ = eng.generate(prompts, tokens_to_generate=12)
        for p, row in zip(prompts, tokens.tolist()):
            seq = list(p)
            for tok in row:
                assert tok == int(plain_toy(seq, w, c)[-1].argmax())
                seq.append(tok)
        replays = sum(r.replays for r in eng.engine._recordings.values())
        assert (replays > 0) == recorded
