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
from yalis_b200.parts.base import FeedForward, Mixer, ParamSpec, PositionEncoding, SlotState, register_part

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
                mixer, names = PartSpec("running_mean", {"hidden_size": h}), dict({"mixer.mix": "mean.mix.weight"}, **common)
            ff, pos = ffn, rot
            if c.get("ffs") and c["ffs"][i] == "routed":
                ff = routed
                names = dict({k: v for k, v in names.items() if not k.startswith("feed_forward.")}, **routed_names)
            if c.get("positions") and c["positions"][i] == "decay":
                pos = decay
            layers.append(LayerSpec(PartSpec("pre_norm_residual"), mixer, ff, norm, norm, pos, f"toy.{i}.", names))
        schedule = tuple(ScheduleEntry(l, c) for l, c in c["schedule"])
        return ModelSpec("ToyForCausalLM", h, c["vocab"], c["max_len"], tuple(layers), schedule, norm, "toy.embed.weight",
                         "toy.head.weight", {"weight": "toy.norm.weight"})


def setup_module(module):
    register_part("mixer", "running_mean", RunningMean, replace=True)
    register_part("feed_forward", "top1_experts", Top1Experts, replace=True)
    register_part("position", "decay", Decay, replace=True)
    registry.register_architecture("ToyForCausalLM", ToyArchitecture, replace=True)


def toy_config(mixers, schedule, window=None, head_dim=8, ffs=None, positions=None):
    return dict(architectures=["ToyForCausalLM"], width=40, heads=4, kv_heads=2, head_dim=head_dim, inner=56, vocab=97,
                max_len=160, eps=1e-5, mixers=mixers, schedule=schedule, window=window, ffs=ffs, positions=positions,
                torch_dtype="bfloat16")


def plain_toy(tokens, w, c):
    """Whole-sequence float32 reference of the toy model, written out here."""
    cfg = dict(num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
               rms_norm_eps=c["eps"], rope_theta=10000.0, rope_scaling=None)
    t = len(tokens)
    pos = torch.arange(t)
    x = w["toy.embed.weight"][torch.tensor(tokens)]
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
        x = x + y
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
    return plain.rms_norm(x, w["toy.norm.weight"], c["eps"]) @ w["toy.head.weight"].T


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
            assert state_entries and all(e.state.shape[0] == 4 for e in state_entries)     # one row per slot
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
