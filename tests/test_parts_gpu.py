"""Each part alone, built from a PartSpec at sizes of its own, against the plain functions."""

import pytest
import torch

import plain_llama as plain
from ctx_helper import DEV, make_cache, make_context
from yalis_b200.config.spec import PartSpec
from yalis_b200.parts.base import ResidualStream, make_part, registered

pytestmark = pytest.mark.gpu


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def test_builtin_kinds_are_registered():
    assert "rms_norm" in registered("norm") and "rotary" in registered("position") and "none" in registered("position")
    assert "paged_attention" in registered("mixer") and "swiglu" in registered("feed_forward")
    assert "pre_norm_residual" in registered("block")
    with pytest.raises(ValueError):
        make_part("mixer", PartSpec("no_such_mixer"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    size, eps = 200, 3e-4
    norm = make_part("norm", PartSpec("rms_norm", {"size": size, "eps": eps}))
    assert norm.param_specs()["weight"].shape == (size,) and norm.param_specs()["weight"].keep_float32
    w = rnd(size, seed=1).abs() + 0.1
    norm.load({"weight": w.to(DEV)})
    x, delta = rnd(6, size, seed=2), rnd(6, size, seed=3).to(dtype)
    stream = ResidualStream(x.clone().to(DEV), dtype)
    stream.add(delta.to(DEV))
    y = norm.forward(stream)
    assert stream.pending is None
    torch.testing.assert_close(stream.x.cpu(), x + delta.float())
    torch.testing.assert_close(y.float().cpu(), plain.rms_norm(x + delta.float(), w, eps).to(dtype).float(), **tol(dtype))
    stream.add(delta.to(DEV))
    rows = torch.tensor([5, 2], dtype=torch.int32, device=DEV)
    yr = norm.forward(stream, rows=rows)                     # chosen rows: the delta stays pending
    assert stream.pending is not None
    ref = plain.rms_norm(x + 2 * delta.float(), w, eps)[[5, 2]]
    torch.testing.assert_close(yr.float().cpu(), ref.to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    hidden, inter = 48, 208
    ff = make_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}))
    specs = ff.param_specs()
    assert specs["gate_proj"].shape == (inter, hidden) and specs["down_proj"].shape == (hidden, inter)
    w = {k: rnd(*v.shape, seed=i, scale=0.2).to(dtype) for i, (k, v) in enumerate(specs.items())}
    ff.load({k: v.to(DEV) for k, v in w.items()})
    x = rnd(9, hidden, seed=7).to(dtype)
    ref = plain.swiglu(x.float(), w["gate_proj"].float(), w["up_proj"].float(), w["down_proj"].float())
    torch.testing.assert_close(ff.forward(x.to(DEV), None).float().cpu(), ref.to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("position_kind", ["rotary", "none"])
def test_attention_part_in_two_steps(dtype, position_kind):
    """The mixer alone: a prompt portion, then the rest beside another request's tokens; the
    outputs equal whole-sequence attention of the plain implementation."""
    hidden, nh, g, hs, page = 40, 6, 2, 16, 4
    theta, scaling = 10000.0, dict(factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=16)
    position = make_part("position", PartSpec(position_kind, {"head_dim": hs, "theta": theta, "scaling": scaling}))
    mixer = make_part("mixer", PartSpec("paged_attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": g,
                                                            "head_dim": hs, "window": None, "scale": None}), position=position)
    req = mixer.cache_request()
    assert (req.num_kv_heads, req.head_dim, req.window) == (g, hs, None)
    w = {k: rnd(*v.shape, seed=i, scale=0.3).to(dtype) for i, (k, v) in enumerate(mixer.param_specs().items())}
    mixer.load({k: v.to(DEV) for k, v in w.items()})
    xa, xb = rnd(21, hidden, seed=11).to(dtype), rnd(6, hidden, seed=12).to(dtype)

    def reference(x):
        t = x.shape[0]
        pos = torch.arange(t)
        xf = x.float()
        q = (xf @ w["q_proj"].float().T).to(dtype).float().view(t, nh, hs)
        k = (xf @ w["k_proj"].float().T).to(dtype).float().view(t, g, hs)
        v = (xf @ w["v_proj"].float().T).to(dtype).float().view(t, g, hs)
        if position_kind == "rotary":
            cos, sin = plain.rope_tables(pos, plain.rope_inverse_frequencies(hs, theta, scaling))
            q, k = plain.apply_rope(q, cos, sin).to(dtype).float(), plain.apply_rope(k, cos, sin).to(dtype).float()
        y = plain.causal_attention(q, k, v, pos, pos).to(dtype).float()
        return (y.reshape(t, nh * hs) @ w["o_proj"].float().T)

    # step 1: 13 tokens of a. step 2: the other 8 of a beside all 6 of b (pages shared in one pool).
    ctx1, _ = make_context([13], [0], page)
    ctx2, n_pages = make_context([8, 6], [13, 0], page)
    cache = make_cache(n_pages, g, page, hs, dtype)
    # both steps must see the same pages for request a: reuse step 2's table for step 1
    ctx1.block_tables["kv_all"] = ctx2.block_tables["kv_all"][:1].contiguous()
    y1 = mixer.forward(xa[:13].to(DEV), ctx1, cache)
    y2 = mixer.forward(torch.cat([xa[13:], xb]).to(DEV), ctx2, cache)
    got_a = torch.cat([y1, y2[:8]]).float().cpu()
    torch.testing.assert_close(got_a, reference(xa).to(dtype).float(), **tol(dtype))
    torch.testing.assert_close(y2[8:].float().cpu(), reference(xb).to(dtype).float(), **tol(dtype))
    assert int(ctx2.error_flag) == 0


def test_block_part_matches_plain_block():
    """The pre-norm residual arrangement with all four parts, float32."""
    hidden, nh, g, hs, inter, eps, page = 32, 4, 4, 8, 72, 1e-5, 8
    norm = PartSpec("rms_norm", {"size": hidden, "eps": eps})
    position = make_part("position", PartSpec("rotary", {"head_dim": hs, "theta": 10000.0, "scaling": None}))
    mixer = make_part("mixer", PartSpec("paged_attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": g,
                                                            "head_dim": hs}), position=position)
    ff = make_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}))
    n1, n2 = make_part("norm", norm), make_part("norm", norm)
    block = make_part("block", PartSpec("pre_norm_residual"),
                      parts={"position": position, "norm_1": n1, "mixer": mixer, "norm_2": n2, "feed_forward": ff})
    names = {"q_proj": "self_attn.q_proj.weight", "k_proj": "self_attn.k_proj.weight", "v_proj": "self_attn.v_proj.weight",
             "o_proj": "self_attn.o_proj.weight", "gate_proj": "mlp.gate_proj.weight", "up_proj": "mlp.up_proj.weight",
             "down_proj": "mlp.down_proj.weight"}
    w = {}
    for i, part in enumerate((mixer, ff)):
        t = {k: rnd(*v.shape, seed=10 * i + j, scale=0.3) for j, (k, v) in enumerate(part.param_specs().items())}
        part.load({k: v.to(DEV) for k, v in t.items()})
        w.update({"model.layers.0." + names[k]: v for k, v in t.items()})
    w1, w2 = rnd(hidden, seed=50).abs() + 0.5, rnd(hidden, seed=51).abs() + 0.5
    n1.load({"weight": w1.to(DEV)}); n2.load({"weight": w2.to(DEV)})
    w["model.layers.0.input_layernorm.weight"], w["model.layers.0.post_attention_layernorm.weight"] = w1, w2
    cfg = dict(num_attention_heads=nh, num_key_value_heads=g, head_dim=hs, rms_norm_eps=eps, rope_theta=10000.0, rope_scaling=None)
    x = rnd(11, hidden, seed=60)
    ctx, n_pages = make_context([11], [0], page)
    stream = ResidualStream(x.clone().to(DEV), torch.float32)
    block.forward(stream, ctx, make_cache(n_pages, g, page, hs, torch.float32))
    stream.flush()
    torch.testing.assert_close(stream.x.cpu(), plain.block(x, w, 0, cfg, torch.arange(11)), rtol=1e-4, atol=1e-5)
