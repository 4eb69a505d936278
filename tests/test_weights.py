"""Weights: the safetensors container, the name/shape check with its one error, random weights."""

import json
import os

import pytest
import torch

from yalis_b200.config.presets import preset
from yalis_b200.config.registry import parse_config
from yalis_b200.engine.model import Model
from yalis_b200.parts.base import ParamSpec
from yalis_b200.weights.loader import WeightError, random_tensor, target_dtype, validate, write_random_model
from yalis_b200.weights.safetensors_io import Checkpoint, write_safetensors


def _model(name):
    arch, cfg = parse_config(preset(name))
    return Model(arch.model_spec(cfg))


def test_container_round_trip_and_official_reader(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
               "d": torch.zeros(0, 4)}
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), tensors)
    with Checkpoint(str(tmp_path)) as ck:
        assert set(ck.names()) == set(tensors)
        for n, t in tensors.items():
            dtype, shape = ck.info(n)
            assert dtype == t.dtype and shape == tuple(t.shape)
            assert torch.equal(ck.get(n).clone(), t)
    from safetensors import safe_open
    with safe_open(str(path), framework="pt") as f:
        assert torch.equal(f.get_tensor("b"), tensors["b"])


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"x": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"y": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    with Checkpoint(str(tmp_path)) as ck:
        assert sorted(ck.names()) == ["x", "y"] and ck.get("y").shape == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "gone.safetensors"}}))
    with pytest.raises(FileNotFoundError):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({}))
    with pytest.raises(RuntimeError):
        Checkpoint(str(tmp_path))


def test_missing_folder_and_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        Checkpoint(str(tmp_path / "none"))
    with pytest.raises(FileNotFoundError):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x00\x01")
    with pytest.raises(RuntimeError):
        Checkpoint(str(tmp_path))


def test_expected_tensors_follow_the_config():
    a, b = _model("tiny-A").expected_tensors(), _model("tiny-B").expected_tensors()
    assert a["model.layers.1.self_attn.k_proj.weight"].shape == (2 * 16, 64)
    assert a["lm_head.weight"].shape == (256, 64) and "lm_head.weight" not in b      # B is tied
    assert b["model.layers.2.mlp.down_proj.weight"].shape == (96, 256)
    assert b["model.norm.weight"].keep_float32 and b["model.norm.weight"].init == "ones"
    assert len(a) == 1 + 2 * 9 + 1 + 1 and len(b) == 1 + 3 * 9 + 1


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(preset("tiny-A"), str(tmp_path / "m"), seed=0)
    with Checkpoint(d) as ck:
        tensors = {n: ck.get(n).clone() for n in ck.names()}
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(3, 3, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # tolerated, as in the reference
    tensors["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with Checkpoint(d) as ck, pytest.raises(WeightError) as e:
        validate(_model("tiny-A").expected_tensors(), ck)
    msg = str(e.value)
    assert "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.7.extra.weight" in msg and "inv_freq" not in msg
    assert "model.layers.1.self_attn.q_proj.weight expected [64, 64], found [3, 3]" in msg
    assert "model.embed_tokens.weight" in msg and "floating-point" in msg
    assert e.value.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]


def test_random_weights_are_seeded_per_tensor(tmp_path):
    d1 = write_random_model(preset("tiny-A"), str(tmp_path / "a"), seed=3)
    d2 = write_random_model(preset("tiny-A"), str(tmp_path / "b"), seed=3)
    d3 = write_random_model(preset("tiny-A"), str(tmp_path / "c"), seed=4)
    with Checkpoint(d1) as c1, Checkpoint(d2) as c2, Checkpoint(d3) as c3:
        name = "model.layers.1.mlp.gate_proj.weight"
        assert torch.equal(c1.get(name).clone(), c2.get(name).clone())
        assert not torch.equal(c1.get(name).clone(), c3.get(name).clone())
        w = c1.get(name).float()
        assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
        assert torch.all(c1.get("model.norm.weight").float() == 1)
        assert c1.info(name)[0] == torch.bfloat16
    cfg = json.load(open(os.path.join(d1, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 64
    # a tensor's values depend on its name and the seed only
    ps = ParamSpec((4, 4))
    assert torch.equal(random_tensor("x", ps, 1), random_tensor("x", ps, 1))
    assert not torch.equal(random_tensor("x", ps, 1), random_tensor("y", ps, 1))


def test_dtype_policy():
    assert target_dtype(ParamSpec((1,)), torch.bfloat16) == torch.bfloat16
    assert target_dtype(ParamSpec((1,)), torch.float32) == torch.float32
    assert target_dtype(ParamSpec((1,), keep_float32=True), torch.bfloat16) == torch.float32
    assert target_dtype(ParamSpec((1,), integer=True), torch.bfloat16) == torch.int32
    # what the checkpoint stores in 32 (or 64) bits stays float32; 16-bit storage follows the engine
    assert target_dtype(ParamSpec((1,)), torch.bfloat16, stored=torch.float32) == torch.float32
    assert target_dtype(ParamSpec((1,)), torch.bfloat16, stored=torch.float64) == torch.float32
    assert target_dtype(ParamSpec((1,)), torch.bfloat16, stored=torch.float16) == torch.bfloat16
    assert target_dtype(ParamSpec((1,)), torch.float32, stored=torch.bfloat16) == torch.float32
    assert target_dtype(ParamSpec((1,), integer=True), torch.bfloat16, stored=torch.int64) == torch.int32


def test_a_tensor_stored_in_32_bit_stays_so(tmp_path):
    """A bfloat16 checkpoint in which one projection and the output matrix are stored in float32: loaded for the
    bfloat16 engine they stay float32 (and the matrix fused from a float32 and two bfloat16 parts is float32)."""
    from yalis_b200.weights.loader import load_weights
    d = write_random_model(preset("tiny-A"), str(tmp_path / "m"), seed=3)
    with Checkpoint(d) as ck:
        tensors = {n: ck.get(n).clone() for n in ck.names()}
    wide = [n for n in tensors if n.endswith("layers.0.self_attn.q_proj.weight") or n.endswith("layers.1.mlp.down_proj.weight")]
    assert len(wide) == 2
    for n in wide:
        tensors[n] = tensors[n].float()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    model = _model("tiny-A")
    load_weights(model, d, "cpu", torch.bfloat16)
    assert model.blocks[0].mixer.w_qkv.dtype == torch.float32 and model.blocks[1].mixer.w_qkv.dtype == torch.bfloat16
    assert model.blocks[1].feed_forward.w_down.dtype == torch.float32 and model.blocks[0].feed_forward.w_down.dtype == torch.bfloat16
    assert model.embedding.dtype == torch.bfloat16
