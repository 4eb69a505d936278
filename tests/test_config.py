"""Configuration: config.json keys -> typed config, defaults, refusals, registry, presets."""

import json
import os

import pytest

from yalis_b200.config import registry
from yalis_b200.config.presets import PRESETS, preset
from yalis_b200.config.registry import ConfigError, parse_config
from yalis_b200.config.runtime import InferenceConfig, ModelConfig
from yalis_b200.config.spec import ModelSpec, ScheduleEntry
from yalis_b200.models.llama import LlamaConfig, RopeScaling


def test_llama_8b_preset_parses_to_typed_config():
    arch, cfg = parse_config(preset("Llama-3-8B"))
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (4096, 32, 32, 8)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (128, 14336, 128256)
    assert cfg.rope_theta == 500000.0 and cfg.rope_scaling is None and not cfg.tie_word_embeddings
    assert cfg.parameter_count() == 8030261248
    spec = arch.model_spec(cfg)
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 32 and len(spec.schedule) == 32
    assert spec.head_name == "lm_head.weight"


def test_defaults_and_derivations():
    raw = dict(architectures=["LlamaForCausalLM"], hidden_size=96, num_hidden_layers=1, num_attention_heads=3,
               intermediate_size=10, vocab_size=7, max_position_embeddings=5)
    _, cfg = parse_config(raw)
    assert cfg.num_key_value_heads == 3          # defaults to the head count
    assert cfg.head_dim == 32                    # hidden / heads
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0


def test_tiny_presets_differ_in_every_size_and_option():
    _, a = parse_config(preset("tiny-A"))
    _, b = parse_config(preset("tiny-B"))
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta",
                "tie_word_embeddings"):
        assert getattr(a, key) != getattr(b, key), key
    assert a.rope_scaling is None and isinstance(b.rope_scaling, RopeScaling)
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads


@pytest.mark.parametrize("patch, fragment", [
    (dict(architectures=["NoSuchModel"]), "not a supported architecture"),
    (dict(architectures=None), "architectures"),
    (dict(hidden_size=None), "hidden_size"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "yarn"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=8.0)), "together"),
    (dict(intermediate_size=None), "intermediate_size"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
])
def test_refusals(patch, fragment):
    raw = preset("tiny-A")
    raw.update(patch)
    with pytest.raises(ConfigError) as e:
        parse_config(raw)
    assert fragment in str(e.value)


def test_round_trip_through_config_json(tmp_path):
    arch, cfg = parse_config(preset("tiny-B"))
    d = arch.config_to_dict(cfg)
    (tmp_path / "config.json").write_text(json.dumps(d))
    arch2, cfg2 = registry.load_config(str(tmp_path))
    assert cfg2 == cfg and arch2 is arch
    with pytest.raises(FileNotFoundError):
        registry.load_config(str(tmp_path / "nowhere"))


def test_reference_preset_names_exist():
    for name in ("Llama-3-8B", "Llama-3-8B-Instruct", "Llama-3.1-8B", "Llama-3.2-1B", "Llama-3.2-3B",
                 "Llama-3.3-70B-Instruct", "Llama-3.1-405B"):
        assert name in PRESETS
    assert preset("meta-llama/Meta-Llama-3-8B")["hidden_size"] == 4096
    with pytest.raises(ValueError):
        preset("Llama-9")


def test_registering_another_architecture():
    class Toy:
        @staticmethod
        def parse_config(raw):
            return raw

        @staticmethod
        def model_spec(cfg):
            raise NotImplementedError

        @staticmethod
        def config_to_dict(cfg):
            return dict(cfg)

    registry.register_architecture("ToyConfigOnly", Toy, replace=True)
    arch, cfg = parse_config(dict(architectures=["ToyConfigOnly"], x=1))
    assert arch is Toy and cfg["x"] == 1
    with pytest.raises(ValueError):
        registry.register_architecture("ToyConfigOnly", Toy)
    with pytest.raises(TypeError):
        registry.register_architecture("Broken", object())


def test_schedule_validation():
    arch, cfg = parse_config(preset("tiny-A"))
    spec = arch.model_spec(cfg)
    kw = {f: getattr(spec, f) for f in spec.__dataclass_fields__}
    kw["schedule"] = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0))   # a layer twice, sharing a cache
    ModelSpec(**kw)
    kw["schedule"] = (ScheduleEntry(0, cache_of=1), ScheduleEntry(1))
    with pytest.raises(ValueError):
        ModelSpec(**kw)
    kw["schedule"] = (ScheduleEntry(5),)
    with pytest.raises(ValueError):
        ModelSpec(**kw)


def test_model_and_inference_config_rules(tmp_path):
    with pytest.raises(ValueError):
        ModelConfig(model_name="x", model_path=str(tmp_path / "missing"))
    with pytest.raises(ValueError):
        ModelConfig(model_name="x", model_path=str(tmp_path), precision="fp16")
    assert ModelConfig(model_name="x", model_path=str(tmp_path), precision="fp32").model_path == str(tmp_path)
    assert ModelConfig(model_name="tiny-A", random_weights=True).random_weights
    ic = InferenceConfig(max_batch_size=3, max_length_of_generated_sequences=77, top_k=5, top_p=0.5, temperature=0.0)
    assert (ic.max_batch_size, ic.max_length, ic.top_k, ic.top_p, ic.temperature) == (3, 77, 5, 0.5, 0.0)
    for bad in (dict(max_batch_size=0), dict(max_length_of_generated_sequences=0), dict(temperature=-1.0),
                dict(top_k=0), dict(top_p=1.5), dict(attention_backend="flash"), dict(attention_backend="sdpa"),
                dict(use_paged_kv_caching=False), dict(page_size=0), dict(num_pages=4, cache_tokens=64),
                dict(memory_fraction=1.5), dict(prefill_chunk=0)):
        with pytest.raises(ValueError):
            InferenceConfig(**bad)
    for gone in (dict(tp_dims=(1, 1, 1)), dict(symmetric_allreduce_strategy=None), dict(prestore_kv_cache=True),
                 dict(use_intra_head_parallelism=False)):
        with pytest.raises(TypeError):          # options for several GPUs do not exist here
            InferenceConfig(**gone)
    assert InferenceConfig(attention_backend="paged").page_size == 64


def test_engine_config_is_typed_and_sizes_the_pool():
    from yalis_b200 import EngineConfig
    ec = EngineConfig(dtype="bf16", page_size=16, max_slots=8, max_context=1000)
    assert ec.dtype == "bfloat16"
    with pytest.raises(Exception):
        ec.page_size = 32                                            # frozen
    assert ec.with_(page_size=32).page_size == 32 and ec.page_size == 16
    assert ec.pool_pages(4096) == 8 * 63                            # every slot at its longest
    assert EngineConfig(page_size=16, num_pages=11).pool_pages(4096) == 11
    assert EngineConfig(page_size=16, cache_tokens=100).pool_pages(4096) == 7
    by_memory = EngineConfig(page_size=16, max_slots=4, max_context=4096, memory_fraction=0.5)
    assert by_memory.pool_pages(8192, free_bytes=1 << 20, bytes_per_page=4096) == 128
    assert by_memory.pool_pages(8192, free_bytes=1 << 40, bytes_per_page=4096) == 4 * 256     # never more than can be mapped
    with pytest.raises(ValueError):
        by_memory.pool_pages(8192, free_bytes=1000, bytes_per_page=4096)
    for bad in (dict(dtype="fp16"), dict(dtype="int8"), dict(page_size=0), dict(max_slots=-1), dict(num_pages=0),
                dict(num_pages=3, memory_fraction=0.5), dict(memory_fraction=0.0), dict(max_tokens_per_step=True)):
        with pytest.raises(ValueError):
            EngineConfig(**bad)
    ic = InferenceConfig(max_batch_size=3, max_length_of_generated_sequences=77, page_size=8, prefill_chunk=24)
    got = ic.engine_config("fp32")
    assert (got.dtype, got.max_slots, got.max_context, got.cache_tokens, got.page_size, got.prefill_chunk) == \
        ("float32", 3, 77, 3 * 77, 8, 24)
