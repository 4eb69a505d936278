"""The Llama 3 dense decoder as an architecture of this engine.

What the reference computes for its ``Llama-3*`` entries
(yalis/external/config.py:755-951: RMSNorm, LLaMAMLP, no parallel residual, no
biases, full rotary, grouped-query attention) is described here as data: a
typed configuration read from the keys of a Hugging Face ``config.json``, and a
``ModelSpec`` that lists, layer by layer, the parts and the names of their
tensors.  No tensor is touched in this file.
"""

from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional

from yalis_b200.config.registry import ConfigError, register_architecture
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule

ARCHITECTURE_NAME = "LlamaForCausalLM"


@dataclass(frozen=True)
class RopeScaling:
    """The llama3 frequency smoothing (yalis/external/model.py:790-807); all
    four numbers come together or not at all (:211-252)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    torch_dtype: str
    bos_token_id: Optional[int]
    eos_token_id: Optional[int]

    @property
    def architecture(self) -> str:
        return ARCHITECTURE_NAME

    def parameter_count(self) -> int:
        c = self
        per_layer = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                     + c.num_attention_heads * c.head_dim * c.hidden_size
                     + 3 * c.hidden_size * c.intermediate_size + 2 * c.hidden_size)
        n = c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size + c.hidden_size
        if not c.tie_word_embeddings:
            n += c.vocab_size * c.hidden_size
        return n


def _require(raw: Dict[str, Any], key: str, kind=int):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks `{key}`")
    v = raw[key]
    if kind is int and (isinstance(v, bool) or not isinstance(v, int) or v <= 0):
        raise ConfigError(f"`{key}` must be a positive integer, got {v!r}")
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or v <= 0:
            raise ConfigError(f"`{key}` must be a positive number, got {v!r}")
        v = float(v)
    return v


def _parse_rope_scaling(raw: Optional[Dict[str, Any]]) -> Optional[RopeScaling]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"`rope_scaling` must be an object, got {raw!r}")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        if any(k in raw for k in ("factor", "low_freq_factor", "high_freq_factor")) and kind is None:
            raise ConfigError("`rope_scaling` has parameters but no `rope_type`")
        return None
    if kind != "llama3":
        raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")
    needed = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
    missing = [k for k in needed if k not in raw]
    if missing:
        # the reference's rule: all adjusted RoPE parameters come together (yalis/external/model.py:240-252)
        raise ConfigError("rope_scaling lacks " + ", ".join(missing) + "; all llama3 parameters must be given together")
    s = RopeScaling(float(raw["factor"]), float(raw["low_freq_factor"]), float(raw["high_freq_factor"]),
                    int(raw["original_max_position_embeddings"]))
    if s.high_freq_factor == s.low_freq_factor:
        raise ConfigError("rope_scaling: high_freq_factor equals low_freq_factor")
    if s.factor <= 0 or s.original_max_position_embeddings <= 0:
        raise ConfigError("rope_scaling: factor and original_max_position_embeddings must be positive")
    return s


class LlamaArchitecture:
    name = ARCHITECTURE_NAME

    @staticmethod
    def parse_config(raw: Dict[str, Any]) -> LlamaConfig:
        hidden = _require(raw, "hidden_size")
        heads = _require(raw, "num_attention_heads")
        # defaults and derivations of yalis/external/config.py:104-135
        kv_heads = raw.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        if not isinstance(kv_heads, int) or kv_heads <= 0 or heads % kv_heads != 0:
            raise ConfigError(f"`num_key_value_heads` ({kv_heads!r}) must divide `num_attention_heads` ({heads})")
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError("`hidden_size` is not a multiple of `num_attention_heads` and `head_dim` is not given")
            head_dim = hidden // heads
        if not isinstance(head_dim, int) or head_dim <= 0:
            raise ConfigError(f"`head_dim` must be a positive integer, got {head_dim!r}")
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key):
                raise ConfigError(f"`{key}` = true is not supported (the Llama 3 layers have no bias)")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"`hidden_act` = {act!r} is not supported (SwiGLU uses silu)")
        eos = raw.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        eps = raw.get("rms_norm_eps", 1e-5)           # yalis/external/config.py:38
        theta = raw.get("rope_theta", 10000.0)        # yalis/external/config.py:78
        if not isinstance(eps, (int, float)) or eps <= 0:
            raise ConfigError(f"`rms_norm_eps` must be positive, got {eps!r}")
        if not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"`rope_theta` must be positive, got {theta!r}")
        return LlamaConfig(
            hidden_size=hidden,
            num_hidden_layers=_require(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_require(raw, "intermediate_size"),   # mandatory: config.py:128-133
            vocab_size=_require(raw, "vocab_size"),
            max_position_embeddings=_require(raw, "max_position_embeddings"),
            rms_norm_eps=float(eps),
            rope_theta=float(theta),
            rope_scaling=_parse_rope_scaling(raw.get("rope_scaling")),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
            bos_token_id=raw.get("bos_token_id"),
            eos_token_id=eos,
        )

    @staticmethod
    def config_to_dict(c: LlamaConfig) -> Dict[str, Any]:
        d = asdict(c)
        d["architectures"] = [ARCHITECTURE_NAME]
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["mlp_bias"] = False
        if c.rope_scaling is not None:
            d["rope_scaling"] = dict(asdict(c.rope_scaling), rope_type="llama3")
        return d

    @staticmethod
    def model_spec(c: LlamaConfig) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps})
        scaling = None if c.rope_scaling is None else asdict(c.rope_scaling)
        position = PartSpec("rotary", {"head_dim": c.head_dim, "theta": c.rope_theta, "scaling": scaling})
        mixer = PartSpec("paged_attention", {
            "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
            "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "window": None, "scale": None,
        })
        ffn = PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size})
        names = {
            "mixer.q_proj": "self_attn.q_proj.weight",
            "mixer.k_proj": "self_attn.k_proj.weight",
            "mixer.v_proj": "self_attn.v_proj.weight",
            "mixer.o_proj": "self_attn.o_proj.weight",
            "feed_forward.gate_proj": "mlp.gate_proj.weight",
            "feed_forward.up_proj": "mlp.up_proj.weight",
            "feed_forward.down_proj": "mlp.down_proj.weight",
            "norm_1.weight": "input_layernorm.weight",
            "norm_2.weight": "post_attention_layernorm.weight",
        }
        layers = tuple(
            LayerSpec(block=PartSpec("pre_norm_residual"),
                      parts={"position": position, "norm_1": norm, "mixer": mixer, "norm_2": norm, "feed_forward": ffn},
                      weight_prefix=f"model.layers.{i}.", weight_names=names)
            for i in range(c.num_hidden_layers))
        return ModelSpec(
            architecture=ARCHITECTURE_NAME,
            hidden_size=c.hidden_size,
            vocab_size=c.vocab_size,
            max_position=c.max_position_embeddings,
            layers=layers,
            schedule=default_schedule(c.num_hidden_layers),
            final_norm=norm,
            embedding_name="model.embed_tokens.weight",
            head_name=None if c.tie_word_embeddings else "lm_head.weight",
            final_norm_names={"weight": "model.norm.weight"},
            eos_token_id=c.eos_token_id,
            bos_token_id=c.bos_token_id,
        )


register_architecture(ARCHITECTURE_NAME, LlamaArchitecture, replace=True)
