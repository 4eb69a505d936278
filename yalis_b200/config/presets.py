"""Named configurations: the dictionaries a ``config.json`` would hold.

The reference chooses a model by name from a registry of size dictionaries
(``Llama-3-8B``, ``Llama-3.2-1B`` ... yalis/external/config.py:755-951, with an
``-Instruct`` twin of each).  The same names are kept here as data for the
random-weights mode and the benchmark; a real checkpoint is run from its own
``config.json`` and never needs this file.  The two ``tiny-*`` entries are the
small test shapes (they differ in every size and option).
"""

from __future__ import annotations

from copy import deepcopy
from typing import Any, Dict

_LLAMA3_SCALING_8 = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                         original_max_position_embeddings=8192)
_LLAMA3_SCALING_32 = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)


def _llama(hidden, layers, heads, kv_heads, inter, max_pos, scaling=None, tied=False, head_dim=None,
           vocab=128256, theta=500000.0, eps=1e-5) -> Dict[str, Any]:
    return dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim or hidden // heads,
        intermediate_size=inter, vocab_size=vocab, max_position_embeddings=max_pos, rms_norm_eps=eps,
        rope_theta=theta, rope_scaling=scaling, tie_word_embeddings=tied, hidden_act="silu",
        attention_bias=False, mlp_bias=False, torch_dtype="bfloat16", bos_token_id=128000, eos_token_id=128001,
    )


_BASE: Dict[str, Dict[str, Any]] = {
    "Llama-3-8B": _llama(4096, 32, 32, 8, 14336, 8192),
    "Llama-3.1-8B": _llama(4096, 32, 32, 8, 14336, 131072, _LLAMA3_SCALING_8),
    "Llama-3-70B": _llama(8192, 80, 64, 8, 28672, 8192),
    "Llama-3.1-70B": _llama(8192, 80, 64, 8, 28672, 131072, _LLAMA3_SCALING_8),
    "Llama-3.1-405B": _llama(16384, 126, 128, 8, 53248, 131072, _LLAMA3_SCALING_8),
    "Llama-3.2-1B": _llama(2048, 16, 32, 8, 8192, 131072, _LLAMA3_SCALING_32, tied=True),
    "Llama-3.2-3B": _llama(3072, 28, 24, 8, 8192, 131072, _LLAMA3_SCALING_32, tied=True),
}

PRESETS: Dict[str, Dict[str, Any]] = {}
for _name, _cfg in _BASE.items():
    PRESETS[_name] = _cfg
    PRESETS[_name + "-Instruct"] = _cfg
PRESETS["Llama-3.3-70B-Instruct"] = _BASE["Llama-3.1-70B"]

# Test shapes. A: GQA x2, no scaling, untied. B: MQA x3 with an odd head count, llama3 scaling whose
# three regimes all occur among 16 frequencies, tied, other eps/theta.
PRESETS["tiny-A"] = dict(
    _llama(64, 2, 4, 2, 176, 128, None, tied=False, head_dim=16, vocab=256, theta=10000.0, eps=1e-5),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
PRESETS["tiny-B"] = dict(
    _llama(96, 3, 3, 1, 256, 256,
           dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                original_max_position_embeddings=32),
           tied=True, head_dim=32, vocab=512, theta=500000.0, eps=1e-6),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
# Head sizes 64 and 128: the shapes that the TMA- and tcgen05-based attention kernels are built for.
PRESETS["tiny-C"] = dict(
    _llama(136, 2, 4, 2, 208, 512,
           dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                original_max_position_embeddings=64),
           tied=False, head_dim=64, vocab=320, theta=10000.0, eps=1e-5),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
PRESETS["tiny-D"] = dict(
    _llama(192, 2, 2, 1, 320, 512, None, tied=True, head_dim=128, vocab=272, theta=500000.0, eps=1e-6),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)


def preset(name: str) -> Dict[str, Any]:
    """A fresh copy of the named configuration dictionary."""
    for key in (name, name.split("/")[-1], name.split("/")[-1].replace("Meta-", "")):
        if key in PRESETS:
            return deepcopy(PRESETS[key])
    raise ValueError(f"{name!r} is not a supported config name (known: {', '.join(sorted(PRESETS))})")
