"""Weights from safetensors by tensor name, and the seeded random-weights mode.

Loading: the model names the tensors it expects with their shapes
(``Model.expected_tensors``); the folder is checked against that list before a
byte is copied, and one ``WeightError`` reports every missing tensor, every
unexpected tensor and every wrong shape together.  (The reference loads with
``strict=True`` and fails on the first kind of mismatch,
yalis/model_loading.py:201-249.)

dtype policy: floating tensors are held in the engine's dtype (bfloat16, or
float32 on the 32-bit path); a parameter its part marks ``keep_float32`` (norm
scales) is held in float32; integer tables are held as int32; and a tensor that
the checkpoint stores in 32 or 64-bit floating point stays float32 whatever the
engine's dtype (whoever stored a matrix that wide in a 16-bit checkpoint meant
it; the products that read it then run on the exact float32 kernels).

Random weights: every matrix and the embedding ~ N(0, 0.02), norm scales 1
(yalis/external/model.py:113-120), from a generator seeded per tensor by
(seed, tensor name), so a tensor's values do not depend on which other tensors
exist.  ``write_random_model`` writes a complete model folder (config.json +
model.safetensors) that loads like any checkpoint.
"""

from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Optional

import torch

from yalis_b200.config.registry import parse_config
from yalis_b200.parts.base import ParamSpec
from .safetensors_io import Checkpoint, write_safetensors

IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)   # dropped by the reference's converter too (convert_hf_checkpoint.py:713)
INIT_STD = 0.02

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


class WeightError(RuntimeError):
    """The model folder does not hold the tensors the model needs."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, wrong_kind):
        self.missing, self.unexpected, self.wrong_shape, self.wrong_kind = missing, unexpected, wrong_shape, wrong_kind
        lines = [f"weights in {model_dir} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, want, got in wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, found {list(got)}")
        for name, why in wrong_kind:
            lines.append(f"  wrong dtype: {name} {why}")
        super().__init__("\n".join(lines))


def target_dtype(ps: ParamSpec, engine_dtype: torch.dtype, stored: Optional[torch.dtype] = None) -> torch.dtype:
    """The dtype a tensor is held in (see the module docstring); ``stored`` is what the checkpoint holds it in."""
    if ps.integer:
        return torch.int32
    if ps.keep_float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype


def validate(expected: Dict[str, ParamSpec], ckpt: Checkpoint) -> None:
    have = set(ckpt.names())
    missing = [n for n in expected if n not in have]
    unexpected = sorted(n for n in have if n not in expected and not n.endswith(IGNORED_SUFFIXES))
    wrong_shape, wrong_kind = [], []
    for name, ps in expected.items():
        if name not in have:
            continue
        dtype, shape = ckpt.info(name)
        if tuple(shape) != tuple(ps.shape):
            wrong_shape.append((name, ps.shape, shape))
        if ps.integer and dtype.is_floating_point:
            wrong_kind.append((name, f"is {dtype}, an integer table is expected"))
        if not ps.integer and not dtype.is_floating_point:
            wrong_kind.append((name, f"is {dtype}, a floating-point tensor is expected"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(ckpt.model_dir, missing, unexpected, wrong_shape, wrong_kind)


def load_weights(model, model_dir: str, device, dtype: torch.dtype) -> None:
    """Check the folder against the model, then move every tensor to the device."""
    expected = model.expected_tensors()
    with Checkpoint(model_dir) as ckpt:
        validate(expected, ckpt)

        def fetch(name: str) -> torch.Tensor:
            t = ckpt.get(name)
            return t.to(device=device, dtype=target_dtype(expected[name], dtype, t.dtype), copy=True)

        model.load(fetch, dtype)


# ---- random weights ------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63)


def random_tensor(name: str, ps: ParamSpec, seed: int, device="cpu", std: float = INIT_STD) -> torch.Tensor:
    """The float32 values of one tensor in random-weights mode."""
    if ps.integer:
        return torch.zeros(ps.shape, dtype=torch.int32, device=device)
    if ps.init == "ones":
        return torch.ones(ps.shape, dtype=torch.float32, device=device)
    if ps.init == "zeros":
        return torch.zeros(ps.shape, dtype=torch.float32, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    return torch.randn(ps.shape, generator=gen, dtype=torch.float32, device=device) * std


def init_random(model, seed: int, device, dtype: torch.dtype) -> None:
    """Fill a model with seeded random weights directly on the device (no files).
    The generator is the device's, so the values differ from ``write_random_model``'s."""
    expected = model.expected_tensors()

    def fetch(name: str) -> torch.Tensor:
        ps = expected[name]
        return random_tensor(name, ps, seed, device=device).to(target_dtype(ps, dtype))

    model.load(fetch, dtype)


def write_random_model(config: Dict[str, Any], out_dir: str, seed: int = 0,
                       storage_dtype: Optional[str] = None, std: float = INIT_STD) -> str:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights.

    ``config`` holds the keys of the architecture's config.json.  Tensors are
    stored in ``storage_dtype`` (default: the config's torch_dtype), so what the
    file holds is exactly representable in that type.  ``std`` widens the normal
    distribution (tests use it to make attention scores far from uniform).
    """
    from yalis_b200.engine.model import Model

    arch, cfg = parse_config(config)
    model = Model(arch.model_spec(cfg))
    as_dict = arch.config_to_dict(cfg)
    name = storage_dtype or as_dict.get("torch_dtype", "bfloat16")
    if name not in _TORCH_DTYPES:
        raise ValueError(f"storage dtype {name!r} is not one of {', '.join(_TORCH_DTYPES)}")
    as_dict["torch_dtype"] = name
    store = _TORCH_DTYPES[name]
    os.makedirs(out_dir, exist_ok=True)
    tensors = {}
    for tname, ps in model.expected_tensors().items():
        t = random_tensor(tname, ps, seed, std=std)
        tensors[tname] = t if ps.integer else t.to(store)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "generator": f"yalis_b200 random weights, seed {seed}"})
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(as_dict, f, indent=2)
    return out_dir
