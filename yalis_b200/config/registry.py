"""The one registry from an architecture's name to its model.

An architecture is an object with
  * ``parse_config(raw: dict) -> config``  a typed, validated configuration
    built from the keys of the architecture's own ``config.json``;
  * ``model_spec(config) -> ModelSpec``     the layers, their parts and their
    order, with the tensor names of every weight;
  * ``config_to_dict(config) -> dict``      the inverse of ``parse_config``
    (used by the random-weights mode to write a model folder).

``config.json`` names its architecture in ``architectures[0]`` (the Hugging Face
convention); everything in the package that needs a model goes through
``load_config`` / ``get_architecture``.  The reference looks models up by a
name registry of dictionaries instead (yalis/external/config.py:183-205, 3249);
its preset names are kept as aliases in ``yalis_b200.config.presets``.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple

_ARCHITECTURES: Dict[str, Any] = {}


class ConfigError(ValueError):
    """A config.json that this package cannot run, with the offending key."""


def register_architecture(name: str, architecture: Any, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    for attr in ("parse_config", "model_spec", "config_to_dict"):
        if not hasattr(architecture, attr):
            raise TypeError(f"architecture {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = architecture


def get_architecture(name: str) -> Any:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"{name!r} is not a supported architecture (known: {', '.join(sorted(_ARCHITECTURES)) or 'none'})"
        ) from None


def architecture_names() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json has no `architectures` entry naming the model class")
    return archs[0]


def parse_config(raw: Dict[str, Any]):
    """(architecture object, typed config) for the dictionary of a config.json."""
    arch = get_architecture(architecture_of(raw))
    return arch, arch.parse_config(raw)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path) as f:
        raw = json.load(f)
    return parse_config(raw)


def _ensure_builtin() -> None:
    # Importing the module registers the architecture it defines.
    from yalis_b200.models import llama  # noqa: F401
