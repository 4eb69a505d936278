"""Tiny model folders for the tests: configurations of the architecture that
differ in every size and option (A and B; C and D have the head sizes 64 and 128 of the
TMA- and tcgen05-based attention kernels), written with seeded random weights into a
temporary folder (never committed)."""

import functools
import os
import tempfile

from yalis_b200.config.presets import preset
from yalis_b200.weights.loader import write_random_model

_ROOT = None


def _root():
    global _ROOT
    if _ROOT is None:
        _ROOT = tempfile.mkdtemp(prefix="yalis_b200_tiny_")
    return _ROOT


# name -> (preset, seed, page size used with it)
TINY = {"A": ("tiny-A", 0, 16), "B": ("tiny-B", 1, 8), "C": ("tiny-C", 2, 16), "D": ("tiny-D", 3, 64)}


@functools.lru_cache(maxsize=None)
def tiny_model_dir(which: str, std: float = 0.02) -> str:
    name, seed, _ = TINY[which]
    d = os.path.join(_root(), f"{name}_std{std}")
    write_random_model(preset(name), d, seed=seed, std=std)
    return d


def page_size_of(which: str) -> int:
    return TINY[which][2]
