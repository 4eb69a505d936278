"""Choosing the next token: the reference's sampler with per-request parameters.

Meaning of the options is the reference's (yalis/external/sampling.py:41-74,
yalis/config.py:88-228):

* ``top_k``: keep the k largest logits (None = off);
* ``temperature``: logits are divided by it when it is > 0;
* ``top_p``: nucleus cut over the sorted probabilities (1.0 = off); the most
  probable token is always kept;
* greedy (argmax) **iff ``temperature == 0`` and ``top_p == 0``** -- with a zero
  temperature alone the reference still draws, from the unscaled softmax.

Unlike the reference, whose parameters and generator are global
(yalis/engine.py:472-474, yalis/initialize.py:27 seeds 1234), every request
carries its own parameters, seed and draw counter, so what a request draws does
not depend on which other requests share its batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from yalis_b200.ops import sampling as ops

DEFAULT_SEED = 1234   # the reference's global seed (yalis/initialize.py:27)
_MIX = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: float = 1.0
    seed: int = DEFAULT_SEED

    def __post_init__(self):
        # the reference's validation (yalis/config.py:173-180)
        if self.temperature is None or self.temperature < 0.0:
            raise ValueError("temperature must be >=0.0.")
        if self.top_k is not None and self.top_k <= 0:
            raise ValueError("top_k must be a positive integer.")
        if self.top_p is None or self.top_p < 0.0 or self.top_p > 1.0:
            raise ValueError("top_p must be in the range [0.0, 1.0].")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 and self.top_p == 0.0


GREEDY = SamplingParams(temperature=0.0, top_p=0.0)


def request_seed(base_seed: int, ordinal: int) -> int:
    """A distinct 64-bit seed for the ordinal-th request under one base seed."""
    return (int(base_seed) + (int(ordinal) + 1) * _MIX) & 0xFFFFFFFFFFFFFFFF


def as_int64(u: int) -> int:
    u &= 0xFFFFFFFFFFFFFFFF
    return u - (1 << 64) if u >= (1 << 63) else u


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], draw_index: Sequence[int]) -> torch.Tensor:
        """int32 [rows] on the device: one token per row of float32 ``logits`` [rows, vocab].
        ``draw_index[i]`` counts the draws request i has made before this one."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(draw_index):
            raise ValueError("one SamplingParams and one draw index per row of logits")
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        host = np.empty((rows, 8), dtype=np.int32)       # packed: temp, top_k, top_p, pad, seed(2), draw(2)
        f = host.view(np.float32)
        q = host.view(np.int64)
        for i, (p, d) in enumerate(zip(params, draw_index)):
            f[i, 0] = p.temperature
            host[i, 1] = p.top_k or 0
            f[i, 2] = p.top_p
            q[i, 2] = as_int64(p.seed)
            q[i, 3] = int(d)
        dev = torch.from_numpy(host).to(self.device, non_blocking=False)
        temperature = dev[:, 0].contiguous().view(torch.float32)
        top_k = dev[:, 1].contiguous()
        top_p = dev[:, 2].contiguous().view(torch.float32)
        wide = dev.view(torch.int64)
        seed = wide[:, 2].contiguous()
        draw = wide[:, 3].contiguous()
        return ops.sample(logits, temperature, top_k, top_p, seed, draw)
