"""Rotary position encoding with the optional llama3 frequency smoothing.

The inverse frequencies are computed once on the host in float32 exactly as the
reference builds its table (yalis/external/model.py:786-807); the angle
``position * inv_freq`` and its sine and cosine are computed in float32 inside
the kernel for the positions of the step, so no table bounds the context.
"""

from __future__ import annotations

from typing import Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import rope_kv_write
from .base import PagedKVCache, PositionEncoding, register_part


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """theta_i = base^(-2i/hs); with ``scaling``: s = clamp((orig/wavelen - low)/(high - low), 0, 1),
    theta_i <- (1 - s) * theta_i / factor + s * theta_i.  float32 [head_dim / 2] on the CPU."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    if scaling is not None:
        wavelen = 2 * torch.pi / inv
        ratio = scaling["original_max_position_embeddings"] / wavelen
        smooth = (ratio - scaling["low_freq_factor"]) / (scaling["high_freq_factor"] - scaling["low_freq_factor"])
        smooth = torch.clamp(smooth, min=0.0, max=1.0)
        inv = (1 - smooth) * (inv / scaling["factor"]) + smooth * inv
    return inv.to(torch.float32)


class RotaryEncoding(PositionEncoding):
    """Parameters: ``head_dim``, ``theta``, ``scaling`` (None or the four llama3 numbers)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        self.inv_freq_host = inverse_frequencies(self.head_dim, float(spec.params["theta"]), spec.params.get("scaling"))
        self.inv_freq: Optional[torch.Tensor] = None

    def load(self, tensors) -> None:
        pass

    def to(self, device) -> None:
        self.inv_freq = self.inv_freq_host.to(device)

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        if self.inv_freq is None or self.inv_freq.device != qkv.device:
            self.to(qkv.device)
        store = cache.writable
        return rope_kv_write(qkv, ctx.positions, ctx.req_of_token, self.inv_freq, cache.k if store else None,
                             cache.v if store else None, ctx.block_tables[cache.group], num_heads, num_kv_heads,
                             head_dim, out_dtype=dtype, bad_flag=ctx.error_flag)

    def rotary_frequencies(self, head_dim: int, device):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        if self.inv_freq is None or self.inv_freq.device != torch.device(device):
            self.to(device)
        return self.inv_freq

    def capture_key(self, host):
        return None


class NoPositionEncoding(PositionEncoding):
    """Stores K and V unrotated (a mixer that wants positions handled elsewhere)."""

    def rotary_frequencies(self, head_dim: int, device):
        return None

    def capture_key(self, host):
        return None

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        store = cache.writable
        return rope_kv_write(qkv, ctx.positions, ctx.req_of_token, None, cache.k if store else None,
                             cache.v if store else None, ctx.block_tables[cache.group], num_heads, num_kv_heads,
                             head_dim, out_dtype=dtype, bad_flag=ctx.error_flag)


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
