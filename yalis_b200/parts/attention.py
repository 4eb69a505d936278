"""Grouped-query causal attention over the paged cache.

qkv = x Wqkv^T; positions are encoded into Q and K and K, V stored (the position
part does both in one kernel); every token attends to the cached keys of its
request up to its own position; the heads are projected back with Wo
(yalis/external/model.py:540-608).  The three projections are stored
concatenated [Wq; Wk; Wv] (the reference interleaves them per KV group,
model.py:544-557, which only serves its tensor-parallel split).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops import attention as attn_ops
from yalis_b200.ops.linear import linear_partial
from .base import NOT_ROTARY, Mixer, PagedKV, PagedKVCache, ParamSpec, PositionEncoding, register_part


class PagedAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``window`` (None = all keys), ``scale`` (None = 1/sqrt(head_dim))."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.g = int(p["num_kv_heads"])
        self.hs = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hs)
        if self.nh % self.g:
            raise ValueError(f"num_heads {self.nh} is not a multiple of num_kv_heads {self.g}")
        if self.hs % 2 or self.hs > 256:
            raise ValueError(f"head_dim {self.hs} is not supported (even, at most 256)")
        if position is None:
            raise ValueError("paged_attention needs a position part (use kind 'none' for no encoding)")
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "q_proj": ParamSpec((self.nh * self.hs, self.hidden)),
            "k_proj": ParamSpec((self.g * self.hs, self.hidden)),
            "v_proj": ParamSpec((self.g * self.hs, self.hidden)),
            "o_proj": ParamSpec((self.hidden, self.nh * self.hs)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()

    def cache_request(self) -> PagedKV:
        return PagedKV(self.g, self.hs, self.window)

    def capture_key(self, host):
        # everything the choice of kernel and its launch depend on besides the shapes of the step's tensors
        per = self.nh // self.g
        if host.max_q_len == 1:
            return host.once(("decode_step_kind",), lambda: attn_ops.decode_step_kind([b + 1 for b in host.ctx_before]))
        return host.once(("portion_step_kind", per, self.g, self.hs),
                         lambda: attn_ops.portion_step_kind(host, per, self.g, self.hs))

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        # QK^T and PV over the keys each token sees (causal; a window bounds them)
        keys = sum(min(ctx_before + t + 1, self.window or (ctx_before + t + 1)) for t in range(q_len)) if self.window \
            else q_len * ctx_before + q_len * (q_len + 1) / 2
        return 4.0 * self.nh * self.hs * keys

    def forward(self, x: torch.Tensor, ctx, cache: PagedKVCache) -> torch.Tensor:
        qkv = linear_partial(x, self.w_qkv)          # [N, width], or float32 partial sums [S, N, width]
        if (attn_ops.USE_FUSED_ROPE and ctx.n_requests * self.g <= 2 * attn_ops.sm_count(x.device)
                and attn_ops.decode_tma_applicable(x.dtype, ctx, self.hs, cache.k.shape[2], self.nh // self.g, self.window)
                and not attn_ops.decode_lean_preferred(ctx.n_requests, self.g, self.hs, attn_ops.step_kind(ctx)[0])):
            # A decode step whose attention blocks fit the GPU at once: the attention kernel rotates Q and the new K
            # itself and stores K, V (one launch less).  With more blocks than that the extra work at the start of
            # every block costs more than the launch (measured at batch 64: 59.5 against 57 us per layer).
            freq = self.position.rotary_frequencies(self.hs, x.device)
            if freq is not NOT_ROTARY:
                y = attn_ops.decode_attention_tma_fused(
                    qkv, freq, cache.writable, cache.k, cache.v, ctx.positions, ctx.q_start,
                    ctx.block_tables[cache.group], self.nh, self.g, self.hs, scale=self.scale,
                    n_splits=attn_ops.decode_tma_splits(ctx.n_requests, self.g, attn_ops.step_kind(ctx)[1]),
                    error_flag=ctx.error_flag,
                    early_fetch=bool(getattr(ctx, "settled", False)))
                return linear_partial(y, self.w_o)
        q = self.position.encode_and_store(qkv, self.nh, self.g, self.hs, ctx, cache, dtype=x.dtype)
        y = attn_ops.paged_attention(q, cache.k, cache.v, ctx, cache.group, self.nh, self.g, self.hs,
                                     scale=self.scale, window=self.window)
        return linear_partial(y, self.w_o)             # the residual stream adds the partial sums


register_part("mixer", "paged_attention", PagedAttention)
