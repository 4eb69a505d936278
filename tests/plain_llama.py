"""Plain, slow Llama 3 dense decoder: whole sequences, no cache, float32 on the CPU.

This file is the oracle of the test-suite. It shares no code with the
``yalis_b200`` package: it reads ``config.json`` itself, takes tensors by their
Hugging Face names and computes every part with ordinary torch operations.
Each function restates one formula of the reference implementation and cites
the place (path inside axonn-ai/yalis : lines).

All arithmetic is done in the dtype of the weights handed in (float32 in the
tests, float64 where a test wants a tighter oracle).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


# --------------------------------------------------------------------------
# configuration (own reading of config.json; defaults of yalis/external/config.py:104-135)
# --------------------------------------------------------------------------

def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    return normalise_config(raw)


def normalise_config(raw: dict) -> dict:
    """Fill the derived sizes the way yalis/external/config.py:104-135 does:
    head size defaults to hidden/heads, KV groups default to the head count."""
    c = dict(raw)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)          # yalis/external/config.py:38
    c.setdefault("rope_theta", 10000.0)         # yalis/external/config.py:78
    c.setdefault("rope_scaling", None)
    c.setdefault("tie_word_embeddings", False)
    return c


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x = wte[idx], no scaling for Llama (yalis/external/model.py:137-141)."""
    return table[token_ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w (yalis/external/model.py:979-986)."""
    ms = torch.mean(x * x, dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """theta_i = base^(-2i/hs) in float32, then the optional llama3 smoothing
    (yalis/external/model.py:786-807)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    if scaling is not None:
        factor = scaling["factor"]
        low = scaling["low_freq_factor"]
        high = scaling["high_freq_factor"]
        orig = scaling["original_max_position_embeddings"]
        wavelen = 2 * torch.pi / inv
        ratio = orig / wavelen
        smooth = torch.clamp((ratio - low) / (high - low), min=0.0, max=1.0)
        inv = (1 - smooth) * (inv / factor) + smooth * inv
    return inv


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor):
    """angle[p, i] = p * theta_i in float32; the halves are repeated
    (yalis/external/model.py:810-820)."""
    ang = torch.outer(positions.float(), inv_freq.float())
    ang = ang.repeat(1, 2)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation: x*cos + [-x2, x1]*sin (yalis/external/model.py:894-909).
    x is [T, heads, hs]; cos and sin are [T, hs]."""
    hs = x.shape[-1]
    x1, x2 = x[..., : hs // 2], x[..., hs // 2:]
    rotated = torch.cat((-x2, x1), dim=-1)
    return x * cos[:, None, :].to(x.dtype) + rotated * sin[:, None, :].to(x.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     q_positions: torch.Tensor, k_positions: torch.Tensor,
                     window: Optional[int] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
    """softmax(Q K^T / sqrt(hs) + mask) V with the mask by absolute position:
    key j is visible to the query at position p iff j <= p
    (yalis/attention/backend_impl/sdpa_and_flex.py:15-19, 301-312; softmax in
    float32, :84-90). Query head h reads KV head h // (heads / groups)
    (sdpa_and_flex.py:59-67).  ``window`` (not used by Llama) further hides keys
    with j <= p - window.
    q [Tq, nh, hs]; k, v [Tk, g, hs]; returns [Tq, nh, hs]."""
    tq, nh, hs = q.shape
    g = k.shape[1]
    per = nh // g
    if scale is None:
        scale = 1.0 / math.sqrt(hs)
    kk = k.repeat_interleave(per, dim=1)            # [Tk, nh, hs]
    vv = v.repeat_interleave(per, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    visible = k_positions[None, :] <= q_positions[:, None]
    if window is not None:
        visible = visible & (k_positions[None, :] > q_positions[:, None] - window)
    s = s.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(s.float(), dim=-1).to(q.dtype)
    return torch.einsum("hqk,khd->qhd", p, vv)


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: torch.Tensor) -> torch.Tensor:
    """QKV projection, RoPE on Q and K, causal attention, output projection
    (yalis/external/model.py:540-608)."""
    nh, g, hs = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    t = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(t, nh, hs)
    k = (x @ w[prefix + "k_proj.weight"].T).view(t, g, hs)
    v = (x @ w[prefix + "v_proj.weight"].T).view(t, g, hs)
    inv = rope_inverse_frequencies(hs, cfg["rope_theta"], cfg["rope_scaling"])
    cos, sin = rope_tables(positions, inv)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    y = causal_attention(q, k, v, positions, positions)
    return y.reshape(t, nh * hs) @ w[prefix + "o_proj.weight"].T


def swiglu(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T), then the down projection
    (yalis/external/model.py:740-744; silu(z) = z * sigmoid(z))."""
    gate = x @ gate_w.T
    up = x @ up_w.T
    return (torch.nn.functional.silu(gate) * up) @ down_w.T


def block(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, cfg: dict,
          positions: torch.Tensor) -> torch.Tensor:
    """Pre-norm residual block: x + attn(norm_1 x), then x + mlp(norm_2 x)
    (yalis/external/model.py:414-438, the non-parallel branch)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", cfg, positions)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                   w[p + "mlp.down_proj.weight"])
    return x


def forward_logits(token_ids: List[int], w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence: embedding, the blocks in order,
    final norm, LM head at every position (yalis/external/model.py:137-197).
    A model with tied embeddings uses the embedding table as the head
    (yalis/external/convert_hf_checkpoint.py:869-875)."""
    ids = torch.tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(token_ids))
    x = embed(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, w, layer, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(prompt: List[int], n_new: int, w: Dict[str, torch.Tensor], cfg: dict) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every new token
    (argmax when temperature is 0, yalis/external/sampling.py:64,74)."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(seq, w, cfg)[-1]
        nxt = int(torch.argmax(logits))
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------
# sampling (yalis/external/sampling.py)
# --------------------------------------------------------------------------

def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: Optional[int],
                          top_p: float) -> torch.Tensor:
    """The probabilities the reference draws from: top-k mask, divide by the
    temperature, top-p mask over the sorted softmax (first entry always kept),
    float32 softmax (yalis/external/sampling.py:16-38, 51-72). logits [V]."""
    logits = logits.float().clone()
    if top_k is not None:
        v, i = torch.topk(logits, min(top_k, logits.numel()))
        masked = torch.full_like(logits, float("-inf"))
        masked[i] = v
        logits = masked
    if temperature > 0.0:
        logits = logits / temperature
    if top_p < 1.0:
        sl, si = torch.sort(logits, descending=True)
        cum = sl.softmax(dim=-1).cumsum(dim=-1)
        remove = cum > top_p
        remove[0] = False
        logits[si[remove]] = float("-inf")
    return torch.softmax(logits, dim=-1)


# --------------------------------------------------------------------------
# weights for the plain model (own reader; float32)
# --------------------------------------------------------------------------

def read_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).to(dtype)
    return out
