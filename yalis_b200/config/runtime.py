"""``ModelConfig`` and ``InferenceConfig``: what a user of the reference passes to
``LLMEngine`` (yalis/config.py:8-228), kept by name so that such code carries
over, and turned into this engine's own ``EngineConfig`` before anything runs.

Only options that mean something on one GPU with a paged cache exist here.  The
reference's options for spreading a model over GPUs or choosing among its
attention libraries are gone, not ignored: passing one is a ``TypeError`` like
any unknown keyword.  ``attention_backend`` and ``use_paged_kv_caching`` are
accepted at the one value that describes this engine, because the reference's
examples pass them.
"""

from __future__ import annotations

import os
from typing import Optional

from .engine_config import EngineConfig
from .presets import PRESETS


class ModelConfig:
    """Which model, where it lies, in which precision.

    ``model_path``: a folder with config.json and model.safetensors; without it the folder is
    ``$YALIS_CACHE/checkpoints/<model_name>`` (``~/.cache/yalis`` when the variable is unset), the
    reference's place (yalis/config.py:52-58).  ``precision``: ``bf16`` or ``fp32`` (the true 32-bit path).
    ``random_weights``: no folder; ``model_name`` is a preset and the weights are drawn on the device from
    ``seed``.
    """

    def __init__(self, model_name: Optional[str] = None, model_path: Optional[str] = None, precision: str = "bf16",
                 random_weights: bool = False, seed: int = 0):
        if model_name is None and model_path is None:
            raise ValueError("ModelConfig: name a model (model_name) or a folder (model_path)")
        if precision == "fp16":
            raise ValueError("ModelConfig: precision fp16 is not offered, weights are held in bfloat16; use bf16 or fp32")
        if precision not in ("bf16", "fp32"):
            raise ValueError(f"ModelConfig: precision {precision!r} is neither bf16 nor fp32")
        if random_weights and model_name not in PRESETS:
            raise ValueError(f"ModelConfig: random_weights wants a preset as model_name ({', '.join(sorted(PRESETS))})")
        self.model_name, self.precision, self.random_weights, self.seed = model_name, precision, random_weights, seed
        if random_weights:
            self.model_path = None
        else:
            if model_path is None:
                root = os.path.expanduser(os.getenv("YALIS_CACHE", "~/.cache/yalis/"))
                model_path = os.path.join(root, "checkpoints", model_name)
            if not os.path.isdir(model_path):
                raise ValueError(f"ModelConfig: no model folder at {model_path}")
            self.model_path = model_path

    def __repr__(self) -> str:
        where = "random weights" if self.random_weights else self.model_path
        return f"ModelConfig({self.model_name or ''} at {where}, {self.precision})"


class InferenceConfig:
    """Limits and defaults of generation, and the engine's memory and batching knobs.

    From the reference, with its meaning (yalis/config.py:93-158): ``max_batch_size`` (most requests alive at
    once), ``max_length_of_generated_sequences`` (most tokens a request may hold, prompt included; kept as
    ``max_length``), ``top_k``, ``top_p``, ``temperature`` (defaults of requests that bring no sampling
    parameters of their own), ``metrics``.  This engine's own: ``page_size``; the pool as one of ``num_pages``,
    ``cache_tokens`` or ``memory_fraction`` (default: ``max_batch_size * max_length`` tokens);
    ``max_tokens_per_step``; ``prefill_chunk``; ``seed`` (of the draws); ``use_graphs``.
    """

    def __init__(self, max_batch_size: int = 1, max_length_of_generated_sequences: int = 1024,
                 top_k: Optional[int] = None, top_p: Optional[float] = 1.0, temperature: Optional[float] = 1.0,
                 metrics: bool = False, attention_backend: Optional[str] = None, use_paged_kv_caching: bool = True,
                 page_size: int = 64, num_pages: Optional[int] = None, cache_tokens: Optional[int] = None,
                 memory_fraction: Optional[float] = None, max_tokens_per_step: int = 2048,
                 prefill_chunk: Optional[int] = None, seed: int = 1234, use_graphs: bool = True):
        if attention_backend not in (None, "paged"):
            raise ValueError(f"InferenceConfig: attention_backend {attention_backend!r} selects nothing here; the engine "
                             "has one attention path, its own paged kernels (leave the option out or pass 'paged')")
        if not use_paged_kv_caching:
            raise ValueError("InferenceConfig: the cache is paged; use_paged_kv_caching cannot be switched off")
        if isinstance(max_length_of_generated_sequences, bool) or not isinstance(max_length_of_generated_sequences, int) \
                or max_length_of_generated_sequences < 1:
            raise ValueError("InferenceConfig: max_length_of_generated_sequences counts tokens, at least 1")
        self.max_batch_size = max_batch_size
        self.max_length = max_length_of_generated_sequences
        self.top_k, self.top_p, self.temperature = top_k, top_p, temperature
        self.metrics = metrics
        self.page_size, self.num_pages, self.cache_tokens, self.memory_fraction = page_size, num_pages, cache_tokens, memory_fraction
        self.max_tokens_per_step, self.prefill_chunk = max_tokens_per_step, prefill_chunk
        self.seed, self.use_graphs = seed, use_graphs
        self.default_sampling()          # validates the three sampling numbers
        self.engine_config("bf16")       # validates the rest

    def default_sampling(self, seed: Optional[int] = None):
        """The sampling parameters of a request that brings none."""
        from yalis_b200.sampling.sampler import SamplingParams
        return SamplingParams(temperature=1.0 if self.temperature is None else self.temperature, top_k=self.top_k,
                              top_p=1.0 if self.top_p is None else self.top_p, seed=self.seed if seed is None else seed)

    def engine_config(self, precision: str, max_context: Optional[int] = None, device: str = "cuda:0") -> EngineConfig:
        pool = dict(num_pages=self.num_pages, cache_tokens=self.cache_tokens, memory_fraction=self.memory_fraction)
        if all(v is None for v in pool.values()):
            pool["cache_tokens"] = self.max_batch_size * self.max_length
        return EngineConfig(dtype=precision, page_size=self.page_size, max_slots=self.max_batch_size,
                            max_tokens_per_step=self.max_tokens_per_step, prefill_chunk=self.prefill_chunk,
                            max_context=max_context or self.max_length, use_graphs=self.use_graphs, device=device, **pool)

    def __repr__(self) -> str:
        shown = ("max_batch_size", "max_length", "top_k", "top_p", "temperature", "page_size", "num_pages", "cache_tokens",
                 "memory_fraction", "max_tokens_per_step", "prefill_chunk", "seed", "use_graphs")
        return "InferenceConfig(" + ", ".join(f"{k}={getattr(self, k)!r}" for k in shown) + ")"
