"""``ModelConfig`` and ``InferenceConfig``: the reference's two user-facing
configuration classes (yalis/config.py:8-228), with the same option names and
meanings where this engine has the option, and the engine's own knobs beside
them.  Architectural numbers never live here: they come from config.json.
"""

from __future__ import annotations

import os
from typing import Literal, Optional, Tuple

from .presets import PRESETS


class ModelConfig:
    """Which model to run and in which precision.

    ``model_name``: a name for messages, or a preset name (``Llama-3-8B`` ...)
    when ``random_weights`` is set.  ``model_path``: folder with config.json
    and model.safetensors; as in the reference it defaults to
    ``$YALIS_CACHE/checkpoints/<model_name>`` (yalis/config.py:52-58) and must
    exist.  ``precision``: ``bf16`` (default) or ``fp32`` (the true 32-bit
    path); the reference's ``fp16`` is refused because weights are kept in
    bfloat16.  ``random_weights``: build the named preset with seeded random
    weights on the device instead of reading a folder.
    """

    def __init__(self, model_name: Optional[str] = None, model_path: Optional[str] = None,
                 precision: Literal["fp32", "bf16"] = "bf16", disable_tp: bool = True,
                 random_weights: bool = False, seed: int = 0):
        self.model_name = model_name
        self.model_path = model_path
        self.precision = precision
        self.disable_tp = disable_tp
        self.random_weights = random_weights
        self.seed = seed
        self._validate()
        if not random_weights:
            self.model_path = self._resolve_model_path(model_path)

    def _resolve_model_path(self, model_path: Optional[str]) -> str:
        if model_path is None:
            cache_dir = os.getenv("YALIS_CACHE", "~/.cache/yalis/")
            model_path = os.path.join(os.path.expanduser(cache_dir), "checkpoints", self.model_name)
        if not os.path.exists(model_path):
            raise ValueError(f"Model path does not exist: {model_path}")
        return model_path

    def _validate(self) -> None:
        if self.model_path is None and self.model_name is None:
            raise ValueError("Either 'model_name' or 'model_path' must be provided.")
        if self.precision == "fp16":
            raise ValueError("Invalid precision: fp16. This engine keeps weights in bfloat16; use 'bf16' or 'fp32'.")
        if self.precision not in {"fp32", "bf16"}:
            raise ValueError(f"Invalid precision: {self.precision}. Supported values are 'fp32', 'bf16'.")
        if self.random_weights and self.model_name not in PRESETS:
            raise ValueError(f"random_weights needs a preset name, one of: {', '.join(sorted(PRESETS))}")

    def __repr__(self) -> str:
        return (f"ModelConfig(model_name={self.model_name}, model_path={self.model_path}, "
                f"precision={self.precision})")


class InferenceConfig:
    """Generation limits, sampling options and the engine's memory and batching knobs.

    Options of the reference kept with their meaning (yalis/config.py:93-158):
    ``max_batch_size`` (most requests alive at once), ``max_length_of_generated_sequences``
    (most tokens a request may hold, prompt included; stored as ``max_length``),
    ``top_k``, ``top_p``, ``temperature``, ``metrics``.  Options that choose among the
    reference's backends or spread the model over GPUs are accepted only at the values
    that describe this engine: one GPU, its own paged attention kernels.

    Own options: ``page_size`` (tokens per cache page), ``cache_tokens`` (size of the page
    pool; default ``max_batch_size * max_length``), ``max_tokens_per_step`` (token budget
    of one step), ``prefill_chunk`` (largest portion of one prompt in a step), ``seed``.
    """

    def __init__(self, max_batch_size: int = 1, max_length_of_generated_sequences: int = 1024,
                 top_k: Optional[int] = None, top_p: Optional[float] = 1.0, temperature: Optional[float] = 1.0,
                 metrics: bool = False, tp_dims: Optional[Tuple[int, int, int]] = None,
                 attention_backend: str = "paged", use_intra_head_parallelism: bool = False,
                 use_paged_kv_caching: bool = True, prestore_kv_cache: bool = True,
                 symmetric_allreduce_strategy: Optional[str] = None,
                 page_size: int = 64, cache_tokens: Optional[int] = None, max_tokens_per_step: int = 2048,
                 prefill_chunk: Optional[int] = None, seed: int = 1234):
        self.max_batch_size = max_batch_size
        self.max_length = max_length_of_generated_sequences
        self.temperature = temperature
        self.top_k = top_k
        self.top_p = top_p
        self.metrics = metrics
        self.tp_dims = tp_dims
        self.attention_backend = attention_backend
        self.use_intra_head_parallelism = use_intra_head_parallelism
        self.use_paged_kv_caching = use_paged_kv_caching
        self.prestore_kv_cache = prestore_kv_cache
        self.symmetric_allreduce_strategy = symmetric_allreduce_strategy
        self.page_size = page_size
        self.cache_tokens = cache_tokens
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk
        self.seed = seed
        self._validate()

    def _validate(self) -> None:
        if self.max_batch_size <= 0:
            raise ValueError("max_batch_size must be a positive integer.")
        if self.max_length <= 0:
            raise ValueError("max_length must be a positive integer.")
        if self.temperature is not None and self.temperature < 0.0:
            raise ValueError("temperature must be >=0.0.")
        if self.top_k is not None and self.top_k <= 0:
            raise ValueError("top_k must be a positive integer.")
        if self.top_p is not None and (self.top_p < 0.0 or self.top_p > 1.0):
            raise ValueError("top_p must be in the range [0.0, 1.0].")
        if self.tp_dims is not None and tuple(self.tp_dims) != (1, 1, 1):
            raise ValueError("tp_dims: this engine runs on one GPU; leave it None or (1, 1, 1).")
        if self.attention_backend not in ("paged", "flash", "sdpa", "flex"):
            raise ValueError(f"Invalid attention backend: {self.attention_backend}.")
        if self.use_intra_head_parallelism:
            raise ValueError("use_intra_head_parallelism splits heads over GPUs; this engine runs on one GPU.")
        if not self.use_paged_kv_caching:
            raise ValueError("use_paged_kv_caching=False: this engine's cache is always paged.")
        if self.symmetric_allreduce_strategy is not None:
            raise ValueError("symmetric_allreduce_strategy applies to several GPUs; this engine runs on one GPU.")
        if self.page_size <= 0 or self.max_tokens_per_step <= 0:
            raise ValueError("page_size and max_tokens_per_step must be positive integers.")
        if self.prefill_chunk is not None and self.prefill_chunk <= 0:
            raise ValueError("prefill_chunk must be a positive integer.")
        if self.cache_tokens is not None and self.cache_tokens <= 0:
            raise ValueError("cache_tokens must be a positive integer.")

    def __repr__(self) -> str:
        keys = ("max_batch_size", "max_length", "top_k", "top_p", "temperature", "metrics", "page_size",
                "cache_tokens", "max_tokens_per_step", "prefill_chunk", "seed")
        return "InferenceConfig(\n" + "".join(f"  {k}={getattr(self, k)},\n" for k in keys) + ")"
