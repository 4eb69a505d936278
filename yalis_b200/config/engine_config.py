"""``EngineConfig``: how the engine runs a model, apart from what the model is.

Everything here is about this machine and this run: precision, the size of
cache pages and of their pool, how many requests may be alive, how many tokens
a step may hold.  Nothing here describes the architecture (that is
config.json's business, read by ``yalis_b200.config.registry``), and nothing of
the architecture is stamped onto it or the other way round; the reference mixes
the two (yalis/model.py:38-44 writes runtime flags into its model config).
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

_DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass(frozen=True)
class EngineConfig:
    """
    dtype               ``bfloat16`` (serving precision) or ``float32`` (the true 32-bit path).
    page_size           tokens per cache page.
    num_pages           pages in the pool of a page group, or
    cache_tokens        the same as a number of tokens, or
    memory_fraction     the share of the device memory still free once the weights are loaded that goes to
                        the pools (at most what ``max_slots`` requests of ``max_context`` tokens can use).
                        At most one of the three; with none the pool holds ``max_slots * max_context`` tokens,
                        capped at 2^20.
    max_slots           most requests alive at once.
    max_tokens_per_step token budget of one step (decoding requests first, the rest to prompt portions).
    prefill_chunk       largest portion of one prompt in a step (None: the step's budget).
    max_context         most tokens a request may hold (None: the model's limit).
    use_graphs          replay recorded steps where a step's shape allows it.
    device              the CUDA device.
    """

    dtype: str = "bfloat16"
    page_size: int = 64
    num_pages: Optional[int] = None
    cache_tokens: Optional[int] = None
    memory_fraction: Optional[float] = None
    max_slots: int = 64
    max_tokens_per_step: int = 2048
    prefill_chunk: Optional[int] = None
    max_context: Optional[int] = None
    use_graphs: bool = True
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype in ("fp16", "float16"):
            raise ValueError("dtype float16: weights are kept in bfloat16 here; choose bfloat16 or float32")
        if self.dtype not in _DTYPE_NAMES:
            raise ValueError(f"dtype {self.dtype!r}: choose one of {', '.join(sorted(set(_DTYPE_NAMES)))}")
        object.__setattr__(self, "dtype", _DTYPE_NAMES[self.dtype])
        for name in ("page_size", "max_slots", "max_tokens_per_step"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v < 1:
                raise ValueError(f"{name} = {v!r}: a whole number of at least 1 is needed")
        for name in ("num_pages", "cache_tokens", "prefill_chunk", "max_context"):
            v = getattr(self, name)
            if v is not None and (isinstance(v, bool) or not isinstance(v, int) or v < 1):
                raise ValueError(f"{name} = {v!r}: leave it None or give a whole number of at least 1")
        given = [n for n in ("num_pages", "cache_tokens", "memory_fraction") if getattr(self, n) is not None]
        if len(given) > 1:
            raise ValueError(f"the pool is sized by one of num_pages, cache_tokens, memory_fraction; got {' and '.join(given)}")
        f = self.memory_fraction
        if f is not None and not (isinstance(f, (int, float)) and 0.0 < float(f) <= 1.0):
            raise ValueError(f"memory_fraction = {f!r}: a share in (0, 1] is needed")

    def with_(self, **changes) -> "EngineConfig":
        """A copy with some fields changed (the dataclass is frozen)."""
        return replace(self, **changes)

    def pool_pages(self, model_max_context: int, free_bytes: Optional[int] = None,
                   bytes_per_page: Optional[int] = None) -> int:
        """Pages of a group that keeps all keys.  ``free_bytes`` and ``bytes_per_page`` (all groups together) are
        needed for ``memory_fraction`` only."""
        context = min(self.max_context or model_max_context, model_max_context)
        most = self.max_slots * -(-context // self.page_size)      # beyond this no page could ever be mapped
        if self.num_pages is not None:
            return self.num_pages
        if self.cache_tokens is not None:
            return max(1, -(-self.cache_tokens // self.page_size))
        if self.memory_fraction is not None:
            if not free_bytes or not bytes_per_page:
                raise ValueError("memory_fraction needs the free device memory and the bytes of a page")
            pages = int(self.memory_fraction * free_bytes) // bytes_per_page
            if pages < 1:
                raise ValueError(f"memory_fraction {self.memory_fraction} of {free_bytes} free bytes holds no page "
                                 f"of {bytes_per_page} bytes")
            return min(pages, most)
        return max(1, min(most, (1 << 20) // self.page_size))
