"""Device memory behind the cache manager: page pools and per-request state.

For every schedule entry of a model the mixer's ``cache_request()`` says what
it keeps: keys and values in pages (``PagedKV``), a fixed-size state per request
(``SlotState``), or nothing.  Paged entries with the same retention rule (all
keys, or a window of W) form one *page group*: they share block tables, so one
page id means the same token range in each of their pools, and every group has
pages of its own.  Each paged entry owns two pools
``[num_pages, kv_heads, page_size, head_dim]`` (a KV head's tokens of one page
are contiguous, so the attention kernels stream whole pages per head); the
reference lays a page out as ``[page, kv_heads, head_dim]`` per token
(yalis/external/model.py:620-627).  Pools are never cleared: what a request can
see is decided by its length and its block table only.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from yalis_b200.parts.base import PagedKV, PagedKVCache, SlotState, SlotStateCache
from .manager import PageGroup


def group_name(request: PagedKV) -> str:
    """Paged entries with the same retention rule share block tables (a page id means the same token range
    in each of their pools); the rule is all a group is known by."""
    return "kv_all" if request.window is None else f"kv_window_{request.window}"


def group_page_bytes(requests: List[Optional[object]], cache_of: List[Optional[int]], page_size: int,
                     element_size: int) -> Dict[str, int]:
    """Bytes that one page id of each group stands for: the K and V pages of every schedule entry of the group
    that keeps a cache of its own."""
    out: Dict[str, int] = {}
    for req, src in zip(requests, cache_of):
        if isinstance(req, PagedKV) and src is None:
            name = group_name(req)
            out[name] = out.get(name, 0) + 2 * req.num_kv_heads * page_size * req.head_dim * element_size
    return out


def window_group_pages(window: int, page_size: int, max_slots: int, step_tokens: int) -> int:
    """Pages a group with a window can have in use at once: per request the window, the tokens of the step that
    is running (their pages are mapped before the step and those behind the window returned after it) and the
    two partly used pages at the ends."""
    return max_slots * (-(-(window + step_tokens) // page_size) + 2)


def plan_groups(requests: List[Optional[object]], page_size: int, num_pages: int, max_context: int,
                max_slots: Optional[int] = None, step_tokens: Optional[int] = None) -> List[PageGroup]:
    """One page group per distinct retention rule among the paged requests.  ``num_pages`` is the pool of a
    group that keeps every key; a group with a window gets no more pages than it can ever use
    (``window_group_pages``) when ``max_slots`` and ``step_tokens`` are known."""
    groups: Dict[str, PageGroup] = {}
    width = -(-max_context // page_size)
    for r in requests:
        if isinstance(r, PagedKV):
            name = group_name(r)
            if name not in groups:
                pages = num_pages
                if r.window is not None and max_slots is not None and step_tokens is not None:
                    pages = min(pages, window_group_pages(r.window, page_size, max_slots, min(step_tokens, max_context)))
                groups[name] = PageGroup(name, page_size, pages, r.window, width)
    return list(groups.values())


class CacheStorage:
    """Allocates what every schedule entry asked for and hands out the per-entry views."""

    def __init__(self, requests: List[Optional[object]], cache_of: List[Optional[int]], groups: List[PageGroup],
                 max_slots: int, device, dtype: torch.dtype):
        by_name = {g.name: g for g in groups}
        self.entries: List[Optional[object]] = []
        self.state_tensors: List[torch.Tensor] = []
        self.bytes = 0
        for i, (req, src) in enumerate(zip(requests, cache_of)):
            if src is not None:
                own = self.entries[src]
                if isinstance(own, PagedKVCache):
                    if not isinstance(req, PagedKV) or (req.num_kv_heads, req.head_dim) != (own.k.shape[1], own.k.shape[3]):
                        raise ValueError(f"schedule entry {i} cannot read the cache of entry {src}: shapes differ")
                    self.entries.append(PagedKVCache(own.k, own.v, own.group, writable=False))
                elif isinstance(own, SlotStateCache):
                    self.entries.append(SlotStateCache(own.state, writable=False))
                else:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {src}, which keeps none")
                continue
            if req is None:
                self.entries.append(None)
            elif isinstance(req, PagedKV):
                g = by_name[group_name(req)]
                shape = (g.num_pages, req.num_kv_heads, g.page_size, req.head_dim)
                k = torch.empty(shape, dtype=dtype, device=device)
                v = torch.empty(shape, dtype=dtype, device=device)
                self.bytes += 2 * k.numel() * k.element_size()
                self.entries.append(PagedKVCache(k, v, g.name))
            elif isinstance(req, SlotState):
                # one row more than there are slots: the row that padding rows of a recorded step point to
                st = torch.zeros((max_slots + 1,) + tuple(req.shape), dtype=req.dtype, device=device)
                self.bytes += st.numel() * st.element_size()
                self.state_tensors.append(st)
                self.entries.append(SlotStateCache(st))
            else:
                raise TypeError(f"schedule entry {i}: unknown cache request {req!r}")

    def reset_slot(self, slot: int) -> None:
        """Zero the per-request state of a newly admitted request."""
        for st in self.state_tensors:
            st[slot].zero_()

    def snapshot_state(self) -> List[torch.Tensor]:
        """Copies of all per-request state (for a trial run whose effects must not stay)."""
        return [st.clone() for st in self.state_tensors]

    def restore_state(self, saved: List[torch.Tensor]) -> None:
        for st, old in zip(self.state_tensors, saved):
            st.copy_(old)
