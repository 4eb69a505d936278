"""The cache manager: request slots, page groups and block tables (host side).

A thin, typed layer over the native allocator (csrc/host/page_allocator.cpp).
It owns no device memory: the pools that the pages index live in
``yalis_b200.cache.storage``.  What it decides:

* a request gets a *slot* for its life (``acquire`` .. ``release``); the slot
  indexes its block-table row in every group and its row in every per-request
  state tensor;
* before a step runs, ``reserve(slot, new_len)`` maps pages so the slot can
  hold ``new_len`` tokens in every group; it returns False, changing nothing,
  when some group has too few free pages (``reserve_many`` does the same for
  all requests of a step together);
* after the step, ``commit(slot, new_len)`` records the length; groups with a
  window give back the pages that no later query can see;
* ``release(slot)`` gives back all pages and the slot at once.

The reference allocates pages for a whole prompt up front, extends by one token
per decode step and frees only through a reset at the start of each generate
call (yalis/attention/paged_kv_cache.cpp:69-165, yalis/engine.py:435-436).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from yalis_b200 import native


class CacheError(RuntimeError):
    """Misuse of the cache manager (a bug in the caller), never a shortage of pages."""


@dataclass(frozen=True)
class PageGroup:
    """A pool of pages shared by the layers with the same retention rule."""

    name: str
    page_size: int
    num_pages: int
    window: Optional[int] = None          # None: keep every key
    max_pages_per_request: int = 0        # width of a block-table row

    def __post_init__(self):
        if self.page_size <= 0 or self.num_pages <= 0 or self.max_pages_per_request <= 0:
            raise ValueError(f"page group {self.name!r}: page_size, num_pages and max_pages_per_request must be positive")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"page group {self.name!r}: window must be positive or None")


def _bind(lib: ctypes.CDLL) -> None:
    if getattr(lib, "_ycm_bound", False):
        return
    c_int, vp = ctypes.c_int, ctypes.c_void_p
    sigs = {
        "ycm_create": (vp, [c_int]),
        "ycm_destroy": (None, [vp]),
        "ycm_last_error": (ctypes.c_char_p, [vp]),
        "ycm_add_group": (c_int, [vp, c_int, c_int, c_int, c_int]),
        "ycm_acquire_slot": (c_int, [vp]),
        "ycm_pages_needed": (c_int, [vp, c_int, c_int, c_int]),
        "ycm_reserve": (c_int, [vp, c_int, c_int]),
        "ycm_reserve_many": (c_int, [vp, c_int, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
        "ycm_commit": (c_int, [vp, c_int, c_int]),
        "ycm_commit_many": (c_int, [vp, c_int, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
        "ycm_release_slot": (c_int, [vp, c_int]),
        "ycm_table": (ctypes.POINTER(ctypes.c_int32), [vp, c_int]),
        "ycm_ctx_len": (ctypes.POINTER(ctypes.c_int32), [vp]),
        "ycm_free_page_count": (c_int, [vp, c_int]),
        "ycm_free_slot_count": (c_int, [vp]),
        "ycm_first_held": (c_int, [vp, c_int, c_int]),
        "ycm_end_mapped": (c_int, [vp, c_int, c_int]),
        "ycm_check": (c_int, [vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib._ycm_bound = True


class CacheManager:
    def __init__(self, max_slots: int, groups: Sequence[PageGroup]):
        if max_slots <= 0:
            raise ValueError("max_slots must be positive")
        names = [g.name for g in groups]
        if len(set(names)) != len(names):
            raise ValueError("page groups must have distinct names")
        self._lib = native.load("host")
        _bind(self._lib)
        self.max_slots = max_slots
        self.groups: List[PageGroup] = list(groups)
        self._index: Dict[str, int] = {}
        self._h = self._lib.ycm_create(max_slots)
        if not self._h:
            raise CacheError("the native cache manager could not be created")
        self._tables: Dict[str, np.ndarray] = {}
        for g in self.groups:
            gi = self._lib.ycm_add_group(self._h, g.page_size, g.num_pages, g.window or 0, g.max_pages_per_request)
            if gi < 0:
                raise CacheError(self._err())
            self._index[g.name] = gi
            p = self._lib.ycm_table(self._h, gi)
            self._tables[g.name] = np.ctypeslib.as_array(p, shape=(max_slots, g.max_pages_per_request))
        self._ctx = np.ctypeslib.as_array(self._lib.ycm_ctx_len(self._h), shape=(max_slots,))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._tables = {}
            self._lib.ycm_destroy(h)

    def _err(self) -> str:
        return self._lib.ycm_last_error(self._h).decode()

    # -- slots ------------------------------------------------------------------------
    def acquire(self) -> Optional[int]:
        """The smallest free slot, or None."""
        s = self._lib.ycm_acquire_slot(self._h)
        return None if s < 0 else s

    def release(self, slot: int) -> int:
        """Give back every page of the slot and the slot; returns the pages given back."""
        r = self._lib.ycm_release_slot(self._h, slot)
        if r < 0:
            raise CacheError(self._err())
        return r

    # -- pages ------------------------------------------------------------------------
    def pages_needed(self, slot: int, new_len: int) -> Dict[str, int]:
        out = {}
        for g in self.groups:
            r = self._lib.ycm_pages_needed(self._h, self._index[g.name], slot, new_len)
            if r < 0:
                raise CacheError(self._err())
            out[g.name] = r
        return out

    def can_reserve(self, slot: int, new_len: int) -> bool:
        need = self.pages_needed(slot, new_len)
        return all(need[g.name] <= self.free_pages(g.name) for g in self.groups) and self.fits(new_len)

    def fits(self, length: int) -> bool:
        """Whether a request of ``length`` tokens fits a block-table row of every group."""
        return all(-(-length // g.page_size) <= g.max_pages_per_request for g in self.groups)

    def reserve(self, slot: int, new_len: int) -> bool:
        r = self._lib.ycm_reserve(self._h, slot, new_len)
        if r == 0:
            return True
        if r == 1:
            return False
        raise CacheError(self._err())

    def reserve_many(self, slots: Sequence[int], new_lens: Sequence[int]) -> bool:
        """``reserve`` for all requests of a step: True and every slot has its pages, or False and nothing
        has changed (slots must be distinct)."""
        n = len(slots)
        if n != len(new_lens):
            raise CacheError("reserve_many: one length per slot")
        if len(set(slots)) != n:
            raise CacheError("reserve_many: a slot is named twice")
        arr = (ctypes.c_int32 * n)
        r = self._lib.ycm_reserve_many(self._h, n, arr(*[int(s) for s in slots]), arr(*[int(l) for l in new_lens]))
        if r == 0:
            return True
        if r == 1:
            return False
        raise CacheError(self._err())

    def commit(self, slot: int, new_len: int) -> int:
        r = self._lib.ycm_commit(self._h, slot, new_len)
        if r < 0:
            raise CacheError(self._err())
        return r

    def commit_many(self, slots: Sequence[int], new_lens: Sequence[int]) -> int:
        """``commit`` for all requests of a step in one call; all are checked before anything changes."""
        n = len(slots)
        if n != len(new_lens):
            raise CacheError("commit_many: one length per slot")
        arr = (ctypes.c_int32 * n)
        r = self._lib.ycm_commit_many(self._h, n, arr(*slots), arr(*new_lens))
        if r < 0:
            raise CacheError(self._err())
        return r

    # -- views ------------------------------------------------------------------------
    def table(self, group: str) -> np.ndarray:
        """int32 [max_slots, width] view of the native block table (-1 = no page)."""
        return self._tables[group]

    def length(self, slot: int) -> int:
        return int(self._ctx[slot])

    def free_pages(self, group: str) -> int:
        return self._lib.ycm_free_page_count(self._h, self._index[group])

    def free_slots(self) -> int:
        return self._lib.ycm_free_slot_count(self._h)

    def held_range(self, group: str, slot: int):
        gi = self._index[group]
        return self._lib.ycm_first_held(self._h, gi, slot), self._lib.ycm_end_mapped(self._h, gi, slot)

    def check(self) -> None:
        """Raise if a page is lost, held twice or free twice."""
        if self._lib.ycm_check(self._h) != 0:
            raise CacheError(self._err())
