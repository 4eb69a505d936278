"""Nested CUDA-event timers keyed by the stack of open names, as the reference's
``Timers`` (yalis/timers.py:6-73): ``start(name)`` / ``stop(name)`` record events on the
current stream, ``get_times()`` synchronises once and returns total milliseconds and
counts per key (a tuple of names from the outermost timer inwards)."""

from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Tuple

import torch


class Timers:
    def __init__(self):
        self._stack: List[str] = []
        self._open: Dict[Tuple[str, ...], torch.cuda.Event] = {}
        self._pairs: Dict[Tuple[str, ...], List[Tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)

    def start(self, name: str) -> None:
        self._stack.append(name)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[tuple(self._stack)] = ev

    def stop(self, name: str) -> None:
        if not self._stack or self._stack[-1] != name:
            raise RuntimeError(f"timer {name!r} is not the innermost open timer ({self._stack})")
        key = tuple(self._stack)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._pairs[key].append((self._open.pop(key), ev))
        self._stack.pop()

    def get_times(self):
        torch.cuda.synchronize()
        times = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._pairs.items()}
        counts = {k: len(v) for k, v in self._pairs.items()}
        return times, counts
