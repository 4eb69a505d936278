"""Builders of replay traces: the same requests cut into steps in four ways.

A trace is a list of step dictionaries in the format ``bin/trace_run`` reads.  Every
builder asks for the logits of every token it feeds, and ``collect`` puts the rows that
come back into one [T, vocab] array per request, so that each way of cutting can be
compared with the plain implementation position by position.
"""

import random
from typing import Dict, List, Tuple

import numpy as np


def round_up(n: int, unit: int = 64) -> int:
    return -(-n // unit) * unit


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, one step each."""
    return [{"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for rid, toks in requests.items()]


def tail_decoded(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for t in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[t]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, List[int]], seed: int = 0) -> List[dict]:
    """Portions of changing size, down to two tokens (and the odd single one)."""
    rng = random.Random(seed)
    steps = []
    for rid, toks in requests.items():
        o = 0
        sizes = [7, 2, 24, 3, 2, 17, 1, 2, 13]
        i = 0
        while o < len(toks):
            c = sizes[i] if i < len(sizes) else rng.choice([2, 2, 3, 5, 9, 16, 31])
            i += 1
            chunk = toks[o:o + c]
            steps.append({"entries": [{"id": rid, "tokens": chunk, "want": list(range(len(chunk)))}], "end": []})
            o += len(chunk)
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests: Dict[str, List[int]], seed: int = 0, max_live: int = 4, tail: int = 8) -> List[dict]:
    """Up to ``max_live`` live requests: portions of some beside decoded tokens of others,
    requests left out of a step now and then, a new request admitted as soon as one ends."""
    rng = random.Random(seed)
    queue = list(requests.items())
    live: Dict[str, Tuple[List[int], int]] = {}
    steps = []
    while queue or live:
        while queue and len(live) < max_live:
            rid, toks = queue.pop(0)
            live[rid] = (toks, 0)
            if rng.random() < 0.3:
                break                      # do not always fill up at once
        entries, end = [], []
        for rid in list(live):
            toks, o = live[rid]
            if len(live) > 1 and rng.random() < 0.2 and entries:
                continue                   # left out of this step, goes on later
            left = len(toks) - o
            c = 1 if left <= tail else min(left - tail, rng.choice([2, 2, 3, 7, 16, 24, 40]))
            chunk = toks[o:o + c]
            entries.append({"id": rid, "tokens": chunk, "want": list(range(len(chunk)))})
            o += c
            live[rid] = (toks, o)
            if o == len(toks):
                end.append(rid)
                del live[rid]
        rng.shuffle(entries)
        steps.append({"entries": entries, "end": end})
    return steps


def number(steps: List[dict], start: int = 0) -> List[dict]:
    return [dict(s, step=start + i) for i, s in enumerate(steps)]


def peak_tokens(steps: List[dict], unit: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``unit``."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round_up(n, unit) for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: List[dict], outputs: Dict[int, np.ndarray], vocab: int) -> Dict[str, np.ndarray]:
    """Per request, the logits of all its positions in order, from the per-step arrays."""
    parts: Dict[str, List[np.ndarray]] = {}
    for s in steps:
        if not any(e["want"] for e in s["entries"]):
            continue
        arr = outputs[s["step"]].reshape(-1, vocab)
        row = 0
        for e in s["entries"]:
            n = len(e["want"])
            parts.setdefault(e["id"], []).append(arr[row:row + n])
            row += n
        assert row == arr.shape[0]
    return {rid: np.concatenate(p) for rid, p in parts.items()}
