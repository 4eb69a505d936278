"""The step context: everything the parts may know about the batch of one step.

A step is a flat list of N tokens from R requests.  Request i contributes
``q_len[i] >= 1`` consecutive tokens that start at position ``ctx_before[i]``
(the number of tokens it already holds): a portion of a prompt of any size, or
one decoded token.  Matrix products see one [N, hidden] matrix; only mixers
look at the request structure.

All device arrays of a step live in one int32 buffer that is filled on the
host in pinned memory and copied once (``StepLayout``); a recorded step keeps
such a buffer of fixed size and pads what a smaller step leaves unused: padding
tokens belong to request -1, padding requests bring no tokens and point to the
slot that belongs to nobody, padding logit rows are -1.  Every kernel skips
those.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class HostStep:
    """The same facts on the host (python lists), for parts that loop over requests or choose
    kernels by lengths.  In a recorded step these are the facts of the step that was recorded:
    a part may use them only as far as its ``capture_key`` covers."""

    slots: List[int]
    q_start: List[int]        # R + 1 offsets into the token list
    ctx_before: List[int]     # tokens each request held before the step
    max_q_len: int
    max_kv_len: int
    memo: Dict[tuple, object] = field(default_factory=dict)    # what parts work out from these facts once per step

    def once(self, key: tuple, work):
        """``work()``, computed the first time ``key`` is asked for in this step (every layer asks the same)."""
        value = self.memo.get(key)
        if value is None:
            value = self.memo[key] = work()
        return value


@dataclass
class StepContext:
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor       # int32 [N]
    positions: torch.Tensor       # int32 [N]   absolute position of each token in its request
    req_of_token: torch.Tensor    # int32 [N]   index into the step's request list (-1: padding)
    q_start: torch.Tensor         # int32 [R+1]
    kv_len: torch.Tensor          # int32 [R]   tokens each request holds after the step
    slots: torch.Tensor           # int32 [R]   state slot of each request (padding: the slot that is nobody's)
    logit_rows: torch.Tensor      # int32 [n_logits] token rows whose logits are wanted (-1: padding)
    block_tables: Dict[str, torch.Tensor]   # group name -> int32 [R, width]
    host: HostStep
    error_flag: Optional[torch.Tensor] = None   # int32 [1]; kernels raise bits in it (bad id, unmapped page, a wait that ran out)
    decode_only: bool = False                    # every request contributes exactly one token
    # The index arrays above reached the device by a copy that finished before the step's first kernel, and the
    # step writes nothing to the cache but its own tokens: kernels may read both ahead of their predecessor.
    settled: bool = False
    extras: dict = field(default_factory=dict)   # lives as long as the step: choices every layer would otherwise repeat
    # A token whose entry in ``token_from_slot`` is not negative is not in ``token_ids``: it is the token an
    # earlier step chose for the request in that slot, kept on the device in ``chosen`` [max_slots + 1].
    token_from_slot: Optional[torch.Tensor] = None
    chosen: Optional[torch.Tensor] = None


class StepLayout:
    """Where each array of a step lies in its one int32 buffer.

    ``n`` tokens, ``r`` requests, ``w`` logit rows, one block table of ``widths[g]`` columns per page group.
    With ``sampling`` the per-row parameters of the token choice follow (temperature and top_p as float32,
    seed and draw counter as int64, 8-byte aligned).  The tables come last, so that a recorded step, whose
    tables have the full row width, can copy everything before them in one piece and of the tables only the
    columns in use.
    """

    def __init__(self, n: int, r: int, w: int, widths: Sequence[int], sampling: bool):
        self.n, self.r, self.w, self.widths, self.sampling = n, r, w, list(widths), sampling
        o = 0

        def take(count: int) -> int:
            nonlocal o
            start = o
            o += count
            return start

        self.tok, self.src, self.pos, self.req = take(n), take(n), take(n), take(n)
        self.qs, self.kv, self.slots, self.rows, self.row_slot = take(r + 1), take(r), take(r), take(w), take(w)
        if sampling:
            self.topk, self.temp, self.topp = take(w), take(w), take(w)
            o += o % 2
            self.seed, self.draw = take(2 * w), take(2 * w)
        self.prefix = o
        self.tables = [take(r * width) for width in self.widths]
        self.total = o

    def views(self, buf, as_numpy: bool):
        """Named views of a buffer (a pinned host tensor as numpy arrays, or a device tensor)."""
        if as_numpy:
            buf = buf.numpy()
        n, r, w = self.n, self.r, self.w
        v = {"tok": buf[self.tok:self.tok + n], "src": buf[self.src:self.src + n], "pos": buf[self.pos:self.pos + n],
             "req": buf[self.req:self.req + n], "qs": buf[self.qs:self.qs + r + 1], "kv": buf[self.kv:self.kv + r],
             "slots": buf[self.slots:self.slots + r], "rows": buf[self.rows:self.rows + w],
             "row_slot": buf[self.row_slot:self.row_slot + w]}
        if self.sampling:
            f32, i64 = (np.float32, np.int64) if as_numpy else (torch.float32, torch.int64)
            v["topk"] = buf[self.topk:self.topk + w]
            v["temp"] = buf[self.temp:self.temp + w].view(f32)
            v["topp"] = buf[self.topp:self.topp + w].view(f32)
            v["seed"] = buf[self.seed:self.seed + 2 * w].view(i64)
            v["draw"] = buf[self.draw:self.draw + 2 * w].view(i64)
        v["tables"] = [buf[o:o + r * width].reshape(r, width) for o, width in zip(self.tables, self.widths)]
        return v
