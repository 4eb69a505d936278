"""The step context: everything the parts may know about the batch of one step.

A step is a flat list of N tokens from R requests.  Request i contributes
``q_len[i] >= 1`` consecutive tokens that start at position ``ctx_before[i]``
(the number of tokens it already holds): a portion of a prompt of any size, or
one decoded token.  Matrix products see one [N, hidden] matrix; only mixers
look at the request structure.

All device arrays of a step live in one int32 buffer that is filled on the
host in pinned memory and copied once.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class HostStep:
    """The same facts on the host (python lists), for parts that loop over requests."""

    slots: List[int]
    q_start: List[int]        # R + 1 offsets into the token list
    ctx_before: List[int]     # tokens each request held before the step
    max_q_len: int
    max_kv_len: int
    # A decode step whose requests are long or differ much in length (see ops.attention.deal_tiles_hint): attention
    # kernels should share the cached keys out evenly among their blocks instead of giving each request its own.
    deal_tiles: bool = False


@dataclass
class StepContext:
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor       # int32 [N]
    positions: torch.Tensor       # int32 [N]   absolute position of each token in its request
    req_of_token: torch.Tensor    # int32 [N]   index into the step's request list (-1: padding)
    q_start: torch.Tensor         # int32 [R+1]
    kv_len: torch.Tensor          # int32 [R]   tokens each request holds after the step
    slots: torch.Tensor           # int32 [R]   state slot of each request
    logit_rows: torch.Tensor      # int32 [n_logits] token rows whose logits are wanted
    block_tables: Dict[str, torch.Tensor]   # group name -> int32 [R, width]
    host: HostStep
    error_flag: Optional[torch.Tensor] = None   # int32 [1]; a kernel sets it on a bad id or page
    decode_only: bool = False                    # every request contributes exactly one token
    # The index arrays above reached the device by a copy that finished before the step's first kernel, and the
    # step writes nothing to the cache but its own tokens: kernels may read both ahead of their predecessor.
    settled: bool = False
    extras: dict = field(default_factory=dict)   # scratch for kernels (split buffers etc.)
