"""The batch of one step: flat token rows of several requests, each a portion of a
prompt or a single decoded token, with what the kernels need to find their cache.

The reference's ``LLMBatch{_tokens, _pos, _token_seq_ids, _logits}``
(src/core/runtime/BatchManager.h:77-99) has the same flat shape, but its graph runs
one contiguous run of one sequence at a time (InferRuntime.cu:429;
QWen3Creator.cpp:267-268).  Here any mix runs as one batch.

All integer arrays are packed into one host buffer and reach the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, starting at the position given by
    the number of tokens it has in the cache, and the places among them (0-based)
    whose logits are wanted."""
    req: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_logit_rows: int
    max_q_len: int
    max_kv_len: int
    token_ids: torch.Tensor       # int32 [T]
    positions: torch.Tensor       # int32 [T]   absolute position of each token in its request
    tok_req: torch.Tensor         # int32 [T]   row (0..B-1) of the token's request in the per-request arrays
    q_start: torch.Tensor         # int32 [B+1] first flat row of each request's tokens (cumulative)
    pos_start: torch.Tensor       # int32 [B]   position of each request's first token of this step
    kv_len: torch.Tensor          # int32 [B]   tokens of each request in the cache after this step
    slots: torch.Tensor           # int32 [B]   state slot of each request
    logit_rows: torch.Tensor      # int32 [R]   flat rows whose logits are wanted
    block_tables: List[torch.Tensor] = field(default_factory=list)   # per group int32 [B, width]
    # host copies, for launch decisions
    h_q_lens: Optional[np.ndarray] = None
    h_pos_start: Optional[np.ndarray] = None
    all_decode: bool = False      # every request brings exactly one token


def build_step_batch(entries: Sequence[StepEntry], starts: Sequence[int], slots: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], device, pad_width_to: int = 1,
                     pinned: bool = False) -> StepBatch:
    """entries[i] starts at position starts[i]; tables[g][i] is request i's block table
    in group g (a list of page ids, -1 for pages that were given back)."""
    B = len(entries)
    q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int32)
    if B == 0 or (q_lens <= 0).any():
        raise ValueError("a step needs at least one request and every request at least one token")
    T = int(q_lens.sum())
    q_start = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    pos_start = np.asarray(starts, dtype=np.int32)
    kv_len = pos_start + q_lens
    token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(np.int32)
    tok_req = np.repeat(np.arange(B, dtype=np.int32), q_lens)
    positions = (np.arange(T, dtype=np.int32) - np.repeat(q_start[:-1], q_lens) + np.repeat(pos_start, q_lens)).astype(np.int32)
    rows = []
    for i, e in enumerate(entries):
        for w in e.want:
            if not (0 <= int(w) < int(q_lens[i])):
                raise ValueError(f"request {e.req!r}: wanted place {w} is outside its {int(q_lens[i])} tokens")
            rows.append(int(q_start[i]) + int(w))
    logit_rows = np.asarray(rows, dtype=np.int32)
    G = len(tables)
    widths = []
    for g in range(G):
        w = max((len(t) for t in tables[g]), default=0)
        w = max(1, -(-w // pad_width_to) * pad_width_to)
        widths.append(w)
    sizes = [T, T, T, B + 1, B, B, B, len(rows)] + [B * w for w in widths]
    total = int(sum(sizes))
    host = torch.empty(total, dtype=torch.int32, pin_memory=pinned)
    hv = host.numpy()
    off = 0
    parts = []
    for arr in (token_ids, positions, tok_req, q_start, pos_start, kv_len,
                np.asarray(slots, dtype=np.int32), logit_rows):
        n = arr.shape[0]
        hv[off:off + n] = arr
        parts.append((off, n))
        off += n
    tparts = []
    for g in range(G):
        w = widths[g]
        bt = np.full((B, w), -1, dtype=np.int32)
        for i, t in enumerate(tables[g]):
            if len(t):
                bt[i, :len(t)] = np.asarray(t, dtype=np.int32)
        hv[off:off + B * w] = bt.reshape(-1)
        tparts.append((off, B, w))
        off += B * w
    dev = host.to(device, non_blocking=pinned) if str(device) != "cpu" else host
    v = [dev[o:o + n] for o, n in parts]
    bts = [dev[o:o + b * w].view(b, w) for o, b, w in tparts]
    return StepBatch(
        num_tokens=T, num_requests=B, num_logit_rows=len(rows),
        max_q_len=int(q_lens.max()), max_kv_len=int(kv_len.max()),
        token_ids=v[0], positions=v[1], tok_req=v[2], q_start=v[3], pos_start=v[4], kv_len=v[5],
        slots=v[6], logit_rows=v[7], block_tables=bts,
        h_q_lens=q_lens, h_pos_start=pos_start, all_decode=bool((q_lens == 1).all()))
