"""The batch of one step: flat token rows of several requests, each a portion of a
prompt or a single decoded token, with what the kernels need to find their cache.

The reference's ``LLMBatch{_tokens, _pos, _token_seq_ids, _logits}``
(src/core/runtime/BatchManager.h:77-99) has the same flat shape, but its graph runs
one contiguous run of one sequence at a time (InferRuntime.cu:429;
QWen3Creator.cpp:267-268).  Here any mix runs as one batch.

All integer arrays are packed into one host buffer (by the host runtime, which holds the positions, slots and
block tables: cache/native.py ``pack_step``) and reach the device in one copy.
A batch may be padded to a fixed number of requests and a fixed block-table width,
so that its device arrays have fixed addresses and sizes (for CUDA graphs); padding
requests bring one token at position 0 whose keys go to a page nobody reads.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

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
    token_src: Optional[Sequence[int]] = None    # per token: row of the previous step's drawn tokens to take the
                                                 # id from on the device, or -1 for the id given in ``tokens``


NUM_FLAT = 10     # flat integer arrays ahead of the block tables in the packed buffer


@dataclass(frozen=True)
class BatchLayout:
    """Sizes of the packed integer buffer: T tokens, B requests, R logit rows, and the
    block-table width of each cache group."""
    T: int
    B: int
    R: int
    widths: Tuple[int, ...]

    def sizes(self) -> List[int]:
        return [self.T, self.T, self.T, self.B + 1, self.B, self.B, self.B, self.R, self.B, self.T] + \
               [self.B * w for w in self.widths]

    @property
    def total(self) -> int:
        return int(sum(self.sizes()))

    def offsets(self) -> List[int]:
        out, off = [], 0
        for n in self.sizes():
            out.append(off)
            off += n
        return out


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
    req_order: Optional[torch.Tensor] = None   # int32 [B] request rows by number of new tokens, then longest context first
    tok_src: Optional[torch.Tensor] = None     # int32 [T] rows of the previous step's drawn tokens (-1: none), or None
    block_tables: List[torch.Tensor] = field(default_factory=list)   # per group int32 [B, width]
    # host copies, for launch decisions
    h_q_lens: Optional[np.ndarray] = None
    h_pos_start: Optional[np.ndarray] = None
    h_sorted_q_lens: Optional[np.ndarray] = None     # q_lens in the order of req_order
    h_sorted_kv_lens: Optional[np.ndarray] = None    # kv_len in the order of req_order (real requests only count)
    # How many requests of the longest context the decoded tokens of this step weigh (sum / longest of the
    # contexts), rounded to a power of two: CudaKernels.key_split_class.  Set by the runner for steps replayed as CUDA graphs, whose launch
    # geometry is fixed when they are captured; None lets the kernel library work it out per launch.
    key_split_class: Optional[int] = None
    all_decode: bool = False      # every request brings exactly one token
    real_requests: int = 0        # requests that are not padding
    real_logit_rows: int = 0
    graph_bucket: Optional[int] = None   # set when the arrays are the fixed ones of a CUDA-graph bucket


def batch_views(dev: torch.Tensor, layout: BatchLayout):
    """Slices of the packed device buffer, in the order of BatchLayout.sizes()."""
    offs, sizes = layout.offsets(), layout.sizes()
    v = [dev[o:o + n] for o, n in zip(offs[:NUM_FLAT], sizes[:NUM_FLAT])]
    bts = [dev[o:o + n].view(layout.B, w) for o, n, w in zip(offs[NUM_FLAT:], sizes[NUM_FLAT:], layout.widths)]
    return v, bts


def batch_from_device(dev: torch.Tensor, layout: BatchLayout, info) -> StepBatch:
    v, bts = batch_views(dev, layout)
    return StepBatch(
        num_tokens=layout.T, num_requests=layout.B, num_logit_rows=layout.R,
        max_q_len=info["max_q_len"], max_kv_len=info["max_kv_len"],
        token_ids=v[0], positions=v[1], tok_req=v[2], q_start=v[3], pos_start=v[4], kv_len=v[5],
        slots=v[6], logit_rows=v[7], req_order=v[8], tok_src=v[9] if info["has_token_src"] else None, block_tables=bts,
        h_q_lens=info["q_lens"], h_pos_start=info["pos_start"], h_sorted_q_lens=info["sorted_q_lens"],
        h_sorted_kv_lens=info["sorted_kv_lens"], all_decode=info["all_decode"],
        real_requests=info["real_requests"], real_logit_rows=info["real_logit_rows"])


def packed_to_device(arr: np.ndarray, layout: BatchLayout, info, device, pinned: bool = False) -> StepBatch:
    """The packed step on ``device``, in one transfer."""
    host = torch.from_numpy(arr)
    if str(device) == "cpu":
        dev = host
    elif pinned:
        dev = host.pin_memory().to(device, non_blocking=True)
    else:
        dev = host.to(device)
    return batch_from_device(dev, layout, info)
