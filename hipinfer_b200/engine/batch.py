"""One step's batch as the kernels see it: flat rows of (token, position, request), per-request
block tables and lengths, the cache slot each row's key and value go to, and the rows whose
logits are wanted. Built on the host from the cache manager's tables, packed into ONE int32
buffer in pinned memory and sent with one copy.

The reference never mixes: `hi_prefill` is one slot's chunk (src/api.cu:1788), `hi_decode`
one token of slots [0, B) (1891); only `verify_step` (2029-2060) runs several consecutive
positions of a slot beside per-row positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """A request's next tokens in this step, and the places among them whose logits are wanted."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    n_rows: int
    n_requests: int
    n_want: int
    tokens: torch.Tensor          # int32 [T]
    positions: torch.Tensor       # int32 [T]
    row_request: torch.Tensor     # int32 [T]  index into this batch's requests
    req_q_start: torch.Tensor     # int32 [R]  first row of the request
    req_q_len: torch.Tensor       # int32 [R]
    req_ctx_len: torch.Tensor     # int32 [R]  tokens in the cache before this step
    req_state_slot: torch.Tensor  # int32 [R]
    want_rows: torch.Tensor       # int32 [W]
    token_map: torch.Tensor       # int32 [T]  >= 0: the row's token is that entry of a device buffer (see runner.step)
    block_tables: List[torch.Tensor]  # per cache group int32 [R, pages]
    slot_maps: List[torch.Tensor]     # per cache group int32 [T]
    # host mirrors, for launch geometry and for parts that loop over requests
    h_q_start: List[int] = field(default_factory=list)
    h_q_len: List[int] = field(default_factory=list)
    h_ctx_len: List[int] = field(default_factory=list)
    h_state_slot: List[int] = field(default_factory=list)
    max_pos: int = 0              # largest position among the rows
    max_q_len: int = 0
    extra: dict = field(default_factory=dict)  # what a kernel dispatcher derived for this batch (cached per step)
    dump: Optional[dict] = None   # debug: planes of the step are recorded here, keyed (order index, name) (parts/planes.py)
    dump_step: int = -1           # the order index the decoder is at


def build_step_batch(entries: Sequence[StepEntry], ctx_lens: Sequence[int], state_slots: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], slot_maps: Sequence[Sequence[Sequence[int]]],
                     n_groups: int, device, table_widths: Optional[Sequence[int]] = None,
                     static: Optional[torch.Tensor] = None, max_pos: Optional[int] = None,
                     token_map: Optional[Sequence[int]] = None, token_arrays: Optional[Sequence] = None) -> StepBatch:
    """entries[r] runs at positions ctx_lens[r].. ; tables[r][g] is the request's block table of
    group g AFTER room was made for this step; slot_maps[r][g][i] the cache slot of its i-th token.
    `table_widths` fixes the block tables' widths and `static` is a device buffer to fill instead
    of a fresh one (both for steps replayed from a CUDA graph, whose addresses and launch
    geometry must not change); `max_pos` then states the bound the geometry was made for.
    `token_arrays`: the entries' tokens as integer arrays, where the caller has them already."""
    R = len(entries)
    q_len = [len(e.tokens) for e in entries]
    T = sum(q_len)
    q_start = [0] * R
    for r in range(1, R):
        q_start[r] = q_start[r - 1] + q_len[r - 1]
    want_rows = [q_start[r] + int(w) for r, e in enumerate(entries) for w in e.want]
    W = len(want_rows)
    widths = [max(1, max((len(tables[r][g]) for r in range(R)), default=1)) for g in range(n_groups)]
    if table_widths is not None:
        assert all(w <= tw for w, tw in zip(widths, table_widths)), "a block table is wider than the graph was made for"
        widths = list(table_widths)
    n_int = 4 * T + 4 * R + W + sum(R * w for w in widths) + n_groups * T
    host = torch.empty(max(n_int, 1), dtype=torch.int32, pin_memory=torch.device(device).type == "cuda")
    buf = host.numpy()
    off = 0

    def put(values, n):
        nonlocal off
        buf[off:off + n] = values
        o = off
        off += n
        return o

    # (numpy, not comprehensions: a prompt portion has thousands of rows)
    if token_arrays is None:
        token_arrays = [np.asarray(e.tokens, dtype=np.int64) for e in entries]
    toks = np.concatenate(token_arrays) if R else np.zeros(0, np.int64)
    pos = np.concatenate([np.arange(ctx_lens[r], ctx_lens[r] + q_len[r]) for r in range(R)]) if R else np.zeros(0, np.int64)
    rowreq = np.repeat(np.arange(R), q_len)
    o_tok, o_pos, o_rr = put(toks, T), put(pos, T), put(rowreq, T)
    o_map = put(list(token_map) if token_map is not None else -1, T)
    o_qs, o_ql, o_cl, o_ss = put(q_start, R), put(q_len, R), put(list(ctx_lens), R), put(list(state_slots), R)
    o_w = put(want_rows, W)
    o_bt = []
    for g in range(n_groups):
        o, w = off, widths[g]
        buf[o:o + R * w] = -1
        for r in range(R):
            row = tables[r][g]
            buf[o + r * w:o + r * w + len(row)] = row
        off += R * w
        o_bt.append(o)
    o_sm = [put(np.concatenate([np.asarray(slot_maps[r][g], dtype=np.int64) for r in range(R)]) if R else [], T)
            for g in range(n_groups)]
    if static is not None:
        assert static.numel() >= n_int
        static[:n_int].copy_(host[:n_int], non_blocking=True)
        dev = static
    else:
        dev = host.to(device, non_blocking=True)

    def view(o, n):
        return dev[o:o + n]

    return StepBatch(
        n_rows=T, n_requests=R, n_want=W, tokens=view(o_tok, T), positions=view(o_pos, T), row_request=view(o_rr, T),
        req_q_start=view(o_qs, R), req_q_len=view(o_ql, R), req_ctx_len=view(o_cl, R), req_state_slot=view(o_ss, R),
        want_rows=view(o_w, W), token_map=view(o_map, T),
        block_tables=[view(o_bt[g], R * widths[g]).view(R, widths[g]) for g in range(n_groups)],
        slot_maps=[view(o_sm[g], T) for g in range(n_groups)],
        h_q_start=q_start, h_q_len=q_len, h_ctx_len=list(ctx_lens), h_state_slot=list(state_slots),
        max_pos=(int(pos.max()) if T else 0) if max_pos is None else max_pos, max_q_len=max(q_len) if q_len else 0)
