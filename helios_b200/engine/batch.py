"""Description of one step's batch, on the host and on the device.

A step runs a flat list of tokens: for every request in it a run of consecutive
tokens (a portion of its prompt, or one decoded token), cut anywhere
(python/helios/exec/model.py:254-277 ``BatchedAttnMeta``;
python/helios/exec/runner.py:188-283 builds the reference's two batches).  All
integer arrays go to the device in one copy from pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class SeqSlice:
    """Host view of one request inside the step."""
    request_id: Hashable
    slot: int
    start_pos: int        # position of its first token in this step
    num_tokens: int
    token_offset: int     # index of its first token in the flat batch


@dataclass
class StepContext:
    act_dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    num_wanted: int
    seqs: List[SeqSlice]
    # device, int32
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T]
    seq_of_token: torch.Tensor       # [T]
    cu_tokens: torch.Tensor          # [S + 1]
    start_pos: torch.Tensor          # [S]
    context_len: torch.Tensor        # [S]  start_pos + num_tokens
    slots: torch.Tensor              # [S]
    want_rows: torch.Tensor          # [R]
    block_tables: List[torch.Tensor]  # per cache group [S, pages]
    # host facts kernels are chosen by
    decode_only: bool = False
    max_tokens_per_seq: int = 0
    max_context_len: int = 0
    # left by the position encoding for the mixers
    rotary_cos: Optional[torch.Tensor] = None
    rotary_sin: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)


def _align4(n: int) -> int:
    return (n + 3) & ~3


def build_context(entries: Sequence[StepEntry], cache, act_dtype: torch.dtype,
                  device: torch.device, table_width: Optional[List[int]] = None) -> StepContext:
    """``cache`` is the cache manager: it knows every request's length, slot and block
    tables (pages for the new tokens must have been taken already)."""
    S = len(entries)
    T = sum(len(e.tokens) for e in entries)
    n_groups = len(cache.groups)
    seqs: List[SeqSlice] = []
    token_ids = np.empty(T, np.int32)
    positions = np.empty(T, np.int32)
    seq_of_token = np.empty(T, np.int32)
    cu = np.zeros(S + 1, np.int32)
    start = np.empty(S, np.int32)
    ctx_len = np.empty(S, np.int32)
    slots = np.empty(S, np.int32)
    want: List[int] = []
    off = 0
    for i, e in enumerate(entries):
        n = len(e.tokens)
        p0 = cache.length(e.request_id)
        seqs.append(SeqSlice(e.request_id, cache.slot(e.request_id), p0, n, off))
        token_ids[off:off + n] = e.tokens
        positions[off:off + n] = np.arange(p0, p0 + n, dtype=np.int32)
        seq_of_token[off:off + n] = i
        start[i], ctx_len[i], slots[i] = p0, p0 + n, seqs[-1].slot
        want.extend(off + int(w) for w in e.want)
        off += n
        cu[i + 1] = off
    want_rows = np.asarray(want, np.int32)
    tables = []
    for g in range(n_groups):
        width = max([len(cache.table(e.request_id, g)) for e in entries] + [1])
        if table_width is not None:
            width = max(width, table_width[g])
        t = np.full((S, width), -1, np.int32)
        for i, e in enumerate(entries):
            row = cache.table(e.request_id, g)
            t[i, :len(row)] = row
        tables.append(t)

    arrays = [token_ids, positions, seq_of_token, cu, start, ctx_len, slots, want_rows] + \
             [t.reshape(-1) for t in tables]
    offsets, total = [], 0
    for a in arrays:
        offsets.append(total)
        total += _align4(a.size)
    host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=(device.type == "cuda"))
    hv = host.numpy()
    for a, o in zip(arrays, offsets):
        hv[o:o + a.size] = a
    dev = host.to(device, non_blocking=True)

    def view(i):
        return dev[offsets[i]:offsets[i] + arrays[i].size]

    n_max = max((len(e.tokens) for e in entries), default=0)
    return StepContext(
        act_dtype=act_dtype, device=device, num_tokens=T, num_seqs=S, num_wanted=len(want),
        seqs=seqs, token_ids=view(0), positions=view(1), seq_of_token=view(2), cu_tokens=view(3),
        start_pos=view(4), context_len=view(5), slots=view(6), want_rows=view(7),
        block_tables=[view(8 + g).view(S, tables[g].shape[1]) for g in range(n_groups)],
        decode_only=(n_max == 1), max_tokens_per_seq=n_max,
        max_context_len=int(ctx_len.max()) if S else 0,
    )
