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
    # left by the plan's position encoding for the mixers that were given none of their own
    rotary_cos: Optional[torch.Tensor] = None
    rotary_sin: Optional[torch.Tensor] = None
    # what the parts make once per step (a position encoding's tables under its identity);
    # emptied when a forward pass begins
    step_tables: dict = field(default_factory=dict)
    # per-request state of the parts of the block that runs now: id(part) -> [slots, ...]
    block_states: dict = field(default_factory=dict)
    # the norm the block after the running one applies first (None: unknown, or the end)
    norm_after_block: object = None
    extras: dict = field(default_factory=dict)

    def part_state(self, part) -> Optional[torch.Tensor]:
        """The [slots, *shape] tensor of a part that declared a ``state_spec`` (not the
        mixer: that one gets its state as an argument); a request's row is its slot."""
        return self.block_states.get(id(part))


def _align4(n: int) -> int:
    return (n + 3) & ~3


class MetaLayout:
    """Where each integer array of a step lies in the one int32 buffer that is copied to
    the device: token ids, positions, request of each token, cumulative tokens, first
    position, context length and slot of each request, wanted rows, and one block table
    [requests, width] per cache group."""

    def __init__(self, num_seqs: int, num_tokens: int, num_wanted: int, table_widths: List[int]) -> None:
        self.S, self.T, self.R = num_seqs, num_tokens, num_wanted
        self.widths = list(table_widths)
        sizes = [num_tokens, num_tokens, num_tokens, num_seqs + 1, num_seqs, num_seqs, num_seqs,
                 num_wanted] + [num_seqs * w for w in self.widths]
        self.sizes = sizes
        self.offsets, total = [], 0
        for n in sizes:
            self.offsets.append(total)
            total += _align4(n)
        self.total = max(total, 4)

    def host_views(self, host: np.ndarray) -> List[np.ndarray]:
        return [host[o:o + n] for o, n in zip(self.offsets, self.sizes)]

    def device_views(self, dev: torch.Tensor) -> List[torch.Tensor]:
        return [dev[o:o + n] for o, n in zip(self.offsets, self.sizes)]


def _fill_decode(layout, entries, cache, pad_page, rows_kept, token_ids, positions, seq_of_token, cu,
                 start, ctx_len, slots, want, tables) -> List[SeqSlice]:
    """``fill_meta`` for a captured decode step (one token a request, one row a request): whole
    arrays at once instead of slices per request, and a block-table row is written again only
    when its request or that request's table has changed since this buffer was last filled
    (``rows_kept``: row -> (request, table version)); with hundreds of requests the per-request
    work of the general path costs more than the step."""
    S, n_real = layout.S, len(entries)
    requests = cache.requests
    lengths, slot_of, seqs = [], [], []
    for i, e in enumerate(entries):
        req = requests[e.request_id]
        lengths.append(req.length)
        slot_of.append(req.slot)
        seqs.append(SeqSlice(e.request_id, req.slot, req.length, 1, i))
        key = (e.request_id, req.version)
        if rows_kept.get(i) != key:
            rows_kept[i] = key
            for g, t in enumerate(tables):
                row = cache.table_array(e.request_id, g)
                t[i, :len(row)] = row
                t[i, len(row):] = -1
    for i in range(n_real, S):
        if rows_kept.get(i) != "padding":
            rows_kept[i] = "padding"
            for g, t in enumerate(tables):
                t[i, :1] = pad_page[g]
                t[i, 1:] = -1
    pad = S - n_real
    token_ids[:S] = [e.tokens[0] for e in entries] + [0] * pad
    positions[:S] = lengths + [0] * pad
    start[:S] = positions[:S]
    ctx_len[:S] = positions[:S] + 1
    slots[:S] = slot_of + [0] * pad
    seq_of_token[:S] = _iota(S)
    want[:S] = seq_of_token[:S]
    cu[:S + 1] = _iota(S + 1)
    return seqs


_iotas: dict = {}


def _iota(n: int) -> np.ndarray:
    a = _iotas.get(n)
    if a is None:
        a = _iotas[n] = np.arange(n, dtype=np.int32)
    return a


def fill_meta(layout: MetaLayout, host: np.ndarray, entries: Sequence[StepEntry], cache,
              pad_page: Optional[List[int]] = None, page_size: int = 1,
              rows_kept: Optional[dict] = None) -> List[SeqSlice]:
    """Write the step's arrays into ``host`` (int32, ``layout.total`` long).  Requests
    beyond ``len(entries)`` up to ``layout.S`` are padding whose keys and values go to the
    spare page ``pad_page[group]`` that no request ever gets; an entry without a wanted place
    gets its last token as one when the layout has a row for every request.  ``rows_kept``:
    what the buffer's block-table rows hold from the fill before (a caller that fills the
    same buffer step after step passes the same dict; see ``_fill_decode``)."""
    v = layout.host_views(host)
    token_ids, positions, seq_of_token, cu, start, ctx_len, slots, want = v[:8]
    tables = [t.reshape(layout.S, w) for t, w in zip(v[8:], layout.widths)]
    if rows_kept is not None and pad_page is not None and layout.S == layout.T \
            and all(len(e.tokens) == 1 and len(e.want) <= 1 for e in entries):
        return _fill_decode(layout, entries, cache, pad_page, rows_kept,
                            token_ids, positions, seq_of_token, cu, start, ctx_len, slots, want, tables)
    if rows_kept is not None:
        rows_kept.clear()
    for t in tables:
        t.fill(-1)
    seqs: List[SeqSlice] = []
    off, nw = 0, 0
    cu[0] = 0
    for i, e in enumerate(entries):
        n = len(e.tokens)
        p0 = cache.length(e.request_id)
        seqs.append(SeqSlice(e.request_id, cache.slot(e.request_id), p0, n, off))
        token_ids[off:off + n] = e.tokens
        positions[off:off + n] = np.arange(p0, p0 + n, dtype=np.int32)
        seq_of_token[off:off + n] = i
        start[i], ctx_len[i], slots[i] = p0, p0 + n, seqs[-1].slot
        for w in e.want:
            want[nw] = off + int(w)
            nw += 1
        if not e.want and pad_page is not None:
            want[nw] = off + n - 1           # a row nobody reads keeps the row count fixed
            nw += 1
        off += n
        cu[i + 1] = off
        for g, t in enumerate(tables):
            row = cache.table_array(e.request_id, g)
            t[i, :len(row)] = row
    # Padding requests (captured graphs): one token each at position 0; the last of them
    # also takes the tokens that fill the step up to ``layout.T``, at positions 0, 1, ...
    # Their keys and values all go to the spare page, whatever their position.
    n_pad = layout.S - len(entries)
    spare = layout.T - off - n_pad
    if spare < 0 or (spare > 0 and n_pad == 0):
        raise ValueError(f"{off} tokens of {len(entries)} requests do not fit a step of "
                         f"{layout.T} tokens and {layout.S} requests")
    for i in range(len(entries), layout.S):
        n = 1 + (spare if i == layout.S - 1 else 0)
        token_ids[off:off + n] = 0
        positions[off:off + n] = np.arange(n, dtype=np.int32)
        seq_of_token[off:off + n] = i
        start[i], ctx_len[i], slots[i] = 0, n, 0
        want[nw] = off
        nw += 1
        off += n
        cu[i + 1] = off
        for g, t in enumerate(tables):
            t[i, :-(-n // page_size)] = pad_page[g]
    return seqs


def context_from_views(layout: MetaLayout, dev: torch.Tensor, seqs: List[SeqSlice],
                       act_dtype: torch.dtype, device: torch.device, max_tokens_per_seq: int,
                       max_context_len: int) -> StepContext:
    v = layout.device_views(dev)
    return StepContext(
        act_dtype=act_dtype, device=device, num_tokens=layout.T, num_seqs=layout.S,
        num_wanted=layout.R, seqs=seqs, token_ids=v[0], positions=v[1], seq_of_token=v[2],
        cu_tokens=v[3], start_pos=v[4], context_len=v[5], slots=v[6], want_rows=v[7],
        block_tables=[t.view(layout.S, w) for t, w in zip(v[8:], layout.widths)],
        decode_only=(max_tokens_per_seq == 1), max_tokens_per_seq=max_tokens_per_seq,
        max_context_len=max_context_len)


def build_context(entries: Sequence[StepEntry], cache, act_dtype: torch.dtype,
                  device: torch.device) -> StepContext:
    """``cache`` is the cache manager: it knows every request's length, slot and block
    tables (pages for the new tokens must have been taken already)."""
    S = len(entries)
    T = sum(len(e.tokens) for e in entries)
    R = sum(len(e.want) for e in entries)
    widths = [max([len(cache.table(e.request_id, g)) for e in entries] + [1])
              for g in range(len(cache.groups))]
    layout = MetaLayout(S, T, R, widths)
    host = torch.empty(layout.total, dtype=torch.int32, pin_memory=(device.type == "cuda"))
    seqs = fill_meta(layout, host.numpy(), entries, cache)
    dev = host.to(device, non_blocking=True)
    n_max = max((len(e.tokens) for e in entries), default=0)
    max_ctx = max((s.start_pos + s.num_tokens for s in seqs), default=0)
    return context_from_views(layout, dev, seqs, act_dtype, device, n_max, max_ctx)
