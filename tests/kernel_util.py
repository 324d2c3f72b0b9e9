"""Helpers for the tests of single kernels: a paged cache built from dense keys and
values with scattered page ids and poisoned free pages, and dense float64 references."""
from __future__ import annotations

from types import SimpleNamespace

import torch


def make_paged_case(seqs, nh, nkv, hd, page_size, dtype, device, seed=0, extra_pages=5,
                    scatter=True):
    """seqs: list of (tokens already in the cache, new tokens).  Returns a namespace with the
    packed q ([T, (nh + 2 nkv) hd], only the q columns matter), pages, block table,
    per-token arrays, and the dense float64 q/k/v per request for the reference."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-(a + n) // page_size) for a, n in seqs) + extra_pages
    order = torch.randperm(total_pages, generator=g).tolist() if scatter else list(range(total_pages))
    k_pages = torch.full((total_pages, nkv, page_size, hd), float("nan"), dtype=torch.float32)
    v_pages = torch.full_like(k_pages, float("nan"))
    width = max(-(-(a + n) // page_size) for a, n in seqs)
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    dense, q_rows, positions, seq_of_token, cu, start = [], [], [], [], [0], []
    next_page = 0
    for i, (a, n) in enumerate(seqs):
        L = a + n
        k = torch.randn(L, nkv, hd, generator=g)
        v = torch.randn(L, nkv, hd, generator=g)
        q = torch.randn(n, nh, hd, generator=g)
        if dtype == torch.bfloat16:
            k, v, q = (t.to(torch.bfloat16).float() for t in (k, v, q))
        dense.append((q.double(), k.double(), v.double(), a))
        for j in range(-(-L // page_size)):
            page = order[next_page]
            next_page += 1
            table[i, j] = page
            lo, hi = j * page_size, min(L, (j + 1) * page_size)
            k_pages[page, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            v_pages[page, :, : hi - lo] = v[lo:hi].transpose(0, 1)
        q_rows.append(q.reshape(n, nh * hd))
        positions.extend(range(a, a + n))
        seq_of_token.extend([i] * n)
        cu.append(cu[-1] + n)
        start.append(a)
    T = cu[-1]
    qkv = torch.zeros(T, (nh + 2 * nkv) * hd)
    qkv[:, : nh * hd] = torch.cat(q_rows)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return SimpleNamespace(
        qkv=qkv.to(device=device, dtype=dtype).contiguous(),
        k_pages=k_pages.to(device=device, dtype=dtype), v_pages=v_pages.to(device=device, dtype=dtype),
        table=table.to(device), positions=i32(positions), seq_of_token=i32(seq_of_token),
        cu_tokens=i32(cu), start_pos=i32(start), dense=dense, seqs=seqs,
        nh=nh, nkv=nkv, hd=hd, page_size=page_size)


def dense_attention(case, scale, window=None):
    """float64 [T, nh * hd]: every new token over keys lo..its position
    (python/helios/exec/paged_attn.py:391-408 with the mask by position)."""
    outs = []
    rep = case.nh // case.nkv
    for q, k, v, a in case.dense:
        n = q.shape[0]
        kk = k.repeat_interleave(rep, dim=1)
        vv = v.repeat_interleave(rep, dim=1)
        scores = torch.einsum("qhd,khd->hqk", q, kk) * scale
        qpos = torch.arange(a, a + n)[:, None]
        kpos = torch.arange(k.shape[0])[None, :]
        mask = kpos > qpos
        if window:
            mask = mask | (kpos <= qpos - window)
        scores = scores.masked_fill(mask[None], float("-inf"))
        outs.append(torch.einsum("hqk,khd->qhd", torch.softmax(scores, -1), vv).reshape(n, -1))
    return torch.cat(outs)


def step_ctx(case):
    """What ops.attention reads of a StepContext."""
    n_max = max(n for _, n in case.seqs)
    return SimpleNamespace(
        seq_of_token=case.seq_of_token, positions=case.positions, cu_tokens=case.cu_tokens,
        start_pos=case.start_pos, num_seqs=len(case.seqs), decode_only=(n_max == 1),
        max_tokens_per_seq=n_max, max_context_len=max(a + n for a, n in case.seqs),
        seqs=[SimpleNamespace(num_tokens=n, start_pos=a) for a, n in case.seqs], extras={})
