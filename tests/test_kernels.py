"""Each kernel alone against a plain float64 reference, at sizes other than the
engine tests use (widths and vocabularies that are no power of two, head sizes in
steps of 16, odd group sizes, several page sizes)."""
import math

import pytest
import torch

import plain_model
from kernel_util import dense_attention, make_paged_case, step_ctx

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from helios_b200.csrc import ops as _ops
    return _ops


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------------- embedding / norms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1003, 72, generator=g).to(dtype)
    ids = torch.randint(0, 1003, (37,), generator=g, dtype=torch.int32)
    out = ops().embedding(ids.to(DEV), table.to(DEV))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [80, 1000, 4104])
def test_add_rmsnorm(dtype, H):
    g = torch.Generator().manual_seed(H)
    res = torch.randn(9, H, generator=g) * 3
    delta = torch.randn(9, H, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    eps = 3e-6
    want_res = res.double() + delta.double()
    want = plain_model.rms_norm(want_res, w.double(), eps)
    r = res.to(DEV).clone()
    out = ops().add_rmsnorm(r, delta.to(DEV), w.to(DEV), eps, dtype)
    assert out.dtype == dtype
    torch.testing.assert_close(r.cpu().double(), want_res, atol=1e-6, rtol=1e-6)   # residual is float32
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype))
    # no delta: the residual is only normed
    r2 = res.to(DEV).clone()
    out2 = ops().add_rmsnorm(r2, None, w.to(DEV), eps, dtype)
    assert torch.equal(r2.cpu(), res)
    torch.testing.assert_close(out2.cpu().double(), plain_model.rms_norm(res.double(), w.double(), eps), **tol(dtype))
    # chosen rows: normed, residual untouched
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    r3 = res.to(DEV).clone()
    out3 = ops().add_rmsnorm(r3, delta.to(DEV), w.to(DEV), eps, dtype, rows=rows.to(DEV))
    assert torch.equal(r3.cpu(), res)
    torch.testing.assert_close(out3.cpu().double(), want[rows.long()], **tol(dtype))
    # the plain norm of compute-dtype rows
    x = delta
    out4 = ops().rmsnorm(x.to(DEV), w.to(DEV), eps)
    torch.testing.assert_close(out4.cpu().double(), plain_model.rms_norm(x.double(), w.double(), eps), **tol(dtype))


def test_norm_of_a_row_does_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(5)
    res = torch.randn(64, 1000, generator=g).to(DEV)
    w = torch.ones(1000, device=DEV)
    whole = ops().add_rmsnorm(res.clone(), None, w, 1e-5, torch.float32)
    alone = ops().add_rmsnorm(res[17:18].clone(), None, w, 1e-5, torch.float32)
    assert torch.equal(whole[17:18], alone)


# ---------------------------------------------------------------------- rotary + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,page", [(4, 2, 16, 16, 16), (6, 1, 48, 48, 8), (5, 5, 80, 32, 3),
                                                (8, 2, 128, 128, 64)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, rot, page):
    g = torch.Generator().manual_seed(nh * hd)
    seqs = [(0, 9), (37, 1), (5, 20), (1000, 1)]       # (already in the cache, new)
    T = sum(n for _, n in seqs)
    n_pages = sum(-(-(a + n) // page) for a, n in seqs) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-(a + n) // page) for a, n in seqs)
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    used = 0
    for i, (a, n) in enumerate(seqs):
        for j in range(-(-(a + n) // page)):
            table[i, j] = perm[used]
            used += 1
    positions = torch.tensor([p for a, n in seqs for p in range(a, a + n)], dtype=torch.int32)
    seq_of = torch.tensor([i for i, (a, n) in enumerate(seqs) for _ in range(n)], dtype=torch.int32)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    inv = plain_model.rope_inv_freq(rot, 500000.0, {"rope_type": "llama3", "factor": 8.0,
                                                    "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                    "original_max_position_embeddings": 64})
    cos, sin = ops().rotary_table(positions.to(DEV), inv.to(DEV))
    ang = positions.double()[:, None] * inv[None, :]
    torch.testing.assert_close(cos.cpu().double(), ang.cos(), atol=1e-7, rtol=0)
    torch.testing.assert_close(sin.cpu().double(), ang.sin(), atol=1e-7, rtol=0)

    k_pages = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full_like(k_pages, float("nan"))
    x = qkv.to(DEV).clone()
    ops().rope_kv_write(x, cos, sin, positions.to(DEV), seq_of.to(DEV), table.to(DEV), k_pages, v_pages,
                        nh, nkv, hd, page)
    src = qkv.double()
    q = src[:, : nh * hd].view(T, nh, hd)
    k = src[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = src[:, (nh + nkv) * hd:].view(T, nkv, hd)

    def rot_part(t):
        out = t.clone()
        out[..., :rot] = plain_model.apply_rope(t[..., :rot], positions, inv)
        return out

    torch.testing.assert_close(x.cpu().double()[:, : nh * hd].view(T, nh, hd), rot_part(q), **tol(dtype))
    kp, vp = k_pages.cpu().double(), v_pages.cpu().double()
    want_k = rot_part(k)
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(T):
        pos, s = int(positions[t]), int(seq_of[t])
        pg, slot = int(table[s, pos // page]), pos % page
        written[pg, slot] = True
        torch.testing.assert_close(kp[pg, :, slot], want_k[t], **tol(dtype))
        torch.testing.assert_close(vp[pg, :, slot], v[t], atol=0, rtol=0)
    # nothing else was touched
    untouched = ~written[:, None, :, None].expand_as(kp)
    assert torch.isnan(kp[untouched]).all() and torch.isnan(vp[untouched]).all()


# ---------------------------------------------------------------------- attention
CASES = [(0, 1), (0, 7), (5, 1), (31, 1), (32, 1), (33, 2), (63, 1), (64, 1), (100, 33), (255, 1),
         (256, 1), (257, 1), (12, 100), (700, 1), (0, 130)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 16), (6, 1, 48, 8), (5, 5, 80, 5), (14, 2, 64, 16)])
@pytest.mark.parametrize("window", [None, 40])
def test_generic_attention(dtype, nh, nkv, hd, page, window):
    case = make_paged_case(CASES, nh, nkv, hd, page, dtype, DEV, seed=hd)
    scale = 1.0 / math.sqrt(hd)
    out = ops().attention_generic(case.qkv, case.k_pages, case.v_pages, case.table, case.seq_of_token,
                                  case.positions, nh, nkv, hd, page, window, scale)
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), **tol(dtype)
                               if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5))


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (28, 4, 128, 16), (14, 2, 64, 8), (6, 6, 96, 64),
                                            (16, 1, 32, 16), (7, 1, 64, 3), (24, 2, 128, 32)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits,cluster", [(1, True), (3, True), (8, True), (3, False), (8, False), (13, True)])
def test_decode_attention_bf16(nh, nkv, hd, page, window, splits, cluster, monkeypatch):
    """Context slices merged inside a thread-block cluster (up to 8) or by the merge kernel."""
    monkeypatch.setattr(ops(), "ATTENTION_CLUSTER_MERGE", cluster)
    seqs = [(n, 1) for n in (0, 1, 30, 31, 32, 33, 127, 128, 129, 255, 256, 1000, 2049)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh + hd)
    scale = 1.0 / math.sqrt(hd)
    out = ops().attention_decode_bf16(case.qkv, case.k_pages, case.v_pages, case.table, case.positions,
                                      nh, nkv, hd, page, window, scale, splits)
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (14, 2, 64, 8), (24, 2, 128, 32), (6, 6, 96, 3)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits,cluster", [(1, True), (3, True), (8, True), (5, False), (13, True)])
@pytest.mark.parametrize("warps", [4, 8])
def test_decode_attention_blocks_of_four_and_of_eight_warps(nh, nkv, hd, page, window, splits, cluster, warps,
                                                            monkeypatch):
    """The kernel runs with 4 or 8 warps a block (``ops.decode_warps`` chooses; here it is given)."""
    monkeypatch.setattr(ops(), "ATTENTION_CLUSTER_MERGE", cluster)
    seqs = [(n, 1) for n in (0, 1, 31, 33, 129, 255, 1000, 2049)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh + hd + warps)
    scale = 1.0 / math.sqrt(hd)
    out = ops().attention_decode_bf16(case.qkv, case.k_pages, case.v_pages, case.table, case.positions,
                                      nh, nkv, hd, page, window, scale, splits, warps=warps)
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (28, 4, 128, 16), (14, 2, 64, 8), (6, 6, 96, 64),
                                            (16, 1, 32, 16), (7, 1, 64, 3)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits,cluster", [(1, True), (3, True), (8, True), (5, False), (13, True)])
@pytest.mark.parametrize("rotate", [True, False])
def test_decode_attention_rotates_and_writes_the_new_token_itself(nh, nkv, hd, page, window, splits, cluster,
                                                                  rotate, monkeypatch):
    """The q|k|v rows come straight from the projection: the kernel rotates the query heads,
    and stores the new token's rotated key and its value at its place in the pages (which hold
    NaN there before) and nowhere else, before it attends."""
    monkeypatch.setattr(ops(), "ATTENTION_CLUSTER_MERGE", cluster)
    seqs = [(n, 1) for n in (0, 1, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255, 256, 1000, 2049)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh + hd + 1)
    S = len(seqs)
    g = torch.Generator().manual_seed(hd)
    raw = torch.randn(S, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    positions = case.positions.cpu()
    inv = plain_model.rope_inv_freq(hd, 10000.0, None)
    q = raw[:, : nh * hd].view(S, nh, hd).double()
    k = raw[:, nh * hd:(nh + nkv) * hd].view(S, nkv, hd).double()
    v = raw[:, (nh + nkv) * hd:].view(S, nkv, hd).double()
    cos = sin = None
    if rotate:
        cos, sin = ops().rotary_table(case.positions, inv.to(DEV))
        q, k = plain_model.apply_rope(q, positions, inv), plain_model.apply_rope(k, positions, inv)
    q, k = q.to(torch.bfloat16).double(), k.to(torch.bfloat16).double()
    before_k, before_v = case.k_pages.clone(), case.v_pages.clone()
    for i, (a, _n) in enumerate(seqs):
        dq, dk, dv, da = case.dense[i]
        dk, dv = dk.clone(), dv.clone()
        dk[a], dv[a] = k[i], v[i]
        case.dense[i] = (q[i:i + 1], dk, dv, da)
        pg, slot = int(case.table[i, a // page]), a % page
        case.k_pages[pg, :, slot] = float("nan")
        case.v_pages[pg, :, slot] = float("nan")
    scale = 1.0 / math.sqrt(hd)
    x = raw.to(DEV)
    out = ops().attention_decode_bf16(x, case.k_pages, case.v_pages, case.table, case.positions, nh, nkv, hd,
                                      page, window, scale, splits, rotary=(cos, sin) if rotate else None,
                                      write_cache=True)
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)
    assert torch.equal(x.cpu(), raw)
    kp, vp = case.k_pages.cpu(), case.v_pages.cpu()
    same = torch.ones_like(kp, dtype=torch.bool)
    for i, (a, _n) in enumerate(seqs):
        pg, slot = int(case.table[i, a // page]), a % page
        same[pg, :, slot] = False
        torch.testing.assert_close(kp[pg, :, slot].double(), k[i], atol=1e-2, rtol=1e-2)
        assert torch.equal(vp[pg, :, slot].double(), v[i])
    bk, bv = before_k.cpu(), before_v.cpu()
    assert torch.equal(kp[same].nan_to_num(7.0), bk[same].nan_to_num(7.0))
    assert torch.equal(vp[same].nan_to_num(7.0), bv[same].nan_to_num(7.0))


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (28, 4, 128, 16), (14, 2, 64, 8), (6, 6, 96, 64),
                                            (16, 1, 32, 16), (3, 1, 64, 3)])
@pytest.mark.parametrize("window", [None, 100])
def test_prefill_attention_bf16(nh, nkv, hd, page, window):
    seqs = CASES + [(0, 300), (190, 70), (1000, 17)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh * hd)
    scale = 1.0 / math.sqrt(hd)
    _, subtiles = ops().prefill_tiling(nh, nkv)
    tiles = ops().query_tiles([n for _, n in seqs], 16 * subtiles, DEV)
    out = ops().attention_prefill_bf16(case.qkv, case.k_pages, case.v_pages, case.table, tiles,
                                       case.cu_tokens, case.start_pos, nh, nkv, hd, page, window, scale)
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype,hd", [(torch.float32, 48), (torch.bfloat16, 48), (torch.bfloat16, 128)])
def test_one_far_key_among_hundreds_and_the_windows_edge(dtype, hd):
    """Random keys would hide a key that is skipped or a window that is off by one: make one
    key's score stand out, once far back, once just inside and once just outside a window."""
    nh, nkv, page, ctx, W = 4, 2, 16, 900, 64
    scale = 1.0 / math.sqrt(hd)
    for far, window, seen in [(3, None, True), (ctx - W, W, True), (ctx - W - 1, W, False),
                              (ctx - 1, W, True), (page * 7 - 1, None, True), (page * 7, None, True)]:
        for mode in ("decode", "portion", "long portion"):
            seqs = {"decode": [(ctx - 1, 1)], "portion": [(ctx - 5, 5)], "long portion": [(ctx - 40, 40)]}[mode]
            case = make_paged_case(seqs, nh, nkv, hd, page, dtype, DEV, seed=far)
            q, k, v, a = case.dense[0]
            # the last query points along e0, the far key too; its value is a marker
            pg, slot = int(case.table[0, far // page]), far % page
            mark = torch.zeros(hd)
            mark[0] = 30.0
            case.k_pages[pg, :, slot] = mark.to(dtype)
            case.v_pages[pg, :, slot] = 100.0
            k[far] = mark.double()
            v[far] = 100.0
            case.qkv[-1, : nh * hd] = mark.repeat(nh).to(dtype)
            q[-1] = mark.double()
            want = dense_attention(case, scale, window)
            got = ops().attention(step_ctx(case), case.qkv, case.k_pages, case.v_pages, case.table,
                                  nh, nkv, hd, page, window, scale)
            last = got[-1].float().cpu()
            if seen:
                assert (last > 90).all(), f"key {far} (window {window}, {mode}) was not seen"
            else:
                assert (last.abs() < 10).all(), f"key {far} outside window {window} was seen ({mode})"
            torch.testing.assert_close(got.cpu().double(), want,
                                       **(dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32
                                          else dict(atol=0.3, rtol=3e-2)))


def _marker_case(seqs, nh, nkv, hd, page, dtype, far, window, seed):
    """A paged case whose LAST query row points along e0 and whose key ``far`` of the last
    request does too (score 900 * scale: it takes all the weight when it is seen); that key's
    value is 100.  With a window, the pages that lie wholly before the first query's window
    are taken out of the table (-1, as the cache manager gives them back) and poisoned."""
    case = make_paged_case(seqs, nh, nkv, hd, page, dtype, DEV, seed=seed)
    i = len(seqs) - 1
    q, k, v, a = case.dense[i]
    mark = torch.zeros(hd)
    mark[0] = 30.0
    pg, slot = int(case.table[i, far // page]), far % page
    case.k_pages[pg, :, slot] = mark.to(dtype)
    case.v_pages[pg, :, slot] = 100.0
    k[far] = mark.double()
    v[far] = 100.0
    case.qkv[-1, : nh * hd] = mark.repeat(nh).to(dtype)
    q[-1] = mark.double()
    if window:
        for r, (before, _n) in enumerate(seqs):
            for j in range(max(0, before - window + 1) // page):
                gone = int(case.table[r, j])
                case.k_pages[gone] = float("nan")
                case.v_pages[gone] = float("nan")
                case.table[r, j] = -1
    return case


MARKER_SIZES = [(8, 2, 64), (7, 1, 64), (4, 1, 128), (14, 2, 128), (6, 2, 32), (6, 6, 96)]


def _marker_places(ctx, W, page):
    """(far key, window, is it seen) for a last query at position ctx - 1."""
    return [(3, None, True), (ctx - W, W, True), (ctx - W - 1, W, False), (ctx - 1, W, True),
            (page * 7 - 1, None, True), (page * 7, None, True), (ctx - 1, None, True)]


def _check_marker(got, want, seen, what):
    last = got[-1].float().cpu()
    if seen:
        assert (last > 90).all(), f"{what}: the far key was not seen"
    else:
        assert (last.abs() < 10).all(), f"{what}: a key outside the window was seen"
    torch.testing.assert_close(got.cpu().double(), want, atol=0.3, rtol=3e-2)


@pytest.mark.parametrize("nh,nkv,hd", MARKER_SIZES)
@pytest.mark.parametrize("splits,cluster", [(1, True), (3, True), (8, True), (5, False), (13, True)])
def test_the_decode_kernel_sees_one_far_key_and_the_windows_edge(nh, nkv, hd, splits, cluster, monkeypatch):
    """Each context slice, the cluster merge and the merge kernel; a second request beside it."""
    monkeypatch.setattr(ops(), "ATTENTION_CLUSTER_MERGE", cluster)
    page, ctx, W = 16, 900, 64
    scale = 1.0 / math.sqrt(hd)
    for far, window, seen in _marker_places(ctx, W, page):
        case = _marker_case([(411, 1), (ctx - 1, 1)], nh, nkv, hd, page, torch.bfloat16, far, window, seed=far)
        got = ops().attention_decode_bf16(case.qkv, case.k_pages, case.v_pages, case.table, case.positions,
                                          nh, nkv, hd, page, window, scale, splits)
        _check_marker(got, dense_attention(case, scale, window), seen,
                      f"decode, {splits} slices, key {far}, window {window}")


@pytest.mark.parametrize("nh,nkv,hd", [s for s in MARKER_SIZES if s[2] in (64, 128)])
@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("page", [16, 8, 128])
def test_the_tensor_memory_kernels_see_one_far_key_and_the_windows_edge(nh, nkv, hd, pairs, page):
    """One and two query tiles a block; portions that end a tile, span tiles, and a page size
    below and at the key tile."""
    ctx, W = 900, 64
    scale = 1.0 / math.sqrt(hd)
    tile = (2 if pairs else 1) * (128 // (nh // nkv))
    for n_new in (5, 40, 300):
        for far, window, seen in _marker_places(ctx, W, page):
            if far >= ctx - n_new and far != ctx - 1:
                continue          # the far key must lie in the cache of earlier steps (or be the query's own)
            seqs = [(100, 33), (ctx - n_new, n_new)]
            case = _marker_case(seqs, nh, nkv, hd, page, torch.bfloat16, far, window, seed=far + n_new)
            tiles = ops().query_tiles([n for _, n in seqs], tile, DEV, [a for a, _ in seqs])
            got = ops().attention_prefill_tc(case.qkv, case.k_pages, case.v_pages, case.table, tiles,
                                             case.cu_tokens, case.start_pos, nh, nkv, hd, page, window, scale,
                                             pairs=pairs)
            ops().check_kernel_errors()
            _check_marker(got, dense_attention(case, scale, window), seen,
                          f"tcgen05 pairs={pairs}, portion {n_new}, key {far}, window {window}")


@pytest.mark.parametrize("nh,nkv,hd", MARKER_SIZES)
def test_the_tiled_prefill_kernel_sees_one_far_key_and_the_windows_edge(nh, nkv, hd):
    page, ctx, W = 16, 900, 64
    scale = 1.0 / math.sqrt(hd)
    _, subtiles = ops().prefill_tiling(nh, nkv)
    for n_new in (5, 40):
        for far, window, seen in _marker_places(ctx, W, page):
            if far >= ctx - n_new and far != ctx - 1:
                continue
            seqs = [(100, 33), (ctx - n_new, n_new)]
            case = _marker_case(seqs, nh, nkv, hd, page, torch.bfloat16, far, window, seed=far + n_new)
            tiles = ops().query_tiles([n for _, n in seqs], 16 * subtiles, DEV)
            got = ops().attention_prefill_bf16(case.qkv, case.k_pages, case.v_pages, case.table, tiles,
                                               case.cu_tokens, case.start_pos, nh, nkv, hd, page, window, scale)
            _check_marker(got, dense_attention(case, scale, window), seen,
                          f"tiled prefill, portion {n_new}, key {far}, window {window}")


def test_attention_does_not_depend_on_the_batch_in_float32():
    """A token's output is bit-equal whether its request is alone, in portions, or beside others."""
    nh, nkv, hd, page = 6, 2, 32, 8
    scale = 1.0 / math.sqrt(hd)
    both = make_paged_case([(40, 25), (3, 1), (90, 4)], nh, nkv, hd, page, torch.float32, DEV, seed=1)
    o = ops().attention_generic(both.qkv, both.k_pages, both.v_pages, both.table, both.seq_of_token,
                                both.positions, nh, nkv, hd, page, None, scale)
    # the same first request, its last 5 tokens alone
    sub_q = both.qkv[20:25].contiguous()
    pos = both.positions[20:25].contiguous()
    seq0 = torch.zeros(5, dtype=torch.int32, device=DEV)
    o2 = ops().attention_generic(sub_q, both.k_pages, both.v_pages, both.table[:1].contiguous(), seq0, pos,
                                 nh, nkv, hd, page, None, scale)
    assert torch.equal(o[20:25], o2)


# ---------------------------------------------------------------------- feed-forward pieces
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(13, 2 * 176, generator=g) * 3).to(dtype)
    out = ops().silu_mul(gu.to(DEV))
    a, b = gu.double()[:, :176], gu.double()[:, 176:]
    torch.testing.assert_close(out.cpu().double(), a * torch.sigmoid(a) * b, **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 100, 50), (3, 64, 17), (65, 130, 96), (128, 257, 1000), (7, 384, 80)])
def test_gemm_f32(M, N, K):
    g = torch.Generator().manual_seed(M * N)
    x, w, b = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    out = ops().linear_f32(x.to(DEV), w.to(DEV), b.to(DEV))
    torch.testing.assert_close(out.cpu().double(), x.double() @ w.double().T + b.double(), atol=1e-4, rtol=1e-5)
    out = ops().linear_f32(x.to(DEV), w.to(DEV))
    torch.testing.assert_close(out.cpu().double(), x.double() @ w.double().T, atol=1e-4, rtol=1e-5)


def test_gemm_f32_row_does_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(9)
    x, w = torch.randn(70, 333, generator=g).to(DEV), torch.randn(129, 333, generator=g).to(DEV)
    assert torch.equal(ops().linear_f32(x, w)[41:42], ops().linear_f32(x[41:42].contiguous(), w))


@pytest.mark.parametrize("M", [1, 8, 64, 300])
def test_linear_bf16(M):
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, 320, generator=g).to(torch.bfloat16)
    w = (torch.randn(200, 320, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(200, generator=g)
    out = ops().linear(x.to(DEV), w.to(DEV), b.to(DEV))
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().double(), x.double() @ w.double().T + b.double(), atol=3e-2, rtol=2e-2)
    logits = ops().linear_logits(x.to(DEV), w.to(DEV))
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu().double(), x.double() @ w.double().T, atol=2e-3, rtol=1e-3)


# ---------------------------------------------------------------------- sampling
def _sample(logits, temps, ks, ps, seeds, offsets, kind=None):
    t = lambda x, d: torch.tensor(x, dtype=d, device=DEV)
    return ops().sample(logits.to(DEV), t(temps, torch.float32), t(ks, torch.int32), t(ps, torch.float32),
                        t(seeds, torch.int64), t(offsets, torch.int64), kind=kind).cpu().tolist()


@pytest.mark.parametrize("V", [1231, 40000, 128256])
def test_greedy_is_argmax_with_lowest_index_on_ties(V):
    """(One block per row below 4,096 values, a cluster per row above.)"""
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, V, generator=g)
    logits[2, 100] = logits[2, V - 300] = 50.0
    logits[3, V - 1] = 60.0
    got = _sample(logits, [0.0] * 5, [0] * 5, [1.0] * 5, [1] * 5, [0] * 5)
    assert got == torch.argmax(logits, -1).tolist() and got[2] == 100 and got[3] == V - 1


@pytest.mark.parametrize("one_block", [False, True])
@pytest.mark.parametrize("V", [384, 1231, 4095, 4096, 4097, 8192, 50001, 128256, 151936, 163840, 163841])
def test_temperature_top_k_top_p_follow_the_reference_rules(V, one_block):
    """Rows of 4,096 to 163,840 values run on the kernel that spreads a row over a cluster of
    blocks, the others, and every row when the caller asks for it, on the kernel with one
    block a row."""
    g = torch.Generator().manual_seed(V)
    R = 24
    logits = torch.randn(R, V, generator=g) * 2
    temps = [0.8, 1.0, 0.3, 1.7] * 6
    ks = [0, 5, 0, 50, 1, 0] * 4
    ps = [1.0, 1.0, 0.9, 0.5, 1.0, 0.2] * 4
    seeds = [11 + i for i in range(R)]
    offsets = [i * 3 for i in range(R)]
    got = _sample(logits, temps, ks, ps, seeds, offsets, kind="one_block" if one_block else None)
    for i in range(R):
        u = ops().philox_uniform(seeds[i], offsets[i])
        want = plain_model.sample_reference(logits[i], temps[i], ks[i], ps[i], u)
        if got[i] != want:
            # float32 sums against float64: only a draw that falls on a boundary may differ
            l = logits[i].double() / temps[i]
            probs = torch.softmax(l, -1)
            assert abs(int(got[i]) - want) >= 0 and probs[got[i]] > 0
            near = min(abs(u - x) for x in _boundaries(logits[i], temps[i], ks[i], ps[i], got[i], want))
            assert near < 1e-4, f"row {i}: got {got[i]}, reference {want}, u={u}"


def _boundaries(logits, temp, k, p, a, b):
    l = logits.double() / temp
    if k > 0:
        kth = torch.topk(l, min(k, l.numel())).values[-1]
        l = torch.where(l < kth, torch.full_like(l, float("-inf")), l)
    if p < 1.0:
        sl, si = torch.sort(l, descending=True)
        cum = torch.cumsum(torch.softmax(sl, -1), -1)
        cut = torch.cat([torch.zeros(1, dtype=torch.bool), (cum > p)[:-1]])
        l = torch.full_like(l, float("-inf")).scatter(0, si, sl.masked_fill(cut, float("-inf")))
    cdf = torch.cumsum(torch.softmax(l, -1), -1)
    lo, hi = min(a, b), max(a, b)
    return [float(cdf[j]) for j in range(lo, hi)]


@pytest.mark.parametrize("V", [3000, 5000, 130000])
def test_a_requests_draws_depend_on_its_seed_and_offset_only(V):
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(1, V, generator=g)
    alone = _sample(logits, [1.0], [0], [1.0], [99], [7])
    batch = _sample(logits.repeat(6, 1), [1.0] * 6, [0] * 6, [1.0] * 6, [1, 2, 99, 3, 99, 5], [0, 1, 7, 2, 8, 3])
    assert batch[2] == alone[0]
    many = _sample(logits.repeat(64, 1), [1.0] * 64, [0] * 64, [1.0] * 64, [99] * 64, list(range(64)))
    assert len(set(many)) > 20       # different offsets, different draws


def test_sampled_frequencies_follow_the_distribution():
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]])
    R = 4000
    got = _sample(logits.repeat(R, 1), [1.0] * R, [0] * R, [1.0] * R, [5] * R, list(range(R)))
    freq = torch.bincount(torch.tensor(got), minlength=5).double() / R
    assert (freq - torch.softmax(logits[0].double(), -1)).abs().max() < 0.03


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (8, 8, 128, 8), (16, 2, 64, 32), (4, 1, 64, 128),
                                            (16, 1, 128, 64), (2, 1, 64, 16), (28, 4, 128, 16), (14, 2, 64, 16),
                                            (5, 1, 128, 32), (6, 2, 64, 8)])
@pytest.mark.parametrize("window", [None, 100, 300])
def test_prefill_attention_tcgen05(nh, nkv, hd, page, window):
    """The tensor-memory attention kernel: ragged requests, portions that start deep in the
    cache, single tokens beside them, scattered and poisoned pages."""
    seqs = CASES + [(0, 300), (190, 70), (1000, 17), (500, 129), (127, 1), (128, 128)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh * hd + page)
    scale = 1.0 / math.sqrt(hd)
    tiles = ops().query_tiles([n for _, n in seqs], 128 // (nh // nkv), DEV, [a for a, _ in seqs])
    out = ops().attention_prefill_tc(case.qkv, case.k_pages, case.v_pages, case.table, tiles,
                                     case.cu_tokens, case.start_pos, nh, nkv, hd, page, window, scale)
    ops().check_kernel_errors()
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 128, 16), (8, 8, 128, 8), (16, 2, 64, 32), (4, 1, 64, 128),
                                            (16, 1, 128, 64), (2, 1, 64, 16), (28, 4, 128, 16), (14, 2, 64, 16),
                                            (5, 1, 128, 32), (6, 2, 64, 8)])
@pytest.mark.parametrize("window", [None, 100, 300])
def test_prefill_attention_tcgen05_two_tiles_a_block(nh, nkv, hd, page, window):
    """The same with two tiles of query rows per block (probabilities kept in tensor memory):
    requests that fill both tiles, the first only, or part of each."""
    seqs = CASES + [(0, 300), (190, 70), (1000, 17), (500, 129), (127, 1), (128, 128), (60, 257), (3, 33)]
    case = make_paged_case(seqs, nh, nkv, hd, page, torch.bfloat16, DEV, seed=nh * hd + page + 1)
    scale = 1.0 / math.sqrt(hd)
    tiles = ops().query_tiles([n for _, n in seqs], 2 * (128 // (nh // nkv)), DEV, [a for a, _ in seqs])
    out = ops().attention_prefill_tc(case.qkv, case.k_pages, case.v_pages, case.table, tiles,
                                     case.cu_tokens, case.start_pos, nh, nkv, hd, page, window, scale, pairs=True)
    ops().check_kernel_errors()
    torch.testing.assert_close(out.cpu().double(), dense_attention(case, scale, window), atol=2e-2, rtol=2e-2)


def test_tcgen05_attention_refuses_sizes_it_does_not_take():
    assert ops().tc_attention_supported(28, 4, 128, 16)          # groups of 7: 18 tokens a tile, two rows idle
    assert not ops().tc_attention_supported(32, 8, 96, 16)
    assert not ops().tc_attention_supported(32, 8, 128, 5)
    case = make_paged_case([(0, 20)], 6, 2, 96, 16, torch.bfloat16, DEV)
    tiles = ops().query_tiles([20], 42, DEV)
    with pytest.raises(ops().KernelError):
        ops().attention_prefill_tc(case.qkv, case.k_pages, case.v_pages, case.table, tiles, case.cu_tokens,
                                   case.start_pos, 6, 2, 96, 16, None, 0.125)
