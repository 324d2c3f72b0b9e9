"""The fused kernels of steps with very few tokens, each against float64 formulas
(python/helios/exec/model.py:109-114 norm, :148-153 rotation, :236-251 projections,
:336-337 feed-forward; python/helios/exec/paged_attn.py:74-85 cache write), at sizes the
engine tests do not have, and the rule that decides when they are used."""
import math

import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from helios_b200.csrc import ops as _ops
    return _ops


def _bf(t):
    return t.to(torch.bfloat16).float()


@pytest.mark.parametrize("T", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(896, 4864), (100, 40), (4096, 4096), (7, 8), (1000, 1224)])
def test_linear_into_the_residual(T, N, K):
    g = torch.Generator().manual_seed(T * N + K)
    res = torch.randn(T, N, generator=g) * 2
    x = _bf(torch.randn(T, K, generator=g))
    w = _bf(torch.randn(N, K, generator=g) * 0.05)
    r = res.to(DEV).clone()
    ops().small_linear_residual(r, x.to(DEV, torch.bfloat16), w.to(DEV, torch.bfloat16))
    want = res.double() + x.double() @ w.double().T
    torch.testing.assert_close(r.cpu().double(), want, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("T", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("I,K", [(4864, 896), (176, 80), (14336, 4096), (3, 16), (1001, 520)])
def test_norm_and_swiglu(T, I, K):
    g = torch.Generator().manual_seed(T * I + K)
    res = torch.randn(T, K, generator=g) * 3
    nw = 1 + 0.1 * torch.randn(K, generator=g)
    w = _bf(torch.randn(2 * I, K, generator=g) * (1.0 / math.sqrt(K)))
    eps = 3e-6
    out = ops().small_norm_swiglu(res.to(DEV), nw.to(DEV), eps, w.to(DEV, torch.bfloat16))
    # exact norm: the kernel rounds residual * weight to bfloat16 and scales by 1/rms after the sums
    h = plain_model.rms_norm(res.double(), nw.double(), eps)
    gate, up = h @ w.double()[:I].T, h @ w.double()[I:].T
    want = gate * torch.sigmoid(gate) * up
    assert out.shape == (T, I) and out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().double(), want, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("T", [1, 4, 8, 11, 16])
@pytest.mark.parametrize("nh,nkv,hd,K,bias,page", [(14, 2, 64, 896, True, 16), (4, 2, 16, 64, False, 8),
                                                   (5, 5, 48, 80, True, 5), (32, 8, 128, 4096, False, 16),
                                                   (6, 1, 24, 96, True, 3)])
@pytest.mark.parametrize("write", [True, False])
def test_norm_projection_rotation_and_cache_write(T, nh, nkv, hd, K, bias, page, write):
    g = torch.Generator().manual_seed(T + nh * hd + K)
    width = (nh + 2 * nkv) * hd
    res = torch.randn(T, K, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(K, generator=g)
    w = _bf(torch.randn(width, K, generator=g) * (1.0 / math.sqrt(K)))
    b = torch.randn(width, generator=g) * 0.5 if bias else None
    eps = 1e-5
    # tokens of three requests at scattered positions, pages scattered too
    n_req = 3
    seq_of = [i % n_req for i in range(T)]
    positions = [7 * (i // n_req) + 3 * (i % n_req) + (40 if i % n_req == 2 else 0) for i in range(T)]
    pages_per = max(positions) // page + 1
    table = torch.randperm(n_req * pages_per + 3, generator=g)[: n_req * pages_per].reshape(n_req, pages_per).int()
    total_pages = n_req * pages_per + 3
    k_pages = torch.full((total_pages, nkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    v_pages = k_pages.clone()
    inv = plain_model.rope_inv_freq(hd, 10000.0, None)
    pos_t = torch.tensor(positions, dtype=torch.float64)
    ang = pos_t[:, None] * inv[None]
    cos, sin = ang.cos().float(), ang.sin().float()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    qkv = ops().small_norm_qkv_rope(res.to(DEV), nw.to(DEV), eps, w.to(DEV, torch.bfloat16),
                                    None if b is None else b.to(DEV), cos.to(DEV), sin.to(DEV), i32(positions),
                                    i32(seq_of), table.to(DEV), k_pages, v_pages, nh, nkv, hd, page,
                                    write_cache=write)
    h = plain_model.rms_norm(res.double(), nw.double(), eps)
    full = h @ w.double().T + (b.double() if bias else 0)
    q = plain_model.apply_rope(full[:, : nh * hd].reshape(T, nh, hd), torch.tensor(positions), inv)
    k = plain_model.apply_rope(full[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), torch.tensor(positions), inv)
    v = full[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    tol = dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(qkv[:, : nh * hd].cpu().double().reshape(T, nh, hd), q, **tol)
    if write:
        seen = torch.zeros(total_pages, page, dtype=torch.bool)
        for t in range(T):
            pg, slot = int(table[seq_of[t], positions[t] // page]), positions[t] % page
            torch.testing.assert_close(k_pages[pg, :, slot].cpu().double(), k[t], **tol)
            torch.testing.assert_close(v_pages[pg, :, slot].cpu().double(), v[t], **tol)
            seen[pg, slot] = True
        # nothing else was written
        for pages in (k_pages, v_pages):
            assert torch.isnan(pages.cpu().float().permute(0, 2, 1, 3)[~seen]).all()
    else:
        torch.testing.assert_close(qkv[:, nh * hd:(nh + nkv) * hd].cpu().double().reshape(T, nkv, hd), k, **tol)
        torch.testing.assert_close(qkv[:, (nh + nkv) * hd:].cpu().double().reshape(T, nkv, hd), v, **tol)
        assert torch.isnan(k_pages.float()).all()


def test_a_row_does_not_depend_on_the_other_tokens_of_the_step():
    """Bit-equal results for a token alone and among fifteen others (T <= 8 and T > 8 run
    different instantiations of the kernel)."""
    g = torch.Generator().manual_seed(3)
    K, I = 896, 4864
    res = torch.randn(16, K, generator=g)
    nw = 1 + 0.1 * torch.randn(K, generator=g)
    w = _bf(torch.randn(2 * I, K, generator=g) * 0.03).to(DEV, torch.bfloat16)
    many = ops().small_norm_swiglu(res.to(DEV), nw.to(DEV), 1e-6, w)
    for t in (0, 7, 8, 15):
        alone = ops().small_norm_swiglu(res[t:t + 1].contiguous().to(DEV), nw.to(DEV), 1e-6, w)
        assert torch.equal(alone[0], many[t])
    wd = _bf(torch.randn(K, I, generator=g) * 0.02).to(DEV, torch.bfloat16)
    r_many = res.to(DEV).clone()
    ops().small_linear_residual(r_many, many, wd)
    r_one = res[9:10].contiguous().to(DEV)
    ops().small_linear_residual(r_one, many[9:10].contiguous(), wd)
    assert torch.equal(r_one[0], r_many[9])


def test_refusals_and_the_rule_of_use():
    o = ops()
    assert not o.small_step_fits(1, 4096, 4096, 14336)           # wide models keep the tcgen05 products
    assert o.small_step_fits(1, 2048, 2048) and o.small_step_fits(16, 896, 896, 4864)
    assert not o.small_step_fits(17, 896, 896) and not o.small_step_fits(1, 100, 100)   # K % 8
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(o.KernelError):
        o.small_linear_residual(torch.zeros(17, 8, device=DEV), x, w)
    with pytest.raises(o.KernelError):
        o.small_norm_swiglu(torch.zeros(2, 60, device=DEV), torch.ones(60, device=DEV), 1e-5,
                            torch.zeros(16, 60, dtype=torch.bfloat16, device=DEV))
