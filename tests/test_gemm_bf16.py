"""The tcgen05 matrix product alone, against float64, over both orientations, split
reductions, the SwiGLU epilogue, float32 output and ragged sizes."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from helios_b200.csrc import ops as _ops
    return _ops


def _case(T, N, K, seed, glu=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn((2 * N if glu else N), K, generator=g) / K ** 0.5).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    return x, w, b


def _close(got, want, scale=1.0):
    torch.testing.assert_close(got.double().cpu(), want, atol=2e-2 * scale, rtol=2e-2)


@pytest.mark.parametrize("T", [1, 8, 16, 17, 40, 64, 100, 128, 129, 300, 1000])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 72), (384, 4096), (1000, 520), (4096, 1024)])
def test_plain_and_bias(T, N, K):
    x, w, b = _case(T, N, K, T + N)
    want = x.double() @ w.double().T
    _close(ops().linear_bf16(x.to(DEV), w.to(DEV)), want)
    _close(ops().linear_bf16(x.to(DEV), w.to(DEV), b.to(DEV)), want + b.double())
    got32 = ops().linear_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert got32.dtype == torch.float32
    torch.testing.assert_close(got32.double().cpu(), want, atol=2e-3, rtol=1e-3)
    ops().check_kernel_errors()


@pytest.mark.parametrize("cluster", [False, True])
@pytest.mark.parametrize("bn", [0, 16, 32, 64, 128])
@pytest.mark.parametrize("splits", [1, 2, 5, 8])
@pytest.mark.parametrize("glu", [False, True])
def test_every_orientation_and_split(bn, splits, glu, cluster):
    """Split reductions both ways: through scratch memory with a ticket per tile, and
    inside a thread-block cluster through distributed shared memory."""
    T = {0: 260, 16: 9, 32: 32, 64: 50, 128: 128}[bn]
    N, K = 392, 1024 + 64 * 3
    x, w, b = _case(T, N, K, bn + splits, glu)
    xd, wd = x.double(), w.double()
    if glu:
        gate, up = xd @ wd[:N].T, xd @ wd[N:].T
        want = gate * torch.sigmoid(gate) * up
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), glu=True, plan=(bn, splits), cluster=cluster)
    else:
        want = xd @ wd.T + b.double()
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), b.to(DEV), plan=(bn, splits), cluster=cluster)
    _close(got, want)
    ops().check_kernel_errors()


def test_split_sum_is_the_same_every_time_and_tickets_return_to_zero():
    x, w, _ = _case(8, 4096, 14336, 3)
    xd, wd = x.to(DEV), w.to(DEV)
    first = ops().linear_bf16(xd, wd, plan=(16, 7), cluster=False)
    for _ in range(5):
        assert torch.equal(ops().linear_bf16(xd, wd, plan=(16, 7), cluster=False), first)
    # the cluster reduction adds the slices in the same order
    for _ in range(3):
        assert torch.equal(ops().linear_bf16(xd, wd, plan=(16, 7), cluster=True), first)
    _, tickets, _ = ops()._gemm_workspace(torch.device(DEV))
    assert int(tickets.abs().sum()) == 0
    _close(first, x.double() @ w.double().T)
    ops().check_kernel_errors()


@pytest.mark.parametrize("T", [3, 64, 2048])
def test_model_sized_products(T):
    # the shapes of the 8B model's layer: fused QKV, output, gate/up with SwiGLU, down
    for N, K, glu in [(6144, 4096, False), (4096, 4096, False), (14336, 4096, True), (4096, 14336, False)]:
        x, w, _ = _case(T, N, K, T + N, glu)
        xd, wd = x.double(), w.double()
        if glu:
            gate, up = xd @ wd[:N].T, xd @ wd[N:].T
            want = gate * torch.sigmoid(gate) * up
            got = ops().linear_swiglu(x.to(DEV), w.to(DEV))
        else:
            want = xd @ wd.T
            got = ops().linear(x.to(DEV), w.to(DEV))
        _close(got, want)
    ops().check_kernel_errors()


def test_k_that_is_no_multiple_of_8_goes_to_the_library_and_is_refused_by_the_kernel():
    x, w, _ = _case(5, 64, 100, 1)
    got = ops().linear(x.to(DEV), w.to(DEV))
    _close(got, x.double() @ w.double().T)
    with pytest.raises(ops().KernelError):
        ops().linear_bf16(x.to(DEV), w.to(DEV))


@pytest.mark.parametrize("two_sm", [False, True])
@pytest.mark.parametrize("T,N,K", [(129, 256, 64), (256, 512, 192), (300, 392, 1224), (2048, 4096, 1024),
                                   (1000, 1000, 520), (513, 6144, 4096)])
@pytest.mark.parametrize("glu", [False, True])
def test_prefill_kernels_one_and_two_sm(T, N, K, glu, two_sm):
    """Tokens on the M axis: one block per 128x256 tile, and the persistent cta_group::2
    kernel (pairs of SMs on 256x256 tiles), ragged in every dimension."""
    x, w, b = _case(T, N, K, T + N + K, glu)
    xd, wd = x.double(), w.double()
    if glu:
        gate, up = xd @ wd[:N].T, xd @ wd[N:].T
        want = gate * torch.sigmoid(gate) * up
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), glu=True, plan=(0, 1), two_sm=two_sm)
    else:
        want = xd @ wd.T + b.double()
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), b.to(DEV), plan=(0, 1), two_sm=two_sm)
    ops().check_kernel_errors()
    _close(got, want)
    got32 = ops().linear_bf16(x.to(DEV), w.to(DEV), glu=glu, plan=(0, 1), two_sm=two_sm, out_dtype=torch.float32)
    ops().check_kernel_errors()
    assert got32.dtype == torch.float32


# ------------------------------------------------------------------ the epilogues of few-token steps
def _norm_case(T, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x, w, b = _case(T, N, K, seed)
    residual = torch.randn(T, N, generator=g) * 3.0
    residual[:, 5 % N] *= 40.0                       # one feature far larger than the rest
    norm_w = 1.0 + 0.3 * torch.randn(N, generator=g)
    return x, w, b, residual, norm_w


@pytest.mark.parametrize("way", ["cluster", "scratch", "whole"])
@pytest.mark.parametrize("T", [1, 8, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(4096, 4096), (896, 4864), (200, 72), (384, 14336)])
def test_a_product_into_the_residual_leaves_the_next_norms_input(T, N, K, way):
    """residual += x W^T (+ bias); out = bfloat16(residual * norm weight); the partial sums of
    squares add up to sum(residual^2): every way the reduction can be split."""
    x, w, b, residual, norm_w = _norm_case(T, N, K, T * 7 + N + K)
    bn = 16 if T <= 16 else 32
    # 2 and 3 slices hold 64 and 43 of a tile's 128 features each (two rows a lane), 5 hold 26
    splits = 1 if way == "whole" else min(2 + (T + N) % 4, max(1, (K // 64) // 2))
    res = residual.to(DEV).clone()
    got = ops().linear_bf16(x.to(DEV), w.to(DEV), b.to(DEV), plan=(bn, splits), cluster=(way == "cluster"),
                            residual=res, norm_weight=norm_w.to(DEV))
    scaled, sumsq = got
    want_res = residual.double() + x.double() @ w.double().T + b.double()
    torch.testing.assert_close(res.double().cpu(), want_res, atol=2e-3, rtol=1e-3)
    assert scaled.dtype == torch.bfloat16 and tuple(sumsq.shape) == (T, 8 * -(-N // 128))
    # bit-equal to rounding what the kernel itself left in the residual
    assert torch.equal(scaled.cpu(), (res.cpu() * norm_w).to(torch.bfloat16))
    torch.testing.assert_close(sumsq.double().sum(1).cpu(), (res.double().cpu() ** 2).sum(1), rtol=1e-5, atol=0)
    # without a norm weight only the residual moves
    res2 = residual.to(DEV).clone()
    assert ops().linear_bf16(x.to(DEV), w.to(DEV), plan=(bn, splits), cluster=(way == "cluster"),
                             residual=res2) is None
    torch.testing.assert_close(res2.double().cpu(), want_res - b.double(), atol=2e-3, rtol=1e-3)
    ops().check_kernel_errors()


@pytest.mark.parametrize("way", ["cluster", "scratch", "whole"])
@pytest.mark.parametrize("glu", [False, True])
@pytest.mark.parametrize("T", [1, 8, 17, 32])
@pytest.mark.parametrize("N,K", [(6144, 4096), (1152, 896), (200, 72)])
def test_a_product_applies_the_tokens_rms_factor(T, N, K, glu, way):
    """Input rows that lack 1 / rms: the accumulators get it before bias or SwiGLU."""
    x, w, b = _case(T, N, K, T + N + K, glu)
    g = torch.Generator().manual_seed(T)
    slots = 8 * -(-K // 128)
    sumsq = torch.rand(T, slots, generator=g) * (K / slots) * torch.linspace(0.1, 30.0, T)[:, None]
    eps = 1e-5
    rstd = torch.rsqrt(sumsq.double().sum(1) / K + eps)[:, None]
    bn = 16 if T <= 16 else 32
    splits = 1 if way == "whole" else min(5, max(1, (K // 64) // 2))
    kw = dict(plan=(bn, splits), cluster=(way == "cluster"), sumsq=sumsq.to(DEV), eps=eps)
    xd, wd = x.double(), w.double()
    if glu:
        gate, up = rstd * (xd @ wd[:N].T), rstd * (xd @ wd[N:].T)
        want = gate * torch.sigmoid(gate) * up
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), glu=True, **kw)
    else:
        want = rstd * (xd @ wd.T) + b.double()
        got = ops().linear_bf16(x.to(DEV), w.to(DEV), b.to(DEV), **kw)
    _close(got, want, scale=float(want.abs().max().clamp(min=1.0)) / 4)
    ops().check_kernel_errors()


def test_two_products_with_the_norm_between_them_folded_in():
    """O-projection into the residual, then gate|up with the token factors: the same as
    add, RMSNorm and the product one after the other."""
    T, H, I = 8, 4096, 1024
    x, wo, _b, residual, norm_w = _norm_case(T, H, H, 99)
    g = torch.Generator().manual_seed(5)
    wgu = (torch.randn(2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16)
    eps = 1e-5
    res = residual.to(DEV).clone()
    scaled, sumsq = ops().linear_bf16(x.to(DEV), wo.to(DEV), residual=res, norm_weight=norm_w.to(DEV))
    got = ops().linear_bf16(scaled, wgu.to(DEV), glu=True, sumsq=sumsq, eps=eps)
    new = residual.double() + x.double() @ wo.double().T
    normed = new * torch.rsqrt((new ** 2).mean(1, keepdim=True) + eps) * norm_w.double()
    gate, up = normed @ wgu.double()[:I].T, normed @ wgu.double()[I:].T
    _close(got, gate * torch.sigmoid(gate) * up, scale=2.0)
    assert ops().DEFERRED_NORM_TOKENS <= ops().DEFERRED_NORM_MOST == 32
    with pytest.raises(ops().KernelError):
        ops().linear_bf16(torch.zeros(40, H, dtype=torch.bfloat16, device=DEV), wo.to(DEV),
                          residual=torch.zeros(40, H, device=DEV))
    ops().check_kernel_errors()
