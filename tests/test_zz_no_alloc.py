"""The allocation-free matrix product (helios_b200/csrc/gemm_bf16_noalloc.h), called
through its exported C symbol the way a host without torch would call it.

Who needs it: a caller that may not allocate device memory when it calls into the
library (a host with a fixed memory plan, a callback or a locked region where the CUDA
allocator must not be entered, a latency-critical path).  The regular product lets its
caller allocate scratch for the partial sums of a split reduction; this one keeps the
scratch in a static device array inside the library, so the caller passes inputs and
outputs only.

The file is named to be collected last: if it fails, a run that stops at the first
failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    from helios_b200.csrc.build import load_library

    lib = load_library("gemm_bf16_noalloc")
    fn = lib.hb_gemm_bf16_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_int
    return fn


def _call(fn, out, x, w, splits):
    """Inputs and outputs are the caller's; the library gets pointers and a stream."""
    err = ctypes.create_string_buffer(256)
    T, K = x.shape
    N = w.shape[0]
    rc = fn(out.data_ptr(), x.data_ptr(), w.data_ptr(), T, N, K, splits,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def test_two_calls_in_a_row_match_the_regular_entry_point():
    from helios_b200.csrc import ops

    fn = _entry()
    g = torch.Generator().manual_seed(7)
    cases = [(8, 4096, 4096, 8), (13, 6144, 1032, 5)]      # (T, N, K, slices); the second leaves stale
    outs = []                                               # partial sums of the first behind
    tensors = []
    for T, N, K, splits in cases:
        x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        tensors.append((x, w, out))
    torch.cuda.synchronize()
    # first call: also does the per-device set-up (outside of any capture)
    rc, msg = _call(fn, tensors[0][2], tensors[0][0], tensors[0][1], cases[0][3])
    assert rc == 0, msg
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rc, msg = _call(fn, tensors[1][2], tensors[1][0], tensors[1][1], cases[1][3])
    assert rc == 0, msg
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the second call changed the device's free memory"
    for (T, N, K, splits), (x, w, out) in zip(cases, tensors):
        want = ops.linear_bf16(x, w, plan=(16, splits))
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
        ref = x.double().cpu() @ w.double().cpu().T
        torch.testing.assert_close(out.double().cpu(), ref, atol=2e-2, rtol=2e-2)
    ops.check_kernel_errors()


def test_unsplit_and_repeated_calls_reuse_the_area():
    fn = _entry()
    g = torch.Generator().manual_seed(8)
    x = torch.randn(3, 520, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(1000, 520, generator=g) / 23).to(torch.bfloat16).to(DEV)
    ref = (x.double().cpu() @ w.double().cpu().T)
    for splits in (1, 4, 2, 4, 1):
        out = torch.zeros(3, 1000, dtype=torch.bfloat16, device=DEV)
        rc, msg = _call(fn, out, x, w, splits)
        assert rc == 0, msg
        torch.testing.assert_close(out.double().cpu(), ref, atol=2e-2, rtol=2e-2)


def test_sizes_beyond_the_maximum_are_refused_with_a_message():
    fn = _entry()
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(17, 128, dtype=torch.bfloat16, device=DEV)
    rc, msg = _call(fn, out, x, w, 1)
    assert rc == 2 and "17" in msg and "maximum" in msg            # too many tokens
    x = torch.zeros(4, 4096, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128 * 100, 4096, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 128 * 100, dtype=torch.bfloat16, device=DEV)
    rc, msg = _call(fn, out, x, w, 16)                              # 100 tiles * 16 slices * 2048 floats
    assert rc == 2 and "scratch floats" in msg
    rc, msg = _call(fn, out, x, w, 65)                              # more slices than k-blocks
    assert rc == 1 and "k_splits" in msg
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 100, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    rc, msg = _call(fn, out, x, w, 1)
    assert rc == 1 and "multiple of 8" in msg
