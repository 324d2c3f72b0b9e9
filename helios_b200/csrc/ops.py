"""Python launchers of the CUDA kernels.

Every function checks its tensors (device, dtype, layout, sizes) and raises a
clear error for a size the kernel does not take; it never computes on the CPU.
Two kinds of matrix product go to the library (cuBLAS through torch), as all of
the reference's do: see ``linear`` and ``GEMM_LIBRARY_TOKEN_RANGE``.  Kernels run
on torch's current stream, so they can be captured into a CUDA graph with the
rest of a step.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p, c_ulonglong
from typing import Optional

import torch

from .build import load_library

_F32, _BF16 = 0, 1
_STATUS = {1: "a size or option this kernel does not take", 2: "the kernel launch failed"}


class KernelError(RuntimeError):
    pass


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)")


def _check(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name} must be a tensor")
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


def _stream() -> int:
    # the raw handle of torch's current stream on the current device (capture streams
    # included); the Python-level Stream object costs several microseconds a launch
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _p(t: Optional[torch.Tensor]) -> int:
    # plain integers: ctypes converts them by the declared argument types, which costs less
    # than building a c_void_p object per argument
    return 0 if t is None else t.data_ptr()


#: launches of this package's own kernels since import (library products are not counted)
launch_count = 0


def _run(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status != 0:
        raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")


_fn_cache = {}


def _fn(lib: str, name: str, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


def preload(names) -> None:
    """Compile (in parallel) and load the named libraries, so that the first step does not
    stop at each one in turn.  A library that is not named here is still compiled and loaded
    when an op first asks for it."""
    from .build import build_all

    names = sorted(set(names) | {"elementwise"})
    build_all(names)
    for n in names:
        load_library(n)


def linear_libraries(dtype: torch.dtype, width: int = 0):
    """Libraries the matrix products of a model of this dtype and width run on."""
    if dtype == torch.float32:
        return ("gemm_f32",)
    return ("gemm_bf16",)


def attention_libraries(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int):
    """Libraries ``attention`` may choose from at these sizes (whatever the page size)."""
    if dtype != torch.bfloat16 or head_dim not in TILED_HEAD_DIMS:
        return ("attention_generic",)
    names = ["attention_bf16"]
    if ATTENTION_TCGEN05 and tc_attention_supported(num_heads, num_kv_heads, head_dim, 16):
        names += ["attention_tc", "attention_pair"]
    return tuple(names)


# ------------------------------------------------------------------ embedding
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """float32 [T, H] rows of ``table`` ([V, H], float32 or bfloat16) at int32 ``ids``."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "table", None, 2)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn("elementwise", "hb_embedding",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _run(f(_p(out), _p(table), _p(ids), T, H, V, _dt(table.dtype), _stream()), "embedding")
    return out


# ------------------------------------------------------------------ norms
def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``residual += delta`` (float32, in place) and the RMS-normed rows in ``out_dtype``.

    With ``rows`` (int32) only those rows are normed and the residual is left as it was.
    """
    _check(residual, "residual", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    n, H = residual.shape
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} entries for width {H}")
    if delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if tuple(delta.shape) != (n, H):
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {(n, H)}")
    n_out = n
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_out = rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
    f = _fn("elementwise", "hb_add_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _run(f(_p(out), _p(residual), _p(delta), _p(weight), _p(rows), n_out, H, float(eps),
           _dt(out_dtype), _stream()), "add_rmsnorm")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _check(x, "x", None, 2)
    _check(weight, "weight", torch.float32, 1)
    n, H = x.shape
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} entries for width {H}")
    out = torch.empty_like(x)
    f = _fn("elementwise", "hb_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _run(f(_p(out), _p(x), _p(weight), n, H, float(eps), _dt(x.dtype), _stream()), "rmsnorm")
    return out


# ------------------------------------------------------------------ rotary + cache write
def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor):
    """cos and sin [T, rot/2] (float32) of position * inv_freq, computed in float64."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float64, 1)
    T, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((T, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    f = _fn("elementwise", "hb_rotary_table",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _run(f(_p(cos), _p(sin), _p(positions), _p(inv_freq), T, half, _stream()), "rotary_table")
    return cos, sin


def rope_kv_write(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                  positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                  k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                  write_cache: bool = True) -> None:
    """Rotate q and k of ``qkv`` ([T, (nh + 2 nkv) hd]) by the tokens' cos/sin rows
    ([T, rot/2], float32; None = no rotation); q stays in place, rotated k and v go to the
    tokens' slots of the cache pages ([pages, nkv, page_size, hd])."""
    _check(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {qkv.shape[1]} is not (nh + 2 nkv) * hd = "
                          f"{(num_heads + 2 * num_kv_heads) * head_dim}")
    rot = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[0] != T:
            raise KernelError(f"cos/sin tables {tuple(cos.shape)}/{tuple(sin.shape)} do not "
                              f"match {T} tokens")
        rot = 2 * cos.shape[1]
        if rot > head_dim:
            raise KernelError(f"rotary dimension {rot} exceeds head_dim {head_dim}")
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    if write_cache:
        for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
            _check(pages, name, qkv.dtype, 4)
            if tuple(pages.shape[1:]) != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name} has shape {tuple(pages.shape)}, expected "
                                  f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    f = _fn("elementwise", "hb_rope_kv_write",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _run(f(_p(qkv), _p(cos), _p(sin), _p(positions), _p(seq_of_token), _p(block_table),
           block_table.shape[1], _p(k_pages) if write_cache else 0,
           _p(v_pages) if write_cache else 0, T, num_heads, num_kv_heads, head_dim,
           rot, page_size, 1 if write_cache else 0, _dt(qkv.dtype), _stream()), "rope_kv_write")


# ------------------------------------------------------------------ attention
def attention_generic(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, seq_of_token: torch.Tensor,
                      positions: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                      page_size: int, window: Optional[int], scale: float) -> torch.Tensor:
    """Attention of every token of the batch over its request's pages; q is read from the
    first ``nh * hd`` columns of ``qkv``.  Returns [T, nh * hd] in qkv's dtype."""
    _check(qkv, "qkv", None, 2)
    _check(k_pages, "k_pages", qkv.dtype, 4)
    _check(v_pages, "v_pages", qkv.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    if head_dim > 256 or head_dim <= 0:
        raise KernelError(f"head_dim {head_dim} is not supported by the attention kernels (1..256)")
    if num_heads % num_kv_heads != 0:
        raise KernelError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
    if tuple(k_pages.shape[1:]) != (num_kv_heads, page_size, head_dim):
        raise KernelError(f"k_pages has shape {tuple(k_pages.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    T = qkv.shape[0]
    out = torch.empty((T, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    f = _fn("attention_generic", "hb_attention_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _run(f(_p(out), _p(qkv), qkv.shape[1], _p(k_pages), _p(v_pages), _p(block_table),
           block_table.shape[1], _p(seq_of_token), _p(positions), T, num_heads, num_kv_heads,
           head_dim, page_size, int(window or 0), float(scale), _dt(qkv.dtype), _stream()),
         "attention_generic")
    return out


# ------------------------------------------------------------------ feed-forward gate
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for ``gate_up`` = [T, 2 I] (gate columns first)."""
    _check(gate_up, "gate_up", None, 2)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even width")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("elementwise", "hb_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _run(f(_p(out), _p(gate_up), T, two_i // 2, _dt(gate_up.dtype), _stream()), "silu_mul")
    return out


# ------------------------------------------------------------------ matrix products
def linear_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed (+ bias [N]) on the float32 FMA pipes."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 2)
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"x has {K} columns but weight has {K2}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError(f"bias has {bias.numel()} entries for {N} outputs")
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    f = _fn("gemm_f32", "hb_gemm_f32",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _run(f(_p(out), _p(x), _p(weight), _p(bias), M, N, K, K, K, N, _stream()), "gemm_f32")
    return out


# Fixed work space of the tensor-core products on a device: partial sums of split
# reductions, one ticket per output tile (zero between launches), and an error word
# that a kernel sets when one of its bounded waits ran out.  Its addresses never
# change, so captured CUDA graphs stay valid.
#: add the partial sums of a split reduction inside a thread-block cluster (through
#: distributed shared memory) where that is possible, instead of through scratch memory
GEMM_CLUSTER_REDUCE = True
#: prefill-sized products (more than 128 tokens, reduction not split) on pairs of SMs
GEMM_TWO_SM = True
_GEMM_SCRATCH_FLOATS = 16 * 1024 * 1024


def _cluster_fits(bn: int, glu: bool) -> bool:
    """Whether a block's float32 partial sums fit the stage buffers they reuse."""
    if bn == 0:
        stage, budget, cols = 48 * 1024, 196 * 1024, 256
    else:
        a_tiles = 2 if glu else 1
        stage, budget, cols = a_tiles * 16384 + bn * 128, 108 * 1024, bn * a_tiles
    stages = max(2, min(8, budget // stage))
    return cols * 128 * 4 <= stages * stage
_GEMM_TICKETS = 1 << 16
_gemm_ws = {}


def _gemm_workspace(device):
    ws = _gemm_ws.get(device)
    if ws is None:
        ws = (torch.empty(_GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_GEMM_TICKETS, dtype=torch.int32, device=device),
              torch.zeros(1, dtype=torch.int32, device=device))
        _gemm_ws[device] = ws
    return ws


def check_kernel_errors(device=None) -> None:
    """Raise if a kernel of this package gave up a bounded wait (synchronises)."""
    for dev, (_s, _t, err) in _gemm_ws.items():
        if device is not None and dev != torch.device(device):
            continue
        code = int(err.item())
        if code:
            err.zero_()
            role = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue"}.get(code, "a role")
            raise KernelError(f"gemm_bf16: {role} gave up waiting on an mbarrier (code {code}); "
                              "the results of that launch are not valid")


_cluster_capacity = {}


def cluster_capacity(bn: int, glu: bool, size: int) -> int:
    """Clusters of ``size`` blocks of the GEMM variant (bn, glu) the device keeps resident
    at once.  The CUDA occupancy calculator is asked (it knows how the SMs are spread over
    the GPCs, which bounds whole clusters); it counts one block per SM where the swapped
    variants run two, so its figure is doubled for them.  Measured on B200: cluster counts
    up to that doubled figure run in one round, beyond it a second round shows."""
    key = (bn, bool(glu), size)
    if key not in _cluster_capacity:
        lib = load_library("gemm_bf16")
        n = int(lib.hb_gemm_bf16_max_clusters(bn, int(glu), size))
        if n <= 0:
            n = sm_count() // size
        _cluster_capacity[key] = n * (2 if bn else 1)
    return _cluster_capacity[key]


_gemm_plans = {}


def gemm_plan(T: int, N: int, K: int, glu: bool):
    """Cached ``_gemm_plan``."""
    key = (T, N, K, bool(glu), GEMM_CLUSTER_REDUCE, GEMM_TWO_SM)
    plan = _gemm_plans.get(key)
    if plan is None:
        plan = _gemm_plans[key] = _gemm_plan(T, N, K, glu)
    return plan


def _gemm_plan(T: int, N: int, K: int, glu: bool):
    """(swap_bn, k_splits) of the tensor-core product for T tokens, N result features.
    Up to 128 tokens run swapped (features on the MMA M axis).  When the tiles alone do not
    fill the SMs, the reduction is split (at least 2 k-blocks a slice; short reductions of
    small models are bound by latency, and more blocks shorten them): with slices as
    thread-block clusters, the count that keeps the most blocks resident in ONE round of
    clusters; else the count that fills the resident blocks."""
    k_blocks = -(-K // 64)
    if T <= 128:
        bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
        tiles = -(-N // 128) * -(-T // bn)
        cols = bn * (2 if glu else 1)
        slots = 2 * sm_count()
    else:
        bn = 0
        tiles = -(-T // 128) * -(-N // (128 if glu else 256))
        cols = 256
        slots = sm_count()
        if GEMM_TWO_SM:
            # the two-SM kernel takes whole reductions only; even with part of the pairs idle
            # it beats the one-SM kernel with a split reduction (20 against 85 microseconds
            # for 512 tokens x 4096 x 4096)
            return bn, 1
    splits = 1
    if tiles < slots:
        most_k = max(1, k_blocks // 2)
        if GEMM_CLUSTER_REDUCE and _cluster_fits(bn, glu):
            best = 0
            for s in range(1, min(8, most_k) + 1):
                # a few clusters over the figure cost less than a smaller cluster size
                if tiles * 15 <= cluster_capacity(bn, glu, s) * 16 and tiles * s > best + best // 16:
                    splits, best = s, tiles * s
        else:
            splits = _wave_splits(tiles, slots, min(16, most_k))
            while splits > 1 and tiles * splits * 128 * cols > _GEMM_SCRATCH_FLOATS:
                splits -= 1
    return bn, splits


def tc_gemm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and weight.dim() == 2 and x.shape[1] == weight.shape[1] and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                glu: bool = False, out_dtype: torch.dtype = torch.bfloat16,
                plan=None, cluster: Optional[bool] = None, two_sm: Optional[bool] = None,
                sumsq: Optional[torch.Tensor] = None, eps: float = 0.0,
                residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                norm_out: Optional[tuple] = None):
    """y = x W^T (+ bias) on tcgen05 tensor cores; bfloat16 operands, float32 accumulate.

    With ``glu`` the weight is [gate rows; up rows] ([2 I, K]) and the result is
    silu(x gate^T) * (x up^T), [T, I].  ``out_dtype`` bfloat16 or float32.  K must be a
    multiple of 8 (TMA rows are 16-byte aligned); any T and N.

    Up to DEFERRED_NORM_MOST tokens there are two more epilogues.  ``sumsq``
    (float32 [T, slots]): ``x`` is residual * norm weight without the token's 1 / rms;
    the accumulators are multiplied by rsqrt(sum(sumsq[t]) / K + eps) before bias or SwiGLU.
    ``residual`` (float32 [T, N]): the product is added into it and None is returned, or,
    with ``norm_weight`` (float32 [N]), the pair (bfloat16(residual * norm_weight),
    partial sums of squares [T, slots]) that a product with ``sumsq`` takes; ``norm_out``
    gives that pair's tensors to write into."""
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    T, K = x.shape
    rows, K2 = weight.shape
    if K != K2:
        raise KernelError(f"x has {K} columns but weight has {K2}")
    if K % 8:
        raise KernelError(f"the tensor-core product needs K to be a multiple of 8, got {K}")
    if glu and rows % 2:
        raise KernelError("a SwiGLU weight needs an even number of rows")
    N = rows // 2 if glu else rows
    if bias is not None:
        if glu:
            raise KernelError("the SwiGLU epilogue takes no bias")
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError(f"bias has {bias.numel()} entries for {N} outputs")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"out_dtype {out_dtype} is not supported")
    few = sumsq is not None or residual is not None
    if few and T > DEFERRED_NORM_MOST:
        raise KernelError(f"the residual and 1 / rms epilogues take at most {DEFERRED_NORM_MOST} tokens, got {T}")
    if sumsq is not None:
        _check(sumsq, "sumsq", torch.float32, 2)
        if sumsq.shape[0] != T or not sumsq.is_contiguous():
            raise KernelError(f"sumsq has shape {tuple(sumsq.shape)} for {T} tokens")
    sumsq_out = None
    if residual is not None:
        _check(residual, "residual", torch.float32, 2)
        if tuple(residual.shape) != (T, N) or not residual.is_contiguous():
            raise KernelError(f"residual has shape {tuple(residual.shape)}, expected ({T}, {N}) contiguous")
        if glu or out_dtype != torch.bfloat16:
            raise KernelError("a product into the residual is a plain bfloat16 one")
        out = None
        if norm_weight is not None:
            _check(norm_weight, "norm_weight", torch.float32, 1)
            if norm_weight.numel() != N:
                raise KernelError(f"norm weight has {norm_weight.numel()} entries for width {N}")
            slots = 8 * -(-N // 128)
            if norm_out is not None:
                out, sumsq_out = norm_out
                _check(out, "norm_out[0]", torch.bfloat16, 2)
                _check(sumsq_out, "norm_out[1]", torch.float32, 2)
                if tuple(out.shape) != (T, N) or tuple(sumsq_out.shape) != (T, slots):
                    raise KernelError("norm_out tensors have the wrong shapes")
            else:
                out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
                sumsq_out = torch.empty((T, slots), dtype=torch.float32, device=x.device)
    elif norm_weight is not None:
        raise KernelError("norm_weight goes with residual")
    else:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if T == 0:
        return out if residual is None else ((out, sumsq_out) if norm_weight is not None else None)
    bn, splits = plan if plan is not None else gemm_plan(T, N, K, glu)
    if few and (bn == 0 or T > bn):
        raise KernelError("the residual and 1 / rms epilogues need the swapped orientation and one token tile")
    if cluster is None:
        cluster = GEMM_CLUSTER_REDUCE
    # slices of a tile as a cluster: at most 8, and the partial sums must fit the stages
    cluster = bool(cluster) and 1 < splits <= 8 and _cluster_fits(bn, glu)
    cluster_arg = 1 if cluster else 0
    if bn == 0 and splits == 1 and (GEMM_TWO_SM if two_sm is None else two_sm):
        cluster_arg = 2                      # prefill tiles on pairs of SMs (cta_group::2)
    scratch, tickets, err = _gemm_workspace(x.device)
    lib = load_library("gemm_bf16")
    if splits > 1 and not cluster:
        lib.hb_gemm_bf16_scratch_floats.restype = ctypes.c_longlong
        need = lib.hb_gemm_bf16_scratch_floats(T, N, bn, int(glu), splits)
        tiles = lib.hb_gemm_bf16_tiles(T, N, bn, int(glu))
        if need > scratch.numel() or tiles > tickets.numel():
            raise KernelError(f"split reduction needs {need} scratch floats and {tiles} tickets; "
                              f"the work space holds {scratch.numel()} and {tickets.numel()}")
    common = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]
    args = (_p(out), _p(x), _p(weight), _p(bias), _p(scratch), _p(tickets), _p(err), T, N, K, K, K, N,
            rows, int(glu), N if glu else 0, 1 if out_dtype == torch.float32 else 0, bn, splits, cluster_arg)
    if few:
        f = _fn("gemm_bf16", "hb_gemm_bf16_fused",
                common + [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p])
        _run(f(*args, _p(residual), _p(norm_weight), _p(sumsq_out), _p(sumsq),
               0 if sumsq is None else sumsq.shape[1], float(eps), _stream()), "gemm_bf16_fused")
        if residual is not None:
            return (out, sumsq_out) if norm_weight is not None else None
        return out
    f = _fn("gemm_bf16", "hb_gemm_bf16", common + [c_void_p])
    _run(f(*args, _stream()), "gemm_bf16")
    return out


#: Steps of at most this many tokens run a layer's RMS norms inside the products around them
#: (see ``linear_bf16``): the products of such a step run swapped, tokens on one narrow tile,
#: on this package's kernel.  The epilogues take up to DEFERRED_NORM_MOST tokens, but their
#: cost grows with the tokens while a norm launch's does not.  Measured, milliseconds a
#: decode step with the norm launches against without: Llama-3.1-8B sizes 4.01 / 3.89 at 8
#: requests, 4.87 / 4.86 at 16, 5.83 / 5.73 at 24, 6.70 / 6.88 at 32; Qwen2.5-7B sizes 3.38 /
#: 3.22 at 8, 4.52 / 4.58 at 32; Qwen2.5-0.5B sizes 1.06 / 1.08 at 24, 1.12 / 1.14 at 32.
DEFERRED_NORM_TOKENS = 16
DEFERRED_NORM_MOST = 32


def deferred_norm_fits(tokens: int, *weights: torch.Tensor) -> bool:
    """Whether a step of ``tokens`` tokens runs these products with the residual and
    1 / rms epilogues: few tokens, and shapes the tensor-core kernel takes."""
    if not 0 < tokens <= DEFERRED_NORM_TOKENS:
        return False
    return all(w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 8 == 0 and w.is_contiguous()
               and w.data_ptr() % 16 == 0 for w in weights)


#: Between the decode kernel's best range (up to 32 tokens: weights streamed once with the
#: tokens on a narrow MMA N axis, a deep ring of weight stages) and the prefill kernel's (pairs
#: of SMs on 256x256 tiles, which need a few hundred tiles to fill 74 pairs) plain products (no
#: bias, bfloat16 out) go to the library (cuBLAS through torch), which the reference uses for
#: every product (python/helios/exec/model.py:170-181).  From 33 tokens on a stage of the decode
#: kernel holds 8-16 KB of tokens beside its 16 KB of weights, the ring gets shallow, and the
#: library is ahead (Llama-3.1-8B sizes at 64 tokens, microseconds in a chain: q|k|v 15.2
#: against 11.5, O 11.1 against 10.0, down 24.3 against 24.2; a decode step of 64 requests
#: 6,300-6,460 against 6,690 tokens/s); from 129 tokens on the two-SM kernel has too few tiles
#: (same sizes, this package's kernel against the library: down 88 / 61 at 513 tokens, 82 / 69
#: at 768, 86 / 83 at 1,024, 171 / 120 at 1,536 with 80 tiles on 74 pairs, 168 / 156 at 2,048,
#: 263 / 271 at 3,072; O 28 / 22, 29 / 22, 30 / 27, 54 / 43, 53 / 50, 84 / 82).  Products with
#: float32 logits, and everything up to 32 tokens, always run on this package's kernels.
#: (0, 0) turns the library off.
GEMM_LIBRARY_TOKEN_RANGE = (33, 1536)
#: gate|up with SwiGLU runs fused on this package's kernels except in these token ranges,
#: where the library's plain product and a gate kernel are ahead (Llama-3.1-8B sizes, fused
#: against library + gate: 73 / 59 at 96 tokens, 82 / 57 at 128; 59 / 67 at 160, 66 / 76 at
#: 256: one full tile of the two-SM kernel; 110 / 93 at 320, 110 / 104 at 384: a second tile
#: that is mostly empty; 111 / 129 at 448, 112 / 141 at 512, 150 / 188 at 640)
GEMM_LIBRARY_GLU_TOKENS = ((33, 128), (257, 383))
#: The library chooses its kernel per shape, which takes about a millisecond of host time
#: the first time a shape is seen; token counts are rounded up to a multiple of this (on a
#: padded copy of the rows) so that a serving run meets a handful of shapes, not hundreds.
#: Up to 128 tokens the step is 8 and up to 256 it is 32 (GEMM_LIBRARY_TOKEN_STEPS_FEW): the
#: padded copy is two launches more per product (the four products of a layer at
#: Llama-3.1-8B sizes and 40 tokens: 105 µs with the copy, 94 without; a decode step of 40
#: requests 7.90 -> 7.60 ms, at Qwen2.5-0.5B sizes 1.26 -> 1.09 ms), and captured steps come
#: in these multiples there anyway.
GEMM_LIBRARY_TOKEN_STEP = 64
GEMM_LIBRARY_TOKEN_STEPS_FEW = ((128, 8), (256, 32))
#: Weight matrices of at most this many bytes (the products of models about 1,000 wide: 2 to
#: 17 MB) go to the library from GEMM_LIBRARY_SMALL_TOKENS[0] tokens on: a product that short
#: is bound by the kernel's own latency, where the tensor-memory kernels (set-up, a cluster for
#: the split reduction) lose to the library's plain ones, and with 896 output features the
#: two-SM kernel has 4 tiles a 256 tokens.  Measured at Qwen2.5-0.5B sizes, microseconds a
#: launch in a chain, this package's kernel against the library, at 24 / 64 / 256 tokens: q|k|v
#: 5.0 / 7.2 / 10.9 against 4.0 / 3.9 / 4.2; down 6.8 / 8.5 / 29.7 against 9.4 / 8.6 / 8.8 (and
#: 30 / 10 at 1,024, 31 / 15 at 2,048, 32 / 27 at 4,096, 64 / 64 at 8,192); gate|up with SwiGLU
#: 14.4 / 18.9 / 16.5 against 8.6 / 8.7 / 12.8 (library product + gate kernel; 26 / 26 at 768,
#: 56 / 58 at 2,048, 96 / 117 at 4,096: GEMM_LIBRARY_SMALL_GLU_TOKENS).  Up to 32 tokens this
#: package's kernels win as a whole (a step of 32 requests: 28,300 against 25,900 tokens/s).
#: 0 bytes turns it off.
GEMM_LIBRARY_SMALL_WEIGHT_BYTES = 20 * 1024 * 1024
GEMM_LIBRARY_SMALL_TOKENS = (33, 4096)
GEMM_LIBRARY_SMALL_GLU_TOKENS = (33, 512)


def _library_range(tokens: int) -> bool:
    lo, hi = GEMM_LIBRARY_TOKEN_RANGE
    return lo <= tokens <= hi


def _small_weight_library(tokens: int, weight: torch.Tensor, glu: bool = False) -> bool:
    lo, hi = GEMM_LIBRARY_SMALL_GLU_TOKENS if glu else GEMM_LIBRARY_SMALL_TOKENS
    return lo <= tokens <= hi and \
        weight.numel() * weight.element_size() <= GEMM_LIBRARY_SMALL_WEIGHT_BYTES


#: Products with a bias take the same way in that range (the library adds the bias, as
#: bfloat16, to its float32 sums before it rounds them): Qwen2.5-7B sizes, 64 requests
#: decoding, 10,550 -> 10,660 tokens/s.
GEMM_LIBRARY_WITH_BIAS = True
_bf16_biases = {}


def _bias_bf16(bias: torch.Tensor) -> torch.Tensor:
    """The bias as bfloat16 for the library, converted once per tensor (a model's biases are
    float32 and do not change)."""
    if bias.dtype == torch.bfloat16:
        return bias
    key = (bias.data_ptr(), bias.numel(), bias.device)
    hit = _bf16_biases.get(key)
    if hit is None or hit[0] is not bias:
        hit = _bf16_biases[key] = (bias, bias.to(torch.bfloat16))
    return hit[1]


def _library_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    T = x.shape[0]
    step = next((st for most, st in GEMM_LIBRARY_TOKEN_STEPS_FEW if T <= most), GEMM_LIBRARY_TOKEN_STEP)
    padded = -(-T // step) * step if step > 1 else T
    if padded == T:
        return torch.nn.functional.linear(x, weight, bias)
    rows = x.new_empty((padded, x.shape[1]))
    rows[:T].copy_(x)
    rows[T:].zero_()                              # they reach no result row, but must not hold NaN
    return torch.nn.functional.linear(rows, weight, bias)[:T]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T + b.  float32: this package's FMA kernel.  bfloat16: the tcgen05 kernels,
    or the library for plain products in the token ranges of GEMM_LIBRARY_TOKEN_RANGE and
    GEMM_LIBRARY_SMALL_TOKENS (small weight matrices); a K that is no multiple of 8 goes to
    the library too, as TMA needs 16-byte rows."""
    if x.dtype == torch.float32:
        return linear_f32(x, weight, bias)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    T = x.shape[0]
    to_library = ((bias is None or GEMM_LIBRARY_WITH_BIAS) and _library_range(T)) \
        or _small_weight_library(T, weight)
    if tc_gemm_supported(x, weight) and not to_library:
        return linear_bf16(x, weight, bias)
    return _library_linear(x, weight, None if bias is None else _bias_bf16(bias))


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for ``w_gate_up`` = [gate rows; up rows]; fused into the
    product's epilogue in bfloat16, two kernels otherwise."""
    if x.dtype == torch.bfloat16 and tc_gemm_supported(x, w_gate_up):
        T = x.shape[0]
        if _small_weight_library(T, w_gate_up, glu=True) or \
                any(lo <= T <= hi for lo, hi in GEMM_LIBRARY_GLU_TOKENS):
            return silu_mul(_library_linear(x, w_gate_up, None))
        return linear_bf16(x, w_gate_up, glu=True)
    return silu_mul(linear(x, w_gate_up))


# ------------------------------------------------------------------ sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed: torch.Tensor, offset: torch.Tensor,
           kind: Optional[str] = None) -> torch.Tensor:
    """One token id per row of float32 ``logits`` [R, V]; per-row options as device tensors
    (temperature float32 with 0 = greedy, top_k int32 with 0 = off, top_p float32,
    seed and offset int64).  ``kind``: what the caller knows of the options, which live on
    the device: "greedy" (every row takes the argmax), "draw" (some rows draw, none has a
    top-k or top-p), "narrow" (some have); it chooses between the kernel with one block a row
    and the one with a cluster of blocks a row (``sampling.cu``), as does the number of
    rows.  "one_block" takes the first whatever the rows; None counts as "narrow"."""
    _check(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _check(temperature, "temperature", torch.float32, 1)
    _check(top_k, "top_k", torch.int32, 1)
    _check(top_p, "top_p", torch.float32, 1)
    _check(seed, "seed", torch.int64, 1)
    _check(offset, "offset", torch.int64, 1)
    for name, t in (("temperature", temperature), ("top_k", top_k), ("top_p", top_p),
                    ("seed", seed), ("offset", offset)):
        if t.numel() != R:
            raise KernelError(f"{name} has {t.numel()} entries for {R} rows")
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "hb_sample",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_void_p])
    _run(f(_p(out), _p(logits), R, V, V, _p(temperature), _p(top_k), _p(top_p), _p(seed),
           _p(offset), _SAMPLE_KINDS[kind], _stream()), "sample")
    return out


_SAMPLE_KINDS = {None: -1, "greedy": 0, "draw": 1, "narrow": 2, "one_block": 3}


def philox_uniform(seed: int, offset: int) -> float:
    """The uniform in [0, 1) that the sampling kernel draws for (seed, offset)."""
    lib = load_library("sampling")
    lib.hb_philox_uniform.argtypes = [c_ulonglong, c_ulonglong]
    lib.hb_philox_uniform.restype = c_float
    return float(lib.hb_philox_uniform(seed & (2**64 - 1), offset & (2**64 - 1)))


def linear_logits(rows: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Output head: float32 logits [R, V] of ``rows`` [R, H] against ``weight`` [V, H]."""
    if rows.dtype == torch.float32:
        return linear_f32(rows, weight, None)
    _check(rows, "rows", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    if tc_gemm_supported(rows, weight):
        return linear_bf16(rows, weight, out_dtype=torch.float32)
    return torch.mm(rows, weight.t(), out_dtype=torch.float32)


TILED_HEAD_DIMS = (32, 64, 96, 128)
#: merge the context slices of decode attention inside a thread-block cluster (up to 8 slices)
ATTENTION_CLUSTER_MERGE = True
#: steps of single tokens: rotary position encoding and cache write inside the decode kernel
ATTENTION_DECODE_ROTARY = True
#: use the tcgen05 attention kernel for batches with prompt portions where its sizes fit
ATTENTION_TCGEN05 = True
#: ... with two tiles of query rows per block when a request brings more than one tile of tokens
ATTENTION_TILE_PAIRS = True
#: ... and the step gives at least this many blocks of two tiles: with fewer, the blocks of one
#: tile (twice as many, each about 1/1.5 as long) still fit the 148 SMs in one round
ATTENTION_PAIR_MIN_BLOCKS = 75
_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the (current) device."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


def _wave_splits(blocks: int, slots: int, most: int) -> int:
    """Number of slices per block so that blocks * slices still fits one round of ``slots``
    resident blocks (at most ``most``)."""
    return max(1, min(most, slots // max(1, blocks)))


_decode_clusters = {}

#: Decode attention blocks have 4 warps, two blocks an SM, or 8 warps, one block an SM, for
#: steps of so few requests that clusters of eight such blocks per (request, KV head) are all
#: resident at once: a warp walks its key tiles one after the other, about 0.8 microseconds
#: each, and with few blocks that chain, not the memory, is what the kernel takes.  Measured,
#: milliseconds a decode step at Llama-3.1-8B sizes, context 4,096 (slices, warps): one request
#: 3.140 (29, 4), 3.129 (8, 4), 3.007 (8, 8), 3.073 (18, 8); two 3.192 (17, 4), 3.164 (8, 8);
#: four 3.365 (9, 4), 3.308 (8, 4), 3.289 (4, 8); eight 3.718 (4, 4), 3.891 (2, 8): once the
#: four-warp blocks fill the SMs they are ahead.  False: always 4.
ATTENTION_DECODE_WIDE_BLOCKS = True


def decode_cluster_capacity(head_dim: int, size: int, warps: int = 4) -> int:
    """Clusters of ``size`` decode-attention blocks of ``warps`` warps the device keeps
    resident at once (the occupancy calculator knows how the SMs are spread over the GPCs,
    which bounds whole clusters: 71 clusters of 4 on a B200 where 74 would fit block by block)."""
    key = (head_dim, size, warps)
    if key not in _decode_clusters:
        n = -1
        if torch.cuda.is_available() and head_dim in TILED_HEAD_DIMS and 1 <= size <= 8:
            n = int(load_library("attention_bf16").hb_attention_decode_max_clusters(head_dim, size, warps))
        _decode_clusters[key] = n if n > 0 else ((2 if warps == 4 else 1) * sm_count()) // size
    return _decode_clusters[key]


#: ... and each of the eight warps still has this many keys (four tiles) of the longest context
#: (Qwen2.5-0.5B sizes at 1,024 tokens, 21 keys a warp: 0.783 against 0.773 ms a step)
ATTENTION_DECODE_WIDE_MIN_KEYS = 64


def decode_warps(blocks: int, n_splits: int, head_dim: int, max_context: int) -> int:
    """Warps per block for ``blocks`` (request, KV head) pairs in ``n_splits`` slices of at most
    ``max_context`` keys together: 8 for slices that run as a cluster in a step small enough
    for clusters of eight, where a warp still has keys enough, else 4."""
    if not (ATTENTION_DECODE_WIDE_BLOCKS and ATTENTION_CLUSTER_MERGE and 1 < n_splits <= 8):
        return 4
    if max_context < ATTENTION_DECODE_WIDE_MIN_KEYS * 8 * n_splits:
        return 4
    fits = min(decode_cluster_capacity(head_dim, n_splits, 8), decode_cluster_capacity(head_dim, 8, 8))
    return 8 if blocks <= fits else 4


def decode_splits(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 128) -> int:
    """Slices of the context per (request, KV head) of the decode attention kernel, by a cost
    model fitted to measurements (64 requests x 8 KV heads of 128 at contexts 1,024 and 4,096;
    it then predicts 40 to 96 requests within 5 %): two blocks of four warps are resident per
    SM, the blocks run in rounds of that many, and a block costs its keys plus a fixed part
    (set-up, merge) worth about 176 keys of 128 values; slices that do not run as a cluster
    need the merge kernel, worth about 300 keys more; a block of eight warps
    (``decode_warps``) walks its keys twice as fast.  A slice has at least 128 keys.  More
    slices are taken when the model gives them 4 % (measured, milliseconds a step at
    Llama-3.1-8B sizes, with the count that a margin of 6 % chose against this one's: 16
    requests x 32,768 keys 15.70 / 14.74, 32 x 16,384 15.91 / 15.06, 64 x 8,192 15.63 / 15.21,
    8 x 32,768 9.23 / 8.98)."""
    blocks = max(1, num_seqs * num_kv_heads)
    slots = 2 * sm_count()
    fixed = 176.0 * 128.0 / max(1, head_dim)
    merge_kernel = 300.0 * 128.0 / max(1, head_dim)
    best, best_cost = 1, None
    for s in range(1, max(1, min(32, max_context // 128)) + 1):
        # 2 to 8 slices run as one cluster per (request, KV head) while all clusters are
        # resident at once; otherwise block by block, with a merge kernel
        if decode_warps(blocks, s, head_dim, max_context) == 8:
            cost = max_context / s / 2 + fixed
        else:
            clustered = 1 < s <= 8 and ATTENTION_CLUSTER_MERGE and blocks <= decode_cluster_capacity(head_dim, s)
            rounds = 1 if clustered else -(-blocks * s // slots)
            cost = rounds * (max_context / s + fixed) + (0.0 if clustered or s == 1 else merge_kernel)
        if best_cost is None or cost < best_cost * 0.96:      # fewer slices unless clearly better
            best, best_cost = s, cost
    return best


def attention_decode_bf16(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          block_table: torch.Tensor, positions: torch.Tensor, num_heads: int,
                          num_kv_heads: int, head_dim: int, page_size: int,
                          window: Optional[int], scale: float, n_splits: int,
                          rotary=None, write_cache: bool = False, warps: Optional[int] = None) -> torch.Tensor:
    """Decode attention (token i is the one new token of request i) on the tensor cores;
    bfloat16, head_dim in TILED_HEAD_DIMS, at most 16 query heads per KV head.

    ``rotary`` = (cos, sin), float32 [requests, head_dim / 2]: the rows of ``qkv`` are not
    rotated yet; the kernel rotates the query heads on the way in.  ``write_cache``: the
    requests' new keys (rotated likewise) and values are still in ``qkv`` and the kernel
    stores them in the pages before it attends.  (Without either, ``rope_kv_write`` must have
    run.)  ``qkv`` itself is left as it was.  ``warps``: 4 (the default) or 8 warps a block
    (``decode_warps``)."""
    _check(qkv, "qkv", torch.bfloat16, 2)
    _check(k_pages, "k_pages", torch.bfloat16, 4)
    _check(v_pages, "v_pages", torch.bfloat16, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    if head_dim not in TILED_HEAD_DIMS:
        raise KernelError(f"head_dim {head_dim} is not one of {TILED_HEAD_DIMS}")
    if num_heads % num_kv_heads or num_heads // num_kv_heads > 16:
        raise KernelError(f"{num_heads} query heads on {num_kv_heads} KV heads: the decode kernel "
                          "takes groups of at most 16")
    if tuple(k_pages.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError(f"cache pages have shape {tuple(k_pages.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    S = qkv.shape[0]
    if block_table.shape[0] != S or positions.numel() != S:
        raise KernelError("decode attention needs one token per request")
    cos = sin = None
    if rotary is not None and rotary[0] is not None:
        cos, sin = rotary
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (S, head_dim // 2) or cos.shape != sin.shape \
                or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError(f"rotary tables have shape {tuple(cos.shape)}, expected ({S}, {head_dim // 2})")
    if (cos is not None or write_cache) and (qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim
                                             or not qkv.is_contiguous()):
        raise KernelError(f"q|k|v rows have {qkv.shape[1]} entries for {num_heads} + 2 x {num_kv_heads} "
                          f"heads of {head_dim}")
    out = torch.empty((S, num_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    part_o = part_ml = None
    # slices as one cluster only while all blocks are resident at once: with several rounds
    # of blocks, clusters (whose blocks must start together) cost more than the merge kernel
    warps = 4 if warps is None else int(warps)
    if warps not in (4, 8):
        raise KernelError(f"decode attention blocks have 4 or 8 warps, not {warps}")
    one_round = n_splits <= 8 and S * num_kv_heads <= decode_cluster_capacity(head_dim, n_splits, warps)
    if n_splits > 8 or (n_splits > 1 and not (ATTENTION_CLUSTER_MERGE and one_round)):
        part_o = torch.empty((S, num_heads, n_splits, head_dim), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((S, num_heads, n_splits, 2), dtype=torch.float32, device=qkv.device)
    f = _fn("attention_bf16", "hb_attention_decode_bf16",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
             c_int, c_int, c_void_p])
    _run(f(_p(out), _p(part_o), _p(part_ml), _p(qkv), qkv.shape[1], _p(k_pages), _p(v_pages),
           _p(block_table), block_table.shape[1], _p(positions), S, num_heads, num_kv_heads,
           head_dim, page_size, int(window or 0), float(scale), int(n_splits), _p(cos), _p(sin),
           1 if write_cache else 0, int(warps), _stream()),
         "attention_decode_bf16")
    return out


def prefill_tiling(num_heads: int, num_kv_heads: int):
    """(query heads per block, 16-token sub-tiles per block) of the prefill kernel."""
    group = num_heads // num_kv_heads
    heads = min(group, 8)
    return heads, max(1, 8 // heads)


def attention_prefill_bf16(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, q_tiles: torch.Tensor,
                           cu_tokens: torch.Tensor, start_pos: torch.Tensor, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int,
                           window: Optional[int], scale: float) -> torch.Tensor:
    """Attention of query-token tiles over the cache, causal by position; ``q_tiles`` is
    int32 [tiles, 2] = (request, first local token) for tiles of
    ``16 * prefill_tiling(...)[1]`` tokens."""
    _check(qkv, "qkv", torch.bfloat16, 2)
    _check(k_pages, "k_pages", torch.bfloat16, 4)
    _check(v_pages, "v_pages", torch.bfloat16, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(q_tiles, "q_tiles", torch.int32, 2)
    _check(cu_tokens, "cu_tokens", torch.int32, 1)
    _check(start_pos, "start_pos", torch.int32, 1)
    if head_dim not in TILED_HEAD_DIMS:
        raise KernelError(f"head_dim {head_dim} is not one of {TILED_HEAD_DIMS}")
    if num_heads % num_kv_heads:
        raise KernelError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
    if tuple(k_pages.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError(f"cache pages have shape {tuple(k_pages.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    heads, subtiles = prefill_tiling(num_heads, num_kv_heads)
    T = qkv.shape[0]
    out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    f = _fn("attention_bf16", "hb_attention_prefill_bf16",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _run(f(_p(out), _p(qkv), qkv.shape[1], _p(k_pages), _p(v_pages), _p(block_table),
           block_table.shape[1], _p(q_tiles), q_tiles.shape[0], _p(cu_tokens), _p(start_pos),
           num_heads, num_kv_heads, head_dim, heads, subtiles, page_size, int(window or 0),
           float(scale), _stream()), "attention_prefill_bf16")
    return out


def tc_attention_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Sizes the tcgen05 prefill attention kernel takes."""
    group = num_heads // max(1, num_kv_heads)
    return (head_dim in (64, 128) and num_heads % num_kv_heads == 0 and group <= 128
            and page_size >= 8 and page_size % 8 == 0 and 128 % page_size == 0)


def attention_prefill_tc(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         block_table: torch.Tensor, q_tiles: torch.Tensor, cu_tokens: torch.Tensor,
                         start_pos: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                         page_size: int, window: Optional[int], scale: float, pairs: bool = False) -> torch.Tensor:
    """Attention of query tiles over the cache on tcgen05 tensor cores; ``q_tiles`` is int32
    [tiles, 2] = (request, first local token) for tiles of ``128 // (nh // nkv)`` tokens, or
    with ``pairs`` of twice as many: then a block works on two tiles of query rows at a time
    (the softmax of one under the products of the other)."""
    _check(qkv, "qkv", torch.bfloat16, 2)
    _check(k_pages, "k_pages", torch.bfloat16, 4)
    _check(v_pages, "v_pages", torch.bfloat16, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(q_tiles, "q_tiles", torch.int32, 2)
    _check(cu_tokens, "cu_tokens", torch.int32, 1)
    _check(start_pos, "start_pos", torch.int32, 1)
    if not tc_attention_supported(num_heads, num_kv_heads, head_dim, page_size):
        raise KernelError(f"the tcgen05 attention kernel does not take {num_heads} heads on "
                          f"{num_kv_heads} KV heads, head_dim {head_dim}, page size {page_size}")
    if tuple(k_pages.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError(f"cache pages have shape {tuple(k_pages.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim}]")
    T = qkv.shape[0]
    out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    _scratch, _tickets, err = _gemm_workspace(qkv.device)
    f = _fn(*(("attention_pair", "hb_attention_prefill_pair") if pairs else
              ("attention_tc", "hb_attention_prefill_tc")),
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _run(f(_p(out), _p(qkv), qkv.shape[1], _p(k_pages), _p(v_pages), k_pages.shape[0], _p(block_table),
           block_table.shape[1], _p(q_tiles), q_tiles.shape[0], _p(cu_tokens), _p(start_pos), num_heads,
           num_kv_heads, head_dim, page_size, int(window or 0), float(scale), _p(err), _stream()),
         "attention_prefill_pair" if pairs else "attention_prefill_tc")
    return out


#: first local token of a tile that holds no work (padding of a captured step's tile list)
EMPTY_TILE_TOKEN = 1 << 30


def query_tile_rows(tokens_per_seq, tile: int, start_positions=None):
    """(request, first local token) of every tile of ``tile`` tokens, as a list.  With
    ``start_positions`` the tiles that see the most keys come first (they run longest)."""
    rows = [(i, t0) for i, n in enumerate(tokens_per_seq) for t0 in range(0, n, tile)]
    if start_positions is not None:
        rows.sort(key=lambda r: -(start_positions[r[0]] + r[1]))
    return rows


def query_tiles(tokens_per_seq, tile: int, device, start_positions=None) -> torch.Tensor:
    """int32 [tiles, 2] on ``device``: ``query_tile_rows`` copied over."""
    host = torch.tensor(query_tile_rows(tokens_per_seq, tile, start_positions), dtype=torch.int32).reshape(-1, 2)
    if torch.device(device).type == "cuda":
        host = host.pin_memory()
    return host.to(device, non_blocking=True)


def _step_tiles(ctx, tile: int, longest_first: bool, device) -> torch.Tensor:
    """The step's query tiles of ``tile`` tokens: made once per step and tile size; a step
    that runs as a captured graph hands out buffers that it refills itself
    (``ctx.extras["tile_provider"]``)."""
    key = ("q_tiles", tile, longest_first)
    tiles = ctx.extras.get(key)
    if tiles is None:
        provider = ctx.extras.get("tile_provider")
        if provider is not None:
            tiles = provider(tile, longest_first)
        else:
            tiles = query_tiles([s.num_tokens for s in ctx.seqs], tile, device,
                                [s.start_pos for s in ctx.seqs] if longest_first else None)
        ctx.extras[key] = tiles
    return tiles


def attention(ctx, qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
              page_size: int, window: Optional[int], scale: float,
              fresh=None) -> torch.Tensor:
    """Attention of the step's tokens over the cache; chooses the kernel by dtype, sizes
    and the shape of the batch described by ``ctx``.  bfloat16 with a tiled head size
    runs on the tensor cores (split-context decode kernel for batches of single tokens,
    tiled kernel otherwise); everything else, and float32, on the generic kernel.

    ``fresh`` = (cos, sin, write_cache): ``qkv`` comes straight from the projection; q and k
    are rotated (tables None: no rotation) and, with ``write_cache``, k and v stored in the
    pages first: inside the decode kernel where that one runs, else by ``rope_kv_write``."""
    decode = (qkv.dtype == torch.bfloat16 and head_dim in TILED_HEAD_DIMS and ctx.decode_only
              and num_heads // num_kv_heads <= 16)
    rotary, write_cache = None, False
    if fresh is not None:
        cos, sin, write = fresh
        if decode and ATTENTION_DECODE_ROTARY and (cos is None or cos.shape[1] * 2 == head_dim):
            rotary, write_cache = (cos, sin), bool(write)
        else:
            rope_kv_write(qkv, cos, sin, ctx.positions, ctx.seq_of_token, block_table, k_pages, v_pages,
                          num_heads, num_kv_heads, head_dim, page_size, write_cache=write)
    if qkv.dtype == torch.bfloat16 and head_dim in TILED_HEAD_DIMS:
        if decode:
            splits = ctx.extras.get("decode_splits")
            if splits is None:
                splits = decode_splits(ctx.num_seqs, num_kv_heads, ctx.max_context_len, head_dim)
            return attention_decode_bf16(qkv, k_pages, v_pages, block_table, ctx.positions,
                                         num_heads, num_kv_heads, head_dim, page_size, window,
                                         scale, splits, rotary, write_cache,
                                         decode_warps(ctx.num_seqs * num_kv_heads, splits, head_dim,
                                                      ctx.max_context_len))
        if (ATTENTION_TCGEN05 and ctx.max_tokens_per_seq >= 16
                and tc_attention_supported(num_heads, num_kv_heads, head_dim, page_size)):
            tile = 128 // (num_heads // num_kv_heads)
            # two tiles of query rows per block when that still gives most SMs a block: a
            # block of two tiles takes about 1.5 times as long as a block of one
            pairs = (ATTENTION_TILE_PAIRS and ctx.max_tokens_per_seq > tile
                     and -(-ctx.num_tokens // (2 * tile)) * num_kv_heads >= ATTENTION_PAIR_MIN_BLOCKS)
            tiles = _step_tiles(ctx, 2 * tile if pairs else tile, True, qkv.device)
            return attention_prefill_tc(qkv, k_pages, v_pages, block_table, tiles, ctx.cu_tokens,
                                        ctx.start_pos, num_heads, num_kv_heads, head_dim, page_size,
                                        window, scale, pairs)
        _heads, subtiles = prefill_tiling(num_heads, num_kv_heads)
        tiles = _step_tiles(ctx, 16 * subtiles, False, qkv.device)
        return attention_prefill_bf16(qkv, k_pages, v_pages, block_table, tiles, ctx.cu_tokens,
                                      ctx.start_pos, num_heads, num_kv_heads, head_dim, page_size,
                                      window, scale)
    return attention_generic(qkv, k_pages, v_pages, block_table, ctx.seq_of_token, ctx.positions,
                             num_heads, num_kv_heads, head_dim, page_size, window, scale)
