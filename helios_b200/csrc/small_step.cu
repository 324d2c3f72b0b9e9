// Matrix products of steps with very few tokens (at most 16: a handful of requests
// decoding), fused with what stands before and after them in a decoder layer
// (python/helios/exec/model.py:373-392 runs norm, projections, rotation, cache write,
// gate and residual adds as separate operations):
//
//   QKV      : RMSNorm of the residual stream -> q|k|v projection (+ bias) -> rotation of
//              q and k (rotate-half) -> q into the step's buffer, k and v into the cache pages
//   GLU      : RMSNorm of the residual stream -> gate|up projection -> silu(gate) * up
//   RESIDUAL : residual stream += x W^T          (output projection, down projection)
//
// At these sizes a product is a stream of weights against a few activation rows, and a
// step is bound by the number of dependent kernels, not by arithmetic: five launches a
// layer instead of eight, and no tensor-memory or TMA set-up on the critical path.
//
// The tokens ride the M axis of mma.sync.m16n8k16 (rows beyond the step's tokens are zero),
// eight weight rows the N axis; a block owns 8 * NT weight rows and ALL of K, its sixteen
// warps take every sixteenth block of 32 k each and add their partial sums through shared
// memory in warp order, so a result does not depend on anything but its own row.  Weights
// go from global memory straight into the B fragments, 16 bytes a thread: within a block
// of 32 k, thread t of a quad holds k 8t..8t+7 of its row, and the two MMAs of the block
// take elements (0,1,2,3) and (4,5,6,7) of every thread's chunk as their k columns
// (2t, 2t+1, 2t+8, 2t+9).  The activations are put into the A fragments by the same rule,
// so every k meets its partner.  A block's first weights are requested before it waits
// for the kernel before it (programmatic dependent launch).
//
// With the norm in front, a block reads the residual rows itself (float32, from L2) in the
// same pass: the A fragments hold bfloat16(residual * norm weight), the sum of squares is
// gathered beside the products, and 1/rms, a factor per token, multiplies the finished sums
// in the epilogue.  Statistics and scaled values are float32
// (python/helios/exec/model.py:109-114); against norming first, only the place of the one
// rounding to bfloat16 moves.
#include "common.cuh"

namespace {

constexpr int SS_WARPS = 16;
constexpr int SS_THREADS = SS_WARPS * 32;

enum { MODE_RESIDUAL = 0, MODE_GLU = 1, MODE_QKV = 2 };

struct SmallArgs {
  const float* residual_in;     // NORM: [T, K] float32
  const float* norm_weight;     // NORM: [K]
  float eps;
  const __nv_bfloat16* x;       // !NORM: [T, K]
  const __nv_bfloat16* w;       // [rows, K]
  const float* bias;            // [rows] or null (QKV only)
  int T, K;
  int n_out;                    // RESIDUAL: rows; GLU: result features I; QKV: (nh + 2 nkv) * hd
  float* residual_out;          // RESIDUAL: [T, n_out]
  __nv_bfloat16* out;           // GLU: [T, n_out]
  int glu_offset;               // GLU: first up row of w
  __nv_bfloat16* qkv;           // QKV: [T, qkv_stride], q heads first
  int qkv_stride;
  const float* cos_tab;         // [T, hd / 2]
  const float* sin_tab;
  const int* positions;         // [T]
  const int* seq_of_token;      // [T]
  const int* block_table;       // [requests, bt_stride]
  int bt_stride;
  __nv_bfloat16* k_pages;       // [pages, nkv, page_size, hd]
  __nv_bfloat16* v_pages;
  int nh, nkv, hd, page_size, write_cache;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Weight row of column n (0..7) of tile `tile`, or -1 beyond the matrix.
template <int MODE>
__device__ __forceinline__ int tile_row(const SmallArgs& a, int tile, int n) {
  if (MODE == MODE_RESIDUAL) {
    const int r = tile * 8 + n;
    return r < a.n_out ? r : -1;
  } else if (MODE == MODE_GLU) {
    const int f = tile * 4 + (n & 3);
    if (f >= a.n_out) return -1;
    return n < 4 ? f : a.glu_offset + f;
  } else {
    const int per_head = a.hd >> 3;
    const int head = tile / per_head, sub = tile - head * per_head;
    if (head >= a.nh + 2 * a.nkv) return -1;
    if (head < a.nh + a.nkv)     // a rotated head: four pairs (d, d + hd/2)
      return head * a.hd + (n < 4 ? sub * 4 + n : (a.hd >> 1) + sub * 4 + (n - 4));
    return head * a.hd + sub * 8 + n;
  }
}

// Bytes between two activation rows in shared memory: 64 beyond a multiple of 128, so the
// 16-byte reads of two neighbouring rows fall into different banks.
__host__ __device__ inline int x_row_bytes(int K) { return ((2 * K + 63) / 128) * 128 + 64; }

// DEEP: twice the weights requested at once (and twice the registers, so one block an SM):
// for long reductions in launches of at most one block per SM, where the second round trip
// to memory would otherwise wait for the first.
template <int MODE, int NT, bool NORM, bool T8, bool DEEP>
__global__ void __launch_bounds__(SS_THREADS, DEEP ? 1 : 2)
small_step_kernel(const SmallArgs a) {
  constexpr int U = (DEEP ? 16 : 8) / NT;   // blocks of 32 k whose weights a warp requests at once
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char xs[];     // [T][x_row_bytes(K)] bfloat16 activations
  __shared__ float red[SS_WARPS][NT][16][8];
  __shared__ float rstd_of[16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int nkb = (a.K + 31) >> 5;
  const int stride = x_row_bytes(a.K);
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

  // this thread's weight rows, as offsets in 16-byte units (rows of K % 8 == 0 values)
  constexpr uint32_t NO_ROW = 0xffffffffu;
  const uint4* w16 = reinterpret_cast<const uint4*>(a.w);
  uint32_t wrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int r = tile_row<MODE>(a, blockIdx.x * NT + j, g);
    wrow[j] = r >= 0 ? (uint32_t)r * (uint32_t)(a.K >> 3) : NO_ROW;
  }
  auto load_w = [&](int kb, uint4 (&w)[NT]) {
    const int k = kb * 32 + t4 * 8;
    const bool ok = kb < nkb && k < a.K;
#pragma unroll
    for (int j = 0; j < NT; ++j) w[j] = (ok && wrow[j] != NO_ROW) ? ldg_stream(w16 + wrow[j] + (k >> 3)) : zero4;
  };

  uint4 wreg[U][NT];
#pragma unroll
  for (int u = 0; u < U; ++u) load_w(warp + u * SS_WARPS, wreg[u]);
  pdl_wait();

  // the step's activations into shared memory, rows beyond the step's tokens zero
  const int chunks = a.K >> 3;              // 16-byte chunks of a row
  if (NORM) {
    // a warp takes a row: bfloat16(residual * norm weight) and the row's sum of squares
    if (warp < a.T) {
      float ss = 0.f;
      unsigned char* dst = xs + (size_t)warp * stride;
      const float* src = a.residual_in + (size_t)warp * a.K;
#pragma unroll 4
      for (int c = lane; c < chunks; c += 32) {
        const float4 p = *reinterpret_cast<const float4*>(src + c * 8);
        const float4 q = *reinterpret_cast<const float4*>(src + c * 8 + 4);
        const float4 wp = *reinterpret_cast<const float4*>(a.norm_weight + c * 8);
        const float4 wq = *reinterpret_cast<const float4*>(a.norm_weight + c * 8 + 4);
        ss += p.x * p.x + p.y * p.y + p.z * p.z + p.w * p.w + q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
        *reinterpret_cast<uint4*>(dst + c * 16) =
            make_uint4(pack2(p.x * wp.x, p.y * wp.y), pack2(p.z * wp.z, p.w * wp.w),
                       pack2(q.x * wq.x, q.y * wq.y), pack2(q.z * wq.z, q.w * wq.w));
      }
      ss = warp_sum(ss);
      if (lane == 0) rstd_of[warp] = rsqrtf(ss / (float)a.K + a.eps);
    }
  } else {
    for (int c = threadIdx.x; c < a.T * chunks; c += SS_THREADS) {
      const int row = c / chunks, cc = c - row * chunks;
      *reinterpret_cast<uint4*>(xs + (size_t)row * stride + cc * 16) =
          *reinterpret_cast<const uint4*>(a.x + (size_t)row * a.K + cc * 8);
    }
  }
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  const unsigned char* x_lo = xs + (size_t)g * stride + t4 * 16;
  const unsigned char* x_hi = xs + (size_t)(g + 8) * stride + t4 * 16;
  for (int kb = warp; kb < nkb; kb += U * SS_WARPS) {
    if (kb != warp) {
#pragma unroll
      for (int u = 0; u < U; ++u) load_w(kb + u * SS_WARPS, wreg[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kbu = kb + u * SS_WARPS;
      const bool in = kbu < nkb && kbu * 32 + t4 * 8 < a.K;
      // rows beyond the step's tokens are not in shared memory: their fragments are zero
      const uint4 lo = (in && g < a.T) ? *reinterpret_cast<const uint4*>(x_lo + kbu * 64) : zero4;
      const uint4 hi = (!T8 && in && g + 8 < a.T) ? *reinterpret_cast<const uint4*>(x_hi + kbu * 64) : zero4;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16(acc[j], lo.x, hi.x, lo.y, hi.y, wreg[u][j].x, wreg[u][j].y);
        mma_bf16(acc[j], lo.z, hi.z, lo.w, hi.w, wreg[u][j].z, wreg[u][j].w);
      }
    }
  }

  // partial sums of the warps: [warp][tile][token][weight row of the tile]
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][j][g][2 * t4] = acc[j][0];
    red[warp][j][g][2 * t4 + 1] = acc[j][1];
    red[warp][j][g + 8][2 * t4] = acc[j][2];
    red[warp][j][g + 8][2 * t4 + 1] = acc[j][3];
  }
  __syncthreads();

  // epilogue: a thread finishes (tile, token, columns p and p + 4)
  const int item = threadIdx.x;
  if (item >= NT * 64) return;
  const int j = item >> 6, token = (item >> 2) & 15, p = item & 3;
  if (token >= a.T) return;
  float v1 = 0.f, v2 = 0.f;
#pragma unroll
  for (int w = 0; w < SS_WARPS; ++w) {
    v1 += red[w][j][token][p];
    v2 += red[w][j][token][p + 4];
  }
  if (NORM) {
    v1 *= rstd_of[token];
    v2 *= rstd_of[token];
  }
  const int tile = blockIdx.x * NT + j;
  const int r1 = tile_row<MODE>(a, tile, p), r2 = tile_row<MODE>(a, tile, p + 4);
  if (MODE == MODE_RESIDUAL) {
    if (r1 >= 0) a.residual_out[(size_t)token * a.n_out + r1] += v1;
    if (r2 >= 0) a.residual_out[(size_t)token * a.n_out + r2] += v2;
  } else if (MODE == MODE_GLU) {
    if (r1 >= 0) a.out[(size_t)token * a.n_out + r1] = __float2bfloat16_rn(v1 / (1.f + __expf(-v1)) * v2);
  } else {
    if (r1 < 0) return;
    if (a.bias != nullptr) {
      v1 += a.bias[r1];
      v2 += a.bias[r2];
    }
    const int head = r1 / a.hd, d1 = r1 - head * a.hd, d2 = r2 - head * a.hd;
    if (head < a.nh + a.nkv) {
      const int half = a.hd >> 1;
      const float c = a.cos_tab[(size_t)token * half + d1], s = a.sin_tab[(size_t)token * half + d1];
      const float o1 = v1 * c - v2 * s, o2 = v2 * c + v1 * s;
      v1 = o1;
      v2 = o2;
    }
    __nv_bfloat16* dst = a.qkv + (size_t)token * a.qkv_stride + (size_t)head * a.hd;   // q, or no cache write
    if (head >= a.nh && a.write_cache) {
      const int pos = a.positions[token];
      const int page = a.block_table[(size_t)a.seq_of_token[token] * a.bt_stride + pos / a.page_size];
      const int slot = pos % a.page_size;
      const bool is_k = head < a.nh + a.nkv;
      const int kvh = is_k ? head - a.nh : head - a.nh - a.nkv;
      dst = (is_k ? a.k_pages : a.v_pages) + (((size_t)page * a.nkv + kvh) * a.page_size + slot) * a.hd;
    }
    dst[d1] = __float2bfloat16_rn(v1);
    dst[d2] = __float2bfloat16_rn(v2);
  }
}

constexpr int SS_MAX_DYNAMIC_SMEM = 160 * 1024;

template <void (*kernel)(const SmallArgs)>
int launch_one(dim3 grid, size_t smem, const SmallArgs& a, cudaStream_t stream) {
  // the limit on dynamic shared memory is an attribute of each kernel on each device
  static bool configured[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HB_LAUNCH_FAILED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SS_MAX_DYNAMIC_SMEM) !=
        cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured[dev] = true;
  }
  hb_launch(kernel, grid, dim3(SS_THREADS), smem, stream, a);
  return hb_check_launch();
}

int sm_count_of_current_device() {
  static int counts[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (counts[dev] == 0) cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev);
  return counts[dev];
}

template <int MODE, bool NORM>
int launch_small(const SmallArgs& a, int tiles, int nt, cudaStream_t stream) {
  const bool t8 = a.T <= 8;
  const size_t smem = (size_t)a.T * x_row_bytes(a.K);
  if (smem > (size_t)SS_MAX_DYNAMIC_SMEM) return HB_BAD_ARGUMENT;
  const int blocks = (tiles + nt - 1) / nt;
  // a warp's share of K in blocks of 32; more than one request of 8 / nt blocks, in a launch
  // that leaves room for one block per SM: the deep variant
  const int per_warp = ((a.K + 31) / 32 + SS_WARPS - 1) / SS_WARPS;
  const bool deep = per_warp * nt > 8 && blocks <= sm_count_of_current_device();
#define HB_SS_CASE(NT_)                                                                                   \
  {                                                                                                       \
    const dim3 grid(blocks);                                                                              \
    if (deep) {                                                                                           \
      if (t8) return launch_one<small_step_kernel<MODE, NT_, NORM, true, true>>(grid, smem, a, stream);   \
      return launch_one<small_step_kernel<MODE, NT_, NORM, false, true>>(grid, smem, a, stream);          \
    }                                                                                                     \
    if (t8) return launch_one<small_step_kernel<MODE, NT_, NORM, true, false>>(grid, smem, a, stream);    \
    return launch_one<small_step_kernel<MODE, NT_, NORM, false, false>>(grid, smem, a, stream);           \
  }
  switch (nt) {
    case 1: HB_SS_CASE(1)
    case 2: HB_SS_CASE(2)
    case 4: HB_SS_CASE(4)
    default: return HB_BAD_ARGUMENT;
  }
#undef HB_SS_CASE
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

// residual[T, N] += x[T, K] w[N, K]^T.  nt = tiles of 8 weight rows per block (1, 2 or 4).
// Most reduction length (K) the kernels take for a step of T tokens: the activations, as
// bfloat16 rows, must fit the block's shared memory.
HB_EXPORT int hb_small_step_max_k(int T) {
  const int rows = T < 1 ? 1 : T;
  return ((SS_MAX_DYNAMIC_SMEM / rows - 64) / 128) * 64;
}

HB_EXPORT int hb_small_linear_residual(float* residual, const void* x, const void* w, int T, int N, int K,
                                       int nt, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return HB_OK;
  if (T > 16 || K <= 0 || (K & 7) || !aligned16(x) || !aligned16(w)) return HB_BAD_ARGUMENT;
  SmallArgs a = {};
  a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w; a.T = T; a.K = K; a.n_out = N;
  a.residual_out = residual;
  return launch_small<MODE_RESIDUAL, false>(a, (N + 7) / 8, nt, stream);
}

// out[T, I] = silu(h gate^T) * (h up^T) with h = RMSNorm(residual) and w = [gate rows; up rows].
HB_EXPORT int hb_small_norm_swiglu(void* out, const float* residual, const float* norm_weight, float eps,
                                   const void* w, int T, int I, int K, int glu_offset, int nt,
                                   cudaStream_t stream) {
  if (T <= 0 || I <= 0) return HB_OK;
  if (T > 16 || K <= 0 || (K & 7) || !aligned16(residual) || !aligned16(norm_weight) || !aligned16(w))
    return HB_BAD_ARGUMENT;
  SmallArgs a = {};
  a.residual_in = residual; a.norm_weight = norm_weight; a.eps = eps;
  a.w = (const __nv_bfloat16*)w; a.T = T; a.K = K; a.n_out = I; a.glu_offset = glu_offset;
  a.out = (__nv_bfloat16*)out;
  return launch_small<MODE_GLU, true>(a, (I + 3) / 4, nt, stream);
}

// q|k|v = RMSNorm(residual) w^T (+ bias); q and k rotated by the tokens' cos/sin rows
// ([T, hd/2]); q to qkv[T, qkv_stride], k and v to the tokens' places in the cache pages
// (or, without write_cache, beside q).
HB_EXPORT int hb_small_norm_qkv_rope(void* qkv, int qkv_stride, const float* residual,
                                     const float* norm_weight, float eps, const void* w, const float* bias,
                                     const float* cos_tab, const float* sin_tab, const int* positions,
                                     const int* seq_of_token, const int* block_table, int bt_stride,
                                     void* k_pages, void* v_pages, int T, int K, int nh, int nkv, int hd,
                                     int page_size, int write_cache, int nt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (T > 16 || K <= 0 || (K & 7) || (hd & 7) || hd <= 0 || nh <= 0 || nkv <= 0 || page_size <= 0 ||
      !aligned16(residual) || !aligned16(norm_weight) || !aligned16(w))
    return HB_BAD_ARGUMENT;
  SmallArgs a = {};
  a.residual_in = residual; a.norm_weight = norm_weight; a.eps = eps;
  a.w = (const __nv_bfloat16*)w; a.bias = bias; a.T = T; a.K = K; a.n_out = (nh + 2 * nkv) * hd;
  a.qkv = (__nv_bfloat16*)qkv; a.qkv_stride = qkv_stride; a.cos_tab = cos_tab; a.sin_tab = sin_tab;
  a.positions = positions; a.seq_of_token = seq_of_token; a.block_table = block_table; a.bt_stride = bt_stride;
  a.k_pages = (__nv_bfloat16*)k_pages; a.v_pages = (__nv_bfloat16*)v_pages;
  a.nh = nh; a.nkv = nkv; a.hd = hd; a.page_size = page_size; a.write_cache = write_cache;
  return launch_small<MODE_QKV, true>(a, (nh + 2 * nkv) * (hd / 8), nt, stream);
}
