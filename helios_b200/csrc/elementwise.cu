// Embedding gather, fused residual-add + RMSNorm, rotary encoding fused with the
// write of keys and values into cache pages, SwiGLU gating.
//
// The residual stream is always float32; "act" tensors (GEMM inputs and
// outputs, cache pages) are float32 or bfloat16 by a type code.  Statistics,
// angles and sums are float32 in both modes.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] (f32) = table[ids[t], :]      python/helios/exec/model.py:486
template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // ids are validated on the host
  const T* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

// bfloat16 table, rows of whole 16-byte chunks: 8 values per thread and trip
__global__ void embedding_bf16x8_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ table,
                                        const int* __restrict__ ids, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  float4* o = reinterpret_cast<float4*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 x = row[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&x);
    o[2 * i] = make_float4(__low2float(p[0]), __high2float(p[0]), __low2float(p[1]), __high2float(p[1]));
    o[2 * i + 1] = make_float4(__low2float(p[2]), __high2float(p[2]), __low2float(p[3]), __high2float(p[3]));
  }
}

HB_EXPORT int hb_embedding(float* out, const void* table, const int* ids, int T, int H, int V,
                           int table_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (table_dt == HB_BF16 && H % 8 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0) {
    hb_launch(embedding_bf16x8_kernel, dim3(T), dim3(256), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V);
    return hb_check_launch();
  }
  HB_DISPATCH_DTYPE(table_dt, TT,
    hb_launch(embedding_kernel<TT>, dim3(T), dim3(256), 0, stream, out, (const TT*)table, ids, H, V));
  return hb_check_launch();
}

// ---------------------------------------------------------------- add + RMSNorm
// residual[r] += delta[r] (if delta); out[i] = residual[r] * rsqrt(mean(residual[r]^2) + eps) * w
// where r = rows ? rows[i] : i.  With `rows` the residual is not written back
// (the final norm runs on the wanted rows only).    python/helios/exec/model.py:109-114
//
// A row is held in registers between the two passes (groups of four values per thread,
// all loads issued before the first use), so a row costs one trip to memory.
template <typename T> struct Vec4 { T v[4]; };

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
  } else {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
  }
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_GROUPS = 8;     // groups of 4 values a thread keeps: rows up to 8192 wide

template <typename TA, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_kernel(TA* __restrict__ out, float* __restrict__ residual, const TA* __restrict__ delta,
                   const float* __restrict__ weight, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * H;
  const TA* d = delta ? delta + (size_t)r * H : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  TA* o = out + (size_t)i * H;
  float ss = 0.f;
  if constexpr (VEC) {
    float v[NORM_GROUPS][4];
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) load4(res + c, v[g]);
    }
    if (d) {
#pragma unroll
      for (int g = 0; g < NORM_GROUPS; ++g) {
        const int c = (g * NORM_THREADS + threadIdx.x) * 4;
        if (c < H) {
          float dv[4];
          load4(d + c, dv);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[g][e] += dv[e];
        }
      }
    }
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        if (write_back) store4(res + c, v[g]);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += v[g][e] * v[g][e];
      }
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        float w[4], y[4];
        load4(weight + c, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = v[g][e] * rstd * w[e];
        store4(o + c, y);
      }
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = res[c];
      if (d) v += to_float(d[c]);
      if (write_back) res[c] = v;
      ss += v * v;
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = res[c];
      if (d && !write_back) v += to_float(d[c]);
      o[c] = from_float<TA>(v * rstd * weight[c]);
    }
  }
}

HB_EXPORT int hb_add_rmsnorm(void* out, float* residual, const void* delta, const float* weight,
                             const int* rows, int n_out, int H, float eps, int act_dt,
                             cudaStream_t stream) {
  if (n_out <= 0) return HB_OK;
  // the register-resident path needs whole groups of four and 16-byte aligned rows
  const bool vec = (H % 4 == 0) && H <= NORM_THREADS * NORM_GROUPS * 4 &&
                   ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                   ((uintptr_t)delta % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                   (act_dt == HB_F32 || H % 8 == 0);
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (vec) hb_launch(add_rmsnorm_kernel<TA, true>, dim3(n_out), dim3(NORM_THREADS), 0, stream, 
        (TA*)out, residual, (const TA*)delta, weight, rows, H, eps);
    else hb_launch(add_rmsnorm_kernel<TA, false>, dim3(n_out), dim3(NORM_THREADS), 0, stream, 
        (TA*)out, residual, (const TA*)delta, weight, rows, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- plain RMSNorm of act rows
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ weight, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const T* xr = x + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) { float v = to_float(xr[c]); ss += v * v; }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  T* o = out + (size_t)blockIdx.x * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    o[c] = from_float<T>(to_float(xr[c]) * rstd * weight[c]);
}

HB_EXPORT int hb_rmsnorm(void* out, const void* x, const float* weight, int n, int H, float eps,
                         int act_dt, cudaStream_t stream) {
  if (n <= 0) return HB_OK;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(rmsnorm_kernel<TA>, dim3(n), dim3(256), 0, stream, (TA*)out, (const TA*)x, weight, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotary tables
// cos/sin[t, j] of angle = position[t] * inv_freq[j], the product and the functions in
// float64, the result rounded to float32 (python/helios/exec/model.py:127-132 builds the
// same table for every position up to max_position_embeddings).
__global__ void rotary_table_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out,
                                    const int* __restrict__ positions,
                                    const double* __restrict__ inv_freq, int T, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, j = idx - t * half;
  double s, c;
  sincos((double)positions[t] * inv_freq[j], &s, &c);
  cos_out[idx] = (float)c;
  sin_out[idx] = (float)s;
}

HB_EXPORT int hb_rotary_table(float* cos_out, float* sin_out, const int* positions,
                              const double* inv_freq, int T, int half, cudaStream_t stream) {
  if (T <= 0 || half <= 0) return HB_OK;
  const int total = T * half;
  hb_launch(rotary_table_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, cos_out, sin_out, positions,
                                                               inv_freq, T, half);
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotary + cache write
// qkv: [T, (nh + 2 nkv) * hd], q heads first, then k heads, then v heads.
// For every token: rotate q and k (rotate-half pairs (j, j + rot/2) by the token's
// cos/sin row, float32; python/helios/exec/model.py:148-153), leave q in place, and
// store the rotated k and the v at the token's place in its pages
// (python/helios/exec/paged_attn.py:74-85): page = block_table[seq, pos / page],
// pages laid out [page, kv head, slot, hd].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ cos_tab,
                                     const float* __restrict__ sin_tab,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int bt_stride,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int nh, int nkv, int hd, int rot, int page_size,
                                     int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  const float* cs = cos_tab + (size_t)t * half;
  const float* sn = sin_tab + (size_t)t * half;
  T* row = qkv + (size_t)t * (size_t)(nh + 2 * nkv) * hd;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  // rotated pairs of q and k heads
  const int n_rot_heads = nh + nkv;
  for (int w = threadIdx.x; w < n_rot_heads * half; w += blockDim.x) {
    const int h = w / half, j = w - h * half;
    T* x = row + (size_t)h * hd;
    const float x1 = to_float(x[j]), x2 = to_float(x[j + half]);
    const float c = cs[j], s = sn[j];
    const T r1 = from_float<T>(x1 * c - x2 * s);
    const T r2 = from_float<T>(x2 * c + x1 * s);
    if (h < nh || !write_cache) {
      x[j] = r1;
      x[j + half] = r2;
    } else {
      T* dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
      dst[j] = r1;
      dst[j + half] = r2;
    }
  }
  if (!write_cache) return;
  // un-rotated tail of k (rot < hd), and v
  if (rot < hd) {
    const int tail = hd - rot;
    for (int w = threadIdx.x; w < nkv * tail; w += blockDim.x) {
      const int h = w / tail, j = rot + (w - h * tail);
      k_pages[((page_base + h) * page_size + slot) * hd + j] = row[(size_t)(nh + h) * hd + j];
    }
  }
  for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
    const int h = w / hd, j = w - h * hd;
    v_pages[((page_base + h) * page_size + slot) * hd + j] = row[(size_t)(nh + nkv + h) * hd + j];
  }
}

// The same, four rotary pairs (or eight copied values) per thread, for full rotation
// (rot == hd) with hd a multiple of 8: one block of work items per token is
// (nh + nkv) * hd / 8 rotations followed by nkv * hd / 8 copies of v.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ cos_tab,
                                         const float* __restrict__ sin_tab,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int bt_stride,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         int nh, int nkv, int hd, int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int half = hd >> 1, quads = half >> 2;            // groups of 4 pairs per head
  const int n_rot = (nh + nkv) * quads;
  const int n_copy = write_cache ? nkv * (hd >> 3) : 0;   // groups of 8 values of v
  if (item >= n_rot + n_copy) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * (size_t)(nh + 2 * nkv) * hd;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  if (item < n_rot) {
    const int h = item / quads, j = (item - h * quads) * 4;
    T* x = row + (size_t)h * hd;
    float x1[4], x2[4], c[4], sn[4], r1[4], r2[4];
    load4(x + j, x1);
    load4(x + j + half, x2);
    load4(cos_tab + (size_t)t * half + j, c);
    load4(sin_tab + (size_t)t * half + j, sn);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // round as the scalar kernel does: each product pair in float32, one rounding to T
      r1[e] = x1[e] * c[e] - x2[e] * sn[e];
      r2[e] = x2[e] * c[e] + x1[e] * sn[e];
    }
    T* dst = x;
    if (h >= nh && write_cache) dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
    store4(dst + j, r1);
    store4(dst + j + half, r2);
  } else {
    const int w = item - n_rot;
    const int per = hd >> 3;
    const int h = w / per, j = (w - h * per) * 8;
    const T* src = row + (size_t)(nh + nkv + h) * hd + j;
    T* dst = v_pages + ((page_base + h) * page_size + slot) * hd + j;
    float a[4], b[4];
    load4(src, a);
    load4(src + 4, b);
    store4(dst, a);
    store4(dst + 4, b);
  }
}

HB_EXPORT int hb_rope_kv_write(void* qkv, const float* cos_tab, const float* sin_tab,
                               const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, void* k_pages,
                               void* v_pages, int T, int nh, int nkv, int hd, int rot,
                               int page_size, int write_cache, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return HB_BAD_ARGUMENT;
  const bool vec = rot == hd && hd % 8 == 0 && (uintptr_t)qkv % 16 == 0 &&
                   (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 &&
                   (uintptr_t)cos_tab % 16 == 0 && (uintptr_t)sin_tab % 16 == 0;
  if (vec) {
    const int items = (nh + nkv) * (hd / 8) + (write_cache ? nkv * (hd / 8) : 0);
    dim3 grid(T, (items + 127) / 128);
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(rope_kv_write_vec_kernel<TA>, dim3(grid), dim3(128), 0, stream, 
          (TA*)qkv, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride,
          (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, page_size, write_cache));
    return hb_check_launch();
  }
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(rope_kv_write_kernel<TA>, dim3(T), dim3(256), 0, stream, 
        (TA*)qkv, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride,
        (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, rot, page_size, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- SwiGLU gate
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]        python/helios/exec/model.py:336-337
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t total, int I) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

HB_EXPORT int hb_silu_mul(void* out, const void* gate_up, int T, int I, int act_dt,
                          cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(silu_mul_kernel<TA>, dim3((unsigned)blocks), dim3(threads), 0, stream, (TA*)out, (const TA*)gate_up, total, I));
  return hb_check_launch();
}
