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
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // ids are validated on the host
  const T* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

HB_EXPORT int hb_embedding(float* out, const void* table, const int* ids, int T, int H, int V,
                           int table_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  HB_DISPATCH_DTYPE(table_dt, TT,
    embedding_kernel<TT><<<T, 256, 0, stream>>>(out, (const TT*)table, ids, H, V));
  return hb_check_launch();
}

// ---------------------------------------------------------------- add + RMSNorm
// residual[r] += delta[r] (if delta); out[i] = residual[r] * rsqrt(mean(residual[r]^2) + eps) * w
// where r = rows ? rows[i] : i.  With `rows` the residual is not written back
// (the final norm runs on the wanted rows only).    python/helios/exec/model.py:109-114
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual,
                                   const TD* __restrict__ delta, const float* __restrict__ weight,
                                   const int* __restrict__ rows, int H, float eps) {
  __shared__ float scratch[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * H;
  const TD* d = delta ? delta + (size_t)r * H : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = res[c];
    if (d) v += to_float(d[c]);
    if (write_back) res[c] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  TO* o = out + (size_t)i * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = res[c];
    if (d && !write_back) v += to_float(d[c]);
    o[c] = from_float<TO>(v * rstd * weight[c]);
  }
}

HB_EXPORT int hb_add_rmsnorm(void* out, float* residual, const void* delta, const float* weight,
                             const int* rows, int n_out, int H, float eps, int act_dt,
                             cudaStream_t stream) {
  if (n_out <= 0) return HB_OK;
  const int threads = H >= 2048 ? 512 : 256;
  HB_DISPATCH_DTYPE(act_dt, TA,
    add_rmsnorm_kernel<TA, TA><<<n_out, threads, 0, stream>>>(
        (TA*)out, residual, (const TA*)delta, weight, rows, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- plain RMSNorm of act rows
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ weight, int H, float eps) {
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
    rmsnorm_kernel<TA><<<n, 256, 0, stream>>>((TA*)out, (const TA*)x, weight, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotary tables
// cos/sin[t, j] of angle = position[t] * inv_freq[j], the product and the functions in
// float64, the result rounded to float32 (python/helios/exec/model.py:127-132 builds the
// same table for every position up to max_position_embeddings).
__global__ void rotary_table_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out,
                                    const int* __restrict__ positions,
                                    const double* __restrict__ inv_freq, int T, int half) {
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
  rotary_table_kernel<<<(total + 127) / 128, 128, 0, stream>>>(cos_out, sin_out, positions,
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

HB_EXPORT int hb_rope_kv_write(void* qkv, const float* cos_tab, const float* sin_tab,
                               const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, void* k_pages,
                               void* v_pages, int T, int nh, int nkv, int hd, int rot,
                               int page_size, int write_cache, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    rope_kv_write_kernel<TA><<<T, 256, 0, stream>>>(
        (TA*)qkv, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride,
        (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, rot, page_size, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- SwiGLU gate
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]        python/helios/exec/model.py:336-337
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t total, int I) {
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
    silu_mul_kernel<TA><<<(unsigned)blocks, threads, 0, stream>>>((TA*)out, (const TA*)gate_up, total, I));
  return hb_check_launch();
}
