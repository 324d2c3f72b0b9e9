// Attention over the paged cache for any batch of tokens: one warp per
// (token, query head).  It serves the float32 path and every size the tiled
// bfloat16 kernels do not take.  A token at position p sees the keys at
// positions lo..p of its own request, lo = max(0, p - window + 1) with a
// window and 0 without, wherever the pages lie
// (python/helios/exec/paged_attn.py:264-295, 368-408; GQA mapping :248-261).
//
// Scores, softmax and the weighted sum are float32.  The keys are walked in
// runs of 32 from `lo`, so the order of every sum depends on the token's
// position alone: not on how the request was cut into steps, nor on the rest of
// the batch.
#include "common.cuh"

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_MAX_HD = 256;

template <typename T>
__global__ void attention_generic_kernel(
    T* __restrict__ out, const T* __restrict__ q, int q_stride,
    const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seq_of_token,
    const int* __restrict__ positions, int n_rows, int nh, int nkv, int hd, int page_size,
    int window, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float q_smem[ATTN_WARPS][ATTN_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ATTN_WARPS + warp;
  if (row >= n_rows) return;
  const int t = row / nh, h = row - t * nh;
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * bt_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float* qs = q_smem[warp];
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = to_float(qrow[d]);
  __syncwarp();

  constexpr int ND = ATTN_MAX_HD / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = lo; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    int page = 0;
    float score = -INFINITY;
    if (valid) {
      page = table[key / page_size];
      const T* kr = k_pages + (((size_t)page * nkv + kvh) * page_size + key % page_size) * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
      score = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int n_valid = min(32, pos - base + 1);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int pagej = __shfl_sync(0xffffffffu, page, j);
      const T* vr = v_pages + (((size_t)pagej * nkv + kvh) * page_size + (base + j) % page_size) * hd;
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = out + (size_t)t * nh * hd + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_float<T>(acc[i] * inv);
  }
}

HB_EXPORT int hb_attention_generic(void* out, const void* q, int q_stride, const void* k_pages,
                                   const void* v_pages, const int* block_table, int bt_stride,
                                   const int* seq_of_token, const int* positions, int T, int nh,
                                   int nkv, int hd, int page_size, int window, float scale,
                                   int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (hd <= 0 || hd > ATTN_MAX_HD || nkv <= 0 || nh % nkv != 0 || page_size <= 0)
    return HB_BAD_ARGUMENT;
  const int n_rows = T * nh;
  const int blocks = (n_rows + ATTN_WARPS - 1) / ATTN_WARPS;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(attention_generic_kernel<TA>, dim3(blocks), dim3(ATTN_WARPS * 32), 0, stream, 
        (TA*)out, (const TA*)q, q_stride, (const TA*)k_pages, (const TA*)v_pages, block_table,
        bt_stride, seq_of_token, positions, n_rows, nh, nkv, hd, page_size, window, scale));
  return hb_check_launch();
}
