// Sampling of one token per logits row, on the device: greedy, or temperature
// with optional top-k and top-p, drawn by inverse CDF from a Philox uniform that
// depends on the request's (seed, offset) only.
//
// Meaning of the options follows python/helios/exec/sampler.py:51-81: temperature 0 is
// argmax of the raw logits; otherwise logits/T; top-k keeps logits >= the k-th
// largest; top-p keeps, in descending order, every token before which the
// cumulative probability is <= top_p (the token that crosses it stays); softmax
// over what is kept.  The reference draws with torch.multinomial from a CPU
// generator per request; here the stream is Philox4x32-10 keyed by the
// request's seed and counted by its own number of sampled tokens, so a request's
// tokens do not depend on what else is in the batch.
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t float_key(float f) {  // order-preserving
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__host__ __device__ inline uint32_t philox_first_word(uint64_t seed, uint64_t offset) {
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

// Block-wide sum in a fixed order; every thread gets the result.
__device__ __forceinline__ float block_sum_all(float v, float* scratch) { return block_sum(v, scratch); }

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float partial[SAMPLE_THREADS];
  __shared__ int s_pick;
  __shared__ float s_prefix;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* l = logits + (size_t)row * ld;

  // ---- argmax, lowest index among equals
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = tid; c < V; c += SAMPLE_THREADS) {
    const float v = l[c];
    if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = s_val[lane]; bi = s_idx[lane];
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { s_val[0] = bv; s_idx[0] = bi; }
  }
  __syncthreads();
  const float mx = s_val[0];
  const int amax = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];
  const float temp = temperature[row];
  if (!(temp > 0.f)) {
    if (tid == 0) out[row] = amax;
    return;
  }
  const float inv_t = 1.f / temp;
  const float mx_t = mx * inv_t;

  // ---- top-k: the largest key c with #(key >= c) >= k
  uint32_t thr = 0;
  const int k = top_k[row];
  if (k > 0 && k < V) {
    uint32_t cand = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t tryk = cand | (1u << bit);
      float cnt = 0.f;
      for (int c = tid; c < V; c += SAMPLE_THREADS) cnt += (float_key(l[c]) >= tryk) ? 1.f : 0.f;
      if (block_sum_all(cnt, scratch) >= (float)k) cand = tryk;
    }
    thr = cand;
  }
  // ---- top-p over what top-k kept: the largest key c with mass(key >= c) > p * Z
  const float pp = top_p[row];
  if (pp < 1.f) {
    float z = 0.f;
    for (int c = tid; c < V; c += SAMPLE_THREADS)
      if (float_key(l[c]) >= thr) z += expf(l[c] * inv_t - mx_t);
    const float Z = block_sum_all(z, scratch);
    const float want = pp * Z;
    uint32_t cand = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t tryk = cand | (1u << bit);
      const uint32_t lim = tryk > thr ? tryk : thr;
      float mass = 0.f;
      for (int c = tid; c < V; c += SAMPLE_THREADS)
        if (float_key(l[c]) >= lim) mass += expf(l[c] * inv_t - mx_t);
      if (block_sum_all(mass, scratch) > want) cand = tryk;
    }
    if (cand > thr) thr = cand;
  }

  // ---- inverse CDF in index order over contiguous chunks
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int c_lo = min(V, tid * chunk), c_hi = min(V, c_lo + chunk);
  float mine = 0.f;
  for (int c = c_lo; c < c_hi; ++c)
    if (float_key(l[c]) >= thr) mine += expf(l[c] * inv_t - mx_t);
  partial[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) total += partial[i];
    const uint32_t r = philox_first_word(seed[row], offset[row]);
    const float u = (float)(r >> 8) * (1.0f / 16777216.0f);
    const float target = u * total;
    float cum = 0.f;
    int pick = -1, last_nonzero = 0;
    float prefix = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) {
      if (partial[i] > 0.f) last_nonzero = i;
      if (pick < 0 && cum + partial[i] > target) { pick = i; prefix = cum; }
      cum += partial[i];
    }
    if (pick < 0) { pick = last_nonzero; prefix = -INFINITY; }  // rounding at the very end
    s_pick = pick;
    s_prefix = prefix;
    partial[0] = target;
  }
  __syncthreads();
  if (tid == s_pick) {
    const float target = partial[0];
    float cum = s_prefix;
    int choice = -1, last_kept = amax;
    for (int c = c_lo; c < c_hi; ++c) {
      if (float_key(l[c]) < thr) continue;
      last_kept = c;
      cum += expf(l[c] * inv_t - mx_t);
      if (cum > target) { choice = c; break; }
    }
    out[row] = choice >= 0 ? choice : last_kept;
  }
}

HB_EXPORT int hb_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature,
                        const int* top_k, const float* top_p, const unsigned long long* seed,
                        const unsigned long long* offset, cudaStream_t stream) {
  if (R <= 0) return HB_OK;
  if (V <= 0) return HB_BAD_ARGUMENT;
  hb_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, out, logits, V, ld, temperature, top_k, top_p,
                                                  seed, offset);
  return hb_check_launch();
}

// The uniform a request draws at (seed, offset): the same function for host-side checks.
HB_EXPORT float hb_philox_uniform(unsigned long long seed, unsigned long long offset) {
  return (float)(philox_first_word(seed, offset) >> 8) * (1.0f / 16777216.0f);
}
