// Sampling of one token per logits row, on the device: greedy, or temperature
// with optional top-k and top-p, drawn by inverse CDF from a Philox uniform that
// depends on the request's (seed, offset) only.
//
// Two kernels: one block per row for any row length, and for rows of 4,096 to 163,840 values
// a thread-block cluster per row that keeps the row in registers (see below).
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

// ---------------------------------------------------------------------------------------------
// The same sampling with a row spread over a thread-block cluster: every block keeps its
// eighth of the row in SHARED MEMORY (as order-preserving keys, a thread's run of values in a
// row of its own), so the threshold searches read global memory once instead of once per
// bit, settle four bits a pass (fifteen thresholds counted side by side), and eight SMs work
// on a row instead of one; three such blocks fit an SM.  Sums keep a fixed order: a
// thread's elements in index order, the block's threads by `block_sum`, the cluster's blocks
// by rank; the draw walks the row in index order as the kernel above does.
constexpr int SC_THREADS = 512;
constexpr int SC_CLUSTER = 8;
constexpr int SC_MOST = 40;          // elements a thread keeps: rows of up to 8 * 512 * 40 values
constexpr int SC_WARPS = SC_THREADS / 32;

__device__ __forceinline__ float key_float(uint32_t k) {   // inverse of float_key
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint32_t sc_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float sc_peer_f32(const float* mine, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote)
               : "r"((uint32_t)__cvta_generic_to_shared(mine)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Fifteen sums over the whole cluster, the same in every thread of every block afterwards:
// warp trees, then the block's warps in turn, then the cluster's blocks by rank.  `slot`
// alternates between calls so that a block may run one call ahead of its peers.
__device__ __forceinline__ void sc_sum15(float (&acc)[15], float (*warp_part)[15], float (*block_part)[16],
                                         float* total, int slot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 15; ++j) acc[j] = warp_sum(acc[j]);
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < 15; ++j) warp_part[warp][j] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x < 15) {
    float t = 0.f;
    for (int w = 0; w < SC_WARPS; ++w) t += warp_part[w][threadIdx.x];
    block_part[slot][threadIdx.x] = t;
  }
  sc_cluster_sync();
  if (threadIdx.x < 15) {
    float t = 0.f;
    for (uint32_t r = 0; r < SC_CLUSTER; ++r) t += sc_peer_f32(&block_part[slot][threadIdx.x], r);
    total[threadIdx.x] = t;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 15; ++j) acc[j] = total[j];
  __syncthreads();                                  // `total` and `warp_part` are free again
}

template <int EPT>
__global__ void __launch_bounds__(SC_THREADS, EPT <= 32 ? 3 : 2)
sample_cluster_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                      const unsigned long long* __restrict__ offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float warp_part[SC_WARPS][15];
  __shared__ float block_part[2][16];
  __shared__ float total[16];
  __shared__ uint32_t s_key[SC_WARPS];
  __shared__ int s_idx[SC_WARPS];
  __shared__ float x_f[4];                 // what a block shows its peers: key, index, total, pick
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = sc_rank();
  const int row = blockIdx.x / SC_CLUSTER;
  const float* l = logits + (size_t)row * ld;
  const int first = ((int)rank * SC_THREADS + tid) * EPT;       // this thread's elements, in index order

  // The block's part of the row comes in with consecutive threads on consecutive values and
  // stays in shared memory as keys, a thread's run of EPT values in a row of EPT + 1 (the runs
  // of a warp's threads then lie in different banks); 0 where the row has ended (no float
  // has key 0 but one NaN).
  extern __shared__ uint32_t keys[];
  {
    const int block_first = (int)rank * SC_THREADS * EPT;
#pragma unroll 8
    for (int c = tid; c < SC_THREADS * EPT; c += SC_THREADS) {
      const int owner = c / EPT, i = c - owner * EPT;
      keys[owner * (EPT + 1) + i] = (block_first + c < V) ? float_key(l[block_first + c]) : 0u;
    }
    __syncthreads();
  }
  const uint32_t* key = keys + tid * (EPT + 1);

  // ---- argmax, lowest index among equals
  uint32_t bk = 0;
  int bi = 0x7fffffff;
#pragma unroll
  for (int i = 0; i < EPT; ++i)
    if (key[i] > bk) { bk = key[i]; bi = first + i; }
  auto better = [](uint32_t k1, int i1, uint32_t k2, int i2) { return k1 > k2 || (k1 == k2 && i1 < i2); };
  for (int o = 16; o > 0; o >>= 1) {
    const uint32_t ok = __shfl_xor_sync(0xffffffffu, bk, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ok, oi, bk, bi)) { bk = ok; bi = oi; }
  }
  if (lane == 0) { s_key[warp] = bk; s_idx[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < SC_WARPS; ++w)
      if (better(s_key[w], s_idx[w], bk, bi)) { bk = s_key[w]; bi = s_idx[w]; }
    x_f[0] = __uint_as_float(bk);
    x_f[1] = __int_as_float(bi);
  }
  sc_cluster_sync();
  bk = 0; bi = 0x7fffffff;
  for (uint32_t r = 0; r < SC_CLUSTER; ++r) {
    const uint32_t ok = __float_as_uint(sc_peer_f32(&x_f[0], r));
    const int oi = __float_as_int(sc_peer_f32(&x_f[1], r));
    if (better(ok, oi, bk, bi)) { bk = ok; bi = oi; }
  }
  const int amax = bi == 0x7fffffff ? 0 : bi;
  const float temp = temperature[row];
  if (!(temp > 0.f)) {                     // the same for the whole cluster: nobody waits for anybody
    if (rank == 0 && tid == 0) out[row] = amax;
    sc_cluster_sync();                     // a peer may still be reading this block's shared memory
    return;
  }
  const float inv_t = 1.f / temp;
  const float mx_t = key_float(bk) * inv_t;
  int slot = 0;
  float acc[15];

  // ---- top-k: the largest key c with #(key >= c) >= k, four bits a pass
  uint32_t thr = 1;                        // keeps every value, and none of the padding
  const int k = top_k[row];
  if (k > 0 && k < V) {
    uint32_t cand = 0;
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
      for (int j = 0; j < 15; ++j) acc[j] = 0.f;
#pragma unroll
      for (int i = 0; i < EPT; ++i) {
        // (what is below the digits settled so far is below every threshold of this pass:
        // after a pass or two that is nearly everything, and whole warps skip it)
        if (key[i] > cand) {
#pragma unroll
          for (int j = 0; j < 15; ++j) acc[j] += (key[i] >= (cand | ((uint32_t)(j + 1) << shift))) ? 1.f : 0.f;
        }
      }
      sc_sum15(acc, warp_part, block_part, total, slot);
      slot ^= 1;
      uint32_t digit = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j)
        if (acc[j] >= (float)k) digit = j + 1;
      cand |= digit << shift;
    }
    if (cand > thr) thr = cand;
  }
  // ---- top-p over what top-k kept: the largest key c with mass(key >= c) > p * Z
  const float pp = top_p[row];
  if (pp < 1.f) {
#pragma unroll
    for (int j = 0; j < 15; ++j) acc[j] = 0.f;
#pragma unroll
    for (int i = 0; i < EPT; ++i)
      if (key[i] >= thr) acc[0] += expf(key_float(key[i]) * inv_t - mx_t);
    sc_sum15(acc, warp_part, block_part, total, slot);
    slot ^= 1;
    const float want = pp * acc[0];
    uint32_t cand = 0;
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
      for (int j = 0; j < 15; ++j) acc[j] = 0.f;
#pragma unroll
      for (int i = 0; i < EPT; ++i) {
        if (key[i] >= thr && key[i] > cand) {
          const float e = expf(key_float(key[i]) * inv_t - mx_t);
#pragma unroll
          for (int j = 0; j < 15; ++j) acc[j] += (key[i] >= (cand | ((uint32_t)(j + 1) << shift))) ? e : 0.f;
        }
      }
      sc_sum15(acc, warp_part, block_part, total, slot);
      slot ^= 1;
      uint32_t digit = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j)
        if (acc[j] > want) digit = j + 1;
      cand |= digit << shift;
    }
    if (cand > thr) thr = cand;
  }

  // ---- inverse CDF in index order: a thread's kept mass, its place among the block's
  // threads (a scan in thread order), the block's place among the blocks (by rank)
  float mine = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i)
    if (key[i] >= thr) mine += expf(key_float(key[i]) * inv_t - mx_t);
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_part[warp][0] = incl;
  __syncthreads();
  float before = incl - mine;                        // exclusive, within the block
  float block_total = 0.f;
  for (int w = 0; w < SC_WARPS; ++w) {
    if (w < warp) before += warp_part[w][0];
    block_total += warp_part[w][0];
  }
  if (tid == 0) x_f[2] = block_total;
  sc_cluster_sync();
  float blocks_before = 0.f, grand = 0.f;
  for (uint32_t r = 0; r < SC_CLUSTER; ++r) {
    const float t = sc_peer_f32(&x_f[2], r);
    if (r < rank) blocks_before += t;
    grand += t;
  }
  const uint32_t word = philox_first_word(seed[row], offset[row]);
  const float target = (float)(word >> 8) * (1.0f / 16777216.0f) * grand;
  const float start = blocks_before + before;
  // the last thread (in index order) that keeps something and starts at or before the target
  const bool candidate = mine > 0.f && start <= target;
  const uint32_t votes = __ballot_sync(0xffffffffu, candidate);
  if (lane == 0) s_idx[warp] = votes ? warp * 32 + (31 - __clz(votes)) : -1;
  __syncthreads();
  if (tid == 0) {
    int best = -1;
    for (int w = 0; w < SC_WARPS; ++w) best = max(best, s_idx[w]);
    x_f[3] = __int_as_float(best < 0 ? -1 : (int)rank * SC_THREADS + best);
  }
  sc_cluster_sync();
  int pick = -1;
  for (uint32_t r = 0; r < SC_CLUSTER; ++r) pick = max(pick, __float_as_int(sc_peer_f32(&x_f[3], r)));
  if (pick < 0) {                                    // nothing kept any mass: cannot happen with finite logits
    if (rank == 0 && tid == 0) out[row] = amax;
  } else if (pick == (int)rank * SC_THREADS + tid) {
    float cum = start;
    int choice = -1, last_kept = amax;
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      if (choice < 0 && key[i] >= thr) {
        last_kept = first + i;
        cum += expf(key_float(key[i]) * inv_t - mx_t);
        if (cum > target) choice = first + i;
      }
    }
    out[row] = choice >= 0 ? choice : last_kept;
  }
  sc_cluster_sync();                                 // nobody leaves while a peer may still read its shared memory
}

template <int EPT>
static int launch_sample_cluster(int* out, const float* logits, int R, int V, int ld, const float* temperature,
                                 const int* top_k, const float* top_p, const unsigned long long* seed,
                                 const unsigned long long* offset, cudaStream_t stream) {
  const size_t smem = (size_t)SC_THREADS * (EPT + 1) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_cluster_kernel<EPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(R * SC_CLUSTER);
  cfg.blockDim = dim3(SC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SC_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hb_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, sample_cluster_kernel<EPT>, out, logits, V, ld, temperature, top_k, top_p, seed, offset);
  return hb_check_launch();
}


// Rows of 4,096 to 163,840 values can go to the cluster kernel (a row of fewer gives eight
// blocks nothing to share out).  It wins while its eight blocks a row find SMs of their own,
// and longer the more passes over the row the options ask for; `kind` says what the caller
// knows of them (the options live on the device): 0 every row takes the argmax, 1 some rows
// draw but none has a top-k or top-p, 2 some have (-1: unknown, taken as 2), 3: the one-block
// kernel whatever the rows.  Measured in chains at 128,256 values, one block / cluster, µs:
// argmax 10 / 6 at 8 rows, 16 / 15 at 64, 24 / 58 at 256; temperature 57 / 13, 84 / 31,
// 95 / 106; top-k 50 and top-p 0.9: 672 / 91, 1,000 / 262, 1,620 / 855.
HB_EXPORT int hb_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature,
                        const int* top_k, const float* top_p, const unsigned long long* seed,
                        const unsigned long long* offset, int kind, cudaStream_t stream) {
  if (R <= 0) return HB_OK;
  if (V <= 0) return HB_BAD_ARGUMENT;
  const int per_thread = (V + SC_CLUSTER * SC_THREADS - 1) / (SC_CLUSTER * SC_THREADS);
  const int most_rows = kind == 0 ? 64 : kind == 1 ? 192 : kind == 3 ? 0 : 1 << 30;
  if (R <= most_rows && V >= 4096 && per_thread <= SC_MOST) {
#define HB_SAMPLE_CASE(EPT_)                                                                          \
    if (per_thread <= EPT_)                                                                            \
      return launch_sample_cluster<EPT_>(out, logits, R, V, ld, temperature, top_k, top_p, seed, offset, stream)
    HB_SAMPLE_CASE(8);
    HB_SAMPLE_CASE(16);
    HB_SAMPLE_CASE(24);
    HB_SAMPLE_CASE(32);
    HB_SAMPLE_CASE(40);
#undef HB_SAMPLE_CASE
  }
  hb_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, out, logits, V, ld, temperature, top_k, top_p,
                                                  seed, offset);
  return hb_check_launch();
}

// The uniform a request draws at (seed, offset): the same function for host-side checks.
HB_EXPORT float hb_philox_uniform(unsigned long long seed, unsigned long long offset) {
  return (float)(philox_first_word(seed, offset) >> 8) * (1.0f / 16777216.0f);
}
