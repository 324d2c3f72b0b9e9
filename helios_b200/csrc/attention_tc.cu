// Prefill / mixed-batch attention over the paged cache on the 5th-generation tensor
// cores (tcgen05.mma with the score and output tiles in tensor memory), bfloat16,
// head sizes 64 and 128.
//
// A block takes one KV head and up to 128 query rows = floor(128/G) consecutive tokens of one
// request times the G query heads that share the KV head (the last rows idle when G does
// not divide 128), and walks the keys the rows may see in
// tiles of 128:
//     TMA        pages of K and V (boxes of page_size x 64 elements, 128-byte swizzle)
//                -> a two-stage ring in shared memory
//     MMA 1      S[128 x 128] = Q K^T           (Q staged once, K-major; K tile K-major)
//     softmax    8 warps, two threads per row: scale, mask by position (causal, window),
//                maximum and sum in float32, P = exp2(.) as bfloat16 into shared
//                memory in the operand layout
//     MMA 2      O[128 x hd] += P V             (V tile as an MN-major operand); the output
//                accumulates in tensor memory over all key tiles, relative to a reference
//                maximum per row that the softmax warps move (rescaling output and sum) only
//                when the true maximum has run ahead of it by more than 2^8; they read the
//                output back once, at the end, and divide by the sum.
// Formulas: python/helios/exec/paged_attn.py:368-408 (scores * scale, key position > query
// position masked, softmax in float32, times V), head mapping :248-261.
//
// Every mbarrier wait is bounded; on a timeout the block raises the error word, frees its
// tensor memory and returns.
#include "tcgen05.cuh"

namespace {

constexpr float LOG2E = 1.4426950408889634f;
constexpr int TILE = 128;            // query rows and keys per tile
constexpr int TC_THREADS = 352;      // warp 0: TMA of K, warp 1: MMA, warps 2-9: softmax, warp 10: TMA of V
constexpr int SOFTMAX_THREADS = 256;

struct AttnArgs {
  __nv_bfloat16* out;
  const __nv_bfloat16* q;
  int q_stride;
  const int* block_table;
  int bt_stride;
  const int* q_tiles;       // (request, first local token) per tile
  const int* cu_tokens;
  const int* start_pos;
  int nh, nkv, page_size, window;
  float scale_log2;
  int* error;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// byte offset of 16-byte chunk `c8` (0..7) of row `row` in a [rows x 128 bytes] tile with
// the 128-byte swizzle (chunk index XOR row mod 8)
__device__ __forceinline__ uint32_t swz(int row, int c8) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((c8 ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            AttnArgs a) {
  constexpr int KH = HD / 64;                       // 64-element halves of the head dimension
  constexpr int HALF_BYTES = TILE * 128;            // one [128 rows x 64 elements] block
  constexpr int QKV_BYTES = KH * HALF_BYTES;        // a Q, K or V tile
  constexpr int P_BYTES = 2 * HALF_BYTES;           // 128 rows x 128 keys
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t S_COL = 0, O_COL = 128;

  extern __shared__ unsigned char smem_raw[];
  pdl_launch_dependents();
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem = q_smem + QKV_BYTES;               // 2 stages
  const uint32_t v_smem = k_smem + 2 * QKV_BYTES;           // 2 stages
  const uint32_t p_smem = v_smem + 2 * QKV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + 5 * QKV_BYTES + P_BYTES);
  // 0,1: K full; 2,3: K empty; 4: q ready; 5: s full; 6: p ready; 7: o full; 8: s free;
  // 9,10: V full; 11,12: V empty
  float* l_exchange = reinterpret_cast<float*>(bars + 14);  // [128]
  float* max_exchange = l_exchange + TILE;                  // [2 tiles][2 halves][128]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(max_exchange + 4 * TILE);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.nh / a.nkv;
  const int TQ = TILE / G;                            // tokens per tile
  // KV heads fastest: the tiles come longest first, and so do the blocks, whatever the head
  const int kvh = blockIdx.x % a.nkv, q_tile = blockIdx.x / a.nkv;
  const int seq = a.q_tiles[2 * q_tile], t0 = a.q_tiles[2 * q_tile + 1];

  if (threadIdx.x == 0) {
    mbar_init(bar(0), 1); mbar_init(bar(1), 1);
    mbar_init(bar(2), 1); mbar_init(bar(3), 1);
    mbar_init(bar(4), SOFTMAX_THREADS / 32);     // one arrival per softmax warp
    mbar_init(bar(5), 1);
    mbar_init(bar(6), SOFTMAX_THREADS / 32);
    mbar_init(bar(7), 1);
    mbar_init(bar(8), SOFTMAX_THREADS / 32);
    mbar_init(bar(9), 1); mbar_init(bar(10), 1);
    mbar_init(bar(11), 1); mbar_init(bar(12), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();     // everything below reads what earlier kernels wrote
  const int tok0 = a.cu_tokens[seq], n_tok = a.cu_tokens[seq + 1] - tok0;
  const int sp = a.start_pos[seq];
  const int p_first = sp + t0;
  const int p_last = sp + min(n_tok, t0 + TQ) - 1;
  const int k_min = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
  const int kt_begin = k_min / TILE, kt_end = p_last / TILE + 1;
  // a tile beyond the request's tokens (padding of a captured step's tile list) has no work
  const int n_it = t0 < n_tok ? kt_end - kt_begin : 0;
  const int* table = a.block_table + (size_t)seq * a.bt_stride;
  const int ps = a.page_size;
  const int pages_per_tile = TILE / ps;

  if (warp == 0 || warp == 10) {
    // ---------------------------------------------------------------- TMA producers
    // Warp 0 copies the K tiles, warp 10 the V tiles, each through a ring of two stages of
    // its own: a K stage is free again as soon as the scores of its tile are computed, long
    // before its V stage, so the next keys arrive while the softmax of this tile still runs.
    // Lane i looks up and copies page i of the tile (the look-ups of a tile's pages would
    // otherwise wait for one another); lane 0 waits for the stage and announces the bytes.
    {
      const bool is_v = warp == 10;
      const CUtensorMap* map = is_v ? &map_v : &map_k;
      const uint32_t ring = is_v ? v_smem : k_smem;
      const int full0 = is_v ? 9 : 0, empty0 = is_v ? 11 : 2;
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const int key_base = (kt_begin + it) * TILE;
        // pages that hold at least one key some row may see (a contiguous run)
        int first = 0, count = 0;
        for (int i = 0; i < pages_per_tile; ++i) {
          const int key0 = key_base + i * ps;
          const bool valid = key0 + ps - 1 >= k_min && key0 <= p_last;
          if (valid) { if (count == 0) first = i; ++count; }
        }
        const bool mine = lane >= first && lane < first + count;
        int row = 0;
        if (mine) row = (table[(key_base + lane * ps) / ps] * a.nkv + kvh) * ps;    // before the wait
        int go = 1;
        if (lane == 0) {
          go = mbar_wait(bar(empty0 + s), ((it >> 1) & 1) ^ 1, abort_flag, a.error, 11) ? 1 : 0;
          if (go) mbar_expect_tx(bar(full0 + s), (uint32_t)(count * ps * 128 * KH));
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) break;
        if (mine) {
          const uint32_t off = (uint32_t)(lane * ps * 128);
#pragma unroll
          for (int hh = 0; hh < KH; ++hh)
            tma_load_2d(ring + s * QKV_BYTES + hh * HALF_BYTES + off, map, bar(full0 + s), hh * 64, row);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_qk = instr_desc(TILE, TILE);
      constexpr uint32_t idesc_pv = instr_desc_b_mn(TILE, HD);
      // S(i+1) = Q K(i+1)^T is issued as soon as the softmax warps have taken S(i) into
      // registers, so that it runs under their exponentials; O_tile(i) = P(i) V(i) follows
      // when P(i) is written.
      bool ok = mbar_wait(bar(4), 0, abort_flag, a.error, 12);
      auto issue_qk = [&](int it) {
        const int s = it & 1;
        if (!mbar_wait(bar(s), (it >> 1) & 1, abort_flag, a.error, 13)) return false;
        tc_fence_after();
        const uint32_t ks = k_smem + s * QKV_BYTES;
#pragma unroll
        for (int hh = 0; hh < KH; ++hh)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + S_COL, smem_desc(q_smem + hh * HALF_BYTES + k * 32),
                      smem_desc(ks + hh * HALF_BYTES + k * 32), idesc_qk, (hh | k) ? 1u : 0u);
        umma_commit(bar(2 + s));      // the K stage is free once the scores are there
        umma_commit(bar(5));
        return true;
      };
      if (ok && n_it > 0) ok = issue_qk(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it) {
          ok = mbar_wait(bar(8), it & 1, abort_flag, a.error, 17);     // S(it) is in registers
          if (!ok) break;
          tc_fence_after();
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        ok = mbar_wait(bar(9 + s), (it >> 1) & 1, abort_flag, a.error, 18);     // V(it) has arrived
        if (!ok) break;
        ok = mbar_wait(bar(6), it & 1, abort_flag, a.error, 14);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vs = v_smem + s * QKV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem_base + O_COL, smem_desc(p_smem + (kk >> 2) * HALF_BYTES + (kk & 3) * 32),
                    smem_desc_mn(vs + kk * 2048, HALF_BYTES, 1024), idesc_pv, (it | kk) ? 1u : 0u);
        umma_commit(bar(11 + s));    // the V stage is free
        umma_commit(bar(7));         // O_tile complete
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- softmax warps
    const int sw = warp - 2;                       // 0..7 (warps 2..9)
    const int quarter = warp & 3;                  // lanes of tensor memory this warp may read
    const int half = sw >> 2;                      // which 64 keys / which half of hd this thread owns
    const int m = quarter * 32 + lane;             // row of the tile
    const int tl = t0 + m / G, g = m % G;
    const bool row_valid = m < TQ * G && tl < n_tok;       // rows beyond TQ * G idle when G does not divide 128
    const int pr = sp + tl;                        // the row's position
    const int tid = threadIdx.x - 64;

    // stage Q: rows = (token, head) pairs, swizzled K-major; invalid rows are zero.  All
    // loads of a thread are issued before the first store (one round trip, not one each).
    {
      constexpr int PER_THREAD = TILE * (HD / 8) / SOFTMAX_THREADS;
      uint4 qv[PER_THREAD];
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) {
        const int idx = tid + i * SOFTMAX_THREADS;
        const int row = idx / (HD / 8), c = idx - row * (HD / 8);
        const int rt = t0 + row / G, rg = row % G;
        qv[i] = make_uint4(0, 0, 0, 0);
        if (row < TQ * G && rt < n_tok)
          qv[i] = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + rt) * a.q_stride +
                                                  (size_t)(kvh * G + rg) * HD + c * 8);
      }
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) {
        const int idx = tid + i * SOFTMAX_THREADS;
        const int row = idx / (HD / 8), c = idx - row * (HD / 8);
        st_shared_v4(q_smem + (c >> 3) * HALF_BYTES + swz(row, c & 7), qv[i].x, qv[i].y, qv[i].z, qv[i].w);
      }
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(4));

    constexpr int OWN = HD / 2;                    // output columns this thread rescales and writes
    // The output accumulates in tensor memory over all key tiles, relative to a reference
    // maximum m_ref per row that is only moved when the true maximum has run ahead of it by
    // more than LAG (then the output and the sum are rescaled); exponentials are at most
    // 2^LAG meanwhile, and the final quotient does not depend on the reference.
    constexpr float LAG = 8.f;
    float m_ref = -INFINITY, l_run = 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int key_base = (kt_begin + it) * TILE;
      if (!mbar_wait(bar(5), it & 1, abort_flag, a.error, 15)) { ok = false; break; }
      tc_fence_after();
      const bool masked_tile = key_base + TILE - 1 > p_first || key_base < k_min ||
                               (a.window > 0 && key_base <= p_last - a.window);
      // this thread's 64 scores stay in registers; the maximum goes over to the other
      // thread of the row through shared memory
      float sv[64];
      {
        float v0[32], v1[32];
        tmem_ld32(lane_addr + S_COL + half * 64, v0);
        tmem_ld32(lane_addr + S_COL + half * 64 + 32, v1);
#pragma unroll
        for (int j = 0; j < 32; ++j) { sv[j] = v0[j]; sv[32 + j] = v1[j]; }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(8));        // the score tile may be overwritten
      if (masked_tile) {
        // columns of this thread's 64 keys the row may see: [lo, hi]
        const int col0 = key_base + half * 64;
        const int hi = pr - col0;
        const int lo = (a.window > 0 ? pr - a.window + 1 : 0) - col0;
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j < lo || j > hi) sv[j] = -INFINITY;
      }
      float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int j = 4; j < 64; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], sv[j]);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      max_exchange[((it & 1) * 2 + half) * TILE + m] = mx;
      named_barrier(2 + quarter, 64);
      mx = fmaxf(mx, max_exchange[((it & 1) * 2 + (half ^ 1)) * TILE + m]) * a.scale_log2;
      // move the reference?  Both threads of a row see the same numbers; the rows of a warp
      // decide together, because tensor memory is read and written by whole warps.
      const bool move = mx > m_ref + LAG || (m_ref == -INFINITY && mx > -INFINITY);
      const bool rescale = __any_sync(0xffffffffu, move) && it > 0;
      float factor = 1.f;
      if (move) {
        factor = fast_exp2(m_ref - mx);          // 0 while nothing has been added yet
        m_ref = mx;
        l_run *= factor;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // the exponentials of this tile, packed, wait in registers: the product of the tile
      // before, which still reads P, finishes under this work
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float p0 = fast_exp2(fmaf(sv[2 * j], a.scale_log2, -m_use));
        const float p1 = fast_exp2(fmaf(sv[2 * j + 1], a.scale_log2, -m_use));
        sum4[j & 3] += p0 + p1;
        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[j] = *reinterpret_cast<uint32_t*>(&pk);
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (it > 0) {
        // P of the tile before has been read, and its product is in the output
        if (!mbar_wait(bar(7), (it - 1) & 1, abort_flag, a.error, 16)) { ok = false; break; }
        tc_fence_after();
        if (rescale) {
#pragma unroll
          for (int c = 0; c < OWN / 32; ++c) {
            float v[32];
            tmem_ld32(lane_addr + O_COL + half * OWN + c * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= factor;
            tmem_st32(lane_addr + O_COL + half * OWN + c * 32, v);
          }
        }
      }
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        st_shared_v4(p_smem + half * HALF_BYTES + swz(m, c8), packed[4 * c8], packed[4 * c8 + 1],
                     packed[4 * c8 + 2], packed[4 * c8 + 3]);
      // V rows of keys past the last position (unwritten slots, pages that were not copied)
      // must not be NaN or Inf when they meet their zero probabilities
      {
        const int s = it & 1;
        auto zero_rows = [&](int row_begin, int row_end) {
          for (int idx = tid + row_begin * KH * 8; idx < row_end * KH * 8; idx += SOFTMAX_THREADS) {
            const int row = idx / (KH * 8), rest = idx - row * (KH * 8);
            st_shared_v4(v_smem + s * QKV_BYTES + (rest >> 3) * HALF_BYTES + row * 128 + (rest & 7) * 16,
                         0, 0, 0, 0);
          }
        };
        if (key_base + TILE - 1 > p_last || key_base < k_min) {
          // the copies of this V tile must have landed first: they bring whole pages
          if (!mbar_wait(bar(9 + s), (it >> 1) & 1, abort_flag, a.error, 19)) { ok = false; break; }
          if (key_base + TILE - 1 > p_last) zero_rows(p_last + 1 - key_base, TILE);
          // pages wholly before the window of the first row were not copied either
          if (key_base < k_min) zero_rows(0, ((k_min - key_base) / ps) * ps);
        }
      }
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(6));
    }
    float o_reg[OWN];
#pragma unroll
    for (int i = 0; i < OWN; ++i) o_reg[i] = 0.f;
    if (ok && n_it > 0) {
      if (mbar_wait(bar(7), (n_it - 1) & 1, abort_flag, a.error, 16)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < OWN / 32; ++c) {
          float v[32];
          tmem_ld32(lane_addr + O_COL + half * OWN + c * 32, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) o_reg[c * 32 + j] = v[j];
        }
        tc_fence_before();
      } else {
        ok = false;
      }
    }

    // the two threads of a row add their sums
    if (half == 1) l_exchange[m] = l_run;
    named_barrier(1, SOFTMAX_THREADS);
    if (half == 0) {
      const float other = l_exchange[m];
      l_exchange[m] = l_run;
      l_run += other;
    }
    named_barrier(1, SOFTMAX_THREADS);
    if (half == 1) l_run += l_exchange[m];
    if (ok && row_valid && !*abort_flag) {
      const float inv = 1.f / l_run;
      __nv_bfloat16* dst = a.out + ((size_t)(tok0 + tl) * a.nh + (kvh * G + g)) * HD + half * OWN;
#pragma unroll
      for (int j = 0; j < OWN; j += 8) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 pk = __floats2bfloat162_rn(o_reg[j + 2 * e] * inv, o_reg[j + 2 * e + 1] * inv);
          w[e] = *reinterpret_cast<uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
int launch_tc(const AttnArgs& a, const void* k_pages, const void* v_pages, long long page_rows, int n_tiles,
              cudaStream_t stream) {
  constexpr int KH = HD / 64;
  constexpr size_t SMEM = 5 * (size_t)KH * TILE * 128 + 2 * TILE * 128 + 1024 + 4096;
  CUtensorMap map_k, map_v;
  if (!make_map(&map_k, k_pages, (uint64_t)page_rows, HD, HD, a.page_size)) return HB_LAUNCH_FAILED;
  if (!make_map(&map_v, v_pages, (uint64_t)page_rows, HD, HD, a.page_size)) return HB_LAUNCH_FAILED;
  auto kernel = attention_prefill_tc_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured = true;
  }
  hb_launch(kernel, dim3(n_tiles * a.nkv), dim3(TC_THREADS), SMEM, stream, map_k, map_v, a);
  return hb_check_launch();
}

}  // namespace

// q_tiles: (request, first local token) for tiles of 128 / (nh / nkv) tokens.  Needs hd in
// {64, 128}, a group size that divides 128, and a page size that is a multiple of 8 and
// divides 128.  num_pages: pages in k_pages / v_pages ([pages, nkv, page_size, hd]).
HB_EXPORT int hb_attention_prefill_tc(void* out, const void* q, int q_stride, const void* k_pages,
                                      const void* v_pages, long long num_pages, const int* block_table,
                                      int bt_stride, const int* q_tiles, int n_tiles, const int* cu_tokens,
                                      const int* start_pos, int nh, int nkv, int hd, int page_size, int window,
                                      float scale, int* error, cudaStream_t stream) {
  if (n_tiles <= 0) return HB_OK;
  if (nkv <= 0 || nh % nkv != 0 || error == nullptr) return HB_BAD_ARGUMENT;
  const int G = nh / nkv;
  if (G > TILE) return HB_BAD_ARGUMENT;
  if (page_size < 8 || page_size % 8 != 0 || TILE % page_size != 0) return HB_BAD_ARGUMENT;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || (q_stride & 7))
    return HB_BAD_ARGUMENT;
  AttnArgs a;
  a.out = (__nv_bfloat16*)out; a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.block_table = block_table; a.bt_stride = bt_stride; a.q_tiles = q_tiles; a.cu_tokens = cu_tokens;
  a.start_pos = start_pos; a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * LOG2E; a.error = error;
  const long long rows = num_pages * nkv * page_size;
  if (hd == 128) return launch_tc<128>(a, k_pages, v_pages, rows, n_tiles, stream);
  if (hd == 64) return launch_tc<64>(a, k_pages, v_pages, rows, n_tiles, stream);
  return HB_BAD_ARGUMENT;
}
