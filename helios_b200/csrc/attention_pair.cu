// Prefill attention over the paged cache on the 5th-generation tensor cores, two query tiles
// per block: bfloat16, head sizes 64 and 128.
//
// A block takes one KV head and TWO tiles of 128 query rows (tile A and tile B: each
// floor(128/G) consecutive tokens of one request times the G query heads that share the KV
// head; B follows A in the request and may be empty).  Both tiles read the same keys, so a
// K or V tile is copied once for 256 rows, and while the softmax of one tile runs the tensor
// cores work for the other:
//     TMA        pages of K and V (boxes of page_size x 64 elements, 128-byte swizzle)
//                -> two rings of two stages in shared memory
//     MMA        S_X[128 x 128] = Q_X K^T for X in {A, B}, into tensor memory
//     softmax    four warps per tile, one thread per row: scale, mask by position (causal,
//                window), maximum and sum in float32, P = exp2(.) as bfloat16 written back
//                into tensor memory over the scores it came from
//     MMA        O_X[128 x hd] += P_X V with P as the operand from tensor memory (V tile as
//                an MN-major operand from shared memory); the output accumulates in tensor
//                memory relative to a reference maximum per row that moves (rescaling output
//                and sum) only when the true maximum has run ahead of it by more than 2^8
// Tensor memory: S_A, S_B, O_A, O_B of 128 columns each, all 512.  The products of a tile
// are issued in the order PV(i), QK(i+1): the tensor cores run them in that order, so the
// scores of the next key tile overwrite P only after it has been read.
// Formulas: python/helios/exec/paged_attn.py:368-408 (scores * scale, key position > query
// position masked, softmax in float32, times V), head mapping :248-261.
//
// Every mbarrier wait is bounded; on a timeout the block raises the error word, frees its
// tensor memory and returns.
#include "tcgen05.cuh"

namespace {

constexpr float LOG2E = 1.4426950408889634f;
constexpr int TILE = 128;             // query rows per tile and keys per key tile
constexpr int PAIR_THREADS = 352;     // warp 0: TMA of K, warp 1: MMA, warps 2-5: softmax A, 6-9: softmax B, warp 10: TMA of V
constexpr int GROUP_THREADS = 128;

struct PairArgs {
  __nv_bfloat16* out;
  const __nv_bfloat16* q;
  int q_stride;
  const int* block_table;
  int bt_stride;
  const int* q_tiles;       // (request, first local token) per pair of tiles
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
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// byte offset of 16-byte chunk `c8` (0..7) of row `row` in a [rows x 128 bytes] tile with
// the 128-byte swizzle (chunk index XOR row mod 8)
__device__ __forceinline__ uint32_t swz(int row, int c8) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((c8 ^ (row & 7)) << 4));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 bfloat16, two to a 32-bit
// column, a row per lane) is read from tensor memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive 32-bit columns of this thread's lane into tensor memory (no wait)
__device__ __forceinline__ void tmem_st16_nowait(uint32_t addr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int HD>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attention_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                              PairArgs a) {
  constexpr int KH = HD / 64;                       // 64-element halves of the head dimension
  constexpr int HALF_BYTES = TILE * 128;            // one [128 rows x 64 elements] block
  constexpr int QKV_BYTES = KH * HALF_BYTES;        // a Q, K or V tile
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ unsigned char smem_raw[];
  pdl_launch_dependents();
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;                             // tiles A and B
  const uint32_t k_smem = q_smem + 2 * QKV_BYTES;           // 2 stages
  const uint32_t v_smem = k_smem + 2 * QKV_BYTES;           // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + 6 * QKV_BYTES);
  // 0,1: K full; 2,3: K empty; 4,5: V full; 6,7: V empty; then per tile X in {0, 1}:
  // 8+X: q ready; 10+X: s full; 12+X: p ready; 14+X: o full
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.nh / a.nkv;
  const int TQ = TILE / G;                            // tokens per tile
  // KV heads fastest: the pairs come longest first, and so do the blocks, whatever the head
  const int kvh = blockIdx.x % a.nkv, q_tile = blockIdx.x / a.nkv;
  const int seq = a.q_tiles[2 * q_tile], t0 = a.q_tiles[2 * q_tile + 1];

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(8), GROUP_THREADS / 32); mbar_init(bar(9), GROUP_THREADS / 32);      // one arrival per warp
    mbar_init(bar(10), 1); mbar_init(bar(11), 1);
    mbar_init(bar(12), GROUP_THREADS / 32); mbar_init(bar(13), GROUP_THREADS / 32);
    mbar_init(bar(14), 1); mbar_init(bar(15), 1);
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
  const int ps = a.page_size;
  const int pages_per_tile = TILE / ps;
  // tokens, positions and key tiles of the two query tiles; a tile without tokens (B past the
  // end of the request, both for the padding of a captured step's list) has no key tiles
  int n_x[2], kt_begin[2], kt_end[2], p_first[2], p_last[2], k_min[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int first = t0 + x * TQ;
    n_x[x] = first < n_tok ? min(TQ, n_tok - first) : 0;
    p_first[x] = sp + first;
    p_last[x] = p_first[x] + n_x[x] - 1;
    k_min[x] = (a.window > 0 && p_first[x] - a.window + 1 > 0) ? p_first[x] - a.window + 1 : 0;
    kt_begin[x] = n_x[x] > 0 ? k_min[x] / TILE : 0;
    kt_end[x] = n_x[x] > 0 ? p_last[x] / TILE + 1 : 0;
  }
  // what the block copies: from the first key tile A sees to the last one B (or A alone) sees
  const int kt0 = kt_begin[0];
  const int kt1 = n_x[1] > 0 ? kt_end[1] : kt_end[0];
  const int n_it = kt1 - kt0;
  const int k_min_all = k_min[0];
  const int p_last_all = n_x[1] > 0 ? p_last[1] : p_last[0];
  auto active = [&](int x, int it) { return kt0 + it >= kt_begin[x] && kt0 + it < kt_end[x]; };
  const int* table = a.block_table + (size_t)seq * a.bt_stride;

  if (warp == 0 || warp == 10) {
    // ---------------------------------------------------------------- TMA producers
    // Warp 0 copies the K tiles, warp 10 the V tiles, each through a ring of two stages of
    // its own.  Lane i looks up and copies page i of the tile; lane 0 waits for the stage and
    // announces the bytes.
    const bool is_v = warp == 10;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    const uint32_t ring = is_v ? v_smem : k_smem;
    const int full0 = is_v ? 4 : 0, empty0 = is_v ? 6 : 2;
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int key_base = (kt0 + it) * TILE;
      // pages that hold at least one key some row may see (a contiguous run)
      int first = 0, count = 0;
      for (int i = 0; i < pages_per_tile; ++i) {
        const int key0 = key_base + i * ps;
        const bool valid = key0 + ps - 1 >= k_min_all && key0 <= p_last_all;
        if (valid) { if (count == 0) first = i; ++count; }
      }
      const bool mine = lane >= first && lane < first + count;
      int row = 0;
      if (mine) row = (table[(key_base + lane * ps) / ps] * a.nkv + kvh) * ps;    // before the wait
      int go = 1;
      if (lane == 0) {
        go = mbar_wait(bar(empty0 + s), ((it >> 1) & 1) ^ 1, abort_flag, a.error, 31) ? 1 : 0;
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
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_qk = instr_desc(TILE, TILE);
      constexpr uint32_t idesc_pv = instr_desc_b_mn(TILE, HD);
      auto issue_qk = [&](int x, int s) {
        const uint32_t ks = k_smem + s * QKV_BYTES, qs = q_smem + x * QKV_BYTES;
#pragma unroll
        for (int hh = 0; hh < KH; ++hh)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + x * TILE, smem_desc(qs + hh * HALF_BYTES + k * 32),
                      smem_desc(ks + hh * HALF_BYTES + k * 32), idesc_qk, (hh | k) ? 1u : 0u);
        umma_commit(bar(10 + x));
      };
      auto issue_pv = [&](int x, int s, bool accumulate) {
        const uint32_t vs = v_smem + s * QKV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_a_tmem(tmem_base + 2 * TILE + x * TILE, tmem_base + x * TILE + kk * 8,
                           smem_desc_mn(vs + kk * 2048, HALF_BYTES, 1024), idesc_pv, (accumulate || kk) ? 1u : 0u);
      };
      int done[2] = {0, 0};            // key tiles of each query tile whose PV is issued
      bool ok = true;
#pragma unroll
      for (int x = 0; x < 2; ++x)
        if (ok && n_x[x] > 0) ok = mbar_wait(bar(8 + x), 0, abort_flag, a.error, 32);
      if (ok) ok = mbar_wait(bar(0), 0, abort_flag, a.error, 33);
      if (ok) {
        tc_fence_after();
        if (active(0, 0)) issue_qk(0, 0);
        if (active(1, 0)) issue_qk(1, 0);
        umma_commit(bar(2));            // the K stage is free once the scores are there
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1, sn = s ^ 1;
        const bool more = it + 1 < n_it;
        ok = mbar_wait(bar(4 + s), (it >> 1) & 1, abort_flag, a.error, 34);         // V(it) has arrived
        if (!ok) break;
        if (active(0, it)) {
          ok = mbar_wait(bar(12), done[0] & 1, abort_flag, a.error, 35);            // P_A(it) is written
          if (!ok) break;
          tc_fence_after();
          issue_pv(0, s, done[0] > 0);
          ++done[0];
          if (!more || !active(0, it + 1)) umma_commit(bar(14));                    // O_A is complete
        }
        if (more) {
          ok = mbar_wait(bar(sn), ((it + 1) >> 1) & 1, abort_flag, a.error, 36);    // K(it+1) has arrived
          if (!ok) break;
          tc_fence_after();
          if (active(0, it + 1)) issue_qk(0, sn);
        }
        if (active(1, it)) {
          ok = mbar_wait(bar(13), done[1] & 1, abort_flag, a.error, 37);
          if (!ok) break;
          tc_fence_after();
          issue_pv(1, s, done[1] > 0);
          ++done[1];
          if (!more || !active(1, it + 1)) umma_commit(bar(15));
        }
        umma_commit(bar(6 + s));       // the V stage is free
        if (more) {
          if (active(1, it + 1)) issue_qk(1, sn);
          umma_commit(bar(2 + sn));
        }
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- softmax warps
    const int x = (warp - 2) >> 2;                 // which query tile
    const int quarter = warp & 3;                  // lanes of tensor memory this warp may read
    const int m = quarter * 32 + lane;             // row of the tile
    const int tl = t0 + x * TQ + m / G, g = m % G;
    const bool row_valid = m < TQ * G && tl < n_tok;       // rows beyond TQ * G idle when G does not divide 128
    const int pr = sp + tl;                        // the row's position
    const int tid = threadIdx.x - 64 - x * GROUP_THREADS;
    const int my_it = kt_end[x] - kt_begin[x];
    const uint32_t s_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + x * TILE;
    const uint32_t o_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + 2 * TILE + x * TILE;

    if (my_it > 0) {
      // stage Q_X: rows = (token, head) pairs, swizzled K-major; invalid rows are zero.  Eight
      // loads of a thread are issued before their stores (one round trip, not one each).
      constexpr int PER_THREAD = TILE * (HD / 8) / GROUP_THREADS;
      constexpr int BATCH = 8;
#pragma unroll
      for (int b0 = 0; b0 < PER_THREAD; b0 += BATCH) {
        uint4 qv[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
          const int idx = tid + (b0 + i) * GROUP_THREADS;
          const int row = idx / (HD / 8), c = idx - row * (HD / 8);
          const int rt = t0 + x * TQ + row / G, rg = row % G;
          qv[i] = make_uint4(0, 0, 0, 0);
          if (row < TQ * G && rt < n_tok)
            qv[i] = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + rt) * a.q_stride +
                                                    (size_t)(kvh * G + rg) * HD + c * 8);
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
          const int idx = tid + (b0 + i) * GROUP_THREADS;
          const int row = idx / (HD / 8), c = idx - row * (HD / 8);
          st_shared_v4(q_smem + x * QKV_BYTES + (c >> 3) * HALF_BYTES + swz(row, c & 7),
                       qv[i].x, qv[i].y, qv[i].z, qv[i].w);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(8 + x));
    }

    // The output accumulates in tensor memory over all key tiles, relative to a reference
    // maximum m_ref per row that is only moved when the true maximum has run ahead of it by
    // more than LAG (then the output and the sum are rescaled); exponentials are at most
    // 2^LAG meanwhile, and the final quotient does not depend on the reference.
    constexpr float LAG = 8.f;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    const int win_lo = a.window > 0 ? pr - a.window + 1 : 0;     // first key position the row sees

    for (int i = 0; i < my_it; ++i) {
      const int it = kt_begin[x] - kt0 + i;        // the block's iteration (stage and parity of V)
      const int key_base = (kt_begin[x] + i) * TILE;
      if (!mbar_wait(bar(10 + x), i & 1, abort_flag, a.error, 38)) { ok = false; break; }
      tc_fence_after();
      const bool masked_tile = key_base + TILE - 1 > p_first[x] || key_base < k_min[x] ||
                               (a.window > 0 && key_base <= p_last[x] - a.window);
      const int hi = pr - key_base, lo = win_lo - key_base;       // columns the row may see: [lo, hi]
      // the row's 128 scores in registers with one load; the maximum first
      float sv[128];
      tmem_ld128(s_addr, sv);
      if (masked_tile) {
#pragma unroll
        for (int j = 0; j < 128; ++j)
          if (j < lo || j > hi) sv[j] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 128; j += 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = max3(mx4[e], sv[j + 2 * e], sv[j + 2 * e + 1]);
      }
      const float mx = fmaxf(max3(mx4[0], mx4[1], mx4[2]), mx4[3]) * a.scale_log2;
      // move the reference?  The rows of a warp decide together, because tensor memory is read
      // and written by whole warps.
      const bool move = mx > m_ref + LAG || (m_ref == -INFINITY && mx > -INFINITY);
      const bool rescale = __any_sync(0xffffffffu, move) && i > 0;
      float factor = 1.f;
      if (move) {
        factor = fast_exp2(m_ref - mx);            // 0 while nothing has been added yet
        m_ref = mx;
        l_run *= factor;
      }
      if (rescale) {
        // the product of the key tile before is complete: the scores of this one were issued
        // after it, and their barrier covers everything issued before
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld32(o_addr + c * 32, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= factor;
          tmem_st32(o_addr + c * 32, v);
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // exponentials, their sum, and P packed into the columns the scores came from
      // (scale, subtraction and the sum two values at a time: packed float32 arithmetic)
      const float2 scale2 = make_float2(a.scale_log2, a.scale_log2), shift2 = make_float2(-m_use, -m_use);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 e = __ffma2_rn(make_float2(sv[c * 32 + 2 * j], sv[c * 32 + 2 * j + 1]), scale2, shift2);
          const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
          sum2[j & 1] = __fadd2_rn(sum2[j & 1], pp);
          __nv_bfloat162 pk = __floats2bfloat162_rn(pp.x, pp.y);
          packed[j] = *reinterpret_cast<uint32_t*>(&pk);
        }
        tmem_st16_nowait(s_addr + c * 16, packed);
      }
      l_run += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      // V rows of keys past the last position (unwritten slots, pages that were not copied)
      // must not be NaN or Inf when they meet their zero probabilities.  The tile whose
      // product is issued first in this iteration does it.
      if ((key_base + TILE - 1 > p_last_all || key_base < k_min_all) && (x == 0 || !active(0, it))) {
        const int s = it & 1;
        auto zero_rows = [&](int row_begin, int row_end) {
          for (int idx = tid + row_begin * KH * 8; idx < row_end * KH * 8; idx += GROUP_THREADS) {
            const int row = idx / (KH * 8), rest = idx - row * (KH * 8);
            st_shared_v4(v_smem + s * QKV_BYTES + (rest >> 3) * HALF_BYTES + row * 128 + (rest & 7) * 16,
                         0, 0, 0, 0);
          }
        };
        // the copies of this V tile must have landed first: they bring whole pages
        if (!mbar_wait(bar(4 + s), (it >> 1) & 1, abort_flag, a.error, 39)) { ok = false; break; }
        if (key_base + TILE - 1 > p_last_all) zero_rows(p_last_all + 1 - key_base, TILE);
        // pages wholly before the window of the first row were not copied either
        if (key_base < k_min_all) zero_rows(0, ((k_min_all - key_base) / ps) * ps);
        fence_async_smem();
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(12 + x));
    }

    if (my_it > 0) {
      if (ok && mbar_wait(bar(14 + x), 0, abort_flag, a.error, 40)) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        __nv_bfloat16* dst = a.out + ((size_t)(tok0 + tl) * a.nh + (kvh * G + g)) * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld32(o_addr + c * 32, v);
          if (row_valid && !*abort_flag) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 pk = __floats2bfloat162_rn(v[j + 2 * e] * inv, v[j + 2 * e + 1] * inv);
                w[e] = *reinterpret_cast<uint32_t*>(&pk);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        tc_fence_before();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);     // copies in flight land before the block leaves
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
int launch_pair(const PairArgs& a, const void* k_pages, const void* v_pages, long long page_rows, int n_pairs,
                cudaStream_t stream) {
  constexpr int KH = HD / 64;
  constexpr size_t SMEM = 6 * (size_t)KH * TILE * 128 + 1024 + 1024;
  CUtensorMap map_k, map_v;
  if (!make_map(&map_k, k_pages, (uint64_t)page_rows, HD, HD, a.page_size)) return HB_LAUNCH_FAILED;
  if (!make_map(&map_v, v_pages, (uint64_t)page_rows, HD, HD, a.page_size)) return HB_LAUNCH_FAILED;
  auto kernel = attention_prefill_pair_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured = true;
  }
  hb_launch(kernel, dim3(n_pairs * a.nkv), dim3(PAIR_THREADS), SMEM, stream, map_k, map_v, a);
  return hb_check_launch();
}

}  // namespace

// q_tiles: (request, first local token) for pairs of tiles, that is for 2 * (128 / (nh / nkv))
// tokens each.  Needs hd in {64, 128}, at most 128 query heads per KV head, and a page size that
// is a multiple of 8 and divides 128.  num_pages: pages in k_pages / v_pages
// ([pages, nkv, page_size, hd]).
HB_EXPORT int hb_attention_prefill_pair(void* out, const void* q, int q_stride, const void* k_pages,
                                        const void* v_pages, long long num_pages, const int* block_table,
                                        int bt_stride, const int* q_tiles, int n_pairs, const int* cu_tokens,
                                        const int* start_pos, int nh, int nkv, int hd, int page_size, int window,
                                        float scale, int* error, cudaStream_t stream) {
  if (n_pairs <= 0) return HB_OK;
  if (nkv <= 0 || nh % nkv != 0 || error == nullptr) return HB_BAD_ARGUMENT;
  const int G = nh / nkv;
  if (G > TILE) return HB_BAD_ARGUMENT;
  if (page_size < 8 || page_size % 8 != 0 || TILE % page_size != 0) return HB_BAD_ARGUMENT;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || (q_stride & 7))
    return HB_BAD_ARGUMENT;
  PairArgs a;
  a.out = (__nv_bfloat16*)out; a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.block_table = block_table; a.bt_stride = bt_stride; a.q_tiles = q_tiles; a.cu_tokens = cu_tokens;
  a.start_pos = start_pos; a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * LOG2E; a.error = error;
  const long long rows = num_pages * nkv * page_size;
  if (hd == 128) return launch_pair<128>(a, k_pages, v_pages, rows, n_pairs, stream);
  if (hd == 64) return launch_pair<64>(a, k_pages, v_pages, rows, n_pairs, stream);
  return HB_BAD_ARGUMENT;
}
