// bfloat16 matrix products y = x W^T on the 5th-generation tensor cores:
// tcgen05.mma (cta_group::1, kind::f16, float32 accumulators in tensor memory),
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle)
// through an mbarrier ring, accumulators read back with tcgen05.ld for the epilogue.
// (python/helios/exec/model.py:236-238, 250-251, 336-337, 493-496 are the products; the
// reference runs them in a library.)
//
// One kernel, two orientations:
//   * tokens on the 128-row MMA M axis, output features on N (prefill);
//   * "swapped" for few tokens (decode): 128 output features on the M axis, the tokens
//     on a narrow N axis, so that a step streams every weight once at full width; the
//     K range can be split over several blocks, whose partial sums the last block to
//     finish adds in a fixed order (scratch memory + a ticket per tile).
// Epilogues: + bias, bfloat16 or float32 out; or SwiGLU, where the block accumulates the
// gate tile and the up tile of the same feature range side by side and writes
// silu(gate) * up.
// Two more for steps of few tokens (swapped orientation), which together take the RMSNorm
// launches out of a decode step: a product can ADD its result into the float32 residual
// stream and leave, for the norm that follows, bfloat16(residual * norm weight) and per-token
// partial sums of squares; and a product whose input was left that way multiplies its
// accumulators by the token's 1 / rms (from those partial sums) before bias or SwiGLU.
//
// One thread issues TMA, one issues MMA, four warps run the epilogue.  Every wait on an
// mbarrier is bounded: when it runs out the block raises an error word in global
// memory, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;          // rows of the A-side tile = MMA M
constexpr int BK = 64;           // 64 bfloat16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;  // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

enum { EPI_STORE = 0, EPI_GLU = 1 };

struct GemmArgs {
  void* out;            // [T, ldo] bfloat16 or float32
  const float* bias;    // [N] or null
  float* scratch;       // partial sums when the K range is split
  int* tickets;         // one per output tile, zero between launches
  int* error;           // set non-zero when a wait ran out
  int T, N, K;          // tokens, output features (for GLU: of the result, = half the weight rows), reduction
  int ldo;
  int glu_offset;       // GLU: row of the weight where the second half ("up") begins
  int out_f32;
  int k_splits;
  int cluster_reduce;   // the K slices of a tile form a thread-block cluster and add their
                        // partial sums through distributed shared memory (no scratch)
  // swapped orientation only:
  float* residual = nullptr;           // [T, N] float32: residual += result (+ bias); then, with
  const float* norm_weight = nullptr;  // a norm weight [N], out = bfloat16(residual * weight) and
  float* sumsq_out = nullptr;          // [T, 8 * feature tiles] partial sums of residual^2
  const float* sumsq_in = nullptr;     // [T, slots_in]: the input rows lack the factor
  int slots_in = 0;                    //   rsqrt(sum(slots) / width + eps), applied to the
  float width = 1.f, eps = 0.f;        //   accumulators here
};

constexpr int SUMSQ_SLOTS = 8;   // partial sums a feature tile leaves per token (K slices or warps)

constexpr uint32_t pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int BN, bool SWAP, int EPI>
struct Config {
  // A-side tiles per stage: two for the swapped SwiGLU (gate rows, up rows)
  static constexpr int A_TILES = (SWAP && EPI == EPI_GLU) ? 2 : 1;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
  // swapped (decode): 108 KB of stages, two blocks per SM; otherwise one block per SM, 196 KB
  static constexpr int BUDGET = SWAP ? 108 * 1024 : 196 * 1024;
  static constexpr int STAGES_FIT = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : (STAGES_FIT < 2 ? 2 : STAGES_FIT);
  static constexpr int MIN_BLOCKS = SWAP ? 2 : 1;
  static constexpr int ACC_COLS = BN * A_TILES;            // float32 columns of tensor memory in use
  static constexpr uint32_t TMEM_COLS = pow2_cols(ACC_COLS);
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment */ +
                                 256 /* barriers */ + (SWAP ? BN * 4 : 0) /* token factors */;
};

// out feature / token of accumulator element (row r of the A-side tile, column c)
template <int BN, bool SWAP, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, Config<BN, SWAP, EPI>::MIN_BLOCKS)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 GemmArgs args) {
  using Cfg = Config<BN, SWAP, EPI>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
  // bars[0..S): full, bars[S..2S): empty, bars[2S]: accumulators ready
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  float* col_scale = reinterpret_cast<float*>(last_flag + 3);     // [BN], one factor per token column

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
  const int kb_total = (args.K + BK - 1) / BK;
  const int kb_per = (kb_total + args.k_splits - 1) / args.k_splits;
  const int kb_begin = split * kb_per;
  const int kb_end = min(kb_total, kb_begin + kb_per);
  const int n_kb = max(0, kb_end - kb_begin);

  auto full_bar = [&](int s) { return smem_u32(bars + s); };
  auto empty_bar = [&](int s) { return smem_u32(bars + Cfg::STAGES + s); };
  const uint32_t acc_bar = smem_u32(bars + 2 * Cfg::STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // rows of the two operands this block reads
  int a_row0, a_row1 = 0, b_row0, b_row1 = 0;
  if (SWAP) {
    a_row0 = tile_a * BM;                       // weight rows (features)
    a_row1 = args.glu_offset + tile_a * BM;     // GLU: the up rows
    b_row0 = tile_b * BN;                       // token rows
  } else {
    a_row0 = tile_a * BM;                       // token rows
    if (EPI == EPI_GLU) {
      b_row0 = tile_b * (BN / 2);               // gate rows
      b_row1 = args.glu_offset + tile_b * (BN / 2);
    } else {
      b_row0 = tile_b * BN;
    }
  }

  // Residual epilogue with the K slices as a cluster: what a thread's first two elements need
  // from global memory (the residual, the norm weight, the bias) does not depend on this
  // kernel's sums; it is fetched as soon as the kernel before is done, under the main loop.
  float early_old[2] = {0.f, 0.f}, early_weight[2] = {0.f, 0.f}, early_bias[2] = {0.f, 0.f};

  if (warp == 0) {
   if (lane == 0) {
    // ------------------------------------------------------------ TMA producer
    // The weights do not depend on the kernel before this one: their copies for the
    // first stages start at once; the activations follow once that kernel is done.
    auto load_weights = [&](int i, int s) {
      const uint32_t sa = base + s * Cfg::STAGE_BYTES;
      const uint32_t sb = sa + Cfg::A_TILES * Cfg::A_BYTES;
      const int k0 = (kb_begin + i) * BK;
      if (SWAP) {
        tma_load_2d(sa, &map_a, full_bar(s), k0, a_row0);
        if (Cfg::A_TILES == 2) tma_load_2d(sa + Cfg::A_BYTES, &map_a, full_bar(s), k0, a_row1);
      } else if (EPI == EPI_GLU) {
        tma_load_2d(sb, &map_b, full_bar(s), k0, b_row0);
        tma_load_2d(sb + Cfg::B_BYTES / 2, &map_b, full_bar(s), k0, b_row1);
      } else {
        tma_load_2d(sb, &map_b, full_bar(s), k0, b_row0);
      }
    };
    auto load_activations = [&](int i, int s) {
      const uint32_t sa = base + s * Cfg::STAGE_BYTES;
      const uint32_t sb = sa + Cfg::A_TILES * Cfg::A_BYTES;
      const int k0 = (kb_begin + i) * BK;
      if (SWAP) tma_load_2d(sb, &map_b, full_bar(s), k0, b_row0);
      else tma_load_2d(sa, &map_a, full_bar(s), k0, a_row0);
    };
    const int pre = n_kb < Cfg::STAGES ? n_kb : Cfg::STAGES;
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(full_bar(i), Cfg::STAGE_BYTES);
      load_weights(i, i);
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i) load_activations(i, i);
    for (int i = pre; i < n_kb; ++i) {
      const int s = i % Cfg::STAGES;
      const uint32_t ph = (i / Cfg::STAGES) & 1;
      if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, args.error, 1)) break;
      mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
      load_weights(i, s);
      load_activations(i, s);
    }
   }
   __syncwarp();
  } else if (warp == 1) {
   if (lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = instr_desc(BM, BN);
    bool ok = true;
    for (int i = 0; i < n_kb && ok; ++i) {
      const int s = i % Cfg::STAGES;
      const uint32_t ph = (i / Cfg::STAGES) & 1;
      ok = mbar_wait(full_bar(s), ph, abort_flag, args.error, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = base + s * Cfg::STAGE_BYTES;
      const uint32_t sb = sa + Cfg::A_TILES * Cfg::A_BYTES;
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        const uint64_t db = smem_desc(sb + k * UMMA_K * 2);
        umma_bf16(tmem_base, smem_desc(sa + k * UMMA_K * 2), db, idesc, acc);
        if (Cfg::A_TILES == 2)
          umma_bf16(tmem_base + BN, smem_desc(sa + Cfg::A_BYTES + k * UMMA_K * 2), db, idesc, acc);
      }
      umma_commit(empty_bar(s));      // the stage is free once these MMAs have read it
    }
    umma_commit(acc_bar);             // accumulators complete
   }
   __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    pdl_wait();                                    // nothing is written before the kernel before is done
    const int quarter = warp & 3;                  // the 32 lanes of tensor memory this warp may read
    const int r = quarter * 32 + lane;             // row of the A-side tile
    if (SWAP && args.residual != nullptr && args.cluster_reduce) {
      const int S = args.k_splits;
      const int r0 = split * BM / S, nrows = (split + 1) * BM / S - r0;
      const int ncols = min(BN, args.T - tile_b * BN);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int e = (int)threadIdx.x - 64 + k * 128;
        if (e < ncols * nrows) {
          const int c = e / nrows;
          const int t = tile_b * BN + c, n = tile_a * BM + r0 + (e - c * nrows);
          if (n < args.N) {
            early_old[k] = __ldcg(args.residual + (size_t)t * args.N + n);
            if (args.norm_weight) early_weight[k] = args.norm_weight[n];
            if (args.bias) early_bias[k] = args.bias[n];
          }
        }
      }
    }
    const bool scaled = SWAP && args.sumsq_in != nullptr;
    if (scaled) {
      // 1 / rms of this tile's tokens, while the products run: a warp per column adds the
      // partial sums in a fixed order
      // (all columns at once: 128 / BN consecutive lanes share a column's partial sums)
      constexpr int PER_COL = BN <= 128 ? 128 / BN : 1;
      const int et = (int)threadIdx.x - 64;
      const int c = et / PER_COL, q = et % PER_COL;
      const int t = tile_b * BN + c;
      float ss = 0.f;
      if (t < args.T) {
        const float* src = args.sumsq_in + (size_t)t * args.slots_in;
#pragma unroll 8
        for (int j = q; j < args.slots_in; j += PER_COL) ss += __ldcg(src + j);
      }
#pragma unroll
      for (int o = PER_COL / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (q == 0) col_scale[c] = t < args.T ? rsqrtf(ss / args.width + args.eps) : 0.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    bool ok = true;
    if (n_kb > 0) ok = mbar_wait(acc_bar, 0, abort_flag, args.error, 3);
    if (*abort_flag) ok = false;
    tc_fence_after();
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int tile_id = tile_b * gridDim.x + tile_a;
    const size_t tile_elems = (size_t)BM * Cfg::ACC_COLS;
    bool finalize = ok;
    if (args.cluster_reduce) {
      // Slices of one tile are the blocks of one cluster.  Each parks its partial sums in
      // its own shared memory (the stage buffers are free now), column-major [col][128].
      finalize = false;
      float* part = reinterpret_cast<float*>(aligned);
      for (int c = 0; c < Cfg::ACC_COLS; c += 16) {
        float v[16];
        if (ok && n_kb > 0) {
          tmem_ld16(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) part[(c + j) * BM + r] = v[j];
      }
    } else if (ok && args.k_splits > 1) {
      // park the partial sums; the last block of the tile adds them up
      float* mine = args.scratch + ((size_t)tile_id * args.k_splits + split) * tile_elems;
      for (int c = 0; c < Cfg::ACC_COLS; c += 16) {
        float v[16];
        if (n_kb > 0) {
          tmem_ld16(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[(size_t)(c + j) * BM + r] = v[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");        // the four epilogue warps
      if (threadIdx.x == 64) {
        const int ticket = atomicAdd(args.tickets + tile_id, 1);
        const int last = (ticket == args.k_splits - 1) ? 1 : 0;
        if (last) args.tickets[tile_id] = 0;                 // ready for the next launch
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      finalize = (*last_flag != 0);
      if (finalize) __threadfence();
    }
    if (finalize) {
      const float* parts = args.scratch + (size_t)tile_id * args.k_splits * tile_elems;
      auto load_chunk = [&](int c, float (&v)[16]) {
        if (args.k_splits > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          for (int sp = 0; sp < args.k_splits; ++sp) {
            const float* p = parts + (size_t)sp * tile_elems;
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __ldcg(p + (size_t)(c + j) * BM + r);
          }
        } else if (n_kb > 0) {
          tmem_ld16(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
      };
      auto store = [&](int t, int n, float val) {
        if (t < args.T && n < args.N) {
          if (args.bias) val += args.bias[n];
          if (args.out_f32) reinterpret_cast<float*>(args.out)[(size_t)t * args.ldo + n] = val;
          else reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)t * args.ldo + n] = __float2bfloat16_rn(val);
        }
      };
      if (EPI == EPI_GLU) {
        constexpr int HALF = SWAP ? BN : BN / 2;   // columns of the gate accumulator
        for (int c = 0; c < HALF; c += 16) {
          if (SWAP && tile_b * BN + c >= args.T) break;           // columns without tokens
          float g[16], u[16];
          load_chunk(c, g);
          load_chunk(HALF + c, u);
          if (scaled) {
#pragma unroll
            for (int j = 0; j < 16; ++j) { g[j] *= col_scale[c + j]; u[j] *= col_scale[c + j]; }
          }
          float val[16];
          // (a row or column beyond the last token holds zeros, and 0 / x takes the division's
          // slow path: the whole warp would wait for it)
          const bool idle_row = !SWAP && tile_a * BM + r >= args.T;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const bool idle = SWAP ? tile_b * BN + c + j >= args.T : idle_row;
            val[j] = idle ? 0.f : g[j] / (1.f + __expf(-g[j])) * u[j];
          }
          if (SWAP) {
#pragma unroll
            for (int j = 0; j < 16; ++j) store(tile_b * BN + c + j, tile_a * BM + r, val[j]);
          } else {
            const int t = tile_a * BM + r, n0 = tile_b * HALF + c;
            if (!args.out_f32 && t < args.T && n0 + 16 <= args.N && (args.ldo & 7) == 0) {
              uint32_t packed[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 p = __floats2bfloat162_rn(val[2 * j], val[2 * j + 1]);
                packed[j] = *reinterpret_cast<uint32_t*>(&p);
              }
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(args.out) + (size_t)t * args.ldo + n0);
              dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) store(t, n0 + j, val[j]);
            }
          }
        }
      } else {
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          load_chunk(c, v);
          if (SWAP && args.residual != nullptr) {
            // into the residual stream; a warp holds 32 features of every token of the tile
            const int n = tile_a * BM + r;
            const int slots = (int)gridDim.x * SUMSQ_SLOTS;
            const bool mine = n < args.N;
            const float bias_n = (mine && args.bias) ? args.bias[n] : 0.f;
            const float weight_n = (mine && args.norm_weight) ? args.norm_weight[n] : 0.f;
            float old[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {                    // the 16 loads in one trip
              const int t = tile_b * BN + c + j;
              old[j] = (mine && t < args.T) ? args.residual[(size_t)t * args.N + n] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = tile_b * BN + c + j;
              if (t < args.T) {                               // the same for the whole warp
                const float nv = old[j] + v[j] + bias_n;
                if (mine) {
                  args.residual[(size_t)t * args.N + n] = nv;
                  if (args.norm_weight)
                    reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)t * args.ldo + n] =
                        __float2bfloat16_rn(nv * weight_n);
                }
                if (args.norm_weight) {
                  const float sq = warp_sum(mine ? nv * nv : 0.f);
                  float* dst = args.sumsq_out + (size_t)t * slots + tile_a * SUMSQ_SLOTS;
                  if (lane == 0) { dst[quarter] = sq; dst[4 + quarter] = 0.f; }
                }
              }
            }
          } else if (SWAP) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              store(tile_b * BN + c + j, tile_a * BM + r, scaled ? v[j] * col_scale[c + j] : v[j]);
          } else {
            const int t = tile_a * BM + r, n0 = tile_b * BN + c;
            if (!args.out_f32 && t < args.T && n0 + 16 <= args.N && (args.ldo & 7) == 0) {
              // 16 bfloat16 of one row: two 16-byte stores
              uint32_t packed[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float lo = v[2 * j], hi = v[2 * j + 1];
                if (args.bias) { lo += args.bias[n0 + 2 * j]; hi += args.bias[n0 + 2 * j + 1]; }
                __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
                packed[j] = *reinterpret_cast<uint32_t*>(&p);
              }
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(args.out) + (size_t)t * args.ldo + n0);
              dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) store(t, n0 + j, v[j]);
            }
          }
        }
      }
    }
  }

  if (args.cluster_reduce) {
    // ---------------------------------------------------------------- reduction inside the cluster
    // After the barrier every block adds up its share of the tile's elements, reading the
    // partial sums of all slices (in slice order) from its peers' shared memory, and writes
    // the result; the second barrier keeps every block's memory alive until all have read.
    cluster_sync_all();
    if (SWAP && args.residual != nullptr) {
      // Into the residual stream: this block adds up rows [r0, r1) of the tile's 128 features
      // for every token of the tile, an element a thread; the squares go through shared
      // memory (behind the partial sums), where four lanes add up a token's in a fixed order.
      if (warp >= 2 && !*abort_flag) {
        const int S = args.k_splits;
        const int r0 = split * BM / S, r1 = (split + 1) * BM / S, nrows = r1 - r0;
        const int ncols = min(BN, args.T - tile_b * BN);
        const int total = ncols * nrows;
        const int slots = (int)gridDim.x * SUMSQ_SLOTS;
        const int et = (int)threadIdx.x - 64;
        float* squares = reinterpret_cast<float*>(aligned) + Cfg::ACC_COLS * BM;     // [ncols][nrows]
        for (int e = et; e < total; e += 128) {
          const int c = e / nrows, rr = r0 + (e - c * nrows);
          const int t = tile_b * BN + c, n = tile_a * BM + rr;
          const bool mine = n < args.N;
          const int k = (e - et) >> 7;               // the first two were fetched under the main loop
          const bool early = k < 2;
          const float old = k == 0 ? early_old[0] : early ? early_old[1]
                            : mine ? args.residual[(size_t)t * args.N + n] : 0.f;
          const float weight_n = k == 0 ? early_weight[0] : early ? early_weight[1]
                                 : (mine && args.norm_weight) ? args.norm_weight[n] : 0.f;
          const float bias_n = k == 0 ? early_bias[0] : early ? early_bias[1]
                               : (mine && args.bias) ? args.bias[n] : 0.f;
          float pv[8];
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)
            pv[sp] = sp < S ? ld_peer_smem(base + (uint32_t)(c * BM + rr) * 4u, sp) : 0.f;
          float val = 0.f;
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) val += pv[sp];
          const float nv = old + val + bias_n;
          if (mine) {
            args.residual[(size_t)t * args.N + n] = nv;
            if (args.norm_weight)
              reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)t * args.ldo + n] = __float2bfloat16_rn(nv * weight_n);
          }
          squares[e] = mine ? nv * nv : 0.f;
        }
        if (args.norm_weight) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int c = et >> 2, q = et & 3;                   // at most 32 token columns (checked at launch)
          float sq = 0.f;
          if (c < ncols)
            for (int i = q; i < nrows; i += 4) sq += squares[c * nrows + i];
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          if (c < ncols && q == 0) {
            float* dst = args.sumsq_out + (size_t)(tile_b * BN + c) * slots + tile_a * SUMSQ_SLOTS;
            dst[split] = sq;
            if (split == 0) for (int sp = S; sp < SUMSQ_SLOTS; ++sp) dst[sp] = 0.f;
          }
        }
      }
    } else if (warp >= 2 && !*abort_flag) {
      constexpr int OUT_COLS = (EPI == EPI_GLU && !SWAP) ? BN / 2 : BN;   // columns of the result tile
      constexpr int GLU_SHIFT = (EPI == EPI_GLU) ? (SWAP ? BN : BN / 2) : 0;
      const uint32_t part_addr = base;
      const int S = args.k_splits;
      // swapped: only the columns that hold tokens are shared out (the others are padding of
      // the MMA's N axis; sums of zeros, whose SwiGLU would also take the slow path of the
      // division)
      const int cols = SWAP ? max(0, min(OUT_COLS, args.T - tile_b * BN)) : OUT_COLS;
      const int total = cols * BM;
      const int per = (total + S - 1) / S;
      const int e_begin = split * per, e_end = min(total, e_begin + per);
      // two elements a thread and pass: the loads of both (from up to 8 peers each) go out
      // before either sum is used
      for (int e0 = e_begin + (int)threadIdx.x - 64; e0 < e_end; e0 += 256) {
        float gv[2][8], uv[2][8], bias_n[2];
        bool live[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int e = e0 + k * 128;
          const int c = e / BM, rr = e - c * BM;
          live[k] = e < e_end && (SWAP || tile_a * BM + rr < args.T);     // not a row beyond the last token
          // the bias goes out with the partial sums, not after them
          const int feature = SWAP ? tile_a * BM + rr : tile_b * OUT_COLS + c;
          bias_n[k] = (args.bias != nullptr && live[k] && feature < args.N) ? args.bias[feature] : 0.f;
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) {
            const bool on = live[k] && sp < S;
            gv[k][sp] = on ? ld_peer_smem(part_addr + (uint32_t)(c * BM + rr) * 4u, sp) : 0.f;
            uv[k][sp] = (EPI == EPI_GLU && on)
                            ? ld_peer_smem(part_addr + (uint32_t)((GLU_SHIFT + c) * BM + rr) * 4u, sp) : 0.f;
          }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (!live[k]) continue;
          const int e = e0 + k * 128;
          const int c = e / BM, rr = e - c * BM;
          float g = 0.f, u = 0.f;                       // the sum in slice order
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) { g += gv[k][sp]; u += uv[k][sp]; }
          if (SWAP && args.sumsq_in != nullptr) { g *= col_scale[c]; u *= col_scale[c]; }
          float val = g;
          if (EPI == EPI_GLU) val = g / (1.f + __expf(-g)) * u;
          int t, n;
          if (SWAP) { t = tile_b * BN + c; n = tile_a * BM + rr; }
          else { t = tile_a * BM + rr; n = tile_b * OUT_COLS + c; }
          if (t < args.T && n < args.N) {
            val += bias_n[k];
            if (args.out_f32) reinterpret_cast<float*>(args.out)[(size_t)t * args.ldo + n] = val;
            else reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)t * args.ldo + n] = __float2bfloat16_rn(val);
          }
        }
      }
    }
    cluster_sync_all();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // copies of this block may still be in flight: give them time to land before the
    // shared memory is handed to another block
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ two-SM persistent kernel (prefill)
// A cluster of two blocks works on tiles of 256 tokens x 256 weight rows with
// tcgen05.mma.cta_group::2: each block stages its 128 token rows and HALF of the weight
// tile (128 rows; for SwiGLU the even block takes the gate rows and the odd block the up
// rows), so a stage is 32 KB instead of 48 KB, six stages fit, and every SM reads two
// thirds of the operand bytes from L2.  The even block's MMA thread issues for the pair;
// barriers: copies of both blocks count on the leader's "full" barriers, one multicast
// commit frees a stage in both blocks and publishes an accumulator to both epilogues, and
// both epilogues hand accumulators back on the leader's "empty" barrier.
constexpr int T2_STAGES = 6;
constexpr int T2_A_BYTES = BM * BK * 2;            // 128 token rows
constexpr int T2_B_BYTES = 128 * BK * 2;           // this block's half of the weight tile
constexpr int T2_STAGE_BYTES = T2_A_BYTES + T2_B_BYTES;
constexpr size_t T2_SMEM = (size_t)T2_STAGES * T2_STAGE_BYTES + 1024 + 256;

template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     GemmArgs args, int tiles_m, int tiles_n) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch_dependents();
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (size_t)T2_STAGES * T2_STAGE_BYTES);
  // [0,S): full (leader's are used), [S,2S): empty, then 2 accumulator-full, 2 accumulator-empty (leader's)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T2_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int kb_total = (args.K + BK - 1) / BK;
  const int n_tiles = tiles_m * tiles_n;             // tiles of 256 x 256
  constexpr int RESULT_COLS = (EPI == EPI_GLU) ? 128 : 256;

  auto full_bar = [&](int s) { return smem_u32(bars + s); };
  auto empty_bar = [&](int s) { return smem_u32(bars + T2_STAGES + s); };
  auto acc_full = [&](int b) { return smem_u32(bars + 2 * T2_STAGES + b); };
  auto acc_empty = [&](int b) { return smem_u32(bars + 2 * T2_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 8);          // four epilogue warps in each of the two blocks
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(tmem_slot), 512);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                      // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int my_tiles = pair < n_tiles ? (n_tiles - 1 - pair) / n_pairs + 1 : 0;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------- TMA producer (both blocks)
      pdl_wait();
      uint32_t it = 0;
      for (int j = 0; j < my_tiles; ++j) {
        const int q = pair + j * n_pairs;
        const int tile_m = q % tiles_m, tile_n = q / tiles_m;
        const int a_row = tile_m * 256 + (int)rank * 128;
        const int b_row = (EPI == EPI_GLU) ? (rank ? args.glu_offset : 0) + tile_n * 128
                                           : tile_n * 256 + (int)rank * 128;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % T2_STAGES;
          const uint32_t ph = (it / T2_STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, args.error, 1)) { j = my_tiles; break; }
          // the leader announces the bytes of BOTH blocks for the stage
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * T2_STAGE_BYTES);
          const uint32_t sa = base + s * T2_STAGE_BYTES;
          const int k0 = kb * BK;
          tma_load_2d_2sm(sa + T2_A_BYTES, &map_b, full_bar(s), k0, b_row);
          tma_load_2d_2sm(sa, &map_a, full_bar(s), k0, a_row);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------------------------------------------------- MMA issuer (leader only)
      constexpr uint32_t idesc = instr_desc(256, 256);
      uint32_t it = 0;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int b = j & 1;
        const uint32_t use = (uint32_t)(j >> 1);
        ok = mbar_wait(acc_empty(b), (use & 1) ^ 1, abort_flag, args.error, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + (uint32_t)(b * 256);
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % T2_STAGES;
          const uint32_t ph = (it / T2_STAGES) & 1;
          ok = mbar_wait(full_bar(s), ph, abort_flag, args.error, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = base + s * T2_STAGE_BYTES, sb = sa + T2_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_2sm(acc_addr, smem_desc(sa + k * UMMA_K * 2), smem_desc(sb + k * UMMA_K * 2), idesc,
                          (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_2sm(empty_bar(s));
        }
        if (ok) umma_commit_2sm(acc_full(b));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue warps (both blocks)
    pdl_wait();
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    for (int j = 0; j < my_tiles; ++j) {
      const int b = j & 1;
      const uint32_t use = (uint32_t)(j >> 1);
      const int q = pair + j * n_pairs;
      const int tile_m = q % tiles_m, tile_n = q / tiles_m;
      if (!mbar_wait(acc_full(b), use & 1, abort_flag, args.error, 3)) break;
      if (*abort_flag) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * 256);
      const int t = tile_m * 256 + (int)rank * 128 + r;
      for (int c = 0; c < RESULT_COLS; c += 16) {
        float val[16];
        if (EPI == EPI_GLU) {
          float g[16], u[16];
          tmem_ld16(taddr + c, g);
          tmem_ld16(taddr + 128 + c, u);
          if (t < args.T) {       // rows beyond the last token hold zeros: 0 / x is the division's slow path
#pragma unroll
            for (int i = 0; i < 16; ++i) val[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
          }
        } else {
          tmem_ld16(taddr + c, val);
        }
        const int n0 = tile_n * RESULT_COLS + c;
        if (t < args.T) {
          if (args.bias) {
#pragma unroll
            for (int i = 0; i < 16; ++i) if (n0 + i < args.N) val[i] += args.bias[n0 + i];
          }
          if (!args.out_f32 && n0 + 16 <= args.N && (args.ldo & 7) == 0) {
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              __nv_bfloat162 p = __floats2bfloat162_rn(val[2 * i], val[2 * i + 1]);
              packed[i] = *reinterpret_cast<uint32_t*>(&p);
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(args.out) + (size_t)t * args.ldo + n0);
            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (n0 + i < args.N) {
                if (args.out_f32) reinterpret_cast<float*>(args.out)[(size_t)t * args.ldo + n0 + i] = val[i];
                else reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)t * args.ldo + n0 + i] = __float2bfloat16_rn(val[i]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(acc_empty(b));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  cluster_sync_all();                      // neither block frees tensor memory the pair still uses
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ host side
constexpr int HB_MAX_DEVICES = 64;
inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= HB_MAX_DEVICES) return -1;
  return dev;
}

template <int BN, bool SWAP, int EPI>
int launch(const void* x, const void* w, const GemmArgs& args, int w_rows, int ldx, int ldw,
           cudaStream_t stream) {
  using Cfg = Config<BN, SWAP, EPI>;
  CUtensorMap map_a, map_b;
  // box rows of the weight-side map: a full tile, or half of it for the two SwiGLU halves
  if (SWAP) {
    if (!make_map(&map_a, w, w_rows, args.K, ldw, BM)) return HB_LAUNCH_FAILED;
    if (!make_map(&map_b, x, args.T, args.K, ldx, BN)) return HB_LAUNCH_FAILED;
  } else {
    if (!make_map(&map_a, x, args.T, args.K, ldx, BM)) return HB_LAUNCH_FAILED;
    if (!make_map(&map_b, w, w_rows, args.K, ldw, EPI == EPI_GLU ? BN / 2 : BN)) return HB_LAUNCH_FAILED;
  }
  auto kernel = gemm_bf16_kernel<BN, SWAP, EPI>;
  // the shared-memory limit is a per-device attribute of the kernel
  static bool configured[HB_MAX_DEVICES] = {};
  const int dev = current_device();
  if (dev < 0) return HB_LAUNCH_FAILED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured[dev] = true;
  }
  dim3 grid;
  if (SWAP) {
    grid = dim3((args.N + BM - 1) / BM, (args.T + BN - 1) / BN, args.k_splits);
  } else {
    const int per_tile = (EPI == EPI_GLU) ? BN / 2 : BN;
    grid = dim3((args.T + BM - 1) / BM, (args.N + per_tile - 1) / per_tile, args.k_splits);
  }
  if (args.cluster_reduce) {
    // the partial sums of a block must fit the stage buffers they reuse
    if ((size_t)Cfg::ACC_COLS * BM * sizeof(float) > (size_t)Cfg::STAGES * Cfg::STAGE_BYTES || args.k_splits > 8)
      return HB_BAD_ARGUMENT;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = args.k_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = hb_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, args);
  } else {
    hb_launch(kernel, grid, dim3(GEMM_THREADS), Cfg::SMEM, stream, map_a, map_b, args);
  }
  return hb_check_launch();
}

template <int EPI>
int launch_2sm(const void* x, const void* w, const GemmArgs& args, int w_rows, int ldx, int ldw,
               cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, x, args.T, args.K, ldx, BM)) return HB_LAUNCH_FAILED;
  if (!make_map(&map_b, w, w_rows, args.K, ldw, 128)) return HB_LAUNCH_FAILED;
  auto kernel = gemm_bf16_2sm_kernel<EPI>;
  static int sm_counts[HB_MAX_DEVICES] = {};         // 0: this device is not set up yet
  const int dev = current_device();
  if (dev < 0) return HB_LAUNCH_FAILED;
  if (sm_counts[dev] == 0) {
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T2_SMEM) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return HB_LAUNCH_FAILED;
    sm_counts[dev] = n;
  }
  const int sm_count = sm_counts[dev];
  const int per_tile = (EPI == EPI_GLU) ? 128 : 256;
  const int tiles_m = (args.T + 255) / 256, tiles_n = (args.N + per_tile - 1) / per_tile;
  const int n_tiles = tiles_m * tiles_n;
  int pairs = sm_count / 2;
  if (n_tiles < pairs) pairs = n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = T2_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hb_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, args, tiles_m, tiles_n);
  return hb_check_launch();
}

// How many clusters of `cluster_size` blocks of this kernel the device keeps resident.
template <int BN, bool SWAP, int EPI>
int max_clusters(int cluster_size) {
  using Cfg = Config<BN, SWAP, EPI>;
  auto kernel = gemm_bf16_kernel<BN, SWAP, EPI>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM) != cudaSuccess)
    return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, cluster_size);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster_size;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) return -1;
  return n;
}

}  // namespace

#ifndef HB_GEMM_BF16_NO_EXPORTS
// Resident clusters of `cluster_size` blocks for the kernel variant a call would use
// (-1 if the query fails).
HB_EXPORT int hb_gemm_bf16_max_clusters(int swap_bn, int glu, int cluster_size) {
  if (cluster_size < 1 || cluster_size > 8) return -1;
#define HB_OCC_CASE(BN_, SWAP_) \
  return glu ? max_clusters<BN_, SWAP_, EPI_GLU>(cluster_size) : max_clusters<BN_, SWAP_, EPI_STORE>(cluster_size)
  switch (swap_bn) {
    case 0: HB_OCC_CASE(256, false);
    case 16: HB_OCC_CASE(16, true);
    case 32: HB_OCC_CASE(32, true);
    case 64: HB_OCC_CASE(64, true);
    case 128: HB_OCC_CASE(128, true);
    default: return -1;
  }
#undef HB_OCC_CASE
}

// Output tiles of a call (N counts the result's features), and the scratch floats it needs
// (0 when the K range is not split).  swap_bn = 0: tiles of 128 tokens x 256 features (128
// result features for SwiGLU); else 128 features x swap_bn tokens.
HB_EXPORT int hb_gemm_bf16_tiles(int T, int N, int swap_bn, int glu) {
  if (swap_bn == 0) {
    const int per = glu ? 128 : 256;
    return ((T + BM - 1) / BM) * ((N + per - 1) / per);
  }
  return ((N + BM - 1) / BM) * ((T + swap_bn - 1) / swap_bn);
}
HB_EXPORT long long hb_gemm_bf16_scratch_floats(int T, int N, int swap_bn, int glu, int k_splits) {
  if (k_splits <= 1) return 0;
  const long long cols = swap_bn == 0 ? 256 : (long long)swap_bn * (glu ? 2 : 1);
  return (long long)hb_gemm_bf16_tiles(T, N, swap_bn, glu) * k_splits * BM * cols;
}

// y[T, N] = x[T, K] w[N, K]^T (+ bias), or SwiGLU over w = [gate rows; up rows] with the up
// rows starting at row glu_offset (then N counts the result's features).
//   swap_bn = 0: tokens on the M axis (tile 128 x 256).  swap_bn in {16, 32, 64, 128}: swapped,
//   that many tokens per tile.  With 1 < k_splits <= 8 and `cluster` set, the slices of a tile
//   run as one thread-block cluster and add up through distributed shared memory; else the
//   partial sums go through `scratch` with one ticket per tile.
static int gemm_bf16_call(void* out, const void* x, const void* w, const float* bias, float* scratch,
                          int* tickets, int* error, int T, int N, int K, int ldx, int ldw, int ldo,
                          int w_rows, int glu, int glu_offset, int out_f32, int swap_bn, int k_splits,
                          int cluster, float* residual, const float* norm_weight, float* sumsq_out,
                          const float* sumsq_in, int slots_in, float eps, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return HB_OK;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || k_splits < 1) return HB_BAD_ARGUMENT;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return HB_BAD_ARGUMENT;
  const bool clustered = k_splits > 1 && k_splits <= 8 && cluster != 0;
  if (k_splits > 1 && !clustered && (scratch == nullptr || tickets == nullptr)) return HB_BAD_ARGUMENT;
  if (k_splits > (K + BK - 1) / BK) return HB_BAD_ARGUMENT;
  if (error == nullptr) return HB_BAD_ARGUMENT;
  if (residual != nullptr || sumsq_in != nullptr) {
    // the epilogues of few-token steps: swapped orientation, one token tile
    if (swap_bn == 0 || T > swap_bn) return HB_BAD_ARGUMENT;
    if (residual != nullptr && swap_bn > 32) return HB_BAD_ARGUMENT;   // room for the squares, four lanes a token
    if (residual != nullptr && (glu || out_f32)) return HB_BAD_ARGUMENT;
    if (norm_weight != nullptr && (residual == nullptr || out == nullptr || sumsq_out == nullptr))
      return HB_BAD_ARGUMENT;
    if (sumsq_in != nullptr && slots_in <= 0) return HB_BAD_ARGUMENT;
  }
  GemmArgs a;
  a.out = out; a.bias = bias; a.scratch = scratch; a.tickets = tickets; a.error = error;
  a.T = T; a.N = N; a.K = K; a.ldo = ldo; a.glu_offset = glu_offset; a.out_f32 = out_f32;
  a.k_splits = k_splits;
  a.cluster_reduce = clustered ? 1 : 0;
  a.residual = residual; a.norm_weight = norm_weight; a.sumsq_out = sumsq_out;
  a.sumsq_in = sumsq_in; a.slots_in = slots_in; a.width = (float)K; a.eps = eps;
#define HB_GEMM_CASE(BN_, SWAP_)                                                              \
  return glu ? launch<BN_, SWAP_, EPI_GLU>(x, w, a, w_rows, ldx, ldw, stream)                 \
             : launch<BN_, SWAP_, EPI_STORE>(x, w, a, w_rows, ldx, ldw, stream)
  if (swap_bn == 0 && k_splits == 1 && cluster == 2)    // prefill: a persistent kernel on pairs of SMs
    return glu ? launch_2sm<EPI_GLU>(x, w, a, w_rows, ldx, ldw, stream)
               : launch_2sm<EPI_STORE>(x, w, a, w_rows, ldx, ldw, stream);
  switch (swap_bn) {
    case 0: HB_GEMM_CASE(256, false);
    case 16: HB_GEMM_CASE(16, true);
    case 32: HB_GEMM_CASE(32, true);
    case 64: HB_GEMM_CASE(64, true);
    case 128: HB_GEMM_CASE(128, true);
    default: return HB_BAD_ARGUMENT;
  }
#undef HB_GEMM_CASE
}

HB_EXPORT int hb_gemm_bf16(void* out, const void* x, const void* w, const float* bias, float* scratch,
                           int* tickets, int* error, int T, int N, int K, int ldx, int ldw, int ldo,
                           int w_rows, int glu, int glu_offset, int out_f32, int swap_bn, int k_splits,
                           int cluster, cudaStream_t stream) {
  return gemm_bf16_call(out, x, w, bias, scratch, tickets, error, T, N, K, ldx, ldw, ldo, w_rows, glu,
                        glu_offset, out_f32, swap_bn, k_splits, cluster, nullptr, nullptr, nullptr,
                        nullptr, 0, 0.f, stream);
}

// The same product with the epilogues of few-token steps (swapped orientation, T <= swap_bn):
//   residual [T, N] float32: residual += x w^T (+ bias) instead of writing the product; with
//   norm_weight [N] also out[T, ldo] = bfloat16(residual * norm_weight) and
//   sumsq_out[T, 8 * ceil(N / 128)] = partial sums of residual^2 over the features, so that
//   rsqrt(sum / N + eps) is the factor that `out` still lacks to be the RMS norm;
//   sumsq_in [T, slots_in]: x lacks such a factor over ITS width K; every accumulator of token
//   t is multiplied by rsqrt(sum(sumsq_in[t]) / K + eps) before bias or SwiGLU.
HB_EXPORT int hb_gemm_bf16_fused(void* out, const void* x, const void* w, const float* bias, float* scratch,
                                 int* tickets, int* error, int T, int N, int K, int ldx, int ldw, int ldo,
                                 int w_rows, int glu, int glu_offset, int out_f32, int swap_bn,
                                 int k_splits, int cluster, float* residual, const float* norm_weight,
                                 float* sumsq_out, const float* sumsq_in, int slots_in, float eps,
                                 cudaStream_t stream) {
  return gemm_bf16_call(out, x, w, bias, scratch, tickets, error, T, N, K, ldx, ldw, ldo, w_rows, glu,
                        glu_offset, out_f32, swap_bn, k_splits, cluster, residual, norm_weight, sumsq_out,
                        sumsq_in, slots_in, eps, stream);
}
#endif  // HB_GEMM_BF16_NO_EXPORTS
