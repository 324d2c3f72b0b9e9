// A whole decode step of the dense GQA decoder (python/helios/exec/model.py:465-496: layers,
// final norm, output head) for at most 8 requests, in ONE persistent kernel.
//
// Why: with a handful of tokens a step is a string of short operations (eight launches a
// layer when each is a kernel of its own), and what bounds it is the ramp between them, not
// the bytes.  Here one block per SM stays resident for the step.  Every layer is five phases,
//   1  RMSNorm -> q|k|v projection (+ bias) -> rotation -> q to a buffer, k and v to the cache
//   2  attention over the paged cache (context slices, merged by whichever slice ends last)
//   3  output projection, added into the residual stream
//   4  RMSNorm -> gate|up projection -> silu(gate) * up
//   5  down projection, added into the residual stream
// then final RMSNorm -> output head.  Between two phases all blocks meet at a barrier in
// global memory; a block requests the first weights of its next phase BEFORE it waits
// there, so the weight stream does not stop at a phase's end.
//
// Products: the tokens ride the M axis of mma.sync.m16n8k16 (rows 8..15 are zero), eight
// weight rows the N axis.  A block owns a contiguous share of a phase's "units" (8 weight
// rows each, for q and k four rotary pairs, for gate|up four gate rows and their up rows)
// and ALL of K: its eight warps take every eighth block of 32 k and add their partial
// sums through shared memory in warp order, so a result depends on nothing but its own row
// and the step's token count.  Weights go from global memory straight into the B fragments
// (16 bytes a thread; the two MMAs of a 32-k block take elements 0..3 and 4..7 of every
// thread's chunk as their k columns, the A fragments follow the same rule), two load steps
// of 12 x 16 bytes a thread in flight per warp: the bytes in flight live in registers, which
// is why a block has 256 threads with many registers each rather than more threads.  With a
// norm in front, the block norms the residual rows into shared memory itself (float32
// statistics, 1/rms applied to the finished sums).
//
// Every wait is bounded: a block that gives up raises the error word, and every block
// leaves at its next barrier.  The kernel is launched cooperatively (all blocks resident).
#include "attention_mma.cuh"

namespace {

constexpr int DS_WARPS = 8;
constexpr int DS_THREADS = DS_WARPS * 32;
constexpr int NT = 4;                 // units of 8 weight rows a block works on at once
constexpr int U = 3;                  // blocks of 32 k per load step and warp
constexpr int MAX_T = 8;
constexpr int ATT_WARPS = 8;          // warps that walk the keys in the attention phase
constexpr int ATT_TILE = 16;          // keys per warp tile
constexpr int MAX_GROUPS = 4;         // cache groups (block tables) a model may have
constexpr uint32_t SPIN_LIMIT = 1u << 22;

enum { MODE_RESIDUAL = 0, MODE_GLU = 1, MODE_QKV = 2, MODE_LOGITS = 3 };
enum { ERR_BARRIER = 21 };

struct DsLayer {
  const __nv_bfloat16* w_qkv;
  const float* b_qkv;
  const __nv_bfloat16* w_o;
  const __nv_bfloat16* w_gate_up;
  const __nv_bfloat16* w_down;
  const float* norm_attn;
  const float* norm_ffn;
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  float eps_attn, eps_ffn;
  int group;                  // which block table
  int window;                 // 0: all keys
  int write_cache;
  int pad;
};

struct DsParams {
  const DsLayer* layers;
  int layer_begin, layer_end;           // layers [begin, end) run
  int run_head;
  int T, H, I, nh, nkv, hd, V, page_size;
  float scale_log2;
  const int* positions;                 // [T]; token t is the one new token of request t
  const int* block_tables[MAX_GROUPS];
  int bt_stride[MAX_GROUPS];
  const float* cos_tab;                 // [T, hd / 2]
  const float* sin_tab;
  float* residual;                      // [T, H]
  __nv_bfloat16* qkv;                   // [T, (nh + 2 nkv) hd]; the q columns are used
  __nv_bfloat16* attn_out;              // [T, nh hd]
  __nv_bfloat16* hmid;                  // [T, I]
  float* part_o;                        // [T nh, splits, hd]
  float* part_ml;                       // [T nh, splits, 2]
  int* tickets;                         // [T nkv], zero between launches
  int splits;
  const float* final_norm;
  float final_eps;
  const __nv_bfloat16* head_w;          // [V, H]
  float* logits;                        // [T, V]
  unsigned* barrier;                    // zero at launch
  int* error;
};

struct Gemv {
  const __nv_bfloat16* w;
  const float* norm_w;        // NORM
  float eps;
  const __nv_bfloat16* x;     // !NORM: [T, K]
  int K, n_units, n_out, glu_offset;
  int layer;                  // QKV: the layer whose bias, pages and block table the epilogue reads
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma8(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8..15 of the A tile (a1, a3) are zero: at most 8 tokens
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bytes between two activation rows in shared memory: 64 beyond a multiple of 128, so the
// 16-byte reads of two neighbouring rows fall into different banks.
__host__ __device__ inline int x_row_bytes(int K) { return ((2 * K + 63) / 128) * 128 + 64; }

// Weight row of column n (0..7) of unit `unit`, or -1 beyond the matrix.
template <int MODE>
__device__ __forceinline__ int unit_row(const DsParams& p, const Gemv& g, int unit, int n) {
  if (MODE == MODE_RESIDUAL || MODE == MODE_LOGITS) {
    const int r = unit * 8 + n;
    return r < g.n_out ? r : -1;
  } else if (MODE == MODE_GLU) {
    const int f = unit * 4 + (n & 3);
    if (f >= g.n_out) return -1;
    return n < 4 ? f : g.glu_offset + f;
  } else {
    const int per_head = p.hd >> 3;
    const int head = unit / per_head, sub = unit - head * per_head;
    if (head >= p.nh + 2 * p.nkv) return -1;
    if (head < p.nh + p.nkv)     // a rotated head: four pairs (d, d + hd/2)
      return head * p.hd + (n < 4 ? sub * 4 + n : (p.hd >> 1) + sub * 4 + (n - 4));
    return head * p.hd + sub * 8 + n;
  }
}

struct Shared {
  float red[DS_WARPS][NT][MAX_T][8];
  float rstd[MAX_T];
  int flag;
};

// ------------------------------------------------------------------ the barrier
// All blocks have arrived `phase` times when the counter reaches phase * gridDim.x.
__device__ __forceinline__ void grid_arrive(const DsParams& p) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_release_add(p.barrier, 1u);
  }
}
// False when the step is aborted (this block or another gave up a wait).
__device__ __forceinline__ bool grid_wait(const DsParams& p, unsigned target, Shared& sh) {
  if (threadIdx.x == 0) {
    int ok = 0;
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
      if (ld_acquire(p.barrier) >= target) { ok = 1; break; }
      if ((i & 63u) == 63u) {
        if (*reinterpret_cast<volatile int*>(p.error) != 0) break;
        __nanosleep(20);
      }
    }
    if (!ok) atomicCAS(p.error, 0, ERR_BARRIER);
    sh.flag = ok;
  }
  __syncthreads();
  const bool ok = sh.flag != 0;
  __syncthreads();
  return ok;
}

// ------------------------------------------------------------------ one product phase
template <int MODE, bool NORM>
__device__ __noinline__ bool gemv_phase(const DsParams& p, const Gemv& g, Shared& sh, unsigned char* xs,
                           unsigned& arrivals, bool wait_first) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, t4 = lane & 3;
  const int K = g.K, nkb = (K + 31) >> 5;
  const int spg = ((nkb + DS_WARPS - 1) / DS_WARPS + U - 1) / U;      // load steps per group of units
  const int u0 = (int)((long long)blockIdx.x * g.n_units / gridDim.x);
  const int u1 = (int)((long long)(blockIdx.x + 1) * g.n_units / gridDim.x);
  const int n_groups = (u1 - u0 + NT - 1) / NT;
  const int total = n_groups * spg;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const uint4* w16 = reinterpret_cast<const uint4*>(g.w);
  const uint32_t row16 = (uint32_t)(K >> 3);
  const bool tok_ok = gq < p.T;

  // Requests of load step s into the buffers (W, X): the weights of the step's NT units for
  // this warp's U blocks of k, and (without a norm) the activation chunks that meet them.
#define DS_ISSUE(s_, W, X, WITH_X)                                                                       \
  {                                                                                                      \
    const int gi_ = (s_) / spg, it_ = (s_) - gi_ * spg;                                                  \
    uint32_t off_[NT];                                                                                   \
    _Pragma("unroll") for (int j = 0; j < NT; ++j) {                                                     \
      const int unit_ = u0 + gi_ * NT + j;                                                               \
      const int r_ = unit_ < u1 ? unit_row<MODE>(p, g, unit_, gq) : -1;                                  \
      off_[j] = r_ >= 0 ? (uint32_t)r_ * row16 : 0xffffffffu;                                            \
    }                                                                                                    \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                                      \
      const int k_ = (warp + DS_WARPS * (it_ * U + u)) * 32 + t4 * 8;                                    \
      const bool in_ = k_ < K;                                                                           \
      _Pragma("unroll") for (int j = 0; j < NT; ++j) {                                                   \
        W[u][j] = zero4;                                                                                 \
        if (in_ && off_[j] != 0xffffffffu) W[u][j] = ldg_stream(w16 + off_[j] + (k_ >> 3));              \
      }                                                                                                  \
      if (!NORM && (WITH_X)) {                                                                           \
        X[u] = zero4;                                                                                    \
        if (in_ && tok_ok) X[u] = __ldcg(reinterpret_cast<const uint4*>(g.x + (size_t)gq * K + k_));     \
      }                                                                                                  \
    }                                                                                                    \
  }

  uint4 w0[U][NT], w1[U][NT], x0[U], x1[U];
  // the weights of the first step do not depend on the phase before: request them, then wait
  // (the activations do depend on it: they are fetched after the wait)
  if (total > 0) DS_ISSUE(0, w0, x0, false)
  if (wait_first) {
    arrivals += gridDim.x;
    if (!grid_wait(p, arrivals, sh)) return false;
  }
  if (total > 0 && !NORM) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (warp + DS_WARPS * u) * 32 + t4 * 8;
      x0[u] = zero4;
      if (k < K && tok_ok) x0[u] = __ldcg(reinterpret_cast<const uint4*>(g.x + (size_t)gq * K + k));
    }
  }

  const int stride = x_row_bytes(K);
  if (NORM && total > 0) {
    // a warp takes a row: bfloat16(residual * norm weight) and the row's 1/rms
    if (warp < MAX_T) {
      float ss = 0.f;
      unsigned char* dst = xs + (size_t)warp * stride;
      const int chunks = K >> 3;
      if (warp < p.T) {
        const float* src = p.residual + (size_t)warp * K;
#pragma unroll 4
        for (int c = lane; c < chunks; c += 32) {
          const float4 a = __ldcg(reinterpret_cast<const float4*>(src + c * 8));
          const float4 q = __ldcg(reinterpret_cast<const float4*>(src + c * 8 + 4));
          const float4 wa = *reinterpret_cast<const float4*>(g.norm_w + c * 8);
          const float4 wq = *reinterpret_cast<const float4*>(g.norm_w + c * 8 + 4);
          ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
          *reinterpret_cast<uint4*>(dst + c * 16) =
              make_uint4(pack_bf16(a.x * wa.x, a.y * wa.y), pack_bf16(a.z * wa.z, a.w * wa.w),
                         pack_bf16(q.x * wq.x, q.y * wq.y), pack_bf16(q.z * wq.z, q.w * wq.w));
        }
      } else {
        for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 16) = zero4;
      }
      ss = warp_sum(ss);
      if (lane == 0) sh.rstd[warp] = rsqrtf(ss / (float)K + g.eps);
    }
    __syncthreads();
  }

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const unsigned char* x_row = xs + (size_t)gq * stride + t4 * 16;

  // the MMAs of load step s from the buffers (W, X)
#define DS_MMA(s_, W, X)                                                                                 \
  {                                                                                                      \
    const int it_ = (s_) % spg;                                                                          \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                                      \
      uint4 xv_ = X[u];                                                                                  \
      if (NORM) {                                                                                        \
        const int kb_ = warp + DS_WARPS * (it_ * U + u);                                                 \
        xv_ = zero4;                                                                                     \
        if (kb_ * 32 + t4 * 8 < K) xv_ = *reinterpret_cast<const uint4*>(x_row + kb_ * 64);              \
      }                                                                                                  \
      _Pragma("unroll") for (int j = 0; j < NT; ++j) {                                                   \
        mma8(acc[j], xv_.x, xv_.y, W[u][j].x, W[u][j].y);                                                \
        mma8(acc[j], xv_.z, xv_.w, W[u][j].z, W[u][j].w);                                                \
      }                                                                                                  \
    }                                                                                                    \
  }

  auto finish_group = [&](int s) {
    const int gi = s / spg, it = s - gi * spg;
    if (it != spg - 1) return;
    // ---- the group's units are complete: add the warps' sums and finish
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      *reinterpret_cast<float2*>(&sh.red[warp][j][gq][2 * t4]) = make_float2(acc[j][0], acc[j][1]);
      acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    }
    __syncthreads();
    const int item = threadIdx.x;
    if (item < NT * MAX_T * 4) {
      const int j = item >> 5, token = (item >> 2) & 7, q = item & 3;
      const int unit = u0 + gi * NT + j;
      if (token < p.T && unit < u1) {
        float v1 = 0.f, v2 = 0.f;
#pragma unroll
        for (int w = 0; w < DS_WARPS; ++w) {
          v1 += sh.red[w][j][token][q];
          v2 += sh.red[w][j][token][q + 4];
        }
        if (NORM) {
          v1 *= sh.rstd[token];
          v2 *= sh.rstd[token];
        }
        const int r1 = unit_row<MODE>(p, g, unit, q), r2 = unit_row<MODE>(p, g, unit, q + 4);
        if (MODE == MODE_RESIDUAL) {
          float* res = p.residual + (size_t)token * g.n_out;
          if (r1 >= 0) res[r1] = __ldcg(res + r1) + v1;
          if (r2 >= 0) res[r2] = __ldcg(res + r2) + v2;
        } else if (MODE == MODE_LOGITS) {
          float* out = p.logits + (size_t)token * g.n_out;
          if (r1 >= 0) out[r1] = v1;
          if (r2 >= 0) out[r2] = v2;
        } else if (MODE == MODE_GLU) {
          if (r1 >= 0) p.hmid[(size_t)token * g.n_out + r1] = __float2bfloat16_rn(v1 / (1.f + __expf(-v1)) * v2);
        } else if (r1 >= 0) {
          // what only this epilogue needs is read here, not kept in registers through the phase
          const DsLayer& L = p.layers[g.layer];
          if (L.b_qkv != nullptr) {
            v1 += L.b_qkv[r1];
            v2 += L.b_qkv[r2];
          }
          const int head = r1 / p.hd, d1 = r1 - head * p.hd, d2 = r2 - head * p.hd;
          if (head < p.nh + p.nkv) {
            const int half = p.hd >> 1;
            const float c = p.cos_tab[(size_t)token * half + d1], sn = p.sin_tab[(size_t)token * half + d1];
            const float o1 = v1 * c - v2 * sn, o2 = v2 * c + v1 * sn;
            v1 = o1;
            v2 = o2;
          }
          __nv_bfloat16* dst = p.qkv + (size_t)token * (p.nh + 2 * p.nkv) * p.hd + (size_t)head * p.hd;
          if (head >= p.nh && L.write_cache) {
            const int pos = p.positions[token];
            const int page = p.block_tables[L.group][(size_t)token * p.bt_stride[L.group] + pos / p.page_size];
            const int slot = pos % p.page_size;
            const bool is_k = head < p.nh + p.nkv;
            const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
            dst = (is_k ? L.k_pages : L.v_pages) + (((size_t)page * p.nkv + kvh) * p.page_size + slot) * p.hd;
          }
          dst[d1] = __float2bfloat16_rn(v1);
          dst[d2] = __float2bfloat16_rn(v2);
        }
      }
    }
    __syncthreads();
  };

  for (int s = 0; s < total; s += 2) {
    if (s + 1 < total) DS_ISSUE(s + 1, w1, x1, true)
    DS_MMA(s, w0, x0)
    finish_group(s);
    if (s + 1 >= total) break;
    if (s + 2 < total) DS_ISSUE(s + 2, w0, x0, true)
    DS_MMA(s + 1, w1, x1)
    finish_group(s + 1);
  }
#undef DS_ISSUE
#undef DS_MMA
  grid_arrive(p);
  return true;
}

// ------------------------------------------------------------------ the attention phase
// Items are (token, KV head, context slice); a block takes every gridDim.x-th item.  The
// warps walk the slice's keys in tiles of 16 (per-warp rings of asynchronous copies), the
// block merges them; the slice of a (token, KV head) that ends last merges the slices.
template <int HD>
__device__ __noinline__ bool attention_phase(const DsParams& p, int layer, Shared& sh, unsigned char* smem_raw,
                                unsigned& arrivals) {
  const DsLayer& Lg = p.layers[layer];
  const __nv_bfloat16* const k_pages = Lg.k_pages;
  const __nv_bfloat16* const v_pages = Lg.v_pages;
  const int window = Lg.window, group = Lg.group;
  constexpr int RS = HD + 8;
  constexpr int TILE_ELEMS = ATT_TILE * RS;
  constexpr int STAGES = HD <= 64 ? 4 : 2;
  arrivals += gridDim.x;
  if (!grid_wait(p, arrivals, sh)) return false;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.nh / p.nkv;
  const int S = p.splits;
  const int n_items = p.T * p.nkv * S;
  const int* table_base = p.block_tables[group];
  const int bt_stride = p.bt_stride[group];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int split = item % S, kvh = (item / S) % p.nkv, seq = item / (S * p.nkv);
    const int pos = p.positions[seq];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - lo + 1;
    const int tiles_total = (n_keys + ATT_TILE - 1) / ATT_TILE;
    const int tiles_per_split = (tiles_total + S - 1) / S;
    const int tile_begin = split * tiles_per_split;
    const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
    const int k_end = pos + 1;
    const int* table = table_base + (size_t)seq * bt_stride;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (warp < ATT_WARPS) {
      __nv_bfloat16* my = smem + (size_t)warp * STAGES * 2 * TILE_ELEMS;
      auto load_tile = [&](int tile, int stage) {
        constexpr int CH = HD / 8;
        int row_id = -1;
        if (lane < ATT_TILE) {
          const int key = lo + tile * ATT_TILE + lane;
          if (key < k_end) {
            const int page = table[key / p.page_size];
            row_id = (page * p.nkv + kvh) * p.page_size + key % p.page_size;
          }
        }
        __nv_bfloat16* kd = my + (size_t)(stage * 2) * TILE_ELEMS;
        __nv_bfloat16* vd = kd + TILE_ELEMS;
#pragma unroll
        for (int it = 0; it < ATT_TILE * CH / 32; ++it) {
          const int idx = it * 32 + lane;
          const int row = idx / CH, c = idx - row * CH;
          const int rid = __shfl_sync(0xffffffffu, row_id, row);
          const size_t base = (size_t)(rid < 0 ? 0 : rid) * HD + c * 8;
          const int bytes = rid < 0 ? 0 : 16;
          cp_async16(kd + row * RS + c * 8, k_pages + base, bytes);
          cp_async16(vd + row * RS + c * 8, v_pages + base, bytes);
        }
      };
      int tile = tile_begin + warp;
#pragma unroll
      for (int s = 0; s < STAGES - 1; ++s) {
        const int tp = tile + s * ATT_WARPS;
        if (tp < tile_end) load_tile(tp, s);
        cp_async_commit();
      }
      // query fragments: rows = the group's heads (zero beyond G)
      uint32_t qa[HD / 16][4];
      {
        const int g0 = lane >> 2, c0 = 2 * (lane & 3);
        const __nv_bfloat16* qrow = p.qkv + (size_t)seq * (p.nh + 2 * p.nkv) * HD + (size_t)kvh * G * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = g0 + (e & 1) * 8;
            const int col = ks * 16 + c0 + (e >> 1) * 8;
            qa[ks][e] = (row < G) ? __ldcg(reinterpret_cast<const unsigned*>(qrow + (size_t)row * HD + col)) : 0u;
          }
        }
      }
      int stage = 0;
      for (; tile < tile_end; tile += ATT_WARPS) {
        const int ahead = tile + (STAGES - 1) * ATT_WARPS;
        int put = stage + STAGES - 1;
        if (put >= STAGES) put -= STAGES;
        if (ahead < tile_end) load_tile(ahead, put);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const __nv_bfloat16* kt = my + (size_t)(stage * 2) * TILE_ELEMS;
        const __nv_bfloat16* vt = kt + TILE_ELEMS;
        float sc[ATT_TILE / 8][4];
#pragma unroll
        for (int i = 0; i < ATT_TILE / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
        qk_tile<HD, ATT_TILE / 8>(sc, qa, kt, lane);
        const int key0 = lo + tile * ATT_TILE + 2 * (lane & 3);
#pragma unroll
        for (int nt = 0; nt < ATT_TILE / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + (e & 1);
            sc[nt][e] = (key < k_end) ? sc[nt][e] * p.scale_log2 : -INFINITY;
          }
        }
        softmax_step<HD, ATT_TILE / 8>(sc, m, l, o);
        pv_tile<HD, ATT_TILE / 8>(o, sc, vt, lane);
        __syncwarp();
        if (++stage == STAGES) stage = 0;
      }
      cp_async_wait<0>();
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      }
    }
    // merge the warps through shared memory (the tile buffers are free now); rows 0..7 only:
    // the groups this kernel takes have at most 8 query heads
    __syncthreads();
    float* red_o = reinterpret_cast<float*>(smem_raw);                  // [warps][8][HD]
    float* red_m = red_o + ATT_WARPS * 8 * HD;                          // [warps][8]
    float* red_l = red_m + ATT_WARPS * 8;
    if (warp < ATT_WARPS) {
      const int g0 = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < HD / 8; ++nt) {
        red_o[((size_t)warp * 8 + g0) * HD + nt * 8 + c0] = o[nt][0];
        red_o[((size_t)warp * 8 + g0) * HD + nt * 8 + c0 + 1] = o[nt][1];
      }
      if ((lane & 3) == 0) {
        red_m[warp * 8 + g0] = m[0];
        red_l[warp * 8 + g0] = l[0];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += DS_THREADS) {
      const int row = idx / HD, d = idx - row * HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, red_m[w * 8 + row]);
      const float m_use = (M == -INFINITY) ? 0.f : M;
      float Lsum = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float f = exp2f(red_m[w * 8 + row] - m_use);
        Lsum += red_l[w * 8 + row] * f;
        acc += red_o[((size_t)w * 8 + row) * HD + d] * f;
      }
      const int h = kvh * G + row;
      if (S == 1) {
        p.attn_out[((size_t)seq * p.nh + h) * HD + d] = __float2bfloat16_rn(acc / Lsum);
      } else {
        const size_t q = ((size_t)seq * p.nh + h) * S + split;
        p.part_o[q * HD + d] = acc;
        if (d == 0) {
          p.part_ml[q * 2] = M;
          p.part_ml[q * 2 + 1] = Lsum;
        }
      }
    }
    if (S > 1) {
      // the slice that ends last merges all slices of its (token, KV head), in slice order
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int ticket = atomicAdd(p.tickets + seq * p.nkv + kvh, 1);
        const int last = ticket == S - 1;
        if (last) p.tickets[seq * p.nkv + kvh] = 0;
        sh.flag = last;
      }
      __syncthreads();
      const bool last = sh.flag != 0;
      if (last) {
        __threadfence();
        for (int idx = threadIdx.x; idx < G * HD; idx += DS_THREADS) {
          const int row = idx / HD, d = idx - row * HD;
          const size_t q = ((size_t)seq * p.nh + kvh * G + row) * S;
          float M = -INFINITY;
          for (int sp = 0; sp < S; ++sp) M = fmaxf(M, __ldcg(p.part_ml + (q + sp) * 2));
          float Lsum = 0.f, acc = 0.f;
          for (int sp = 0; sp < S; ++sp) {
            const float f = exp2f(__ldcg(p.part_ml + (q + sp) * 2) - M);
            Lsum += __ldcg(p.part_ml + (q + sp) * 2 + 1) * f;
            acc += __ldcg(p.part_o + (q + sp) * HD + d) * f;
          }
          p.attn_out[((size_t)seq * p.nh + kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / Lsum);
        }
      }
    }
    __syncthreads();           // the tile buffers are reused by the block's next item
  }
  grid_arrive(p);
  return true;
}

// ------------------------------------------------------------------ the kernel
template <int HD>
__global__ void __launch_bounds__(DS_THREADS, 1)
decode_step_kernel(const DsParams p) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ Shared sh;
  unsigned arrivals = 0;
  bool first = true;
  for (int li = p.layer_begin; li < p.layer_end; ++li) {
    const DsLayer& L = p.layers[li];
    Gemv g = {};
    g.w = L.w_qkv; g.norm_w = L.norm_attn; g.eps = L.eps_attn; g.K = p.H; g.layer = li;
    g.n_units = (p.nh + 2 * p.nkv) * (p.hd >> 3); g.n_out = (p.nh + 2 * p.nkv) * p.hd;
    if (!gemv_phase<MODE_QKV, true>(p, g, sh, dyn, arrivals, !first)) return;
    first = false;
    if (!attention_phase<HD>(p, li, sh, dyn, arrivals)) return;
    g = Gemv{};
    g.w = L.w_o; g.x = p.attn_out; g.K = p.nh * p.hd; g.n_units = (p.H + 7) >> 3; g.n_out = p.H;
    if (!gemv_phase<MODE_RESIDUAL, false>(p, g, sh, dyn, arrivals, true)) return;
    g = Gemv{};
    g.w = L.w_gate_up; g.norm_w = L.norm_ffn; g.eps = L.eps_ffn; g.K = p.H;
    g.n_units = (p.I + 3) >> 2; g.n_out = p.I; g.glu_offset = p.I;
    if (!gemv_phase<MODE_GLU, true>(p, g, sh, dyn, arrivals, true)) return;
    g = Gemv{};
    g.w = L.w_down; g.x = p.hmid; g.K = p.I; g.n_units = (p.H + 7) >> 3; g.n_out = p.H;
    if (!gemv_phase<MODE_RESIDUAL, false>(p, g, sh, dyn, arrivals, true)) return;
  }
  if (p.run_head) {
    Gemv g = {};
    g.w = p.head_w; g.norm_w = p.final_norm; g.eps = p.final_eps; g.K = p.H;
    g.n_units = (p.V + 7) >> 3; g.n_out = p.V;
    if (!gemv_phase<MODE_LOGITS, true>(p, g, sh, dyn, arrivals, !first)) return;
  }
}

template <int HD>
size_t step_smem(int H) {
  constexpr int RS = HD + 8;
  constexpr int STAGES = HD <= 64 ? 4 : 2;
  const size_t tiles = (size_t)ATT_WARPS * STAGES * 2 * ATT_TILE * RS * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)(ATT_WARPS * 8 * HD + 2 * ATT_WARPS * 8) * sizeof(float);
  const size_t x = (size_t)MAX_T * x_row_bytes(H);
  size_t need = tiles > merge ? tiles : merge;
  return need > x ? need : x;
}

template <int HD>
int launch_step(const DsParams& p, cudaStream_t stream) {
  auto kernel = decode_step_kernel<HD>;
  const size_t smem = step_smem<HD>(p.H);
  if (smem > 200 * 1024) return HB_BAD_ARGUMENT;
  static int blocks_of[64] = {};          // per device: blocks of a launch (0: not set up yet)
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HB_LAUNCH_FAILED;
  if (blocks_of[dev] == 0) {
    int sms = 0, per_sm = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, DS_THREADS, 200 * 1024) != cudaSuccess ||
        sms <= 0 || per_sm < 1)
      return HB_LAUNCH_FAILED;
    blocks_of[dev] = sms;                 // one block per SM, all resident at once
  }
  void* args[] = {const_cast<DsParams*>(&p)};
  if (cudaLaunchCooperativeKernel((const void*)kernel, dim3(blocks_of[dev]), dim3(DS_THREADS), args, smem,
                                  stream) != cudaSuccess)
    return HB_LAUNCH_FAILED;
  return hb_check_launch();
}

}  // namespace

HB_EXPORT int hb_decode_step_layer_bytes() { return (int)sizeof(DsLayer); }
HB_EXPORT int hb_decode_step_param_bytes() { return (int)sizeof(DsParams); }

// Runs layers [layer_begin, layer_end) and, with run_head, the final norm and the output head
// for the step described by `params` (a DsParams, passed as bytes).  The barrier word and the
// tickets must be zero; the residual holds the embedded tokens (or what the layers before left).
HB_EXPORT int hb_decode_step(const void* params, cudaStream_t stream) {
  const DsParams& p = *reinterpret_cast<const DsParams*>(params);
  if (p.T < 1 || p.T > MAX_T || p.nkv < 1 || p.nh % p.nkv || p.nh / p.nkv > 8 || (p.H & 7) || (p.I & 7) ||
      ((p.nh * p.hd) & 7) || (p.hd & 7) || p.splits < 1 || p.page_size < 1 || p.layer_begin < 0 ||
      p.layer_end < p.layer_begin)
    return HB_BAD_ARGUMENT;
  switch (p.hd) {                       // head sizes in steps of 16
    case 16: return launch_step<16>(p, stream);
    case 32: return launch_step<32>(p, stream);
    case 48: return launch_step<48>(p, stream);
    case 64: return launch_step<64>(p, stream);
    case 80: return launch_step<80>(p, stream);
    case 96: return launch_step<96>(p, stream);
    case 112: return launch_step<112>(p, stream);
    case 128: return launch_step<128>(p, stream);
    default: return HB_BAD_ARGUMENT;
  }
}
