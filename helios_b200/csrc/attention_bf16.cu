// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// float32 accumulate), for head sizes 32, 64, 96 and 128.
//
//   * decode: one query token per request.  A block takes one (request, KV head,
//     slice of the context); the query heads that share the KV head are the rows
//     of one MMA tile, so every key and value is read once for the whole group.
//     Up to 8 slices run as one thread-block cluster and are merged through distributed
//     shared memory; more are merged by a second kernel (flash-decoding).  A block has 4
//     or 8 warps, each with key tiles of its own.  The kernel can take the
//     step's rotary position encoding and cache write with it: every block rotates its
//     query heads in registers, and the one warp whose tile holds the request's new
//     token rotates that key and puts it and the value into the cache first
//     (python/helios/exec/model.py:148-153, paged_attn.py:74-85), which saves a launch.
//   * prefill / mixed: tiles of query tokens of one request against the keys the
//     cache holds for it, causal by position (and a window), whatever mix of
//     prompt portions and single tokens the batch is.
//
// Math follows python/helios/exec/paged_attn.py:264-408 (scores = q.k * scale, mask,
// softmax in float32, times V); pages are [page, kv head, slot, head_dim] as in
// paged_attn.py:49.  Scores, the running maximum, the sum and the output
// accumulators are float32; probabilities are rounded to bfloat16 for the PV
// product, as the reference casts them to the value dtype (paged_attn.py:293).
#include <type_traits>
#include "common.cuh"
#include "attention_mma.cuh"

namespace {

// ------------------------------------------------------------------------ decode
// (warps per decode block, a template parameter: 4, two blocks an SM, or 8, one block an SM,
// where so few blocks run that each warp's chain of key tiles, not the memory, bounds the kernel)
constexpr int DEC_TILE = 16;      // keys per warp tile
constexpr int DEC_STAGES = 3;     // tiles a warp keeps in shared memory (all but one in flight)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The online-softmax step of the decode kernel over a tile's scaled, masked scores (log2
// domain).  Without WIDE only the first eight rows of the MMA tile are query heads: the
// second row group (rows 8-15, zero queries) is left out and its probabilities are zero.
// The output and the sum are rescaled only in tiles where some row's maximum grew (a
// warp-wide vote; otherwise every factor would be exactly 1).
template <int HD, int NT, bool WIDE>
__device__ __forceinline__ void decode_softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2],
                                                    float (&o)[HD / 8][4]) {
  constexpr int R = WIDE ? 2 : 1;
  float m_new[2] = {m[0], m[1]};
  bool grew = false;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    m_new[r] = fmaxf(m[r], mx);
    grew = grew || m_new[r] > m[r];
  }
  if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float corr = fast_exp2(m[r] - ((m_new[r] == -INFINITY) ? 0.f : m_new[r]));
      l[r] *= corr;
#pragma unroll
      for (int nt = 0; nt < HD / 8; ++nt) {
        o[nt][2 * r] *= corr;
        o[nt][2 * r + 1] *= corr;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = m_new[r];
    const float m_use = (m_new[r] == -INFINITY) ? 0.f : m_new[r];
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][2 * r] = fast_exp2(s[nt][2 * r] - m_use);
      s[nt][2 * r + 1] = fast_exp2(s[nt][2 * r + 1] - m_use);
      sum += s[nt][2 * r] + s[nt][2 * r + 1];
    }
    l[r] += sum;
  }
  if (!WIDE) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) s[nt][2] = s[nt][3] = 0.f;
  }
}

template <int HD, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
decode_attention_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, const __nv_bfloat16* __restrict__ q,
                        int q_stride, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages,
                        const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ positions, int nh, int nkv, int page_size,
                        int window, float scale_log2, int n_splits, int cluster_merge,
                        const float* __restrict__ rot_cos, const float* __restrict__ rot_sin,
                        __nv_bfloat16* k_write, __nv_bfloat16* v_write) {
  // rot_cos / rot_sin [requests, HD / 2]: q (and the new key) still lack their rotation.
  // k_write / v_write (the cache again, writable): the new token's key and value are still
  // in the q|k|v row and go into the cache here.
  pdl_launch_dependents();
  constexpr int RS = HD + 8;
  constexpr int TILE_ELEMS = DEC_TILE * RS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = nh / nkv;
  const int pos = positions[seq];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // Tiles start at a multiple of the tile size where pages hold whole tiles: then every tile's
  // keys are consecutive slots of ONE page.  Keys of the first tile from before the window
  // are zero-filled and masked.
  const bool whole_pages = page_size % DEC_TILE == 0;
  const int first = whole_pages ? lo - lo % DEC_TILE : lo;
  const int n_keys = pos - first + 1;
  // slices of whole tiles
  const int tiles_total = (n_keys + DEC_TILE - 1) / DEC_TILE;
  const int tiles_per_split = (tiles_total + n_splits - 1) / n_splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + tiles_per_split);
  const int k_end = pos + 1;
  const int* table = block_table + (size_t)seq * bt_stride;

  __nv_bfloat16* my = smem + (size_t)warp * DEC_STAGES * 2 * TILE_ELEMS;   // [stage][k|v][tile]
  // A tile is DEC_TILE rows of HD/8 16-byte chunks; consecutive lanes copy consecutive
  // chunks, so a warp instruction reads 512 contiguous bytes.  Where the tile's keys are
  // consecutive slots of ONE page (page_size a multiple of the tile) the whole tile is one
  // contiguous stretch of the cache: one look-up in the block table and one address per
  // warp.  Otherwise lane r first finds the cache row of key r.
  auto load_tile = [&](int tile, int stage) {
    constexpr int CH = HD / 8;
    __nv_bfloat16* kd = my + (size_t)(stage * 2) * TILE_ELEMS;
    __nv_bfloat16* vd = kd + TILE_ELEMS;
    if (whole_pages) {
      const int key_first = first + tile * DEC_TILE;
      const int page = table[key_first / page_size];
      const size_t base = ((size_t)(page * nkv + kvh) * page_size + key_first % page_size) * HD + lane * 8;
      const int rows_valid = k_end - key_first;            // >= 1; rows from there on are zero-filled,
      const int rows_skipped = lo - key_first;             // and so are rows before the window
#pragma unroll
      for (int it = 0; it < DEC_TILE * CH / 32; ++it) {
        const int idx = it * 32 + lane;
        const int row = idx / CH, c = idx - row * CH;
        const int bytes = (row < rows_valid && row >= rows_skipped) ? 16 : 0;
        cp_async16(kd + row * RS + c * 8, k_pages + base + it * 256, bytes);
        cp_async16(vd + row * RS + c * 8, v_pages + base + it * 256, bytes);
      }
      return;
    }
    int row_id = -1;
    if (lane < DEC_TILE) {
      const int key = first + tile * DEC_TILE + lane;
      if (key < k_end) {
        const int page = table[key / page_size];
        row_id = (page * nkv + kvh) * page_size + key % page_size;
      }
    }
#pragma unroll
    for (int it = 0; it < DEC_TILE * CH / 32; ++it) {
      const int idx = it * 32 + lane;
      const int row = idx / CH, c = idx - row * CH;
      const int rid = __shfl_sync(0xffffffffu, row_id, row);
      const size_t base = (size_t)(rid < 0 ? 0 : rid) * HD + c * 8;
      const int bytes = rid < 0 ? 0 : 16;
      cp_async16(kd + row * RS + c * 8, k_pages + base, bytes);
      cp_async16(vd + row * RS + c * 8, v_pages + base, bytes);
    }
  };

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // prologue: DEC_STAGES - 1 tiles in flight.  Keys of earlier steps do not depend on the
  // kernel before this one (the block tables and positions were copied before the step's
  // first kernel): their tiles are fetched while that kernel still runs.  The tile with
  // the token's own key, which that kernel writes, and the query follow after the wait.
  int tile = tile_begin + warp;
  bool early[DEC_STAGES - 1];
#pragma unroll
  for (int p = 0; p < DEC_STAGES - 1; ++p) {
    const int tp = tile + p * WARPS;
    early[p] = tp < tile_end && tp < tiles_total - 1;
    if (early[p]) load_tile(tp, p);
  }
  pdl_wait();
  {
    // the warp whose tile holds the request's own token (the last tile) writes its key and
    // value before it fetches that tile
    const int last_tile = tiles_total - 1;
    if (k_write != nullptr && last_tile >= tile_begin && last_tile < tile_end &&
        (last_tile - tile_begin) % WARPS == warp) {
      const int page = table[pos / page_size];
      const size_t dst = ((size_t)(page * nkv + kvh) * page_size + pos % page_size) * HD;
      const __nv_bfloat16* k_new = q + (size_t)seq * q_stride + (size_t)(nh + kvh) * HD;
      const __nv_bfloat16* v_new = k_new + (size_t)nkv * HD;
      for (int j = 2 * lane; j < HD / 2; j += 64) {
        const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(k_new + j));
        const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(k_new + j + HD / 2));
        float2 r1 = x1, r2 = x2;
        if (rot_cos != nullptr) {
          const float2 c = *reinterpret_cast<const float2*>(rot_cos + (size_t)seq * (HD / 2) + j);
          const float2 sn = *reinterpret_cast<const float2*>(rot_sin + (size_t)seq * (HD / 2) + j);
          r1 = make_float2(x1.x * c.x - x2.x * sn.x, x1.y * c.y - x2.y * sn.y);
          r2 = make_float2(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y);
        }
        *reinterpret_cast<__nv_bfloat162*>(k_write + dst + j) = __floats2bfloat162_rn(r1.x, r1.y);
        *reinterpret_cast<__nv_bfloat162*>(k_write + dst + j + HD / 2) = __floats2bfloat162_rn(r2.x, r2.y);
      }
      for (int j = 8 * lane; j < HD; j += 256)
        *reinterpret_cast<uint4*>(v_write + dst + j) = *reinterpret_cast<const uint4*>(v_new + j);
      __syncwarp();           // the copies below, by other lanes, read these rows
    }
  }
#pragma unroll
  for (int p = 0; p < DEC_STAGES - 1; ++p) {
    const int tp = tile + p * WARPS;
    if (tp < tile_end && !early[p]) load_tile(tp, p);
    cp_async_commit();
  }

  // query fragments: rows = the group's heads (zero beyond G)
  uint32_t qa[HD / 16][4];
  {
    const int g0 = lane >> 2, c0 = 2 * (lane & 3);
    const __nv_bfloat16* qrow = q + (size_t)seq * q_stride + (size_t)kvh * G * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = g0 + (e & 1) * 8;
        const int col = ks * 16 + c0 + (e >> 1) * 8;
        qa[ks][e] = (row < G) ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)row * HD + col) : 0u;
      }
    }
    if (rot_cos != nullptr) {
      // rotate-half pairs (j, j + HD / 2): both values of a pair are in this thread's fragments
      const float* cs = rot_cos + (size_t)seq * (HD / 2);
      const float* sn = rot_sin + (size_t)seq * (HD / 2);
#pragma unroll
      for (int ks = 0; ks < HD / 32; ++ks) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = ks * 16 + c0 + (e >> 1) * 8;
          const float2 c = *reinterpret_cast<const float2*>(cs + col);
          const float2 sv = *reinterpret_cast<const float2*>(sn + col);
          const float2 x1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qa[ks][e]));
          const float2 x2 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qa[ks + HD / 32][e]));
          __nv_bfloat162 r1 = __floats2bfloat162_rn(x1.x * c.x - x2.x * sv.x, x1.y * c.y - x2.y * sv.y);
          __nv_bfloat162 r2 = __floats2bfloat162_rn(x2.x * c.x + x1.x * sv.x, x2.y * c.y + x1.y * sv.y);
          qa[ks][e] = *reinterpret_cast<uint32_t*>(&r1);
          qa[ks + HD / 32][e] = *reinterpret_cast<uint32_t*>(&r2);
        }
      }
    }
  }

  // the key tiles of this warp; `wide` (a compile-time tag): more than eight query heads
  // share the KV head, so both row groups of the MMA tile are live
  auto run = [&](auto wide) {
    constexpr bool WIDE = decltype(wide)::value;
    int stage = 0;
    for (; tile < tile_end; tile += WARPS) {
      const int ahead = tile + (DEC_STAGES - 1) * WARPS;
      int put = stage + DEC_STAGES - 1;
      if (put >= DEC_STAGES) put -= DEC_STAGES;
      if (ahead < tile_end) load_tile(ahead, put);
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();
      __syncwarp();
      const __nv_bfloat16* kt = my + (size_t)(stage * 2) * TILE_ELEMS;
      const __nv_bfloat16* vt = kt + TILE_ELEMS;
      float s[DEC_TILE / 8][4];
#pragma unroll
      for (int i = 0; i < DEC_TILE / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      qk_tile<HD, DEC_TILE / 8>(s, qa, kt, lane);
      const int tile_key0 = first + tile * DEC_TILE;
      if (tile_key0 + DEC_TILE > k_end || tile_key0 < lo) {
        // the last tile (keys beyond the token's own) or the first (keys before the window)
        const int key0 = tile_key0 + 2 * (lane & 3);
#pragma unroll
        for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + (e & 1);
            s[nt][e] = (key < k_end && key >= lo) ? s[nt][e] * scale_log2 : -INFINITY;
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < (WIDE ? 4 : 2); ++e) s[nt][e] *= scale_log2;
        }
      }
      decode_softmax_step<HD, DEC_TILE / 8, WIDE>(s, m, l, o);
      pv_tile<HD, DEC_TILE / 8>(o, s, vt, lane);
      __syncwarp();
      if (++stage == DEC_STAGES) stage = 0;
    }
  };
  if (G > 8) run(std::true_type()); else run(std::false_type());
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }

  // merge the block's warps through shared memory (reusing the tile buffers)
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(smem_raw);                 // [warps][16][HD]
  float* red_m = red_o + WARPS * 16 * HD;                        // [warps][16]
  float* red_l = red_m + WARPS * 16;
  float* cta_o = red_l + WARPS * 16;                             // [16][HD] this block's merged partial
  float* cta_ml = cta_o + 16 * HD;                                   // [16][2]
  {
    const int g0 = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = g0 + (e >> 1) * 8, col = nt * 8 + c0 + (e & 1);
        red_o[((size_t)warp * 16 + row) * HD + col] = o[nt][e];
      }
    }
    if ((lane & 3) == 0) {
      red_m[warp * 16 + g0] = m[0];
      red_m[warp * 16 + g0 + 8] = m[1];
      red_l[warp * 16 + g0] = l[0];
      red_l[warp * 16 + g0 + 8] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += WARPS * 32) {
    const int row = idx / HD, d = idx - row * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, red_m[w * 16 + row]);
    const float m_use = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = exp2f(red_m[w * 16 + row] - m_use);
      L += red_l[w * 16 + row] * f;
      acc += red_o[((size_t)w * 16 + row) * HD + d] * f;
    }
    const int h = kvh * G + row;
    if (n_splits == 1) {
      out[((size_t)seq * nh + h) * HD + d] = __float2bfloat16_rn(acc / L);
    } else if (cluster_merge) {
      // the slices of this (request, KV head) are one thread-block cluster: park the block's
      // partial result in its own shared memory for the merge below
      cta_o[idx] = acc;
      if (d == 0) {
        cta_ml[2 * row] = M;
        cta_ml[2 * row + 1] = L;
      }
    } else {
      const size_t p = ((size_t)seq * nh + h) * n_splits + split;
      part_o[p * HD + d] = acc;
      if (d == 0) {
        part_ml[p * 2] = M;
        part_ml[p * 2 + 1] = L;
      }
    }
  }
  if (n_splits > 1 && cluster_merge) {
    // every block merges its share of the G x HD outputs, reading all slices' partial
    // results (in slice order) from its peers' shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    const uint32_t o_addr = (uint32_t)__cvta_generic_to_shared(cta_o);
    const uint32_t ml_addr = (uint32_t)__cvta_generic_to_shared(cta_ml);
    auto peer = [](uint32_t addr, uint32_t rank) {
      uint32_t remote;
      float v;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
      return v;
    };
    const int total = G * HD;
    const int per = (total + n_splits - 1) / n_splits;
    const int e_end = min(total, (split + 1) * per);
    for (int idx = split * per + threadIdx.x; idx < e_end; idx += WARPS * 32) {
      const int row = idx / HD, d = idx - row * HD;
      float ms[8], ls[8], os[8];
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        const bool on = sp < n_splits;
        ms[sp] = on ? peer(ml_addr + (uint32_t)(2 * row) * 4u, sp) : -INFINITY;
        ls[sp] = on ? peer(ml_addr + (uint32_t)(2 * row + 1) * 4u, sp) : 0.f;
        os[sp] = on ? peer(o_addr + (uint32_t)idx * 4u, sp) : 0.f;
      }
      float M = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) M = fmaxf(M, ms[sp]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        const float f = exp2f(ms[sp] - M);
        L += ls[sp] * f;
        acc += os[sp] * f;
      }
      out[((size_t)seq * nh + kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / L);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
}

template <int HD>
__global__ void decode_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;   // seq * nh + head
  const float* ml = part_ml + row * n_splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += ml[2 * s + 1] * exp2f(ml[2 * s] - M);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      acc += part_o[(row * n_splits + s) * HD + d] * exp2f(ml[2 * s] - M);
    out[row * HD + d] = __float2bfloat16_rn(acc / L);
  }
}

// ------------------------------------------------------------------------ prefill / mixed
constexpr int PRE_WARPS = 8;
constexpr int PRE_TILE = 64;   // keys per block tile

template <int HD>
__global__ void __launch_bounds__(PRE_WARPS * 32)
prefill_attention_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                         int q_stride, const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ q_tiles, const int* __restrict__ cu_tokens,
                         const int* __restrict__ start_pos, int nh, int nkv, int heads_per_block,
                         int token_subtiles, int page_size, int window, float scale_log2) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int RS = HD + 8;
  constexpr int TILE_ELEMS = PRE_TILE * RS;
  constexpr int CHUNKS = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [stage][k|v][tile]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = nh / nkv;
  const int head_blocks = (G + heads_per_block - 1) / heads_per_block;
  const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y - kvh * head_blocks;
  const int seq = q_tiles[2 * blockIdx.x], t0 = q_tiles[2 * blockIdx.x + 1];
  const int tok0 = cu_tokens[seq], n_tok = cu_tokens[seq + 1] - tok0;
  if (t0 >= n_tok) return;      // padding of a captured step's tile list
  const int sp = start_pos[seq];
  const int BQ = 16 * token_subtiles;
  const int p_first = sp + t0;
  const int p_last = sp + min(n_tok, t0 + BQ) - 1;
  const int k_min = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int* table = block_table + (size_t)seq * bt_stride;

  const int head_local = warp % heads_per_block, sub = warp / heads_per_block;
  const int g_in_kv = hb * heads_per_block + head_local;
  const bool active = sub < token_subtiles && g_in_kv < G && (t0 + sub * 16) < n_tok;
  const int h = kvh * G + g_in_kv;
  const int g0 = lane >> 2, c0 = 2 * (lane & 3);
  // the two rows of this thread: local tokens and their positions
  const int tl0 = t0 + sub * 16 + g0, tl1 = tl0 + 8;
  const int pr0 = sp + tl0, pr1 = sp + tl1;

  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tl = (e & 1) ? tl1 : tl0;
      const int col = ks * 16 + c0 + (e >> 1) * 8;
      qa[ks][e] = (active && tl < n_tok)
          ? *reinterpret_cast<const uint32_t*>(q + (size_t)(tok0 + tl) * q_stride + (size_t)h * HD + col)
          : 0u;
    }
  }

  auto load_tile = [&](int kt, int stage) {
    __nv_bfloat16* kd = smem + (size_t)(stage * 2) * TILE_ELEMS;
    __nv_bfloat16* vd = kd + TILE_ELEMS;
    for (int idx = threadIdx.x; idx < PRE_TILE * CHUNKS; idx += PRE_WARPS * 32) {
      const int row = idx / CHUNKS, c = idx - row * CHUNKS;
      const int key = kt * PRE_TILE + row;
      const bool valid = key >= k_min && key <= p_last;
      size_t base = 0;
      if (valid) {
        const int page = table[key / page_size];
        base = (((size_t)page * nkv + kvh) * page_size + key % page_size) * HD + c * 8;
      }
      const int bytes = valid ? 16 : 0;
      cp_async16(kd + row * RS + c * 8, k_pages + base, bytes);
      cp_async16(vd + row * RS + c * 8, v_pages + base, bytes);
    }
  };

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int kt_begin = k_min / PRE_TILE, kt_end = p_last / PRE_TILE + 1;
  // the key range this warp's 16 rows can see
  const int w_pmin = sp + t0 + sub * 16, w_pmax = min(w_pmin + 15, p_last);
  const int w_kmin = (window > 0 && w_pmin - window + 1 > 0) ? w_pmin - window + 1 : 0;

  load_tile(kt_begin, 0);
  cp_async_commit();
  int stage = 0;
  for (int kt = kt_begin; kt < kt_end; ++kt, stage ^= 1) {
    if (kt + 1 < kt_end) load_tile(kt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int key_base = kt * PRE_TILE;
    if (active && key_base <= w_pmax && key_base + PRE_TILE - 1 >= w_kmin) {
      const __nv_bfloat16* ktile = smem + (size_t)(stage * 2) * TILE_ELEMS;
      const __nv_bfloat16* vtile = ktile + TILE_ELEMS;
      float s[PRE_TILE / 8][4];
#pragma unroll
      for (int i = 0; i < PRE_TILE / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      qk_tile<HD, PRE_TILE / 8>(s, qa, ktile, lane);
#pragma unroll
      for (int nt = 0; nt < PRE_TILE / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_base + nt * 8 + c0 + (e & 1);
          const int pr = (e >> 1) ? pr1 : pr0;
          const bool ok = key <= pr && (window <= 0 || key > pr - window);
          s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
        }
      }
      softmax_step<HD, PRE_TILE / 8>(s, m, l, o);
      pv_tile<HD, PRE_TILE / 8>(o, s, vtile, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (!active) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int tl = r ? tl1 : tl0;
    if (tl >= n_tok) continue;
    const float inv = 1.f / l[r];
    __nv_bfloat16* orow = out + ((size_t)(tok0 + tl) * nh + h) * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      *reinterpret_cast<uint32_t*>(orow + nt * 8 + c0) =
          pack_bf16(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    }
  }
}

template <int HD, int WARPS>
int launch_decode(void* out, float* part_o, float* part_ml, const void* q, int q_stride,
                  const void* k_pages, const void* v_pages, const int* block_table, int bt_stride,
                  const int* positions, int S, int nh, int nkv, int page_size, int window,
                  float scale, int n_splits, const float* rot_cos, const float* rot_sin,
                  int write_cache, cudaStream_t stream) {
  constexpr int RS = HD + 8;
  // the new keys and values go into the very pages the kernel reads
  __nv_bfloat16* k_write = write_cache ? (__nv_bfloat16*)const_cast<void*>(k_pages) : nullptr;
  __nv_bfloat16* v_write = write_cache ? (__nv_bfloat16*)const_cast<void*>(v_pages) : nullptr;
  size_t smem = (size_t)WARPS * DEC_STAGES * 2 * DEC_TILE * RS * sizeof(__nv_bfloat16);
  const size_t red = (size_t)(WARPS * 16 * (HD + 2) + 16 * (HD + 2)) * sizeof(float);
  if (red > smem) smem = red;
  auto kernel = decode_attention_kernel<HD, WARPS>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured = true;
  }
  dim3 grid(n_splits, nkv, S);
  const int cluster_merge = (n_splits > 1 && n_splits <= 8 && part_o == nullptr) ? 1 : 0;
  if (cluster_merge) {
    // the slices of one (request, KV head) as a cluster: merged through distributed shared memory
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = n_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = hb_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, q_stride,
                       (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, bt_stride,
                       positions, nh, nkv, page_size, window, scale * LOG2E, n_splits, 1,
                       rot_cos, rot_sin, k_write, v_write);
    return hb_check_launch();
  }
  hb_launch(kernel, dim3(grid), dim3(WARPS * 32), smem, stream, 
      (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, q_stride,
      (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, bt_stride,
      positions, nh, nkv, page_size, window, scale * LOG2E, n_splits, 0,
      rot_cos, rot_sin, k_write, v_write);
  if (n_splits > 1)
    hb_launch(decode_merge_kernel<HD>, dim3(S * nh), dim3(HD < 128 ? HD : 128), 0, stream, 
        (__nv_bfloat16*)out, part_o, part_ml, n_splits);
  return hb_check_launch();
}

// Clusters of `cluster_size` decode blocks the device keeps resident at once (-1 if the
// query fails): whole clusters are placed inside a GPC, so this can be fewer than the blocks
// that would fit one by one.
template <int HD, int WARPS>
int decode_max_clusters(int cluster_size) {
  constexpr int RS = HD + 8;
  size_t smem = (size_t)WARPS * DEC_STAGES * 2 * DEC_TILE * RS * sizeof(__nv_bfloat16);
  const size_t red = (size_t)(WARPS * 16 * (HD + 2) + 16 * (HD + 2)) * sizeof(float);
  if (red > smem) smem = red;
  auto kernel = decode_attention_kernel<HD, WARPS>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster_size, 1, 1);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) return -1;
  return n;
}

template <int HD>
int launch_prefill(void* out, const void* q, int q_stride, const void* k_pages, const void* v_pages,
                   const int* block_table, int bt_stride, const int* q_tiles, int n_tiles,
                   const int* cu_tokens, const int* start_pos, int nh, int nkv, int heads_per_block,
                   int token_subtiles, int page_size, int window, float scale, cudaStream_t stream) {
  constexpr int RS = HD + 8;
  const size_t smem = (size_t)4 * PRE_TILE * RS * sizeof(__nv_bfloat16);
  auto kernel = prefill_attention_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    configured = true;
  }
  const int G = nh / nkv;
  const int head_blocks = (G + heads_per_block - 1) / heads_per_block;
  dim3 grid(n_tiles, nkv * head_blocks);
  hb_launch(kernel, dim3(grid), dim3(PRE_WARPS * 32), smem, stream, 
      (__nv_bfloat16*)out, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages,
      (const __nv_bfloat16*)v_pages, block_table, bt_stride, q_tiles, cu_tokens, start_pos, nh, nkv,
      heads_per_block, token_subtiles, page_size, window, scale * LOG2E);
  return hb_check_launch();
}

}  // namespace

#define HB_DISPATCH_HD(hd, ...)                         \
  switch (hd) {                                         \
    case 32: { constexpr int HD = 32; __VA_ARGS__; }    \
    case 64: { constexpr int HD = 64; __VA_ARGS__; }    \
    case 96: { constexpr int HD = 96; __VA_ARGS__; }    \
    case 128: { constexpr int HD = 128; __VA_ARGS__; }  \
    default: return HB_BAD_ARGUMENT;                    \
  }

// Decode: S requests, one token each (token i belongs to request i).  Needs the group
// size nh / nkv <= 16.  part_o: float [S, nh, n_splits, hd], part_ml: float
// [S, nh, n_splits, 2]; both unused when n_splits == 1.  With 2..8 slices and part_o null
// the slices run as one thread-block cluster and are merged through distributed shared
// memory instead of a second kernel.
//   q is a row of q|k|v per request ([nh + 2 nkv] heads, q_stride elements apart).  With
//   rot_cos / rot_sin (float [S, hd / 2]) the query heads are rotated on the way in (rotate-half
//   pairs (j, j + hd / 2)); with write_cache the request's key (rotated likewise) and value are
//   taken from that row and stored at its position in the pages before the kernel attends.
//   Without either, q must be rotated and the cache written already.
HB_EXPORT int hb_attention_decode_bf16(void* out, float* part_o, float* part_ml, const void* q,
                                       int q_stride, const void* k_pages, const void* v_pages,
                                       const int* block_table, int bt_stride, const int* positions,
                                       int S, int nh, int nkv, int hd, int page_size, int window,
                                       float scale, int n_splits, const float* rot_cos,
                                       const float* rot_sin, int write_cache, int warps,
                                       cudaStream_t stream) {
  if (S <= 0) return HB_OK;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || page_size <= 0 || n_splits < 1 ||
      (warps != 4 && warps != 8))
    return HB_BAD_ARGUMENT;
  if ((rot_cos == nullptr) != (rot_sin == nullptr)) return HB_BAD_ARGUMENT;
  if (write_cache && (q_stride < (nh + 2 * nkv) * hd || (q_stride & 7) || ((uintptr_t)q & 15)))
    return HB_BAD_ARGUMENT;
#define HB_DECODE(W)                                                                              \
  HB_DISPATCH_HD(hd, return (launch_decode<HD, W>(out, part_o, part_ml, q, q_stride, k_pages, v_pages, \
                                                  block_table, bt_stride, positions, S, nh, nkv,      \
                                                  page_size, window, scale, n_splits, rot_cos,        \
                                                  rot_sin, write_cache, stream)))
  if (warps == 8) HB_DECODE(8);
  HB_DECODE(4);
#undef HB_DECODE
}

HB_EXPORT int hb_attention_decode_max_clusters(int hd, int cluster_size, int warps) {
  if (cluster_size < 1 || cluster_size > 8 || (warps != 4 && warps != 8)) return -1;
  if (warps == 8) HB_DISPATCH_HD(hd, return (decode_max_clusters<HD, 8>(cluster_size)));
  HB_DISPATCH_HD(hd, return (decode_max_clusters<HD, 4>(cluster_size)));
}

// Prefill / mixed: q_tiles holds (request, first local token) for every tile of
// 16 * token_subtiles query tokens; heads_per_block * token_subtiles <= 8.
HB_EXPORT int hb_attention_prefill_bf16(void* out, const void* q, int q_stride, const void* k_pages,
                                        const void* v_pages, const int* block_table, int bt_stride,
                                        const int* q_tiles, int n_tiles, const int* cu_tokens,
                                        const int* start_pos, int nh, int nkv, int hd,
                                        int heads_per_block, int token_subtiles, int page_size,
                                        int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return HB_OK;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0 || heads_per_block < 1 || token_subtiles < 1 ||
      heads_per_block * token_subtiles > PRE_WARPS)
    return HB_BAD_ARGUMENT;
  HB_DISPATCH_HD(hd, return launch_prefill<HD>(out, q, q_stride, k_pages, v_pages, block_table,
                                               bt_stride, q_tiles, n_tiles, cu_tokens, start_pos,
                                               nh, nkv, heads_per_block, token_subtiles, page_size,
                                               window, scale, stream));
}
