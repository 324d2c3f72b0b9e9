// Tiles of attention on mma.sync.m16n8k16 (bfloat16 operands, float32 accumulators), shared
// by the attention kernels that read keys and values from padded rows in shared memory:
// S += Q K^T, the online-softmax step, O += P V, and the 16-byte asynchronous copy.
// Math of python/helios/exec/paged_attn.py:264-295 (scores, float32 softmax, times V).
#pragma once
#include "common.cuh"

namespace {

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One query row group (16 rows) against a tile of NT*8 keys held in shared memory
// (rows of HD + 8 bfloat16): S += Q K^T.
template <int HD, int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qa)[HD / 16][4],
                                        const __nv_bfloat16* k_tile, int lane) {
  constexpr int RS = HD + 8;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t r[4];
      const int row = 16 * np + (lane >> 4) * 8 + (lane & 7);
      const int col = ks * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(r, k_tile + row * RS + col);
      mma_bf16(s[2 * np], qa[ks], r[0], r[1]);
      mma_bf16(s[2 * np + 1], qa[ks], r[2], r[3]);
    }
  }
}

// O += P V for the same tile; P comes from the score fragments.
template <int HD, int NT>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const float (&p)[NT][4],
                                        const __nv_bfloat16* v_tile, int lane) {
  constexpr int RS = HD + 8;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t pa[4];
    pa[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    pa[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    pa[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    pa[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t r[4];
      const int row = 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int col = 16 * dp + (lane >> 4) * 8;
      ldmatrix_x4_trans(r, v_tile + row * RS + col);
      mma_bf16(o[2 * dp], pa, r[0], r[1]);
      mma_bf16(o[2 * dp + 1], pa, r[2], r[3]);
    }
  }
}

// Online softmax step over the masked scores of a tile (log2 domain).
template <int HD, int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2],
                                             float (&o)[HD / 8][4]) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
    mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float corr = exp2f(m[r] - m_use);
    m[r] = m_new;
    l[r] *= corr;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      o[nt][2 * r] *= corr;
      o[nt][2 * r + 1] *= corr;
    }
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][2 * r] = exp2f(s[nt][2 * r] - m_use);
      s[nt][2 * r + 1] = exp2f(s[nt][2 * r + 1] - m_use);
      sum += s[nt][2 * r] + s[nt][2 * r + 1];
    }
    l[r] += sum;
  }
}

}  // namespace
