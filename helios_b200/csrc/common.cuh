// Shared device helpers for the helios_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define HB_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes returned by every launcher.
enum {
  HB_OK = 0,
  HB_BAD_ARGUMENT = 1,      // a size this kernel does not take
  HB_LAUNCH_FAILED = 2,     // cudaGetLastError() after the launch
};

// Element types by code, as the Python side passes them.
enum { HB_F32 = 0, HB_BF16 = 1 };

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block in a fixed order (warp tree, then warps 0..n-1 in turn), so
// the result for a row never depends on what else is in the launch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += scratch[w];
    scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch: a kernel lets the next kernel of the stream start while it
// still runs (launch_dependents) and itself waits for the kernel before it to finish, with
// its writes visible, before touching anything that kernel may have written (wait).  What a
// kernel does before its wait (set-up, fetching weights) overlaps the tail of its
// predecessor.  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <cstdlib>
static inline bool hb_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = std::getenv("HELIOS_B200_NO_PDL");
    on = (e != nullptr && e[0] == '1') ? 0 : 1;
  }
  return on == 1;
}

// Launch with the programmatic-stream-serialization attribute (plain launch when disabled).
template <typename... KArgs, typename... Args>
static inline void hb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hb_pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int hb_check_launch() {
  return cudaGetLastError() == cudaSuccess ? HB_OK : HB_LAUNCH_FAILED;
}

#define HB_DISPATCH_DTYPE(code, T, ...)                         \
  do {                                                          \
    if ((code) == HB_F32) { using T = float; __VA_ARGS__; }     \
    else if ((code) == HB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return HB_BAD_ARGUMENT;                                \
  } while (0)
