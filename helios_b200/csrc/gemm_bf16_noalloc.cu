// The allocation-free variant of the decode matrix product: same kernel as
// gemm_bf16.cu (included below without its exported launchers), scratch in a
// static device array.  Contract and limits: gemm_bf16_noalloc.h.
#define HB_GEMM_BF16_NO_EXPORTS
#include "gemm_bf16.cu"

#include <cstdio>
#include <cstring>

#include "gemm_bf16_noalloc.h"

namespace {

// layout of the scratch area: [0, 4) error word; [256, 256 + 4 * MAX_TILES) tickets;
// from PARTIALS_OFFSET on, float partial sums
constexpr size_t TICKETS_OFFSET = 256;
constexpr size_t PARTIALS_OFFSET = 8192;
static_assert(TICKETS_OFFSET + 4 * HB_GEMM_NOALLOC_MAX_TILES <= PARTIALS_OFFSET, "tickets overlap the sums");
constexpr size_t PARTIAL_FLOATS = (HB_GEMM_NOALLOC_SCRATCH_BYTES - PARTIALS_OFFSET) / sizeof(float);

// In host code this name is only a handle for cudaGetSymbolAddress: it is NOT the
// device address, and passing it to a kernel would make the kernel fault (or, where the
// GPU can reach host memory, scribble over the wrong bytes).
static __device__ __align__(256) unsigned char g_noalloc_scratch[HB_GEMM_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = HB_MAX_DEVICES;
// device address of the array, per device.  Written without a lock: two host threads that
// make the first call on a device at once would both look the same address up.
unsigned char* g_scratch_ptr[MAX_DEVICES] = {};

int fail(int code, char* err, int err_len, const char* fmt, long long a = 0, long long b = 0) {
  if (err != nullptr && err_len > 0) std::snprintf(err, (size_t)err_len, fmt, a, b);
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int hb_gemm_bf16_noalloc(void* out, const void* x, const void* w, int T, int N, int K, int k_splits,
                         cudaStream_t stream, char* err, int err_len) {
  if (err != nullptr && err_len > 0) err[0] = '\0';
  if (out == nullptr || x == nullptr || w == nullptr)
    return fail(HB_NOALLOC_BAD_ARGUMENT, err, err_len, "hb_gemm_bf16_noalloc: out, x and w must not be null");
  if (T < 1 || N < 1 || K < 1)
    return fail(HB_NOALLOC_BAD_ARGUMENT, err, err_len, "hb_gemm_bf16_noalloc: T, N and K must be positive");
  if (T > HB_GEMM_NOALLOC_MAX_TOKENS)
    return fail(HB_NOALLOC_TOO_LARGE, err, err_len,
                "hb_gemm_bf16_noalloc: T = %lld exceeds the maximum of %lld tokens", T,
                HB_GEMM_NOALLOC_MAX_TOKENS);
  if ((K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return fail(HB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "hb_gemm_bf16_noalloc: K = %lld must be a multiple of 8 and x, w 16-byte aligned", K);
  if (k_splits < 1 || k_splits > (K + BK - 1) / BK)
    return fail(HB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "hb_gemm_bf16_noalloc: k_splits = %lld must lie in 1..ceil(K / 64) = %lld", k_splits,
                (K + BK - 1) / BK);
  const long long tiles = (N + BM - 1) / BM;
  const long long floats = k_splits > 1 ? tiles * k_splits * (long long)BM * 16 : 0;
  if (k_splits > 1 && tiles > HB_GEMM_NOALLOC_MAX_TILES)
    return fail(HB_NOALLOC_TOO_LARGE, err, err_len,
                "hb_gemm_bf16_noalloc: %lld output tiles exceed the maximum of %lld", tiles,
                HB_GEMM_NOALLOC_MAX_TILES);
  if (floats > (long long)PARTIAL_FLOATS)
    return fail(HB_NOALLOC_TOO_LARGE, err, err_len,
                "hb_gemm_bf16_noalloc: the split needs %lld scratch floats, the static area holds %lld",
                floats, (long long)PARTIAL_FLOATS);

  // ---- set-up, once per device, with that device current
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
    return fail(HB_NOALLOC_SETUP_FAILED, err, err_len, "hb_gemm_bf16_noalloc: no current CUDA device");
  bool first = false;
  if (g_scratch_ptr[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (rc != cudaSuccess || ptr == nullptr)
      return fail(HB_NOALLOC_SETUP_FAILED, err, err_len,
                  "hb_gemm_bf16_noalloc: cudaGetSymbolAddress failed with code %lld", (long long)rc);
    g_scratch_ptr[dev] = ptr;
    first = true;
  }
  unsigned char* scratch = g_scratch_ptr[dev];
  int* error_word = reinterpret_cast<int*>(scratch);

  // The error word of earlier launches.  A kernel that gives up a bounded wait sets it and
  // nothing but this block clears it, so a code is never lost: it is reported by the first
  // call that finds the stream idle (reading it earlier would make this call wait for the
  // work in flight).  The read is a copy on `stream` itself, not on the legacy default
  // stream, so it neither waits for other streams nor disturbs a capture elsewhere.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(stream, &capturing);
  if (!first && capturing == cudaStreamCaptureStatusNone && cudaStreamQuery(stream) == cudaSuccess) {
    int code = 0;
    if (cudaMemcpyAsync(&code, error_word, sizeof(int), cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
        cudaStreamSynchronize(stream) == cudaSuccess && code != 0) {
      cudaMemsetAsync(error_word, 0, sizeof(int), stream);
      return fail(HB_NOALLOC_KERNEL_GAVE_UP, err, err_len,
                  "hb_gemm_bf16_noalloc: an earlier launch gave up a bounded wait (code %lld)", code);
    }
  }
  // The tickets start at zero (the last block of a tile resets its ticket, but a launch that
  // gave up may have left some behind); the partial sums need no clearing.  On the first call
  // the error word is cleared too: the array's initial contents are not relied on.
  if (first && cudaMemsetAsync(error_word, 0, sizeof(int), stream) != cudaSuccess)
    return fail(HB_NOALLOC_LAUNCH_FAILED, err, err_len, "hb_gemm_bf16_noalloc: cudaMemsetAsync failed");
  if (cudaMemsetAsync(scratch + TICKETS_OFFSET, 0, 4 * HB_GEMM_NOALLOC_MAX_TILES, stream) != cudaSuccess)
    return fail(HB_NOALLOC_LAUNCH_FAILED, err, err_len, "hb_gemm_bf16_noalloc: cudaMemsetAsync failed");

  GemmArgs a;
  a.out = out;
  a.bias = nullptr;
  a.scratch = reinterpret_cast<float*>(scratch + PARTIALS_OFFSET);
  a.tickets = reinterpret_cast<int*>(scratch + TICKETS_OFFSET);
  a.error = error_word;
  a.T = T; a.N = N; a.K = K; a.ldo = N; a.glu_offset = 0; a.out_f32 = 0;
  a.k_splits = k_splits;
  a.cluster_reduce = 0;
  const int rc = launch<16, true, EPI_STORE>(x, w, a, N, K, K, stream);
  if (rc != HB_OK)
    return fail(HB_NOALLOC_LAUNCH_FAILED, err, err_len, "hb_gemm_bf16_noalloc: the kernel launch failed");
  return HB_NOALLOC_OK;
}
