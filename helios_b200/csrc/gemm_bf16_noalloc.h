/* helios_b200: a decode-sized bfloat16 matrix product that allocates nothing.
 *
 * This entry point has no counterpart in the reference project (anish41338/helios
 * leaves its products to a library).  It exists for callers that must not, or
 * cannot, allocate device memory when they call into this library:
 *
 *   - hosts that hand the GPU's memory out once, up front, to a pool of their own
 *     (a serving process with a fixed memory plan, an embedded runtime) and treat
 *     any later allocation by a library as an error;
 *   - callers in a place where the CUDA allocator must not be entered: inside a
 *     host callback, while holding a lock the allocator may also want, or in a
 *     phase in which cudaMalloc's implicit device synchronisation would stall
 *     other streams;
 *   - latency-critical paths where the time an allocation takes, or its failure
 *     under memory pressure, is not acceptable.
 *
 * The regular entry point (hb_gemm_bf16) splits the reduction over several
 * thread blocks and parks their partial sums in scratch memory that the caller
 * (the Python side, through torch) allocates.  Here the same kernel uses a
 * scratch area that is part of the library image itself: a file-scope
 * `static __device__` array of HB_GEMM_NOALLOC_SCRATCH_BYTES (8 MiB).  Every
 * device that loads the library holds those 8 MiB until the process exits.
 *
 *   y[T, N] = x[T, K] * w[N, K]^T      bfloat16 in, bfloat16 out, float32 accumulate
 *
 * Limits (a call beyond them is refused, nothing is launched):
 *   1 <= T <= 16; K a positive multiple of 8; x and w 16-byte aligned and densely
 *   packed (row strides K); 1 <= k_splits <= ceil(K / 64); and, when k_splits > 1,
 *     ceil(N / 128) * k_splits * 2048 floats  <= the scratch area's float capacity
 *     ceil(N / 128)                           <= HB_GEMM_NOALLOC_MAX_TILES.
 *   (N = 4096 with 9 slices, or N = 6144 with 6, use about 2.3 MiB.)
 *
 * The caller owns x, w and out (device memory, out = T * N bfloat16).  The
 * function calls no cudaMalloc, cudaFree or any other allocating routine; it
 * issues one cudaMemsetAsync (the tickets must start at zero; the partial sums
 * need no clearing, every slot is written before it is read) and one kernel
 * launch on `stream`.
 *
 * First call on a device: the address of the scratch array is looked up with
 * cudaGetSymbolAddress (the array's name is only a host-side handle, not a
 * device pointer) and the kernel's shared-memory limit is raised; both are kept
 * per device.  This set-up happens inside the first call for each device, with
 * that device current.  Make that first call outside of any stream capture, and
 * from one host thread.
 *
 * All calls on a device share the one scratch area, and it keeps what the last
 * call left there.  Two calls that overlap on the GPU (different streams, or
 * different host threads) race on it: keep calls on one device in one stream
 * order.
 *
 * Returns 0 on success, else one of the codes below; if `err` is not NULL a
 * one-line message is written there (at most err_len bytes, always terminated).
 * A kernel that gave up a bounded wait leaves a code in the scratch area's error
 * word.  It is read, reported (HB_NOALLOC_KERNEL_GAVE_UP) and cleared by the first
 * later call on that device that finds `stream` idle: reading it while work is in
 * flight would make the call wait.  A caller that issues calls back to back
 * without ever letting the stream drain therefore hears of it late, but the code
 * is not lost.  That read is a 4-byte copy on `stream` followed by a wait for it.
 */
#ifndef HELIOS_B200_GEMM_BF16_NOALLOC_H
#define HELIOS_B200_GEMM_BF16_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_GEMM_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
#define HB_GEMM_NOALLOC_MAX_TILES 1024
#define HB_GEMM_NOALLOC_MAX_TOKENS 16

enum {
  HB_NOALLOC_OK = 0,
  HB_NOALLOC_BAD_ARGUMENT = 1,     /* a null pointer, misalignment, K not a multiple of 8, ... */
  HB_NOALLOC_TOO_LARGE = 2,        /* T, the tile count or the partial sums exceed the maximum */
  HB_NOALLOC_SETUP_FAILED = 3,     /* cudaGetSymbolAddress or another set-up call failed */
  HB_NOALLOC_LAUNCH_FAILED = 4,
  HB_NOALLOC_KERNEL_GAVE_UP = 5    /* an earlier launch on this device ran out of a bounded wait */
};

int hb_gemm_bf16_noalloc(void* out, const void* x, const void* w, int T, int N, int K,
                         int k_splits, cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
#endif
