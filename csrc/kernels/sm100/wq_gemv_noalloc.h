// Allocation-free entry point of the mixed-bit GEMV.  It has no counterpart in the reference engine.
//
// Who needs it: callers that must not (or cannot) allocate device memory at the moment they want a GEMV -- code that
// runs while a memory-budget cap leaves no headroom, plug-ins that are handed a fixed set of buffers by their host
// application, and hosts that forbid cudaMalloc on their hot path because it synchronises the device.  The regular
// entry point (b2_wq_gemv) expects the caller to bring split-k scratch memory, work counters and a status word; this
// one keeps them in a fixed array inside the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch serves: b2_wq_gemv_scratch_floats(n, k, ks, rb, m) <= this many floats and
// n / 32 <= B2_NOALLOC_MAX_ITEMS.  The array costs (floats * 4 + items * 4 + 256) bytes of device memory on every GPU
// that loads the library, until the process exits.
#define B2_NOALLOC_SCRATCH_FLOATS (1 << 20)   /* 4 MiB */
#define B2_NOALLOC_MAX_ITEMS 8192

// y[m][ldy] (bf16) = x[m][ldx] (bf16) * W^T, W an FM-layout quantised linear (n rows, k columns).
//   * Returns 0 on success, 1 for a bad or too large argument set (the message names the limit; nothing is launched),
//     2 when a CUDA call failed.  `err` (optional, >= 160 bytes) receives a human-readable reason.
//   * Allocates nothing: no cudaMalloc / cudaFree, no library call that allocates.
//   * The first call on a device resolves the address of the built-in scratch array (cudaGetSymbolAddress).  Make that
//     first call outside of any stream capture.
//   * All calls share the one scratch array.  The work counters in it are cleared at the start of every call, so a
//     call never depends on what an earlier one left behind; two calls that overlap in time on the GPU (different
//     streams, no dependency) would race on it -- serialise them.
//   * After the call has finished on the device, *status_out (device pointer, optional) holds 0 or the kernel's
//     status code (3 = a bounded wait ran out).
__attribute__((visibility("default")))
int b2_wq_gemv_noalloc(const uint8_t* wq, int n, int k, int bits, int group, int ks, const void* x_bf16, long ldx, int m,
                       void* y_bf16, long ldy, int* status_out, cudaStream_t stream, char* err);

#ifdef __cplusplus
}
#endif
