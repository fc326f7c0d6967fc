// Split-K GEMM for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library.
//
// Who needs it.  The serving engine sizes the paged KV cache to take whatever HBM the weights leave
// (about 90 % of the card), so once it is up there may be no room for one more cudaMalloc, and a
// program that embeds the library through the C API may own the rest of the GPU itself and forbid
// allocations on its latency-critical thread (a device allocation can stall behind other work on
// the GPU).  Such a caller cannot hand the GEMM the scratch buffer that its split-K reduction
// needs.  Here that scratch lives inside the library: a fixed array in device memory
// (JIB_NOALLOC_SCRATCH_BYTES plus a few KiB of counters) that every GPU which loads the library
// holds from load until the process exits.  The call itself makes no cudaMalloc / cudaFree and uses
// no allocating library routine; inputs and the output are still the caller's buffers.
//
// What it computes.  out[T][N] (bf16, row stride N) = x[T][K] (bf16, row stride K) times the
// transpose of w[N][K] (bf16, row stride K), fp32 accumulation, with the K range cut into `splits`
// parts (0 = let the library choose) exactly as jib_gemm_bf16 does.  T <= 256.
//
// Limits and errors.  The partial sums need
//     ceil(N/128) * splits * max(16, pow2ceil(T)) * 128 * 4 bytes  <=  JIB_NOALLOC_SCRATCH_BYTES
// and ceil(N/128) <= JIB_NOALLOC_MAX_TILES.  A call beyond either limit returns
// JIB_E_NOALLOC_TOO_LARGE and launches nothing.  Other failures the host can see (bad arguments,
// alignment, a refused launch) return the JIB_E_* codes of jib_kernels.h.  Pointers must be 16-byte
// aligned and K a multiple of 8.  With splits = 0 the count follows the SM count of the current
// device (queried once per device), by the same rule as jib_gemm_bf16.
//
// Faults found on the device.  The kernel's waits are bounded and its scratch indices checked; when
// a wait runs out or an index is out of range it records a code in four status words inside the
// built-in array and finishes normally, so the return value of the launch cannot show it.  Each
// call clears those words; read them with jib_gemm_bf16_noalloc_status() after the call (same
// stream) and before the next call on that device.
//
// First call.  The first call on each device looks up the device address of the built-in array
// (with that device current) and remembers it; make that first call outside any stream capture.
//
// Sharing.  All calls on a device share the one array.  Each call clears the tile counters that must
// start at zero before it launches; partial sums need no clearing.  Two calls whose kernels overlap
// on the GPU (different streams, or different host threads on different streams) race on the array:
// serialise them, e.g. by using one stream.
#pragma once
#include <stddef.h>

#include "jib_kernels.h"

#define JIB_NOALLOC_SCRATCH_BYTES (8u << 20)
#define JIB_NOALLOC_MAX_TILES 4096
#define JIB_E_NOALLOC_TOO_LARGE (-7)

#ifdef __cplusplus
extern "C" {
#endif

JIB_EXPORT int jib_gemm_bf16_noalloc(const void * x, const void * w, void * out, int T, int N, int K, int splits, void * stream);

// Bytes of partial-sum scratch a call with these sizes needs (for callers that want to check first).
JIB_EXPORT size_t jib_gemm_bf16_noalloc_need(int T, int N, int K, int splits);

// Copies the status words {code, site, block, extra} of the last call on the current device to out[4] (host memory) in
// stream order; code 0 = no fault, 1 = a bounded wait ran out, 2 = an index was out of range.  Allocates nothing.
JIB_EXPORT int jib_gemm_bf16_noalloc_status(int * out, void * stream);

#ifdef __cplusplus
}
#endif
