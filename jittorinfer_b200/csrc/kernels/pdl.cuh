// Programmatic dependent launch (PDL) helpers.
//
// Every kernel of the library is launched with the "programmatic stream serialization" attribute: its CTAs may
// become resident while the previous kernel on the stream is still draining, run their prologue (barrier
// initialisation, TMEM allocation, tensor-map prefetch, reading launch-invariant inputs) and then block in
// pdl_wait() until the previous grid has completed and its writes are visible.  Rules every kernel follows:
//   * pdl_launch_dependents() first thing (lets the next kernel's CTAs be scheduled early);
//   * pdl_wait() before the first read of anything an earlier kernel produced, before ANY global write, and on
//     every path that leaves the kernel — the chain "N waits for N-1" is what orders N against all earlier work.
// Captured into CUDA graphs the attribute becomes a programmatic dependency edge.  JIB_PDL=0 turns it off.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <stdlib.h>
#include <string.h>
#include <utility>

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Where a kernel lets its dependents start.  Default: first thing (the next kernels become resident as early as the SMs have
// room and park in pdl_wait()).  -DJIB_PDL_LATE: only once the kernel's own loads have been issued (PDL_TRIGGER_LATE() sites;
// kernels without such a site release their dependents when their CTAs exit), so that parked CTAs do not share the SMs
// with the running kernel for its whole duration.
#ifdef JIB_PDL_LATE
#define PDL_TRIGGER_TOP() \
    do {                  \
    } while (0)
#define PDL_TRIGGER_LATE() pdl_launch_dependents()
#else
#define PDL_TRIGGER_TOP() pdl_launch_dependents()
#define PDL_TRIGGER_LATE() \
    do {                   \
    } while (0)
#endif

namespace jib {

inline bool pdl_enabled() {
    static const bool on = [] {
        const char * e = getenv("JIB_PDL");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to one (function, device) pair: a process that launches on several
// GPUs (layer split) has to set it on each.  `done` is the caller's per-kernel table, one atomic flag per device ordinal.
constexpr int MAX_DEVICES = 64;
template <typename K>
inline bool ensure_dyn_smem(K kern, int bytes, std::atomic<unsigned char> (&done)[MAX_DEVICES]) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return false;
    if (done[dev].load(std::memory_order_acquire)) return true;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    done[dev].store(1, std::memory_order_release);
    return true;
}

// Small latency-bound kernels run their body twice: once "dry" (same instructions, no stores, indices that come from memory
// replaced by safe ones) while they still wait for the previous kernel, then for real.  A kernel's first pass over cold code
// costs an instruction-cache miss every few instructions; the dry pass takes those misses in the shadow of the previous
// kernel.  JIB_WARM=0 turns the dry passes off (A/B measurements).
inline int warm_enabled() {
    static const int on = [] {
        const char * e = getenv("JIB_WARM");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return on;
}

// ... for launches of up to `WARM_MAX_ROWS` rows only: in a grid of thousands of CTAs every CTA would pay for the dry pass while
// only the first one on each SM finds cold code.
constexpr int WARM_MAX_ROWS = 256;
inline int warm_for(long long rows) { return (warm_enabled() && rows <= WARM_MAX_ROWS) ? 1 : 0; }

// cluster_z > 1: consecutive blockIdx.z values form a thread-block cluster of that size.
template <typename... P, typename... A>
inline cudaError_t launch_pdl_cluster(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                                      A &&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned) cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<A>(args)...);
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A &&... args) {
    return launch_pdl_cluster(kern, grid, block, smem, stream, 1, std::forward<A>(args)...);
}

}  // namespace jib

// kern may contain template commas: pass it in parentheses, e.g. JIB_LAUNCH((rmsnorm_kernel<256, 4>), grid, ...)
#define JIB_LAUNCH(kern, grid, block, smem, stream, ...) (void) jib::launch_pdl(kern, dim3(grid), dim3(block), smem, stream, __VA_ARGS__)
