// Bounds-check build (-DJIB_BOUNDS_CHECK): index checks that are silent clamps or skips in the normal build also record
// the offending value in the status words (code JIB_ERR_BOUNDS, a site number, blockIdx.x, the value) so that the host
// sees it through ops.native.check_status().  Nothing traps: the kernel carries on with the clamped value.  The normal
// build compiles JIB_BC to nothing.  Stands in for compute-sanitizer's memcheck on machines where that tool cannot run.
#pragma once
#include <cuda_runtime.h>

#include "jib_kernels.h"

#ifdef JIB_BOUNDS_CHECK
static __device__ int * jib_bc_status = nullptr;        // one per translation unit, set by jib_bounds_status_<unit>()
__device__ __forceinline__ void jib_bc_report(int site, int extra) {
    int * st = jib_bc_status;
    if (st != nullptr && atomicCAS(st, 0, 2 /* JIB_ERR_BOUNDS */) == 0) {
        st[1] = site;
        st[2] = (int) blockIdx.x;
        st[3] = extra;
    }
}
#define JIB_BC(cond, site, extra)                         \
    do {                                                  \
        if (!(cond)) jib_bc_report((site), (int) (extra)); \
    } while (0)
#define JIB_BC_DEFINE_SETTER(unit)                                                                              \
    extern "C" JIB_EXPORT int jib_bounds_status_##unit(int * status) {                                          \
        return cudaMemcpyToSymbol(jib_bc_status, &status, sizeof(status)) == cudaSuccess ? 0 : JIB_E_LAUNCH;    \
    }
#else
#define JIB_BC(cond, site, extra) \
    do {                          \
    } while (0)
#define JIB_BC_DEFINE_SETTER(unit)
#endif
