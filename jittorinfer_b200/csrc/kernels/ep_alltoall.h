// Context of the expert-parallel all-to-all kernels (ep_alltoall.cu).  Every pointer array is indexed by rank and
// holds that rank's buffer as mapped into this process (CUDA IPC), the entry [rank] being the local allocation.
#pragma once
#include <stdint.h>

#include "comm_fused.cuh"

struct JibEpCtx {
    __nv_bfloat16 * xrecv[JIB_AR_MAX_WORLD];   // [2][max_recv_rows][d]   token rows dispatched to this rank's experts
    int * meta[JIB_AR_MAX_WORLD];              // [2][max_recv_rows]      return tag per row: source rank << 24 | pair index
    int * counts[JIB_AR_MAX_WORLD];            // [2][world][E_local*world] pairs per expert of every source rank
    __nv_bfloat16 * yret[JIB_AR_MAX_WORLD];    // [2][max_pairs][d]       expert outputs returned for this rank's pairs
    unsigned * flags[JIB_AR_MAX_WORLD];        // [n_sites][3][world]     epoch flags: counts / rows / outputs arrived
    unsigned * epoch;                          // this rank's step counter
    int * status;                              // this rank's status words (code, site, block, extra)
    int world, rank, n_sites, E_local, d, max_recv_rows, max_pairs;
    unsigned spin_limit;                       // polls a wait on a peer's flag may take; 0 = JIB_AR_SPIN_LIMIT
};

#ifdef __CUDACC__
__device__ __forceinline__ void jib_ep_report(int * status, int code, int site, int extra) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = site;
        status[2] = (int) blockIdx.x;
        status[3] = extra;
    }
}
#endif
