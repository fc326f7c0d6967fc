// Device-side pieces of the one-shot peer-memory all-reduce, shared by the stand-alone kernel (comm_fused.cu)
// and the GEMM epilogue (gemm_tcgen05.cu).  See comm_fused.cu for the protocol.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define JIB_AR_MAX_WORLD 8
#ifndef JIB_AR_SPIN_LIMIT
#define JIB_AR_SPIN_LIMIT (1u << 20)      // polls of ~1-2 us each (a flag load plus a short sleep): gives up after 1-2 s,
                                          // enough for host-side skew between ranks (graph capture, first-use loads)
#endif

struct JibArCtx {
    float * recv[JIB_AR_MAX_WORLD];       // receive buffer of every rank (peer-mapped): [2][world][max_rows][d_max] fp32
    unsigned * flags[JIB_AR_MAX_WORLD];   // flag array of every rank (peer-mapped): [n_sites][world][max_tiles]
    unsigned * epoch;                     // this rank's step counter (device memory)
    int * status;                         // this rank's status words (code, site, block, extra)
    int world, rank, n_sites, max_rows, d_max, max_tiles;
};

#ifdef __CUDACC__
__device__ __forceinline__ void jib_st_release_sys(unsigned * p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned jib_ld_acquire_sys(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 jib_ld_cg4(const float * p) { return __ldcg((const float4 *) p); }

// Called by `nthreads` threads (a multiple of 32, named barrier 1) after they stored their partials to the peers.
// local_tid in [0, nthreads).  Returns false if a source never signalled within the poll budget.
__device__ __forceinline__ bool jib_ar_signal_and_wait(const JibArCtx & ar, int site, int tile, unsigned epoch, int nthreads,
                                                       int local_tid) {
    __shared__ int s_ok;
    __threadfence_system();                       // my partial rows are visible to every GPU before any flag is
    if (local_tid == 0) s_ok = 1;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    const size_t slot = ((size_t) site * ar.world) * ar.max_tiles + tile;
    if (local_tid < ar.world)                     // tell peer `local_tid` that slot [rank] of this tile is complete
        jib_st_release_sys(ar.flags[local_tid] + slot + (size_t) ar.rank * ar.max_tiles, epoch);
    if (local_tid < ar.world) {                   // wait for source `local_tid`
        const unsigned * f = ar.flags[ar.rank] + slot + (size_t) local_tid * ar.max_tiles;
        bool got = false;
        for (unsigned i = 0; i < JIB_AR_SPIN_LIMIT; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        if (!got) {
            s_ok = 0;
            if (ar.status != nullptr && atomicCAS(ar.status, 0, 1 /* wait timeout */) == 0) {
                ar.status[1] = 40 + local_tid;    // site code: 40 + source rank
                ar.status[2] = tile;
                ar.status[3] = site;
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    return s_ok != 0;
}
#endif
