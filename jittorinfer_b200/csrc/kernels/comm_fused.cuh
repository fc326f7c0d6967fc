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
    // two-shot path for large batches (prefill): a tile's partials go to one owner rank only, the owner reduces and
    // stores the bf16 result into every rank's result buffer.  All NULL / 0 when not allocated.
    float * recv2[JIB_AR_MAX_WORLD];      // [2][world][max_rows2][d_max] fp32 partials of the tiles this rank owns
    void * out2[JIB_AR_MAX_WORLD];        // [2][max_rows2][d_max] bf16 reduced result (identical on every rank)
    unsigned * flags2[JIB_AR_MAX_WORLD];  // [n_sites][max_tiles] "tile reduced and delivered" flags
    int max_rows2;
    // all-gather of token rows (sequence-parallel prefill): every rank stores its rows into every rank's gather buffer
    void * xg[JIB_AR_MAX_WORLD];          // [2][max_rows2][d_max] bf16 gathered rows
    unsigned * flags3[JIB_AR_MAX_WORLD];  // [n_sites][world] "rows of source s have landed" flags
    int * ag_counter;                     // this rank's block counter of the push kernel (zero between launches)
    unsigned spin_limit;                  // polls a wait on a peer's flag may take before it gives up; 0 = JIB_AR_SPIN_LIMIT
};

#ifdef __CUDACC__
#include "timeline.cuh"
__device__ __forceinline__ void jib_st_release_sys(unsigned * p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned jib_ld_acquire_sys(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 jib_ld_cg4(const float * p) { return __ldcg((const float4 *) p); }
__device__ __forceinline__ unsigned jib_ar_limit(const JibArCtx & ar) { return ar.spin_limit != 0 ? ar.spin_limit : JIB_AR_SPIN_LIMIT; }

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
    if (local_tid == 0) JIB_TS(10, site, tile, ar.rank);
    if (local_tid < ar.world) {                   // wait for source `local_tid`
        const unsigned * f = ar.flags[ar.rank] + slot + (size_t) local_tid * ar.max_tiles;
        bool got = false;
        for (unsigned i = 0, lim = jib_ar_limit(ar); i < lim; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        JIB_TS(11, site, tile, local_tid);
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
    if (local_tid == 0) JIB_TS(12, site, tile, ar.rank);
    return s_ok != 0;
}
// Two-shot exchange for one tile, called by `nthreads` threads (named barrier 1) after they stored their fp32 partial
// of the tile into slot [rank] of the owner's recv2.  Signals the owner; returns once the flag wait of this thread's
// role is over.  Owner side: wait for every source's partial (returns true so that the caller reduces + delivers and
// then calls jib_ar2_deliver_and_wait); non-owners skip straight to jib_ar2_deliver_and_wait.
__device__ __forceinline__ bool jib_ar2_signal_owner(const JibArCtx & ar, int site, int tile, int owner, unsigned epoch, int nthreads,
                                                     int local_tid) {
    __shared__ int s_ok2;
    __threadfence_system();
    if (local_tid == 0) s_ok2 = 1;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    const size_t slot = ((size_t) site * ar.world) * ar.max_tiles + tile;
    if (local_tid == 0) {
        jib_st_release_sys(ar.flags[owner] + slot + (size_t) ar.rank * ar.max_tiles, epoch);
        JIB_TS(20, site, tile, owner);
    }
    if (ar.rank == owner && local_tid < ar.world) {
        const unsigned * f = ar.flags[ar.rank] + slot + (size_t) local_tid * ar.max_tiles;
        bool got = false;
        for (unsigned i = 0, lim = jib_ar_limit(ar); i < lim; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        JIB_TS(21, site, tile, local_tid);
        if (!got) {
            s_ok2 = 0;
            if (ar.status != nullptr && atomicCAS(ar.status, 0, 1 /* wait timeout */) == 0) {
                ar.status[1] = 50 + local_tid;    // site code: 50 + source rank (two-shot, partials)
                ar.status[2] = tile;
                ar.status[3] = site;
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    return s_ok2 != 0;
}

// Owner: after storing the reduced tile into every rank's out2, publish it.  Everyone: wait until the owner published.
__device__ __forceinline__ bool jib_ar2_deliver_and_wait(const JibArCtx & ar, int site, int tile, int owner, unsigned epoch, int nthreads,
                                                         int local_tid) {
    __shared__ int s_ok3;
    const size_t slot = (size_t) site * ar.max_tiles + tile;
    if (ar.rank == owner) {
        __threadfence_system();
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (local_tid < ar.world) jib_st_release_sys(ar.flags2[local_tid] + slot, epoch);
    }
    if (local_tid == 0) {
        s_ok3 = 1;
        const unsigned * f = ar.flags2[ar.rank] + slot;
        bool got = false;
        for (unsigned i = 0, lim = jib_ar_limit(ar); i < lim; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        JIB_TS(22, site, tile, owner);
        if (!got) {
            s_ok3 = 0;
            if (ar.status != nullptr && atomicCAS(ar.status, 0, 1 /* wait timeout */) == 0) {
                ar.status[1] = 58;                // two-shot: the owner never delivered
                ar.status[2] = tile;
                ar.status[3] = site;
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    return s_ok3 != 0;
}
#endif
