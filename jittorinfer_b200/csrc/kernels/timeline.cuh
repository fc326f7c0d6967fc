// Timeline build (-DJIB_TIMELINE): device-side time stamps of the collective phases.
//
// JIB_TS(kind, a, b, c) appends {globaltimer ns, kind, a, b, c} to a ring in device memory that the host registered with
// jib_timeline_set_<unit>() (one pointer set per translation unit, like the bounds-check build).  The normal build
// compiles JIB_TS to nothing, so the production kernels carry no trace of it.  Stamps are taken by single threads at
// points where they already synchronise (after a flag store, after a flag wait), never inside the spin itself.
//
// kinds: 10 one-shot all-reduce: this rank's partials are stored and signalled   (a = call site, b = tile, c = rank)
//        11 one-shot: the partial of source rank c has arrived
//        12 one-shot: all sources seen, reduction starts
//        20 two-shot: partial stored at the tile owner and signalled (c = owner)
//        21 two-shot, owner: the partial of source rank c has arrived
//        22 two-shot: the owner's reduced tile has been delivered here
//        30 GEMM with a fused collective: accumulators complete (main loop over)  (a = call site, b = tile, c = split)
// Times are per GPU (%globaltimer of the stamping GPU): compare stamps of one rank only.
#pragma once
#include <cuda_runtime.h>

#include "jib_kernels.h"

#ifdef JIB_TIMELINE
struct JibStamp {
    unsigned long long t;
    int kind, a, b, c;
};
static __device__ JibStamp * jib_tl_buf = nullptr;
static __device__ unsigned * jib_tl_head = nullptr;
static __device__ unsigned jib_tl_cap = 0;
__device__ __forceinline__ void jib_stamp(int kind, int a, int b, int c) {
    JibStamp * buf = jib_tl_buf;
    if (buf == nullptr) return;
    const unsigned i = atomicAdd(jib_tl_head, 1u);
    if (i >= jib_tl_cap) return;                 // ring full: later stamps are dropped, the head keeps counting
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    buf[i].t = t;
    buf[i].kind = kind;
    buf[i].a = a;
    buf[i].b = b;
    buf[i].c = c;
}
#define JIB_TS(kind, a, b, c) jib_stamp((kind), (int) (a), (int) (b), (int) (c))
#define JIB_TL_DEFINE_SETTER(unit)                                                                        \
    extern "C" JIB_EXPORT int jib_timeline_set_##unit(void * buf, unsigned * head, unsigned cap) {        \
        JibStamp * b = (JibStamp *) buf;                                                                  \
        if (cudaMemcpyToSymbol(jib_tl_buf, &b, sizeof(b)) != cudaSuccess) return JIB_E_LAUNCH;            \
        if (cudaMemcpyToSymbol(jib_tl_head, &head, sizeof(head)) != cudaSuccess) return JIB_E_LAUNCH;     \
        return cudaMemcpyToSymbol(jib_tl_cap, &cap, sizeof(cap)) == cudaSuccess ? 0 : JIB_E_LAUNCH;       \
    }
#else
#define JIB_TS(kind, a, b, c) \
    do {                      \
    } while (0)
#define JIB_TL_DEFINE_SETTER(unit)
#endif
