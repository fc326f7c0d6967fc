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
//        100 + kernel id: phase stamps of a kernel's CTAs (a = linear block index, b = blocks in the grid, c = phase:
//            0 entry, 1 past the wait for the previous kernel, 9 exit; 2..8 kernel specific).  Kernel ids: 1 gemm
//            (2 operand loads issued, 4 accumulators complete, 5 split partial published, 6 result stored), 2 mla_flash
//            (4 first score tile, 6 result stored), 3 mla_combine, 4 rmsnorm, 5 mla_qkv_post, 6 embed_gather,
//            7 gather_rows, 8 argmax, 9 router_logits, 10 moe_gate, 11 moe_permute, 12 moe_combine, 13 moe_combine_norm,
//            14 moe_route_fused, 15 topk
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
// phase stamp by thread `tid` of every CTA
#define JIB_KS_T(id, phase, tid)                                                                                     \
    do {                                                                                                             \
        if (threadIdx.x == (tid))                                                                                    \
            jib_stamp(100 + (id), (int) (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)),            \
                      (int) (gridDim.x * gridDim.y * gridDim.z), (phase));                                           \
    } while (0)
#define JIB_KS(id, phase) JIB_KS_T(id, phase, 0)
// the same by whichever single thread executes it
#define JIB_KS_ANY(id, phase)                                                                                  \
    jib_stamp(100 + (id), (int) (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)),              \
              (int) (gridDim.x * gridDim.y * gridDim.z), (phase))
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
#define JIB_KS_T(id, phase, tid) \
    do {                         \
    } while (0)
#define JIB_KS(id, phase) \
    do {                  \
    } while (0)
#define JIB_KS_ANY(id, phase) \
    do {                      \
    } while (0)
#define JIB_TL_DEFINE_SETTER(unit)
#endif
