// Thin inline-PTX layer for the Blackwell (sm_100a) async machinery used by the GEMM and attention
// kernels: mbarriers, TMA tensor copies, tcgen05 MMA with TMEM accumulators, tcgen05.ld.
//
// Conventions
//  * every wait is bounded: it returns false after JIB_SPIN_LIMIT polls and the caller records a
//    status word and leaves through the normal exit path (TMEM freed, no trap);
//  * TMA loads never use cluster multicast;
//  * shared-memory operand tiles are K-major rows of 128 bytes with the 128-byte swizzle, i.e. exactly
//    what a TMA box of {64 bf16, rows} with CU_TENSOR_MAP_SWIZZLE_128B writes.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef JIB_SPIN_LIMIT
#define JIB_SPIN_LIMIT (1u << 22)
#endif

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
        "elect.sync R|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One wait attempt: the thread may be suspended until the phase completes, but for no longer than the hint (the time a
// try_wait without a hint may stay suspended is implementation-defined, which would make a poll count meaningless).
#ifndef JIB_SUSPEND_NS
#define JIB_SUSPEND_NS 20000        // 0: never suspend, poll with test_wait only (a build variant, to compare wake-up latency)
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    const uint32_t suspend_hint_ns = JIB_SUSPEND_NS;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false if the phase did not complete within the time budget.  One try_wait may itself block for an
// implementation-defined while, so a poll count alone bounds nothing in wall time: the budget is JIB_WAIT_NS on
// %globaltimer (checked every 16 unsuccessful polls; these barriers pace a CTA's own pipeline, where a healthy wait takes
// microseconds), with the poll count as a second limit.
#ifndef JIB_WAIT_NS
#define JIB_WAIT_NS 2000000000ull
#endif
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Non-blocking test of a phase (try_wait may suspend the thread for an implementation-defined time; this one never does).
__device__ __forceinline__ bool mbar_test_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity) {
#if JIB_SUSPEND_NS > 0
    if (mbar_try_wait(bar, parity)) return true;          // the common case: one (possibly suspending) wait is enough
#endif
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 0; i < JIB_SPIN_LIMIT; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((i & 15) == 15) {
            if (globaltimer_ns() - t0 > JIB_WAIT_NS) return false;
#if JIB_SUSPEND_NS > 0
            __nanosleep(64);
#else
            if (i > 4096) __nanosleep(64);                // a long wait: stop taking issue slots from the warps that work
#endif
        }
    }
    return false;
}

// ---- TMA --------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap * m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 3-D tiled load global -> shared, completion on an mbarrier (bytes). No multicast.
__device__ __forceinline__ void tma_load_3d(void * dst, const CUtensorMap * m, uint64_t * bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// The same with an L2 eviction policy for the loaded lines.  evict_first: data read once per forward pass (the weights of a
// decode step, tens of GB) leaves the L2 before anything else does, so that activations, small tables and kernel code stay.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_3d_hint(void * dst, const CUtensorMap * m, uint64_t * bar, int x, int y, int z, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void * dst, const CUtensorMap * m, uint64_t * bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// ---- TMEM -------------------------------------------------------------------------------------
// Whole-warp calls. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t * dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------------
// Shared-memory operand descriptor, K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart.
// `addr` may point at a 32-byte K sub-step inside the swizzle atom (the tile base is 1024-B aligned).
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr & 0x3FFFF) >> 4);
    d |= (uint64_t) 1 << 16;                 // leading byte offset: unused for swizzled K-major
    d |= (uint64_t) (1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t) 1 << 46;                 // descriptor version (Blackwell)
    d |= (uint64_t) 2 << 61;                 // SWIZZLE_128B
    return d;
}
// MN-major, 128-byte swizzle: the tile is stored as [k][mn] with mn contiguous; 64 mn-elements (128 B)
// per swizzle row, 8 k-rows per 1024-B atom.  lbo = byte distance between 64-element mn chunks,
// sbo = byte distance between 8-row k groups.
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr & 0x3FFFF) >> 4);
    d |= (uint64_t) ((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t) ((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 2 << 61;
    return d;
}
// Instruction descriptor, kind::f16, bf16 x bf16 -> fp32.  a_mn / b_mn: 1 when that operand is MN-major.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn = 0, int b_mn = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) a_mn << 15) | ((uint32_t) b_mn << 16) |
           ((uint32_t) (N >> 3) << 17) | ((uint32_t) (M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t) accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]  (A read from tensor memory; used for P*V in attention).
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t) accumulate)
        : "memory");
}
// Arrive on an mbarrier when all previously issued MMAs of this thread have completed.
__device__ __forceinline__ void mma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- TMEM -> registers ------------------------------------------------------------------------
// 32 lanes x 32-bit, 16 consecutive columns: thread i of the warp receives lane (base_lane+i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// one column (same address in every lane of the warp): thread i receives lane (base_lane+i) of that column
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// registers -> TMEM, 16 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace sm100

// ---- status words -----------------------------------------------------------------------------
// A kernel that gives up on a wait stores a code here (first writer wins) and returns normally.
// Layout: [0] code, [1] site, [2] blockIdx.x, [3] extra.
enum JibStatusCode : int { JIB_OK = 0, JIB_ERR_WAIT_TIMEOUT = 1, JIB_ERR_BOUNDS = 2, JIB_ERR_ALIGN = 3 };

__device__ __forceinline__ void jib_report(int * status, int code, int site, int extra) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = site;
        status[2] = (int) blockIdx.x;
        status[3] = extra;
    }
}
