// Expert-parallel all-to-all over NVLink peer memory: dispatch of token rows to the ranks that own their experts and
// the return of the expert outputs, issued from inside kernels (no NCCL, no host synchronisation).
//
// The reference has no all-to-all: under expert parallelism every rank holds all tokens, runs its local experts over
// them and the post-MLP all-reduce doubles as the combine (src/llama-graph-deepseek2.cpp:365-368;
// ggml/src/ggml-cann/aclnn_ops.cpp:2134-2168 picks the local rows on the host after a device-to-host copy and a stream
// synchronise).  Here attention is data-parallel -- every rank has its own tokens -- and one MoE layer is
//
//   plan     (1 CTA)   count my (token, expert) pairs per expert, push the count vector to every rank, wait for
//                      everybody's, and derive from the full table: my experts' row segments (seg, for the grouped
//                      GEMM) and, for each of my pairs, the exact row it occupies in the owner's expert-sorted buffer;
//   push     (n CTAs)  store every pair's hidden row (and a return tag) straight into the owner's buffer over NVLink;
//                      the last CTA to finish signals all ranks, waits for their signals and turns the tags of the
//                      rows that arrived into return addresses;
//   experts            the two grouped tcgen05 GEMMs over the receive buffer; the down-projection's epilogue stores
//                      each output row through its return address, i.e. directly into the source rank's memory;
//   combine  (T CTAs)  signal "my outputs are delivered", wait for every rank's signal, then
//                      out[t] = residual + shared + sum_j w[t][j] * returned[t][j].
//
// Every wait is a bounded ld.acquire.sys spin that records a status word and returns.  Flags carry the step epoch and
// are never reset; buffers are double-buffered by call-site parity as in comm_fused.cu: a rank can run at most one
// collective phase ahead of the slowest rank, because each phase needs every rank's signal of the phase before.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_fused.cuh"
#include "ep_alltoall.h"
#include "jib_kernels.h"
#include "pdl.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int EP_MAX_E = 256;

__device__ __forceinline__ int ep_parity(const JibEpCtx & c, int site, unsigned epoch) {
    return (site + (int) (epoch % 2u) * (c.n_sites & 1)) & 1;
}

__device__ __forceinline__ unsigned * ep_flag(const JibEpCtx & c, int on_rank, int site, int phase, int src) {
    return c.flags[on_rank] + ((size_t) site * 3 + phase) * c.world + src;
}

// Threads [0, world) of the calling block: release-store `epoch` into flag (site, phase, my rank) of every rank, then
// spin (bounded) on the local flags of every source.  All threads of the block must call it.  Returns false on expiry.
__device__ bool ep_signal_and_wait(const JibEpCtx & c, int site, int phase, unsigned epoch, bool do_signal) {
    __shared__ int s_ok;
    __threadfence_system();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int) threadIdx.x < c.world) {
        if (do_signal) jib_st_release_sys(ep_flag(c, (int) threadIdx.x, site, phase, c.rank), epoch);
        const unsigned * f = ep_flag(c, c.rank, site, phase, (int) threadIdx.x);
        bool got = false;
        for (unsigned i = 0, lim = c.spin_limit != 0 ? c.spin_limit : JIB_AR_SPIN_LIMIT; i < lim; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        if (!got) {
            s_ok = 0;
            if (c.status != nullptr && atomicCAS(c.status, 0, 1 /* wait timeout */) == 0) {
                c.status[1] = 60 + phase * 10 + (int) threadIdx.x;      // 60/70/80 + source rank: plan / push / return
                c.status[2] = site;
                c.status[3] = (int) epoch;
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// ---- plan ------------------------------------------------------------------------------------------------------------
// ids [n] global expert ids of my pairs (pair i = token i / k, slot i % k).  Outputs: seg [E_local + 1] row segments of my
// experts in my receive buffer; pair_dst [n] = owner rank << 27 | row in the owner's buffer (-1: dropped, buffer full).
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int * __restrict__ ids, int n, JibEpCtx c, int site, int * __restrict__ seg,
                                                      int * __restrict__ pair_dst) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    __shared__ int cnt[EP_MAX_E];                 // my pairs per global expert
    __shared__ int base[EP_MAX_E];                // first row of my pairs for expert e in its owner's buffer
    __shared__ int tot[EP_MAX_E];                 // rows of expert e over all ranks
    const unsigned epoch = *c.epoch;
    const int par = ep_parity(c, site, epoch);
    const int E = c.E_local * c.world;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < E; e += nw) {
        int cn = 0;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            cn += __popc(__ballot_sync(0xffffffffu, i < n && ids[i] == e));
        }
        if (lane == 0) cnt[e] = cn;
    }
    __syncthreads();
    // my count vector goes to row [rank] of every rank's table
    for (int i = threadIdx.x; i < E * c.world; i += blockDim.x) {
        const int p = i / E, e = i % E;
        c.counts[p][((size_t) par * c.world + c.rank) * E + e] = cnt[e];
    }
    const bool ok = ep_signal_and_wait(c, site, 0, epoch, true);
    const int * tab = c.counts[c.rank] + (size_t) par * c.world * E;       // [world][E], written by the peers
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0, before = 0;
        for (int r = 0; r < c.world; ++r) {
            const int v = ok ? __ldcg(tab + (size_t) r * E + e) : (r == c.rank ? cnt[e] : 0);
            t += v;
            if (r < c.rank) before += v;
        }
        tot[e] = t;
        base[e] = before;
    }
    __syncthreads();
    if ((int) threadIdx.x < c.world) {            // exclusive prefix of the totals within each owner's expert range
        int acc = 0;
        for (int le = 0; le < c.E_local; ++le) {
            const int e = (int) threadIdx.x * c.E_local + le;
            const int t = tot[e];
            if ((int) threadIdx.x == c.rank) seg[le] = acc;
            base[e] += acc;
            acc += t;
        }
        if ((int) threadIdx.x == c.rank) {
            seg[c.E_local] = min(acc, c.max_recv_rows);
            if (acc > c.max_recv_rows) jib_ep_report(c.status, 2 /* bounds */, 61, acc);
        }
    }
    __syncthreads();
    if ((int) threadIdx.x <= c.E_local && seg[threadIdx.x] > c.max_recv_rows) seg[threadIdx.x] = c.max_recv_rows;
    for (int e = warp; e < E; e += nw) {          // stable: pairs of one expert keep their token order
        int b = base[e];
        const int owner = e / c.E_local;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < n && ids[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int row = b + __popc(m & ((1u << lane) - 1));
                pair_dst[i] = row < c.max_recv_rows ? (owner << 27) | row : -1;
            }
            b += __popc(m);
        }
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (ids[i] < 0 || ids[i] >= E) pair_dst[i] = -1;
}

// ---- push ------------------------------------------------------------------------------------------------------------
// x [T][d] my tokens; one warp per pair copies the row into the owner's receive buffer and writes the return tag.
// done_counter: one int, zero between launches.  row_ptr [max_recv_rows]: return address of every row I received.
__global__ void __launch_bounds__(256) ep_push_kernel(const bf16 * __restrict__ x, const int * __restrict__ pair_dst, int n, int k,
                                                     JibEpCtx c, int site, const int * __restrict__ seg, int * done_counter,
                                                     unsigned long long * __restrict__ row_ptr) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    const unsigned epoch = *c.epoch;
    const int par = ep_parity(c, site, epoch);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vec = c.d / 8;                      // uint4 per row
    for (int i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
        const int dst = pair_dst[i];
        if (dst < 0) continue;
        const int owner = dst >> 27, row = dst & ((1 << 27) - 1);
        const uint4 * src = (const uint4 *) (x + (size_t) (i / k) * c.d);
        uint4 * out = (uint4 *) (c.xrecv[owner] + ((size_t) par * c.max_recv_rows + row) * c.d);
        for (int v = lane; v < vec; v += 32) out[v] = src[v];
        if (lane == 0) c.meta[owner][(size_t) par * c.max_recv_rows + row] = (c.rank << 24) | i;
    }
    __shared__ int s_last;
    __threadfence_system();                       // this block's rows are visible to every GPU before the count
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(done_counter, 1) == (int) gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *done_counter = 0;
    // all my rows are on their way: tell every rank, wait until every rank's rows for me have landed
    const bool ok = ep_signal_and_wait(c, site, 1, epoch, true);
    const int n_rows = ok ? seg[c.E_local] : 0;
    const int * meta = c.meta[c.rank] + (size_t) par * c.max_recv_rows;
    for (int r = threadIdx.x; r < c.max_recv_rows; r += blockDim.x) {
        unsigned long long addr = 0;
        if (r < n_rows) {
            const int m = __ldcg(meta + r);
            const int src = (m >> 24) & 0xff, pair = m & 0xffffff;
            if (src < c.world && pair < c.max_pairs) addr = (unsigned long long) (c.yret[src] + ((size_t) par * c.max_pairs + pair) * c.d);
            else jib_ep_report(c.status, 2 /* bounds */, 71, m);
        }
        row_ptr[r] = addr;
    }
}

// ---- combine ---------------------------------------------------------------------------------------------------------
// Runs after this rank's down-projection (stream order), whose epilogue delivered the outputs of my experts to their
// sources.  out[t] = residual[t] + shared[t] + sum_j wts[t][j] * yret[t*k + j].
__global__ void __launch_bounds__(256) ep_combine_kernel(const float * __restrict__ wts, const int * __restrict__ pair_dst,
                                                        const bf16 * __restrict__ shared, const bf16 * __restrict__ residual,
                                                        bf16 * __restrict__ out, int T, int k, JibEpCtx c, int site) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    const unsigned epoch = *c.epoch;
    const int par = ep_parity(c, site, epoch);
    const bool ok = ep_signal_and_wait(c, site, 2, epoch, blockIdx.x == 0);
    const int t = blockIdx.x;
    if (t >= T) return;
    const bf16 * y = c.yret[c.rank] + (size_t) par * c.max_pairs * c.d;
    for (int i = threadIdx.x; i < c.d / 8; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int j = 0; j < k && ok; ++j) {
            if (pair_dst[(size_t) t * k + j] < 0) continue;
            const float w = wts[(size_t) t * k + j];
            const uint4 raw = __ldcg((const uint4 *) (y + ((size_t) t * k + j) * c.d) + i);
            const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(p[q]);
                acc[2 * q] += w * f.x;
                acc[2 * q + 1] += w * f.y;
            }
        }
        const bf16 * extra[2] = {shared, residual};
        for (int s = 0; s < 2; ++s) {
            if (extra[s] == nullptr) continue;
            const uint4 raw = ((const uint4 *) (extra[s] + (size_t) t * c.d))[i];
            const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(p[q]);
                acc[2 * q] += f.x;
                acc[2 * q + 1] += f.y;
            }
        }
        uint4 o;
        __nv_bfloat162 * po = (__nv_bfloat162 *) &o;
#pragma unroll
        for (int q = 0; q < 4; ++q) po[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        ((uint4 *) (out + (size_t) t * c.d))[i] = o;
    }
}

}  // namespace

extern "C" {

JIB_EXPORT int jib_ep_plan(const int * ids, int T, int k, const JibEpCtx * c, int site, int * seg, int * pair_dst, void * stream) {
    if (c->E_local * c->world > EP_MAX_E || c->world > JIB_AR_MAX_WORLD || site < 0 || site >= c->n_sites || T * k > c->max_pairs ||
        T * k >= (1 << 24))
        return JIB_E_ARG;
    JIB_LAUNCH((ep_plan_kernel), 1, 1024, 0, (cudaStream_t) stream, ids, T * k, *c, site, seg, pair_dst);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

JIB_EXPORT int jib_ep_push(const void * x, const int * pair_dst, int T, int k, const JibEpCtx * c, int site, const int * seg,
                           int * done_counter, void * row_ptr, void * stream) {
    if (c->d % 8 || site < 0 || site >= c->n_sites) return JIB_E_ARG;
    const int n = T * k;
    const int grid = n > 0 ? (n + 7) / 8 : 1;     // an idle rank still signals and waits
    JIB_LAUNCH((ep_push_kernel), grid, 256, 0, (cudaStream_t) stream, (const bf16 *) x, pair_dst, n, k, *c, site, seg, done_counter,
               (unsigned long long *) row_ptr);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

JIB_EXPORT int jib_ep_combine(const float * wts, const int * pair_dst, const void * shared, const void * residual, void * out, int T, int k,
                              const JibEpCtx * c, int site, void * stream) {
    if (c->d % 8 || site < 0 || site >= c->n_sites) return JIB_E_ARG;
    JIB_LAUNCH((ep_combine_kernel), T > 0 ? T : 1, 256, 0, (cudaStream_t) stream, wts, pair_dst, (const bf16 *) shared,
               (const bf16 *) residual, (bf16 *) out, T, k, *c, site);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

}  // extern "C"
