// Peer-memory collectives over NVLink / NVSwitch issued from inside kernels: no NCCL on these paths.
//
// The reference's only device collective is a blocking HcclAllReduce (fp32) after o_proj and after the
// FFN/MoE block, 120 times per decoded token for DeepSeek-V2 (ggml/src/ggml-cann/aclnn_ops.cpp:522-536;
// src/llama-graph-deepseek2.cpp:294-297, 365-368).  Here each rank owns a buffer that every peer maps through
// CUDA IPC ("symmetric" layout: same offsets on every rank) and the reduction is one-shot:
//   push   every rank stores its fp32 partial rows into slot [my_rank] of every peer's receive buffer,
//   signal st.release.sys of the step epoch into a per-(site, source, tile) flag on the peer,
//   wait   ld.acquire.sys spin on the local flags of all sources — bounded; on expiry a status word is set,
//   reduce sum the slots in rank order (bitwise identical on every rank), add the residual, store bf16.
// The same push/wait/reduce sequence is the epilogue of the tcgen05 GEMM (gemm_tcgen05.cu, args.ar) so that the
// transfer of one tile overlaps the MMA work of the others; this file holds the stand-alone all-reduce used
// after the MoE combine, the epoch kernel and the IPC plumbing.
//
// Flags are never reset: they carry the step epoch, a device-side counter bumped once per forward pass, and
// each collective call site of the model owns its own flag rows.  Receive buffers are double-buffered by the
// parity of (site + epoch * n_sites): consecutive collectives always use different halves, so a fast rank
// cannot overwrite data a slow rank is still reducing.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "comm_fused.cuh"
#include "jib_kernels.h"
#include "pdl.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__global__ void epoch_bump_kernel(unsigned * epoch) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    *epoch += 1;
}

// One CTA per (8 rows, 512 features).  x: fp32 or bf16 partial [T][d]; out bf16 [T][d] = sum over ranks + residual.
template <typename TIn>
__global__ void __launch_bounds__(128) allreduce_oneshot_kernel(const TIn * __restrict__ x, const bf16 * __restrict__ residual,
                                                                bf16 * __restrict__ out, int T, int d, JibArCtx ar, int site) {
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    const unsigned epoch = *ar.epoch;
    const int parity = (site + (int) (epoch % 2u) * (ar.n_sites & 1)) & 1;
    const int f0 = blockIdx.x * 512, r0 = blockIdx.y * 8;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int f = f0 + threadIdx.x * 4;
    const int rows = min(8, T - r0);
    const size_t half = (size_t) ar.world * ar.max_rows * ar.d_max;        // floats per parity half
    if (f < d) {       // push my partial into slot [rank] of every peer
        for (int j = 0; j < rows; ++j) {
            float4 v;
            if (sizeof(TIn) == 4) {
                v = *(const float4 *) ((const float *) x + (size_t) (r0 + j) * d + f);
            } else {
                const uint2 raw = *(const uint2 *) ((const bf16 *) x + (size_t) (r0 + j) * d + f);
                const float2 a = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.x);
                const float2 b = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.y);
                v = make_float4(a.x, a.y, b.x, b.y);
            }
            const size_t off = (size_t) parity * half + ((size_t) ar.rank * ar.max_rows + (r0 + j)) * ar.d_max + f;
            for (int p = 0; p < ar.world; ++p) *(float4 *) (ar.recv[p] + off) = v;
        }
    }
    jib_ar_signal_and_wait(ar, site, tile, epoch, 128, (int) threadIdx.x);
    if (f < d) {       // reduce in rank order
        for (int j = 0; j < rows; ++j) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < ar.world; ++s) {
                const float4 v = jib_ld_cg4(ar.recv[ar.rank] + (size_t) parity * half + ((size_t) s * ar.max_rows + (r0 + j)) * ar.d_max + f);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            if (residual) {
                const uint2 raw = *(const uint2 *) (residual + (size_t) (r0 + j) * d + f);
                const float2 a = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.x);
                const float2 b = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.y);
                acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
            }
            uint2 o;
            *(__nv_bfloat162 *) &o.x = __floats2bfloat162_rn(acc.x, acc.y);
            *(__nv_bfloat162 *) &o.y = __floats2bfloat162_rn(acc.z, acc.w);
            *(uint2 *) (out + (size_t) (r0 + j) * d + f) = o;
        }
    }
}

// Two-shot variant for large T: one CTA per (32 rows, 512 features) tile.  The tile's partials go to one owner rank
// (tile % world), which reduces them in rank order, adds the residual and stores the bf16 result into every rank's
// result buffer (ar.out2); every rank's CTA of that tile returns once the owner has delivered.
template <typename TIn>
__global__ void __launch_bounds__(128) allreduce_twoshot_kernel(const TIn * __restrict__ x, const bf16 * __restrict__ residual, int T, int d,
                                                                JibArCtx ar, int site, int rs_rows) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    const unsigned epoch = *ar.epoch;
    const int parity = (site + (int) (epoch % 2u) * (ar.n_sites & 1)) & 1;
    const int f0 = blockIdx.x * 512, r0 = blockIdx.y * 32;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int owner = tile % ar.world;
    const int f = f0 + threadIdx.x * 4;
    const int rows = min(32, T - r0);
    const size_t half = (size_t) ar.world * ar.max_rows2 * ar.d_max;
    const size_t ohalf = (size_t) ar.max_rows2 * ar.d_max;
    if (f < d) {
        float * dst = ar.recv2[owner] + (size_t) parity * half;
        for (int j = 0; j < rows; ++j) {
            float4 v;
            if (sizeof(TIn) == 4) {
                v = *(const float4 *) ((const float *) x + (size_t) (r0 + j) * d + f);
            } else {
                const uint2 raw = *(const uint2 *) ((const bf16 *) x + (size_t) (r0 + j) * d + f);
                const float2 a = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.x);
                const float2 b = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.y);
                v = make_float4(a.x, a.y, b.x, b.y);
            }
            *(float4 *) (dst + ((size_t) ar.rank * ar.max_rows2 + (r0 + j)) * ar.d_max + f) = v;
        }
    }
    const bool ok = jib_ar2_signal_owner(ar, site, tile, owner, epoch, 128, (int) threadIdx.x);
    if (ar.rank == owner && ok && f < d) {
        for (int j = 0; j < rows; ++j) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < ar.world; ++s) {
                const float4 v = jib_ld_cg4(ar.recv2[ar.rank] + (size_t) parity * half + ((size_t) s * ar.max_rows2 + (r0 + j)) * ar.d_max + f);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            if (residual) {
                const uint2 raw = *(const uint2 *) (residual + (size_t) (r0 + j) * d + f);
                const float2 a = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.x);
                const float2 b = __bfloat1622float2(*(const __nv_bfloat162 *) &raw.y);
                acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
            }
            uint2 o;
            *(__nv_bfloat162 *) &o.x = __floats2bfloat162_rn(acc.x, acc.y);
            *(__nv_bfloat162 *) &o.y = __floats2bfloat162_rn(acc.z, acc.w);
            const size_t oi = (size_t) parity * ohalf + (size_t) (r0 + j) * ar.d_max + f;
            if (rs_rows > 0) {        // reduce-scatter: only the rank that owns this row gets it
                *(uint2 *) ((bf16 *) ar.out2[min((r0 + j) / rs_rows, ar.world - 1)] + oi) = o;
            } else {
                for (int p = 0; p < ar.world; ++p) *(uint2 *) ((bf16 *) ar.out2[p] + oi) = o;
            }
        }
    }
    jib_ar2_deliver_and_wait(ar, site, tile, owner, epoch, 128, (int) threadIdx.x);
}

// All-gather of token rows: this rank's R rows (x_loc [R][d] bf16) go to rows [rank*R, rank*R + R) of every rank's gather
// buffer.  One warp per row.  The last block to finish publishes "my rows have landed" to every rank; with `wait` it
// then also waits for every source (bounded), so that the buffer is complete when the kernel ends -- without it the
// consumer (the GEMM's TMA warp) waits per token tile on the same flags.
__global__ void __launch_bounds__(256) allgather_push_kernel(const bf16 * __restrict__ x_loc, int R, int d, JibArCtx ar, int site, int wait) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    const unsigned epoch = *ar.epoch;
    const int par = (site >> 1) & 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t half = (size_t) ar.max_rows2 * ar.d_max;
    for (int i = blockIdx.x * 8 + warp; i < R; i += gridDim.x * 8) {
        const uint4 * src = (const uint4 *) (x_loc + (size_t) i * d);
        const size_t off = (size_t) par * half + ((size_t) ar.rank * R + i) * ar.d_max;
        for (int p = 0; p < ar.world; ++p) {
            uint4 * dst = (uint4 *) ((bf16 *) ar.xg[p] + off);
            for (int v = lane; v < d / 8; v += 32) dst[v] = src[v];
        }
    }
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ar.ag_counter, 1) == (int) gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *ar.ag_counter = 0;
    __threadfence_system();
    if ((int) threadIdx.x < ar.world)
        jib_st_release_sys(ar.flags3[threadIdx.x] + (size_t) site * ar.world + ar.rank, epoch);
    if (wait && (int) threadIdx.x < ar.world) {
        const unsigned * f = ar.flags3[ar.rank] + (size_t) site * ar.world + threadIdx.x;
        bool got = false;
        for (unsigned i = 0, lim = jib_ar_limit(ar); i < lim; ++i) {
            if (jib_ld_acquire_sys(f) == epoch) { got = true; break; }
            __nanosleep(40);
        }
        if (!got && ar.status != nullptr && atomicCAS(ar.status, 0, 1 /* wait timeout */) == 0) {
            ar.status[1] = 90 + (int) threadIdx.x;     // site code: 90 + source rank (all-gather)
            ar.status[2] = 0;
            ar.status[3] = site;
        }
    }
}

}  // namespace

JIB_TL_DEFINE_SETTER(comm)

extern "C" {

// 1 when the library was built with -DJIB_TIMELINE
JIB_EXPORT int jib_timeline_enabled(void) {
#ifdef JIB_TIMELINE
    return 1;
#else
    return 0;
#endif
}

// ---- IPC plumbing (cudaMalloc'd buffers exchanged as 64-byte handles by the Python side) --------------------
JIB_EXPORT int jib_symm_alloc(size_t bytes, void ** ptr_out, void * handle_out /*64 bytes*/) {
    void * p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return JIB_E_LAUNCH;
    if (cudaMemset(p, 0, bytes) != cudaSuccess) return JIB_E_LAUNCH;
    if (cudaDeviceSynchronize() != cudaSuccess) return JIB_E_LAUNCH;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return JIB_E_DRIVER;
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return 0;
}
JIB_EXPORT int jib_symm_open(const void * handle, void ** ptr_out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void * p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return JIB_E_DRIVER;
    *ptr_out = p;
    return 0;
}
JIB_EXPORT int jib_symm_close(void * ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : JIB_E_DRIVER; }
JIB_EXPORT int jib_symm_free(void * ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : JIB_E_DRIVER; }

JIB_EXPORT int jib_ar_epoch_bump(unsigned * epoch, void * stream) {
    JIB_LAUNCH((epoch_bump_kernel), 1, 1, 0, (cudaStream_t) stream, epoch);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

// Stand-alone one-shot all-reduce of a [T][d] partial (fp32 or bf16) + residual -> bf16.
JIB_EXPORT int jib_allreduce_oneshot(const void * x, int x_f32, const void * residual, void * out, int T, int d, const JibArCtx * ar,
                                     int site, void * stream) {
    if (T <= 0) return 0;
    if (d % 4 || d > ar->d_max || T > ar->max_rows || site < 0 || site >= ar->n_sites) return JIB_E_ARG;
    dim3 grid((d + 511) / 512, (T + 7) / 8);
    if ((int) (grid.x * grid.y) > ar->max_tiles) return JIB_E_ARG;
    if (x_f32)
        JIB_LAUNCH((allreduce_oneshot_kernel<float>), grid, 128, 0, (cudaStream_t) stream, (const float *) x, (const bf16 *) residual, (bf16 *) out, T, d, *ar, site);
    else
        JIB_LAUNCH((allreduce_oneshot_kernel<bf16>), grid, 128, 0, (cudaStream_t) stream, (const bf16 *) x, (const bf16 *) residual, (bf16 *) out, T, d, *ar, site);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

// Two-shot all-reduce of a [T][d] partial (+ residual); the bf16 result lands in ar->out2[rank] at the call site's
// half (site & 1; n_sites must be even), row stride d_max.
// rs_rows > 0 turns it into a reduce-scatter by token rows: row i is delivered only to rank i / rs_rows.
JIB_EXPORT int jib_allreduce_twoshot(const void * x, int x_f32, const void * residual, int T, int d, const JibArCtx * ar, int site,
                                     int rs_rows, void * stream) {
    if (T <= 0) return 0;
    if (d % 4 || d > ar->d_max || T > ar->max_rows2 || ar->recv2[0] == nullptr || (ar->n_sites & 1) || site < 0 || site >= ar->n_sites)
        return JIB_E_ARG;
    dim3 grid((d + 511) / 512, (T + 31) / 32);
    if ((int) (grid.x * grid.y) > ar->max_tiles) return JIB_E_ARG;
    if (x_f32)
        JIB_LAUNCH((allreduce_twoshot_kernel<float>), grid, 128, 0, (cudaStream_t) stream, (const float *) x, (const bf16 *) residual, T, d, *ar, site, rs_rows);
    else
        JIB_LAUNCH((allreduce_twoshot_kernel<bf16>), grid, 128, 0, (cudaStream_t) stream, (const bf16 *) x, (const bf16 *) residual, T, d, *ar, site, rs_rows);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

// All-gather of [R][d] bf16 rows per rank into ar->xg[rank] (half (site >> 1) & 1, row stride d_max).
JIB_EXPORT int jib_allgather_rows(const void * x_loc, int R, int d, const JibArCtx * ar, int site, int wait, void * stream) {
    if (R <= 0) return 0;
    if (d % 8 || d > ar->d_max || R * ar->world > ar->max_rows2 || ar->xg[0] == nullptr || site < 0 || site >= ar->n_sites) return JIB_E_ARG;
    const int grid = (R + 7) / 8;
    JIB_LAUNCH((allgather_push_kernel), grid, 256, 0, (cudaStream_t) stream, (const bf16 *) x_loc, R, d, *ar, site, wait);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

}  // extern "C"
