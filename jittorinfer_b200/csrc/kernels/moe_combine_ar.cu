// Expert combine + all-reduce over peer memory (+ residual, + the next block's RMSNorm) in one launch, for decode batches.
//
// Reference: the MoE block of a tensor/expert-parallel rank ends in MoeFinalizeRouting (weighted top-k sum of the local
// experts' rows, ggml/src/ggml-cann/aclnn_ops.cpp:2540-2542) followed by a blocking HcclAllReduce that doubles as the
// expert-parallel combine (src/llama-graph-deepseek2.cpp:365-368), the residual add and, in the next block, the attention
// RMSNorm: four device passes and a host sync.  Here one CTA owns a token row: it forms the row's partial sum in fp32
// registers (no bf16 rounding before the reduction), stores it into slot [rank] of every peer's receive buffer, signals,
// waits (bounded) for the other ranks' partials of the same row, reduces them in rank order (so every rank gets bitwise
// the same row), adds the residual, stores the bf16 row and -- because it holds the complete row -- also the RMSNorm of
// it for the next block.  The exchange uses the one-shot buffers and flags of comm_fused (tile index = token row).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_fused.cuh"
#include "jib_kernels.h"
#include "pdl.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// NT threads, each owns MAXV groups of 8 consecutive columns (group i = threadIdx.x + it * NT), d <= NT * MAXV * 8.
template <int NT, int MAXV>
__global__ void __launch_bounds__(NT) moe_combine_ar_kernel(const bf16 * __restrict__ y, const int * __restrict__ dest,
                                                            const float * __restrict__ wts, const bf16 * __restrict__ shared,
                                                            const bf16 * __restrict__ residual, const float * __restrict__ norm_w,
                                                            bf16 * __restrict__ out, bf16 * __restrict__ out_norm, int k, int d,
                                                            float eps, JibArCtx ar, int site) {
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int nv = d / 8;
    const unsigned epoch = *ar.epoch;
    const int parity = (site + (int) (epoch % 2u) * (ar.n_sites & 1)) & 1;
    const size_t half = (size_t) ar.world * ar.max_rows * ar.d_max;        // floats per parity half
    float vals[MAXV][8];

    // 1. this rank's partial of the row, pushed into slot [rank] of every rank's receive buffer
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int j = 0; j < k; ++j) {
                const int row = dest[(size_t) t * k + j];
                if (row < 0) continue;                     // expert of another rank
                const float w = wts[(size_t) t * k + j];
                const uint4 raw = ((const uint4 *) (y + (size_t) row * d))[i];
                const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(p[q]);
                    acc[2 * q] += w * f.x;
                    acc[2 * q + 1] += w * f.y;
                }
            }
            if (shared) {                                  // this rank's shard of the shared experts
                const uint4 raw = ((const uint4 *) (shared + (size_t) t * d))[i];
                const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(p[q]);
                    acc[2 * q] += f.x;
                    acc[2 * q + 1] += f.y;
                }
            }
            const size_t off = (size_t) parity * half + ((size_t) ar.rank * ar.max_rows + t) * ar.d_max + (size_t) i * 8;
            const float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
            for (int p = 0; p < ar.world; ++p) {
                float4 * dst = (float4 *) (ar.recv[p] + off);
                dst[0] = lo;
                dst[1] = hi;
            }
        }
    }
    // 2. signal every rank, wait for every rank's partial of this row (bounded; a timeout is reported in ar.status)
    jib_ar_signal_and_wait(ar, site, t, epoch, NT, (int) threadIdx.x);

    // 3. reduce in rank order, add the residual, store the row; keep the rounded values for the norm
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int s = 0; s < ar.world; ++s) {
                const float * src = ar.recv[ar.rank] + (size_t) parity * half + ((size_t) s * ar.max_rows + t) * ar.d_max + (size_t) i * 8;
                const float4 a = jib_ld_cg4(src), b = jib_ld_cg4(src + 4);
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
            if (residual) {
                const uint4 raw = ((const uint4 *) (residual + (size_t) t * d))[i];
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
            ((uint4 *) (out + (size_t) t * d))[i] = o;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(po[q]);
                vals[it][2 * q] = f.x;
                vals[it][2 * q + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    if (out_norm == nullptr) return;                       // uniform over the CTA
    // 4. RMSNorm of the complete row for the next block
    ss = warp_sum_f(ss);
    {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        if (l == 0) red[w] = ss;
        __syncthreads();
        float tsum = l < NT / 32 ? red[l] : 0.f;
        ss = warp_sum_f(tsum);
    }
    const float inv = rsqrtf(ss / (float) d + eps);
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            const float4 w0 = ((const float4 *) norm_w)[2 * i], w1 = ((const float4 *) norm_w)[2 * i + 1];
            uint4 o;
            __nv_bfloat162 * po = (__nv_bfloat162 *) &o;
            po[0] = __floats2bfloat162_rn(vals[it][0] * inv * w0.x, vals[it][1] * inv * w0.y);
            po[1] = __floats2bfloat162_rn(vals[it][2] * inv * w0.z, vals[it][3] * inv * w0.w);
            po[2] = __floats2bfloat162_rn(vals[it][4] * inv * w1.x, vals[it][5] * inv * w1.y);
            po[3] = __floats2bfloat162_rn(vals[it][6] * inv * w1.z, vals[it][7] * inv * w1.w);
            ((uint4 *) (out_norm + (size_t) t * d))[i] = o;
        }
    }
}

}  // namespace

JIB_TL_DEFINE_SETTER(combine_ar)

// out [T][d] bf16 = sum over ranks of (sum_j wts[t][j] * y[dest[t][j]] + shared[t]) + residual[t]; with norm_w also
// out_norm = rmsnorm(out) * norm_w.  T <= ar->max_rows and T <= ar->max_tiles (one tile per token row); d == multiple of 8.
extern "C" JIB_EXPORT int jib_moe_combine_allreduce(const void * y, const int * dest, const float * wts, const void * shared,
                                                    const void * residual, const float * norm_w, void * out, void * out_norm, int T,
                                                    int k, int d, float eps, const JibArCtx * ar, int site, void * stream) {
    if (T <= 0) return 0;
    if (d % 8 || d > ar->d_max || ar->d_max % 4 || T > ar->max_rows || T > ar->max_tiles || site < 0 || site >= ar->n_sites) return JIB_E_ARG;
    if ((norm_w == nullptr) != (out_norm == nullptr)) return JIB_E_ARG;
    const int nv = d / 8;
    cudaStream_t s = (cudaStream_t) stream;
#define JIB_CAR(NT, MAXV)                                                                                                          \
    JIB_LAUNCH((moe_combine_ar_kernel<NT, MAXV>), T, NT, 0, s, (const bf16 *) y, dest, wts, (const bf16 *) shared, (const bf16 *) residual, \
               norm_w, (bf16 *) out, (bf16 *) out_norm, k, d, eps, *ar, site)
    if (nv <= 128) JIB_CAR(128, 1);
    else if (nv <= 256) JIB_CAR(256, 1);
    else if (nv <= 1024) JIB_CAR(256, 4);
    else return JIB_E_ARG;
#undef JIB_CAR
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}
