// Weight-absorbed MLA attention over the paged latent cache, split-KV ("flash-decoding") form.
//
// The reference composes this from four matmuls and a softmax that materialise [S, T*H] scores in HBM and
// keeps a second, transposed copy of the latent (src/llama-graph-attn.cpp:219-342); its mask is a dense
// host-built [n_kv x T] matrix (src/llama-context.cpp:326-423).  Here one kernel streams each latent row
// once per (token, head-group, kv-split), keeps scores on chip, derives causality from sequence lengths,
// and a small second kernel merges the split partials (m, l, o).
//
// This file is the CUDA-core (SIMT) implementation: any q_len, any head count that is a multiple of 16.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "jib_kernels.h"
#include "pdl.cuh"
#include "timeline.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int HG = 16;        // heads per block
constexpr int PC = 32;        // kv positions per chunk
constexpr int NT = 256;

// grid: (T, n_splits, H/HG).  part_o [T][n_splits][H][r] (unnormalised), part_ml [T][n_splits][H][2].
template <int R, int DR>
__global__ void __launch_bounds__(NT) mla_attn_split_kernel(const bf16 * __restrict__ q, const bf16 * __restrict__ cache,
                                                            const int * __restrict__ block_tables, int max_blocks,
                                                            const int * __restrict__ seq_lens, const int * __restrict__ q_start, int n_seqs,
                                                            int H, int block_size, float scale, int n_splits, float * __restrict__ part_o,
                                                            float * __restrict__ part_ml, bf16 * __restrict__ o_lat) {
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    constexpr int D = R + DR;              // 576
    constexpr int ROWB = D * 2 + 16;       // padded smem row (bytes): conflict-free 16-byte reads across rows
    extern __shared__ __align__(16) uint8_t smem[];
    float * qs = (float *) smem;                               // [HG][D]
    uint8_t * lat = smem + HG * D * sizeof(float);             // [PC][ROWB]
    float * ps = (float *) (lat + PC * ROWB);                  // [HG][PC]
    const int t = blockIdx.x, sp = blockIdx.y, hg = blockIdx.z;
    const int tid = threadIdx.x;

    // which sequence owns token t (q_start is ascending)
    int lo = 0, hi = n_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (q_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int q0 = q_start[b], q1 = q_start[b + 1];
    const int S = seq_lens[b];
    const int n_kv = (t < q1 && S > 0) ? S - (q1 - q0) + (t - q0) + 1 : 0;   // causal: positions [0, pos]
    int chunk = (n_kv + n_splits - 1) / n_splits;
    chunk = (chunk + PC - 1) / PC * PC;
    if (chunk < 2 * PC) chunk = 2 * PC;
    const int k0 = sp * chunk;
    const int k1 = min(n_kv, k0 + chunk);

    const int h_local = tid >> 4;           // 0..15 : head inside the group
    const int sub = tid & 15;
    const int h = hg * HG + h_local;
    const size_t pidx = ((size_t) t * n_splits + sp) * H + h;

    if (k0 >= k1) {
        if (n_splits > 1) {
            if (sub == 0 && h < H) { part_ml[pidx * 2] = -INFINITY; part_ml[pidx * 2 + 1] = 0.f; }
        } else {
            for (int i = sub; i < R && h < H; i += 16) o_lat[((size_t) t * H + h) * R + i] = __float2bfloat16(0.f);
        }
        return;
    }

    for (int i = tid; i < HG * D; i += NT) {
        const int hh = i / D, dd = i - hh * D;
        qs[i] = hg * HG + hh < H ? __bfloat162float(q[((size_t) t * H + hg * HG + hh) * D + dd]) * scale : 0.f;
    }

    float acc[R / 16];                      // dims: (sub*2 + 32*i, +1), i < R/32
#pragma unroll
    for (int i = 0; i < R / 16; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int * bt = block_tables + (size_t) b * max_blocks;

    for (int c0 = k0; c0 < k1; c0 += PC) {
        __syncthreads();
        // stage PC latent rows (16-byte vectors; D*2/16 = 72 vectors per row)
        constexpr int VPR = D * 2 / 16;
        for (int i = tid; i < PC * VPR; i += NT) {
            const int j = i / VPR, v = i - j * VPR;
            const int p = c0 + j;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (p < k1) {
                const int blk = bt[p / block_size];
                val = ((const uint4 *) (cache + ((size_t) blk * block_size + p % block_size) * D))[v];
            }
            *(uint4 *) (lat + j * ROWB + v * 16) = val;
        }
        __syncthreads();
        // scores: thread (h_local, sub) -> positions sub and sub+16
        float s0 = 0.f, s1 = 0.f;
        {
            const float * qh = qs + h_local * D;
            const uint8_t * r0 = lat + sub * ROWB;
            const uint8_t * r1 = lat + (sub + 16) * ROWB;
#pragma unroll 4
            for (int v = 0; v < VPR; ++v) {
                const uint4 a = *(const uint4 *) (r0 + v * 16);
                const uint4 bq = *(const uint4 *) (r1 + v * 16);
                const __nv_bfloat162 * pa = (const __nv_bfloat162 *) &a;
                const __nv_bfloat162 * pb = (const __nv_bfloat162 *) &bq;
                const float4 qa = *(const float4 *) (qh + v * 8);
                const float4 qb = *(const float4 *) (qh + v * 8 + 4);
                float2 f;
                f = __bfloat1622float2(pa[0]); s0 += f.x * qa.x + f.y * qa.y;
                f = __bfloat1622float2(pa[1]); s0 += f.x * qa.z + f.y * qa.w;
                f = __bfloat1622float2(pa[2]); s0 += f.x * qb.x + f.y * qb.y;
                f = __bfloat1622float2(pa[3]); s0 += f.x * qb.z + f.y * qb.w;
                f = __bfloat1622float2(pb[0]); s1 += f.x * qa.x + f.y * qa.y;
                f = __bfloat1622float2(pb[1]); s1 += f.x * qa.z + f.y * qa.w;
                f = __bfloat1622float2(pb[2]); s1 += f.x * qb.x + f.y * qb.y;
                f = __bfloat1622float2(pb[3]); s1 += f.x * qb.z + f.y * qb.w;
            }
        }
        if (c0 + sub >= k1) s0 = -INFINITY;
        if (c0 + sub + 16 >= k1) s1 = -INFINITY;
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run, mx);
        const float p0 = __expf(s0 - m_new), p1 = __expf(s1 - m_new);
        float ls = p0 + p1;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
        const float corr = __expf(m_run - m_new);
        l_run = l_run * corr + ls;
        m_run = m_new;
        ps[h_local * PC + sub] = p0;
        ps[h_local * PC + sub + 16] = p1;
#pragma unroll
        for (int i = 0; i < R / 16; ++i) acc[i] *= corr;
        __syncwarp();
        // o += p * c : this thread's dims are words (sub + 16*i) of each latent row
        const float * ph = ps + h_local * PC;
#pragma unroll 2
        for (int j = 0; j < PC; ++j) {
            const float pj = ph[j];
            const __nv_bfloat162 * rowp = (const __nv_bfloat162 *) (lat + j * ROWB);
#pragma unroll
            for (int i = 0; i < R / 32; ++i) {
                const float2 f = __bfloat1622float2(rowp[sub + 16 * i]);
                acc[2 * i] += pj * f.x;
                acc[2 * i + 1] += pj * f.y;
            }
        }
    }

    if (h >= H) {
        // padding head of a partial head group: nothing to store
    } else if (n_splits > 1) {
        float * po = part_o + pidx * R;
#pragma unroll
        for (int i = 0; i < R / 32; ++i) *(float2 *) (po + 2 * (sub + 16 * i)) = make_float2(acc[2 * i], acc[2 * i + 1]);
        if (sub == 0) { part_ml[pidx * 2] = m_run; part_ml[pidx * 2 + 1] = l_run; }
    } else {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16 * po = o_lat + ((size_t) t * H + h) * R;
#pragma unroll
        for (int i = 0; i < R / 32; ++i)
            *(__nv_bfloat162 *) (po + 2 * (sub + 16 * i)) = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
    }
}

// grid (T, H); 128 threads. Merges split partials.
template <int R>
__device__ __noinline__ void mla_combine_head(const float * __restrict__ part_o, const float * __restrict__ part_ml, int n_splits, int H,
                                              bf16 * __restrict__ o_lat, float * wsm, bool dry) {
    // n_splits <= 32: warp 0 turns the (m, l) pairs into normalised weights, then every thread sums its
    // dims over the splits with independent loads.  dry: same instructions, no stores (see pdl.cuh: warm_enabled).
    const int t = blockIdx.x, h = blockIdx.y;
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        float m = -INFINITY, l = 0.f;
        if (s < n_splits) {
            const size_t pidx = ((size_t) t * n_splits + s) * H + h;
            m = part_ml[pidx * 2];
            l = part_ml[pidx * 2 + 1];
        }
        float M = m;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w = (l > 0.f && M > -INFINITY) ? __expf(m - M) : 0.f;
        float L = l * w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        wsm[s] = L > 0.f ? w / L : 0.f;
    }
    __syncthreads();
    // float4 per thread, 8 splits unrolled: enough independent loads in flight to cover L2 latency
    for (int i = threadIdx.x * 4; i < R; i += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) {
            const float w = wsm[s];
            const float4 v = *(const float4 *) (part_o + (((size_t) t * n_splits + s) * H + h) * R + i);
            if (w > 0.f) {                       // empty splits never wrote part_o
                acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
            }
        }
        __nv_bfloat162 * po = (__nv_bfloat162 *) (o_lat + ((size_t) t * H + h) * R + i);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        if (!dry) {
            po[0] = lo;
            po[1] = hi;
        }
    }
    __syncthreads();
}

template <int R>
__global__ void mla_attn_combine_kernel(const float * __restrict__ part_o, const float * __restrict__ part_ml, int n_splits, int H,
                                        bf16 * __restrict__ o_lat, int warm) {
    JIB_KS(3, 0);
    PDL_TRIGGER_TOP();
    __shared__ float wsm[32];
    if (warm) mla_combine_head<R>(part_o, part_ml, n_splits, H, o_lat, wsm, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(3, 1);
    mla_combine_head<R>(part_o, part_ml, n_splits, H, o_lat, wsm, false);
    JIB_KS(3, 9);
}

}  // namespace

JIB_TL_DEFINE_SETTER(attn)

extern "C" int jib_mla_attention(const void * q, const void * cache, const int * block_tables, int max_blocks, const int * seq_lens,
                                 const int * q_start, int n_seqs, int T, int H, int r, int dr, int block_size, float scale, int n_splits,
                                 float * part_o, float * part_ml, void * o_lat, void * stream) {
    if (T <= 0) return 0;
    if (n_splits < 1) return JIB_E_ARG;
    cudaStream_t s = (cudaStream_t) stream;
    dim3 grid(T, n_splits, (H + HG - 1) / HG);
#define JIB_MLA_CASE(R_, DR_)                                                                                                   \
    if (r == R_ && dr == DR_) {                                                                                                  \
        constexpr int D = R_ + DR_;                                                                                              \
        const size_t smem = HG * D * sizeof(float) + PC * (D * 2 + 16) + HG * PC * sizeof(float);                                \
        static bool attr = false;                                                                                                \
        if (!attr) {                                                                                                             \
            if (cudaFuncSetAttribute(mla_attn_split_kernel<R_, DR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != \
                cudaSuccess)                                                                                                     \
                return JIB_E_LAUNCH;                                                                                             \
            attr = true;                                                                                                         \
        }                                                                                                                        \
        JIB_LAUNCH((mla_attn_split_kernel<R_, DR_>), grid, NT, smem, s, (const bf16 *) q, (const bf16 *) cache, block_tables, max_blocks,  \
                                                              seq_lens, q_start, n_seqs, H, block_size, scale, n_splits, part_o, \
                                                              part_ml, (bf16 *) o_lat);                                          \
        if (cudaGetLastError() != cudaSuccess) return JIB_E_LAUNCH;                                                              \
        if (n_splits > 1) {                                                                                                      \
            JIB_LAUNCH((mla_attn_combine_kernel<R_>), dim3(T, H), 128, 0, s, part_o, part_ml, n_splits, H, (bf16 *) o_lat, jib::warm_for(T));                \
            if (cudaGetLastError() != cudaSuccess) return JIB_E_LAUNCH;                                                          \
        }                                                                                                                        \
        return 0;                                                                                                                \
    }
    JIB_MLA_CASE(512, 64)
    JIB_MLA_CASE(64, 16)
#undef JIB_MLA_CASE
    return JIB_E_ARG;
}

// Merge of split-KV partials (m, l, o) written by either attention kernel.  r in {512, 64}.
extern "C" int jib_mla_combine(const float * part_o, const float * part_ml, int n_splits, int T, int H, int r, void * o_lat,
                               void * stream) {
    if (T <= 0) return 0;
    if (n_splits < 1 || n_splits > 32) return JIB_E_ARG;
    cudaStream_t s = (cudaStream_t) stream;
    if (r == 512) JIB_LAUNCH((mla_attn_combine_kernel<512>), dim3(T, H), 128, 0, s, part_o, part_ml, n_splits, H, (bf16 *) o_lat, jib::warm_for(T));
    else if (r == 64) JIB_LAUNCH((mla_attn_combine_kernel<64>), dim3(T, H), 128, 0, s, part_o, part_ml, n_splits, H, (bf16 *) o_lat, jib::warm_for(T));
    else return JIB_E_ARG;
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}
