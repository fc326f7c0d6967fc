// Memory-bound kernels: embedding gather, fused residual-add + RMSNorm, the MLA "post" kernel
// (latent RMSNorm + YaRN RoPE + paged cache write + q RoPE), argmax / top-k over the vocabulary,
// KV block copy and row gather.  All use 16-byte vector accesses and fp32 statistics.
//
// Reference ops replaced: ascendc_get_row_* (ggml/src/ggml-cann/aclnn_ops.cpp:4404-4500), aclnnRmsNorm
// (3140-3229), ggml_cann_rope + concat + cpy/scatter-update (5160-5260, 6052-6129), aclnnTopk presample
// (ggml/src/ggml-cann/aclnn_ops.h:675-708), the defrag copy graph (src/llama-graph-defrag.cpp:23-85).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "bounds_check.cuh"
#include "jib_kernels.h"
#include "pdl.cuh"
#include "timeline.cuh"
#include "sm100.cuh"

namespace {

typedef __nv_bfloat16 bf16;

struct alignas(16) bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int NT>
__device__ __forceinline__ float block_sum(float v, float * red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = l < NT / 32 ? red[l] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

// ---------------------------------------------------------------------------------------------
__global__ void embed_gather_kernel(const bf16 * __restrict__ table, const int * __restrict__ ids, bf16 * __restrict__ out, int d,
                                    int n_vocab) {
    JIB_KS(6, 0);
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(6, 1);
    const int t = blockIdx.x;
    int id = ids[t];
    JIB_BC(id >= 0 && id < n_vocab, 12, id);
    id = id < 0 ? 0 : (id >= n_vocab ? n_vocab - 1 : id);
    const uint4 * src = (const uint4 *) (table + (size_t) id * d);
    uint4 * dst = (uint4 *) (out + (size_t) t * d);
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
    JIB_KS(6, 9);
}

// out_sum = x + residual (bf16-rounded), out_norm = rmsnorm(out_sum) * w.  One block per row.
// dry: the same instructions without the stores (see pdl.cuh: warm_enabled).
template <int NT, int MAXV>
__device__ __noinline__ void rmsnorm_row(const bf16 * __restrict__ x, const bf16 * __restrict__ residual, const float * __restrict__ w,
                                         bf16 * __restrict__ out_norm, bf16 * __restrict__ out_sum, int d, long long x_stride, float eps,
                                         float * red, bool dry) {
    const int t = blockIdx.x;
    const bf16x8 * xr = (const bf16x8 *) (x + (size_t) t * x_stride);
    const bf16x8 * rr = residual ? (const bf16x8 *) (residual + (size_t) t * d) : nullptr;
    const int nv = d / 8;
    float vals[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            bf16x8 a = xr[i];
            if (rr) {
                bf16x8 b = rr[i];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 fa = __bfloat1622float2(a.v[j]), fb = __bfloat1622float2(b.v[j]);
                    a.v[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
                }
            }
            if (out_sum && !dry) ((bf16x8 *) (out_sum + (size_t) t * d))[i] = a;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(a.v[j]);
                vals[it][2 * j] = f.x;
                vals[it][2 * j + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = block_sum<NT>(ss, red);
    const float inv = rsqrtf(ss / (float) d + eps);
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            const float4 w0 = ((const float4 *) w)[2 * i], w1 = ((const float4 *) w)[2 * i + 1];
            bf16x8 o;
            o.v[0] = __floats2bfloat162_rn(vals[it][0] * inv * w0.x, vals[it][1] * inv * w0.y);
            o.v[1] = __floats2bfloat162_rn(vals[it][2] * inv * w0.z, vals[it][3] * inv * w0.w);
            o.v[2] = __floats2bfloat162_rn(vals[it][4] * inv * w1.x, vals[it][5] * inv * w1.y);
            o.v[3] = __floats2bfloat162_rn(vals[it][6] * inv * w1.z, vals[it][7] * inv * w1.w);
            if (!dry) ((bf16x8 *) (out_norm + (size_t) t * d))[i] = o;
        }
    }
}

template <int NT, int MAXV>
__global__ void __launch_bounds__(NT) rmsnorm_kernel(const bf16 * __restrict__ x, const bf16 * __restrict__ residual,
                                                     const float * __restrict__ w, bf16 * __restrict__ out_norm,
                                                     bf16 * __restrict__ out_sum, int d, long long x_stride, float eps, int warm) {
    JIB_KS(4, 0);
    PDL_TRIGGER_TOP();
    __shared__ float red[32];
    if (warm) rmsnorm_row<NT, MAXV>(x, residual, w, out_norm, out_sum, d, x_stride, eps, red, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(4, 1);
    rmsnorm_row<NT, MAXV>(x, residual, w, out_norm, out_sum, d, x_stride, eps, red, false);
    JIB_KS(4, 9);
}

// One block per token: c = rmsnorm(ckv[:r]) * w -> cache[slot][:r]; k_pe = rope(ckv[r:]) -> cache[slot][r:];
// q_pe = rope(q[h][dn:]) -> q_out[t][h][r:].  rope_table [max_pos][dr/2][2] holds (cos, sin) * magnitude.
// dry: the same instructions without stores or status reports.
template <int NT>
__device__ __noinline__ void mla_qkv_post_row(const bf16 * __restrict__ q, long long q_stride, const bf16 * __restrict__ ckv,
                                              long long ckv_stride, const float * __restrict__ kv_norm_w, float eps,
                                              const float * __restrict__ rope_table, const int * __restrict__ positions,
                                              const int * __restrict__ slot_mapping, bf16 * __restrict__ cache, bf16 * __restrict__ q_out,
                                              long long qo_row, long long qo_head, int H, int dn, int dr, int r, int max_pos,
                                              long long n_slots, int * status, float * red, bool dry) {
    const int t = blockIdx.x;
    const int slot = slot_mapping[t];
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (slot >= 0 && !dry) jib_report(status, JIB_ERR_BOUNDS, 10, pos);
        pos = pos < 0 ? 0 : max_pos - 1;
    }
    const float * cs = rope_table + (size_t) pos * dr;       // dr/2 pairs * 2
    const bf16 * crow = ckv + (size_t) t * ckv_stride;
    // latent RMSNorm
    float ss = 0.f;
    for (int i = threadIdx.x; i < r; i += NT) {
        const float v = __bfloat162float(crow[i]);
        ss += v * v;
    }
    ss = block_sum<NT>(ss, red);
    const float inv = rsqrtf(ss / (float) r + eps);
    const bool write_kv = slot >= 0 && slot < n_slots;
    if (slot >= n_slots && !dry) jib_report(status, JIB_ERR_BOUNDS, 11, slot);
    if (write_kv) {
        bf16 * dst = cache + (size_t) slot * (r + dr);
        for (int i = threadIdx.x; i < r; i += NT) {
            const bf16 v = __float2bfloat16(__bfloat162float(crow[i]) * inv * kv_norm_w[i]);
            if (!dry) dst[i] = v;
        }
        for (int i = threadIdx.x; i < dr / 2; i += NT) {
            const float x0 = __bfloat162float(crow[r + 2 * i]), x1 = __bfloat162float(crow[r + 2 * i + 1]);
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const __nv_bfloat162 v = __floats2bfloat162_rn(x0 * c - x1 * s, x0 * s + x1 * c);
            if (!dry) *(__nv_bfloat162 *) (dst + r + 2 * i) = v;
        }
    }
    // q rope: H * dr/2 pairs
    const int half = dr / 2;
    const bf16 * qrow = q + (size_t) t * q_stride;
    bf16 * qo = q_out + (size_t) t * qo_row;      // q_out points at the first RoPE element of token 0, head 0
    for (int i = threadIdx.x; i < H * half; i += NT) {
        const int h = i / half, p = i - h * half;
        const __nv_bfloat162 xx = *(const __nv_bfloat162 *) (qrow + (size_t) h * (dn + dr) + dn + 2 * p);
        const float2 f = __bfloat1622float2(xx);
        const float c = cs[2 * p], s = cs[2 * p + 1];
        const __nv_bfloat162 v = __floats2bfloat162_rn(f.x * c - f.y * s, f.x * s + f.y * c);
        if (!dry) *(__nv_bfloat162 *) (qo + (size_t) h * qo_head + 2 * p) = v;
    }
}

template <int NT>
__global__ void __launch_bounds__(NT) mla_qkv_post_kernel(const bf16 * __restrict__ q, long long q_stride, const bf16 * __restrict__ ckv,
                                                          long long ckv_stride, const float * __restrict__ kv_norm_w, float eps,
                                                          const float * __restrict__ rope_table, const int * __restrict__ positions,
                                                          const int * __restrict__ slot_mapping, bf16 * __restrict__ cache,
                                                          bf16 * __restrict__ q_out, long long qo_row, long long qo_head, int H, int dn,
                                                          int dr, int r, int max_pos, long long n_slots, int * status, int warm) {
    JIB_KS(5, 0);
    PDL_TRIGGER_TOP();
    __shared__ float red[32];
    // positions / slot_mapping are step inputs, uploaded before the first kernel of the step: valid during the dry pass
    if (warm) mla_qkv_post_row<NT>(q, q_stride, ckv, ckv_stride, kv_norm_w, eps, rope_table, positions, slot_mapping, cache, q_out, qo_row,
                                   qo_head, H, dn, dr, r, max_pos, n_slots, status, red, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(5, 1);
    mla_qkv_post_row<NT>(q, q_stride, ckv, ckv_stride, kv_norm_w, eps, rope_table, positions, slot_mapping, cache, q_out, qo_row, qo_head, H,
                         dn, dr, r, max_pos, n_slots, status, red, false);
    JIB_KS(5, 9);
}

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2key(float f) {   // order-preserving float -> uint
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <int NT>
__global__ void __launch_bounds__(NT) argmax_kernel(const float * __restrict__ logits, int * __restrict__ out, int V) {
    JIB_KS(8, 0);
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(8, 1);
    __shared__ unsigned long long best_s[NT / 32];
    const float * row = logits + (size_t) blockIdx.x * V;
    // pack (key, ~index) so that max picks the largest value and, among equals, the lowest index
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < V; i += NT) {
        float v = row[i];
        if (v != v) v = -FLT_MAX;
        const unsigned long long p = ((unsigned long long) f2key(v) << 32) | (uint32_t) (0x7fffffff - i);
        best = p > best ? p : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < NT / 32 ? best_s[threadIdx.x] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (threadIdx.x == 0) out[blockIdx.x] = 0x7fffffff - (int) (best & 0xffffffffu);
    }
    JIB_KS(8, 9);
}

// Exact top-k (k <= 128) of one row per block: 3-pass radix select of the k-th key (11+11+10 bits), then
// collect and rank-sort the winners (descending, ties by lower index).
template <int NT>
__global__ void __launch_bounds__(NT) topk_kernel(const float * __restrict__ logits, float * __restrict__ vals, int * __restrict__ ids,
                                                  int V, int k) {
    JIB_KS(15, 0);
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(15, 1);
    __shared__ int hist[2048];
    __shared__ uint32_t s_prefix, s_mask;
    __shared__ int s_need, s_cnt_gt, s_cnt_eq;
    __shared__ float c_val[128];
    __shared__ int c_idx[128];
    const float * row = logits + (size_t) blockIdx.x * V;
    if (threadIdx.x == 0) { s_prefix = 0; s_mask = 0; s_need = k; }
    const int shifts[3] = {21, 10, 0};
    const int bits[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; ++pass) {
        for (int i = threadIdx.x; i < 2048; i += NT) hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, mask = s_mask;
        const int sh = shifts[pass], nb = 1 << bits[pass];
        for (int i = threadIdx.x; i < V; i += NT) {
            float v = row[i];
            if (v != v) v = -FLT_MAX;
            const uint32_t key = f2key(v);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & (nb - 1)], 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int need = s_need, b = nb - 1;
            for (; b > 0; --b) {
                if (hist[b] >= need) break;
                need -= hist[b];
            }
            s_need = need;                       // still needed inside bin b
            s_prefix = prefix | ((uint32_t) b << sh);
            s_mask = mask | ((uint32_t) (nb - 1) << sh);
        }
        __syncthreads();
    }
    // s_prefix is now the exact key of the k-th largest element; s_need of the equal ones are taken
    const uint32_t kth = s_prefix;
    if (threadIdx.x == 0) { s_cnt_gt = 0; s_cnt_eq = 0; }
    __syncthreads();
    const int n_gt = k - s_need;
    for (int i = threadIdx.x; i < V; i += NT) {
        float v = row[i];
        if (v != v) v = -FLT_MAX;
        const uint32_t key = f2key(v);
        if (key > kth) {
            const int p = atomicAdd(&s_cnt_gt, 1);
            if (p < 128) { c_val[p] = v; c_idx[p] = i; }
        }
    }
    __syncthreads();
    // equal keys: take the lowest indices first -> scan in index order by a single warp-free loop over candidates
    // (ties at the cut are rare; a serial pass by one thread keeps the result deterministic)
    if (threadIdx.x == 0) {
        int taken = 0;
        for (int i = 0; i < V && taken < s_need; ++i) {
            float v = row[i];
            if (v != v) v = -FLT_MAX;
            if (f2key(v) == kth) {
                c_val[n_gt + taken] = v;
                c_idx[n_gt + taken] = i;
                ++taken;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x < k) {
        const float v = c_val[threadIdx.x];
        const int id = c_idx[threadIdx.x];
        int rank = 0;
        for (int j = 0; j < k; ++j) {
            const float o = c_val[j];
            rank += (o > v) || (o == v && c_idx[j] < id);
        }
        vals[(size_t) blockIdx.x * k + rank] = v;
        ids[(size_t) blockIdx.x * k + rank] = id;
    }
    JIB_KS(15, 9);
}

__global__ void kv_block_copy_kernel(bf16 * cache, long long layer_stride, const int * __restrict__ src, const int * __restrict__ dst,
                                     int block_elems) {
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    const int i = blockIdx.x, l = blockIdx.y;
    const uint4 * s = (const uint4 *) (cache + (size_t) l * layer_stride + (size_t) src[i] * block_elems);
    uint4 * d = (uint4 *) (cache + (size_t) l * layer_stride + (size_t) dst[i] * block_elems);
    for (int j = threadIdx.x; j < block_elems / 8; j += blockDim.x) d[j] = s[j];
}

__global__ void gather_rows_kernel(const bf16 * __restrict__ x, const int * __restrict__ src_row, bf16 * __restrict__ out, int d, int n_src) {
    JIB_KS(7, 0);
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(7, 1);
    const int rrow = blockIdx.x;
    const int s = src_row[rrow];
    JIB_BC(s < n_src, 13, s);
    if (s < 0 || s >= n_src) return;   // unowned / out-of-range row: leave the destination untouched
    const uint4 * src = (const uint4 *) (x + (size_t) s * d);
    uint4 * dst = (uint4 *) (out + (size_t) rrow * d);
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
    JIB_KS(7, 9);
}

inline int launched() { return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH; }

}  // namespace

JIB_BC_DEFINE_SETTER(elementwise)
JIB_TL_DEFINE_SETTER(elementwise)

extern "C" {

// 1 when the library was built with -DJIB_BOUNDS_CHECK
JIB_EXPORT int jib_bounds_check_enabled(void) {
#ifdef JIB_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}

int jib_embed_gather(const void * table, const int * ids, void * out, int T, int d, int n_vocab, void * stream) {
    if (T <= 0) return 0;
    if (d % 8) return JIB_E_ARG;
    JIB_LAUNCH((embed_gather_kernel), T, 128, 0, (cudaStream_t) stream, (const bf16 *) table, ids, (bf16 *) out, d, n_vocab);
    return launched();
}

int jib_rmsnorm(const void * x, const void * residual, const float * w, void * out_norm, void * out_sum, int T, int d,
                long long x_stride, float eps, void * stream) {
    if (T <= 0) return 0;
    if (d % 8 || x_stride % 8) return JIB_E_ARG;
    cudaStream_t s = (cudaStream_t) stream;
    const int nv = d / 8;
    if (nv <= 128)
        JIB_LAUNCH((rmsnorm_kernel<128, 1>), T, 128, 0, s, (const bf16 *) x, (const bf16 *) residual, w, (bf16 *) out_norm, (bf16 *) out_sum, d, x_stride, eps, jib::warm_for(T));
    else if (nv <= 256)
        JIB_LAUNCH((rmsnorm_kernel<256, 1>), T, 256, 0, s, (const bf16 *) x, (const bf16 *) residual, w, (bf16 *) out_norm, (bf16 *) out_sum, d, x_stride, eps, jib::warm_for(T));
    else if (nv <= 1024)
        JIB_LAUNCH((rmsnorm_kernel<256, 4>), T, 256, 0, s, (const bf16 *) x, (const bf16 *) residual, w, (bf16 *) out_norm, (bf16 *) out_sum, d, x_stride, eps, jib::warm_for(T));
    else if (nv <= 2048)
        JIB_LAUNCH((rmsnorm_kernel<512, 4>), T, 512, 0, s, (const bf16 *) x, (const bf16 *) residual, w, (bf16 *) out_norm, (bf16 *) out_sum, d, x_stride, eps, jib::warm_for(T));
    else
        return JIB_E_ARG;
    return launched();
}

int jib_mla_qkv_post(const void * q, long long q_stride, const void * ckv, long long ckv_stride, const float * kv_norm_w, float eps,
                     const float * rope_table, const int * positions, const int * slot_mapping, void * cache, void * q_out,
                     long long qo_row, long long qo_head, int T, int H, int dn, int dr, int r, int max_pos, long long n_slots, int * status,
                     void * stream) {
    if (T <= 0) return 0;
    if ((dr & 1) || (dn & 1) || (r & 1) || (q_stride & 1) || (qo_row & 1) || (qo_head & 1) || ((uintptr_t) q_out & 3)) return JIB_E_ARG;
    JIB_LAUNCH((mla_qkv_post_kernel<256>), T, 256, 0, (cudaStream_t) stream, (const bf16 *) q, q_stride, (const bf16 *) ckv, ckv_stride, kv_norm_w,
                                                                    eps, rope_table, positions, slot_mapping, (bf16 *) cache,
                                                                    (bf16 *) q_out, qo_row, qo_head, H, dn, dr, r, max_pos, n_slots, status,
                                                                    jib::warm_for(T));
    return launched();
}

int jib_argmax(const float * logits, int * out, int n, int V, void * stream) {
    if (n <= 0) return 0;
    JIB_LAUNCH((argmax_kernel<1024>), n, 1024, 0, (cudaStream_t) stream, logits, out, V);
    return launched();
}

int jib_topk(const float * logits, float * vals, int * ids, int n, int V, int k, void * stream) {
    if (n <= 0) return 0;
    if (k < 1 || k > 128 || k > V) return JIB_E_ARG;
    JIB_LAUNCH((topk_kernel<1024>), n, 1024, 0, (cudaStream_t) stream, logits, vals, ids, V, k);
    return launched();
}

int jib_kv_block_copy(void * cache, long long layer_stride_elems, int n_layers, const int * src, const int * dst, int n, int block_elems,
                      void * stream) {
    if (n <= 0) return 0;
    if (block_elems % 8) return JIB_E_ARG;
    JIB_LAUNCH((kv_block_copy_kernel), dim3(n, n_layers), 256, 0, (cudaStream_t) stream, (bf16 *) cache, layer_stride_elems, src, dst, block_elems);
    return launched();
}

int jib_gather_rows(const void * x, const int * src_row, void * out, int rows, int d, int n_src, void * stream) {
    if (rows <= 0) return 0;
    if (d % 8) return JIB_E_ARG;
    JIB_LAUNCH((gather_rows_kernel), rows, 128, 0, (cudaStream_t) stream, (const bf16 *) x, src_row, (bf16 *) out, d, n_src);
    return launched();
}

}  // extern "C"
