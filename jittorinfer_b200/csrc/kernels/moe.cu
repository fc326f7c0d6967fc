// MoE routing kernels: fused router (fp32 matmul + softmax/sigmoid + [group-limited] top-k + renorm/scale),
// expert-sorted permutation with device-side segment offsets, and the weighted top-k combine.
//
// Reference: router + softmax + full argsort + slice + gather + scale as separate graph ops
// (src/llama-graph-ffn.cpp:145-197), aclnnMoeInitRouting + a device->host copy and host binary search for the
// local expert range (ggml/src/ggml-cann/aclnn_ops.cpp:2129-2168), aclnnMoeFinalizeRoutingV2 (2540-2542).
// Here nothing leaves the device and expert-parallel ranks simply mark foreign experts as "not local".
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "bounds_check.cuh"
#include "jib_kernels.h"
#include "pdl.cuh"
#include "timeline.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAX_E = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Router logits in fp32: logits[t][e] = sum_i g[t][i] * w_router[e][i].
// One expert per CTA, 256 threads; thread i owns the 8-element chunks i, i + 256, ... of the d axis (its router row slice
// stays in registers), tokens are walked in groups of 8 so that every load of a group is independent -- the kernel is
// latency-bound, so memory-level parallelism is what matters.
//
// With norm_w the rows of x are first RMS-normalised: thread mapping, accumulation order and reduction tree are those of
// rmsnorm_kernel<256, *> (elementwise.cu), so the bf16 row the dot product sees -- and the row CTA (t mod gridDim.x)
// stores to g_out -- is bit for bit what that kernel would have produced.
constexpr int GATE_TG = 8;
constexpr int GATE_NT = 256;
constexpr int GATE_MAXC = 4;      // 8-element chunks per thread: d <= 4 * 256 * 8 = 8192

struct alignas(16) bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __noinline__ void router_rows(const bf16 * __restrict__ x, const float * __restrict__ w_router, const float * __restrict__ norm_w,
                                            float eps, bf16 * __restrict__ g_out, float * __restrict__ logits, int t_begin, int t_end,
                                            int T, int d, int E, int e, float (*red)[GATE_TG], float * inv_s, bool dry = false) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nv = d / 8;
    float4 w[GATE_MAXC][2];
    float4 nw[GATE_MAXC][2];
#pragma unroll
    for (int c = 0; c < GATE_MAXC; ++c) {
        const int i = threadIdx.x + c * GATE_NT;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        w[c][0] = i < nv ? ((const float4 *) (w_router + (size_t) e * d))[2 * i] : z;
        w[c][1] = i < nv ? ((const float4 *) (w_router + (size_t) e * d))[2 * i + 1] : z;
        nw[c][0] = (norm_w != nullptr && i < nv) ? ((const float4 *) norm_w)[2 * i] : z;
        nw[c][1] = (norm_w != nullptr && i < nv) ? ((const float4 *) norm_w)[2 * i + 1] : z;
    }
    for (int t0 = t_begin; t0 < t_end; t0 += GATE_TG) {
        if (norm_w != nullptr) {
            // sum of squares per token, then 1 / rms: warp w finishes token t0 + w
            float ss[GATE_TG];
#pragma unroll
            for (int j = 0; j < GATE_TG; ++j) ss[j] = 0.f;
#pragma unroll
            for (int c = 0; c < GATE_MAXC; ++c) {
                const int i = threadIdx.x + c * GATE_NT;
                if (i < nv) {
#pragma unroll
                    for (int j = 0; j < GATE_TG; ++j) {
                        const int t = min(t0 + j, T - 1);
                        const bf16x8 a = ((const bf16x8 *) (x + (size_t) t * d))[i];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 f = __bfloat1622float2(a.v[q]);
                            ss[j] += f.x * f.x + f.y * f.y;
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < GATE_TG; ++j) {
                const float s = warp_sum(ss[j]);
                if (lane == 0) red[warp][j] = s;
            }
            __syncthreads();
            {
                float t = lane < GATE_NT / 32 ? red[lane][warp] : 0.f;
                t = warp_sum(t);
                if (lane == 0) inv_s[warp] = rsqrtf(t / (float) d + eps);
            }
            __syncthreads();
        }
        float acc[GATE_TG];
#pragma unroll
        for (int j = 0; j < GATE_TG; ++j) acc[j] = 0.f;
#pragma unroll
        for (int c = 0; c < GATE_MAXC; ++c) {
            const int i = threadIdx.x + c * GATE_NT;
            if (i < nv) {
#pragma unroll
                for (int j = 0; j < GATE_TG; ++j) {
                    const int t = min(t0 + j, T - 1);
                    bf16x8 a = ((const bf16x8 *) (x + (size_t) t * d))[i];
                    if (norm_w != nullptr) {
                        const float inv = inv_s[j];
                        const float2 f0 = __bfloat1622float2(a.v[0]), f1 = __bfloat1622float2(a.v[1]);
                        const float2 f2 = __bfloat1622float2(a.v[2]), f3 = __bfloat1622float2(a.v[3]);
                        a.v[0] = __floats2bfloat162_rn(f0.x * inv * nw[c][0].x, f0.y * inv * nw[c][0].y);
                        a.v[1] = __floats2bfloat162_rn(f1.x * inv * nw[c][0].z, f1.y * inv * nw[c][0].w);
                        a.v[2] = __floats2bfloat162_rn(f2.x * inv * nw[c][1].x, f2.y * inv * nw[c][1].y);
                        a.v[3] = __floats2bfloat162_rn(f3.x * inv * nw[c][1].z, f3.y * inv * nw[c][1].w);
                        if (g_out != nullptr && !dry && t0 + j < t_end && (t0 + j) % (int) gridDim.x == (int) blockIdx.x)
                            ((bf16x8 *) (g_out + (size_t) (t0 + j) * d))[i] = a;
                    }
                    const float2 f0 = __bfloat1622float2(a.v[0]), f1 = __bfloat1622float2(a.v[1]);
                    const float2 f2 = __bfloat1622float2(a.v[2]), f3 = __bfloat1622float2(a.v[3]);
                    acc[j] += w[c][0].x * f0.x + w[c][0].y * f0.y + w[c][0].z * f1.x + w[c][0].w * f1.y +
                              w[c][1].x * f2.x + w[c][1].y * f2.y + w[c][1].z * f3.x + w[c][1].w * f3.y;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < GATE_TG; ++j) {
            const float s = warp_sum(acc[j]);
            if (lane == 0) red[warp][j] = s;
        }
        __syncthreads();
        if (threadIdx.x < GATE_TG && t0 + threadIdx.x < t_end) {
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < GATE_NT / 32; ++q) s += red[q][threadIdx.x];
            if (!dry) logits[(size_t) (t0 + threadIdx.x) * E + e] = s;
        }
        __syncthreads();
    }
}

// grid (E, ceil(T/64))
__global__ void __launch_bounds__(GATE_NT) router_logits_kernel(const bf16 * __restrict__ g, const float * __restrict__ w_router,
                                                                float * __restrict__ logits, int T, int d, int E, int warm) {
    JIB_KS(9, 0);
    PDL_TRIGGER_TOP();
    __shared__ float red[GATE_NT / 32][GATE_TG];
    if (warm)          // one token group, no stores: the code and this expert's router row are on the SM before the inputs are
        router_rows(g, w_router, nullptr, 0.f, nullptr, logits, blockIdx.y * 64, min(T, (int) blockIdx.y * 64 + GATE_TG), T, d, E,
                    blockIdx.x, red, nullptr, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(9, 1);
    router_rows(g, w_router, nullptr, 0.f, nullptr, logits, blockIdx.y * 64, min(T, (int) (blockIdx.y + 1) * 64), T, d, E, blockIdx.x, red,
                nullptr);
    JIB_KS(9, 9);
}

// Gating of one token by one warp: softmax/sigmoid over the logits, optional group-limited masking, k rounds of arg-max.
// prob / sel: MAX_E floats each, gscore: 32 floats, all private to the warp.  Not inlined: the fused router calls it twice
// (a dry run, then the real one) and both calls must execute the same copy of the code.
__device__ __noinline__ void gate_token(const float * __restrict__ logits_row, const float * __restrict__ bias, int * __restrict__ ids,
                                           float * __restrict__ wts, int t, int E, int k, int n_group, int topk_group, float scale,
                                           int norm, int sigmoid, int n_shared, int group_top2, float * prob, float * sel,
                                           float * gscore, int * ids_copy = nullptr, bool dry = false) {
    // dry: runs the same instructions on whatever `prob` holds and stores nothing -- a caller that is still waiting for its
    // inputs uses it to pull this code into the SM's instruction cache ahead of the real call
    const int lane = threadIdx.x & 31;
    const int ld = k + n_shared;
    if (!dry)
        for (int e = lane; e < E; e += 32) prob[e] = __ldcg(logits_row + e);      // possibly written by other CTAs: from L2
    __syncwarp();
    // softmax / sigmoid over E (E <= 256 -> 8 per lane)
    float mx = -FLT_MAX;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, prob[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float p = sigmoid ? 1.f / (1.f + expf(-prob[e])) : expf(prob[e] - mx);
        prob[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        if (!sigmoid) prob[e] = prob[e] / sum;
        sel[e] = prob[e] + (bias ? bias[e] : 0.f);
    }
    __syncwarp();
    if (n_group > 1) {
        const int gs = E / n_group;
        if (lane < n_group) {
            // a group's score: its best expert (DeepSeek-V2) or the sum of its two best (DeepSeek-V3)
            float m = -FLT_MAX, m2 = -FLT_MAX;
            for (int j = 0; j < gs; ++j) {
                const float v = sel[lane * gs + j];
                if (v > m) { m2 = m; m = v; } else if (v > m2) { m2 = v; }
            }
            gscore[lane] = (group_top2 && gs >= 2) ? m + m2 : m;
        }
        __syncwarp();
        // keep the topk_group best groups (ties -> lower group id): rank of my group
        if (lane < n_group) {
            int rank = 0;
            const float mine = gscore[lane];
            for (int j = 0; j < n_group; ++j) rank += (gscore[j] > mine) || (gscore[j] == mine && j < lane);
            if (rank >= topk_group)
                for (int j = 0; j < gs; ++j) sel[lane * gs + j] = -INFINITY;
        }
        __syncwarp();
    }
    // k rounds of warp arg-max (ties -> lower expert id); lane `round` keeps that round's pick
    float wsum = 0.f, my_w = 0.f;
    int my_id = 0;
    for (int round = 0; round < k; ++round) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sel[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) bi = 0;     // a -inf that was already masked can only be re-picked when fewer than k experts are eligible
        const float p = prob[bi];
        if (lane == round) { my_id = bi; my_w = p; }
        if (lane == 0) sel[bi] = -INFINITY;
        wsum += p;
        __syncwarp();
    }
    if (lane < k) {
        float w = my_w;
        if (norm) w /= wsum;
        if (!dry) {
            ids[(size_t) t * ld + lane] = my_id;
            wts[(size_t) t * ld + lane] = w * scale;
        }
        if (ids_copy != nullptr) ids_copy[t * ld + lane] = my_id;
    } else if (lane < ld) {
        // shared experts ride along as always-selected experts E, E+1, ... with weight 1
        if (!dry) {
            ids[(size_t) t * ld + lane] = E + (lane - k);
            wts[(size_t) t * ld + lane] = 1.f;
        }
        if (ids_copy != nullptr) ids_copy[t * ld + lane] = E + (lane - k);
    }
}

// One warp per token.
__global__ void __launch_bounds__(32) moe_gate_kernel(const float * __restrict__ logits, const float * __restrict__ bias,
                                                      int * __restrict__ ids, float * __restrict__ wts, int E, int k, int n_group,
                                                      int topk_group, float scale, int norm, int sigmoid, int n_shared,
                                                      int group_top2, int warm) {
    JIB_KS(10, 0);
    PDL_TRIGGER_TOP();
    __shared__ float prob[MAX_E];
    __shared__ float sel[MAX_E];
    __shared__ float gscore[32];
    const int t = blockIdx.x;
    if (warm) {
        for (int e = threadIdx.x & 31; e < MAX_E; e += 32) prob[e] = (float) ((e * 37 + t) & 63);
        __syncwarp();
        gate_token(nullptr, bias == nullptr ? nullptr : (const float *) prob, nullptr, nullptr, 0, E, k, n_group, topk_group, scale, norm,
                   sigmoid, n_shared, group_top2, prob, sel, gscore, nullptr, true);
        __syncwarp();
    }
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(10, 1);
    gate_token(logits + (size_t) t * E, bias, ids, wts, t, E, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2, prob,
               sel, gscore);
    JIB_KS(10, 9);
}

// Stable counting sort of n (token, slot) pairs by local expert id, by all threads of one CTA (a multiple of 32).
// seg[e] .. seg[e+1] delimit expert e's rows; src_token[row] = token feeding sorted row; dest[i] = row or -1.
// Every warp walks the id list twice per expert it owns, so `ids` should sit in shared memory (SORT_SMEM_MAX ids fit the
// callers' staging buffers); a global pointer works too, at an L2 round trip per 32 ids.
constexpr int SORT_SMEM_MAX = 4096;
__device__ __noinline__ void sort_pairs(const int * __restrict__ ids, int n, int k, int expert_base, int E_local, int * __restrict__ seg,
                                           int * __restrict__ src_token, int * __restrict__ dest, int * count, int * offs,
                                           bool dry = false, int * __restrict__ active = nullptr) {
    // dry: same instructions, no global stores (instruction-cache warm-up, see gate_token)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < E_local; e += nw) {
        int c = 0;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < n && ids[i] - expert_base == e;
            c += __popc(__ballot_sync(0xffffffffu, hit));
        }
        if (lane == 0) count[e] = c;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        // exclusive prefix over the experts by one warp (E_local <= 256: 8 per lane)
        int run = 0;
        for (int e0 = 0; e0 < E_local; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < E_local ? count[e] : 0;
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            if (e < E_local) offs[e] = run + inc - c;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) offs[E_local] = run;
        if (active != nullptr && !dry) {
            // the experts that have rows, in order, then -1: grouped launches of small batches cover this list only
            int n_act = 0;
            for (int e0 = 0; e0 < E_local; e0 += 32) {
                const int e = e0 + lane;
                const bool has = e < E_local && count[e] > 0;
                const unsigned m = __ballot_sync(0xffffffffu, has);
                if (has) active[n_act + __popc(m & ((1u << lane) - 1))] = e;
                n_act += __popc(m);
            }
            for (int i = n_act + lane; i < E_local; i += 32) active[i] = -1;
        }
    }
    __syncthreads();
    if (!dry) {
        for (int e = threadIdx.x; e <= E_local; e += blockDim.x) seg[e] = offs[e];
        for (int i = offs[E_local] + threadIdx.x; i < n; i += blockDim.x) src_token[i] = -1;   // rows no local expert owns
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int le = ids[i] - expert_base;
            if (le < 0 || le >= E_local) dest[i] = -1;
        }
    }
    for (int e = warp; e < E_local; e += nw) {
        int base = offs[e];
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < n && ids[i] - expert_base == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit && !dry) {
                const int row = base + __popc(m & ((1u << lane) - 1));
                dest[i] = row;
                if (row < n) src_token[row] = i / k;
            }
            base += __popc(m);
        }
    }
}

__global__ void __launch_bounds__(1024) moe_permute_kernel(const int * __restrict__ ids, int n, int k, int expert_base, int E_local,
                                                          int * __restrict__ seg, int * __restrict__ src_token, int * __restrict__ dest,
                                                          int warm, int * __restrict__ active) {
    JIB_KS(11, 0);
    PDL_TRIGGER_TOP();
    __shared__ int count[MAX_E + 1];
    __shared__ int offs[MAX_E + 1];
    __shared__ int ids_s[SORT_SMEM_MAX];
    if (warm) {
        for (int i = threadIdx.x; i < 32; i += blockDim.x) ids_s[i] = expert_base + (i % max(E_local, 1));
        __syncthreads();
        sort_pairs(ids_s, min(n, 32), k, expert_base, E_local, nullptr, nullptr, nullptr, count, offs, true);
        __syncthreads();
    }
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(11, 1);
    if (n <= SORT_SMEM_MAX) {
        for (int i = threadIdx.x; i < n; i += blockDim.x) ids_s[i] = ids[i];
        __syncthreads();
    }
    sort_pairs(n <= SORT_SMEM_MAX ? ids_s : ids, n, k, expert_base, E_local, seg, src_token, dest, count, offs, false, active);
    JIB_KS(11, 9);
}

// ---- the same sort for large n (prefill) on many CTAs: histogram per 1024-pair chunk, scan, stable scatter ----------
// tmp: int[n_chunks][E_local], chunk c covers pairs [c*1024, (c+1)*1024).
constexpr int PERM_CHUNK = 1024;

__global__ void __launch_bounds__(PERM_CHUNK) permute_count_kernel(const int * __restrict__ ids, int n, int expert_base, int E_local,
                                                                   int * __restrict__ tmp) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    __shared__ int hist[MAX_E];
    for (int e = threadIdx.x; e < E_local; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * PERM_CHUNK + threadIdx.x;
    if (i < n) {
        const int le = ids[i] - expert_base;
        if (le >= 0 && le < E_local) atomicAdd(&hist[le], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E_local; e += blockDim.x) tmp[(size_t) blockIdx.x * E_local + e] = hist[e];
}

// One CTA: tmp[c][e] becomes the first sorted row of chunk c's pairs of expert e; seg[e] the expert's first row.
__global__ void __launch_bounds__(MAX_E) permute_scan_kernel(int * __restrict__ tmp, int n_chunks, int E_local, int n, int * __restrict__ seg,
                                                            int * __restrict__ src_token) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    __shared__ int total[MAX_E + 1];
    const int e = threadIdx.x;
    int acc = 0;
    if (e < E_local) {
        for (int c = 0; c < n_chunks; ++c) {
            const int v = tmp[(size_t) c * E_local + e];
            tmp[(size_t) c * E_local + e] = acc;       // rows of expert e in earlier chunks
            acc += v;
        }
        total[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int x = 0; x < E_local; ++x) { const int v = total[x]; total[x] = run; run += v; }
        total[E_local] = run;
    }
    __syncthreads();
    if (e < E_local) {
        seg[e] = total[e];
        for (int c = 0; c < n_chunks; ++c) tmp[(size_t) c * E_local + e] += total[e];
    }
    if (threadIdx.x == 0) seg[E_local] = total[E_local];
    for (int i = total[E_local] + threadIdx.x; i < n; i += blockDim.x) src_token[i] = -1;      // rows no local expert owns
}

__global__ void __launch_bounds__(PERM_CHUNK) permute_scatter_kernel(const int * __restrict__ ids, int n, int k, int expert_base, int E_local,
                                                                     const int * __restrict__ tmp, int * __restrict__ src_token,
                                                                     int * __restrict__ dest) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    extern __shared__ int warp_cnt[];              // [32 warps][E_local]: pairs of expert e in warp w, then their prefix over w
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int x = threadIdx.x; x < 32 * E_local; x += blockDim.x) warp_cnt[x] = 0;
    __syncthreads();
    const int i = blockIdx.x * PERM_CHUNK + threadIdx.x;
    int le = -1;
    if (i < n) {
        le = ids[i] - expert_base;
        if (le < 0 || le >= E_local) le = -1;
    }
    // lanes of this warp with the same expert: rank among them keeps the order of the pair indices
    const unsigned same = __match_any_sync(0xffffffffu, le);
    const int rank = __popc(same & ((1u << lane) - 1));
    if (le >= 0 && rank == 0) warp_cnt[warp * E_local + le] = __popc(same);
    __syncthreads();
    for (int e = threadIdx.x; e < E_local; e += blockDim.x) {      // exclusive prefix over the 32 warps
        int run = 0;
        for (int w = 0; w < 32; ++w) { const int v = warp_cnt[w * E_local + e]; warp_cnt[w * E_local + e] = run; run += v; }
    }
    __syncthreads();
    if (i < n) {
        if (le < 0) {
            dest[i] = -1;
        } else {
            const int row = tmp[(size_t) blockIdx.x * E_local + le] + warp_cnt[warp * E_local + le] + rank;
            dest[i] = row;
            if (row < n) src_token[row] = i / k;
        }
    }
}

// ---- decode batches (T <= 64): [RMSNorm,] router logits, gating and the expert sort in ONE launch -------------------
// grid (E), 256 threads.  CTA e computes the logits of expert e for all tokens (router_rows; with norm_w it normalises the
// rows itself and the CTAs share out the stores of the normalised rows to g_out); the CTA that finishes last (a counter
// that it also resets) then gates every token, one warp per token, and sorts the (token, slot) pairs by local expert.
// Three (with the norm: four) launches fewer per MoE layer of a decode step.
constexpr int ROUTE_MAX_T = 64;
__global__ void __launch_bounds__(GATE_NT) moe_route_fused_kernel(const bf16 * __restrict__ g, const float * __restrict__ w_router,
                                                                  const float * __restrict__ bias, float * __restrict__ logits,
                                                                  int * __restrict__ ids, float * __restrict__ wts, int * __restrict__ seg,
                                                                  int * __restrict__ src_token, int * __restrict__ dest,
                                                                  int * __restrict__ counter, int T, int d, int E, int k, int n_group,
                                                                  int topk_group, float scale, int norm, int sigmoid, int n_shared,
                                                                  int group_top2, int expert_base, int E_local,
                                                                  const float * __restrict__ norm_w, float eps, bf16 * __restrict__ g_out,
                                                                  int warm) {
    JIB_KS(14, 0);
    PDL_TRIGGER_TOP();
    __shared__ float red[GATE_NT / 32][GATE_TG];
    __shared__ float inv_s[GATE_TG];
    __shared__ int s_last;
    __shared__ float prob_s[GATE_NT / 32][MAX_E];
    __shared__ float sel_s[GATE_NT / 32][MAX_E];
    __shared__ float gscore_s[GATE_NT / 32][32];
    __shared__ int ids_s[ROUTE_MAX_T * 32];      // k + n_shared <= 32 columns
    __shared__ int count[MAX_E + 1];
    __shared__ int offs[MAX_E + 1];
    const int warp = threadIdx.x >> 5;
    if (warm) {
        // While the previous kernel is still running: walk the gating and sorting code once on scratch values, storing
        // nothing, so that whichever CTA turns out to be last finds that code in its SM's instruction cache.
        for (int e = threadIdx.x & 31; e < MAX_E; e += 32) prob_s[warp][e] = (float) ((e * 37 + warp) & 63);
        __syncwarp();
        gate_token(nullptr, bias == nullptr ? nullptr : (const float *) prob_s[warp], nullptr, nullptr, 0, E, k, n_group, topk_group, scale,
                   norm, sigmoid, n_shared, group_top2, prob_s[warp], sel_s[warp], gscore_s[warp], ids_s, true);
        __syncthreads();
        sort_pairs(ids_s, k + n_shared, k + n_shared, expert_base, E_local, nullptr, nullptr, nullptr, count, offs, true);
        __syncthreads();
    }
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(14, 1);
    router_rows(g, w_router, norm_w, eps, g_out, logits, 0, T, T, d, E, blockIdx.x, red, inv_s);
    JIB_KS(14, 2);
    // ---- last CTA to finish carries on ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(counter, 1) == (int) gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *counter = 0;      // ready for the next launch
    __threadfence();
    JIB_KS(14, 3);

    // ---- gating: warp w takes tokens w, w + 8, ... ----
    for (int t = warp; t < T; t += GATE_NT / 32) {
        gate_token(logits + (size_t) t * E, bias, ids, wts, t, E, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2,
                   prob_s[warp], sel_s[warp], gscore_s[warp], ids_s);
        __syncwarp();
    }
    __syncthreads();         // ids of all tokens are in shared memory
    JIB_KS(14, 4);
    sort_pairs(ids_s, T * (k + n_shared), k + n_shared, expert_base, E_local, seg, src_token, dest, count, offs, false, seg + E_local + 1);
    JIB_KS(14, 9);
}

// (expert, token tile) pairs of a grouped launch, one CTA: see jib_moe_tile_list.
__global__ void __launch_bounds__(256) tile_list_kernel(const int * __restrict__ seg, int E_local, int bn, int * __restrict__ out, int cap) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    __shared__ int first[MAX_E + 1];
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int run = 0;
        for (int e0 = 0; e0 < E_local; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < E_local ? (seg[e + 1] - seg[e] + bn - 1) / bn : 0;
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            if (e < E_local) first[e] = run + inc - c;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) first[E_local] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E_local; e += blockDim.x)
        for (int i = first[e], t = 0; i < first[e + 1]; ++i, ++t)
            if (i < cap) out[i] = (t << 16) | e;
    for (int i = first[E_local] + threadIdx.x; i < cap; i += blockDim.x) out[i] = -1;
}

// out[t] = residual[t] + shared[t] + sum_j wts[t][j] * y[dest[t][j]]   (fp32 accumulate, bf16 out)
// dry: the same instructions with row 0 in place of the sorted-row indices (which are not valid yet) and no stores.
__device__ __noinline__ void moe_combine_row(const bf16 * __restrict__ y, const int * __restrict__ dest, const float * __restrict__ wts,
                                             const bf16 * __restrict__ shared, const bf16 * __restrict__ residual, bf16 * __restrict__ out,
                                             int k, int d, bool dry) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int j = 0; j < k; ++j) {
            const int row = dry ? 0 : dest[(size_t) t * k + j];
            JIB_BC(row < (int) gridDim.x * k, 14, row);
            if (row < 0) continue;
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
        if (shared) {
            const uint4 raw = ((const uint4 *) (shared + (size_t) t * d))[i];
            const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(p[q]);
                acc[2 * q] += f.x;
                acc[2 * q + 1] += f.y;
            }
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
        if (!dry) ((uint4 *) (out + (size_t) t * d))[i] = o;
    }
}

__global__ void moe_combine_kernel(const bf16 * __restrict__ y, const int * __restrict__ dest, const float * __restrict__ wts,
                                   const bf16 * __restrict__ shared, const bf16 * __restrict__ residual, bf16 * __restrict__ out, int k,
                                   int d, int warm) {
    JIB_KS(12, 0);
    PDL_TRIGGER_TOP();
    if (warm) moe_combine_row(y, dest, wts, shared, residual, out, k, d, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(12, 1);
    moe_combine_row(y, dest, wts, shared, residual, out, k, d, false);
    JIB_KS(12, 9);
}

// ---- combine fused with the RMSNorm that follows it (the next block's attention norm) ---------------------------------
// One CTA per token keeps the token's whole output row in registers: out = bf16(residual + shared + sum_j w_j y_j) as
// moe_combine_kernel computes it, then out_norm = rmsnorm(out) * norm_w from the bf16-rounded values, with the thread
// mapping and reduction order of rmsnorm_kernel<NT, MAXV> (elementwise.cu), so both results equal the two-launch path
// bit for bit.  One launch fewer per MoE layer.
template <int NT>
__device__ __forceinline__ float block_sum_nt(float v, float * red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = l < NT / 32 ? red[l] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

template <int NT, int MAXV>
__device__ __noinline__ void moe_combine_norm_row(const bf16 * __restrict__ y, const int * __restrict__ dest, const float * __restrict__ wts,
                                                  const bf16 * __restrict__ shared, const bf16 * __restrict__ residual,
                                                  const float * __restrict__ norm_w, bf16 * __restrict__ out, bf16 * __restrict__ out_norm,
                                                  int k, int d, float eps, float * red, bool dry) {
    const int t = blockIdx.x;
    const int nv = d / 8;
    float vals[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = threadIdx.x + it * NT;
        if (i < nv) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int j = 0; j < k; ++j) {
                const int row = dry ? 0 : dest[(size_t) t * k + j];
                if (row < 0) continue;
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
            if (shared) {
                const uint4 raw = ((const uint4 *) (shared + (size_t) t * d))[i];
                const __nv_bfloat162 * p = (const __nv_bfloat162 *) &raw;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(p[q]);
                    acc[2 * q] += f.x;
                    acc[2 * q + 1] += f.y;
                }
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
            if (!dry) ((uint4 *) (out + (size_t) t * d))[i] = o;
#pragma unroll
            for (int q = 0; q < 4; ++q) {                 // the norm sees what the next kernel would have read back
                const float2 f = __bfloat1622float2(po[q]);
                vals[it][2 * q] = f.x;
                vals[it][2 * q + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = block_sum_nt<NT>(ss, red);
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
            if (!dry) ((uint4 *) (out_norm + (size_t) t * d))[i] = o;
        }
    }
}

template <int NT, int MAXV>
__global__ void __launch_bounds__(NT) moe_combine_norm_kernel(const bf16 * __restrict__ y, const int * __restrict__ dest,
                                                              const float * __restrict__ wts, const bf16 * __restrict__ shared,
                                                              const bf16 * __restrict__ residual, const float * __restrict__ norm_w,
                                                              bf16 * __restrict__ out, bf16 * __restrict__ out_norm, int k, int d,
                                                              float eps, int warm) {
    JIB_KS(13, 0);
    PDL_TRIGGER_TOP();
    __shared__ float red[32];
    if (warm) moe_combine_norm_row<NT, MAXV>(y, dest, wts, shared, residual, norm_w, out, out_norm, k, d, eps, red, true);
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    JIB_KS(13, 1);
    moe_combine_norm_row<NT, MAXV>(y, dest, wts, shared, residual, norm_w, out, out_norm, k, d, eps, red, false);
    JIB_KS(13, 9);
}

inline int launched() { return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH; }

// JIB_ROUTE_WARM=0: the fused router does not pre-walk its gating / sorting code while it waits (A/B measurements).
inline bool route_warm() {
    static const bool on = [] {
        const char * e = getenv("JIB_ROUTE_WARM");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

}  // namespace

JIB_BC_DEFINE_SETTER(moe)
JIB_TL_DEFINE_SETTER(moe)

extern "C" {

int jib_moe_gate(const void * g, const float * w_router, const float * bias, float * logits, int * ids, float * wts, int T, int d,
                 int E, int k, int n_group, int topk_group, float scale, int norm, int sigmoid, int n_shared, int group_top2,
                 void * stream) {
    if (T <= 0) return 0;
    if (E > MAX_E || k + n_shared > 32 || n_shared < 0 || k > E || d % 8 || d > GATE_MAXC * GATE_NT * 8 || n_group > 32 || (n_group > 1 && E % n_group)) return JIB_E_ARG;
    JIB_LAUNCH((router_logits_kernel), dim3(E, (T + 63) / 64), GATE_NT, 0, (cudaStream_t) stream, (const bf16 *) g, w_router, logits, T, d, E,
               jib::warm_for(T));
    if (cudaGetLastError() != cudaSuccess) return JIB_E_LAUNCH;
    JIB_LAUNCH((moe_gate_kernel), T, 32, 0, (cudaStream_t) stream, logits, bias, ids, wts, E, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2,
               jib::warm_for(T));
    return launched();
}

// jib_moe_gate followed by jib_moe_permute (over the k + n_shared columns) in one launch; T <= 64.  counter: one device int,
// zero between launches.  norm_w != NULL: g holds un-normalised rows; they are RMS-normalised (weights norm_w, eps) on the
// fly and also stored to g_out [T][d] -- what jib_rmsnorm would have produced.
int jib_moe_route_fused(const void * g, const float * w_router, const float * bias, float * logits, int * ids, float * wts, int * seg,
                        int * src_token, int * dest, int * counter, int T, int d, int E, int k, int n_group, int topk_group, float scale,
                        int norm, int sigmoid, int n_shared, int group_top2, int expert_base, int E_local, const float * norm_w, float eps,
                        void * g_out, void * stream) {
    if (T <= 0) return 0;
    if (T > ROUTE_MAX_T || counter == nullptr || E_local > MAX_E || E_local < 1) return JIB_E_ARG;
    if (E > MAX_E || k + n_shared > 32 || n_shared < 0 || k > E || d % 8 || d > GATE_MAXC * GATE_NT * 8 || n_group > 32 || (n_group > 1 && E % n_group)) return JIB_E_ARG;
    if (norm_w != nullptr && g_out == nullptr) return JIB_E_ARG;
    JIB_LAUNCH((moe_route_fused_kernel), E, GATE_NT, 0, (cudaStream_t) stream, (const bf16 *) g, w_router, bias, logits, ids, wts, seg,
               src_token, dest, counter, T, d, E, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2, expert_base, E_local,
               norm_w, eps, (bf16 *) g_out, route_warm() ? 1 : 0);
    return launched();
}

int jib_moe_permute(const int * ids, int T, int k, int expert_base, int E_local, int * seg, int * src_token, int * dest, void * stream) {
    if (T <= 0) return 0;
    if (E_local > MAX_E) return JIB_E_ARG;
    JIB_LAUNCH((moe_permute_kernel), 1, 1024, 0, (cudaStream_t) stream, ids, T * k, k, expert_base, E_local, seg, src_token, dest,
               jib::warm_for(T), seg + E_local + 1);
    return launched();
}

int jib_moe_tile_list(const int * seg, int E_local, int bn, int * out, int cap, void * stream) {
    if (E_local <= 0 || E_local > MAX_E || bn <= 0 || cap <= 0) return JIB_E_ARG;
    JIB_LAUNCH((tile_list_kernel), 1, 256, 0, (cudaStream_t) stream, seg, E_local, bn, out, cap);
    return launched();
}

// Same contract as jib_moe_permute, for large n: three launches over ceil(n / 1024) CTAs.  tmp: device int[ceil(T*k/1024) * E_local].
int jib_moe_permute_multi(const int * ids, int T, int k, int expert_base, int E_local, int * seg, int * src_token, int * dest, int * tmp,
                          void * stream) {
    if (T <= 0) return 0;
    if (E_local > MAX_E || tmp == nullptr) return JIB_E_ARG;
    const int n = T * k;
    const int n_chunks = (n + PERM_CHUNK - 1) / PERM_CHUNK;
    const size_t smem = (size_t) 32 * E_local * sizeof(int);
    if (smem > 48 * 1024) return JIB_E_ARG;
    JIB_LAUNCH((permute_count_kernel), n_chunks, PERM_CHUNK, 0, (cudaStream_t) stream, ids, n, expert_base, E_local, tmp);
    JIB_LAUNCH((permute_scan_kernel), 1, MAX_E, 0, (cudaStream_t) stream, tmp, n_chunks, E_local, n, seg, src_token);
    JIB_LAUNCH((permute_scatter_kernel), n_chunks, PERM_CHUNK, smem, (cudaStream_t) stream, ids, n, k, expert_base, E_local,
               (const int *) tmp, src_token, dest);
    return launched();
}

int jib_moe_combine(const void * y, const int * dest, const float * wts, const void * shared, const void * residual, void * out, int T,
                    int k, int d, void * stream) {
    if (T <= 0) return 0;
    if (d % 8) return JIB_E_ARG;
    JIB_LAUNCH((moe_combine_kernel), T, 256, 0, (cudaStream_t) stream, (const bf16 *) y, dest, wts, (const bf16 *) shared, (const bf16 *) residual,
                                                              (bf16 *) out, k, d, jib::warm_for(T));
    return launched();
}

// jib_moe_combine followed by jib_rmsnorm(out, norm_w) in one launch: out [T][d] and out_norm [T][d], both bf16.
int jib_moe_combine_norm(const void * y, const int * dest, const float * wts, const void * shared, const void * residual,
                         const float * norm_w, void * out, void * out_norm, int T, int k, int d, float eps, void * stream) {
    if (T <= 0) return 0;
    if (d % 8 || norm_w == nullptr || out_norm == nullptr) return JIB_E_ARG;
    const int nv = d / 8;
    cudaStream_t s = (cudaStream_t) stream;
#define JIB_CN(NT, MAXV)                                                                                                         \
    JIB_LAUNCH((moe_combine_norm_kernel<NT, MAXV>), T, NT, 0, s, (const bf16 *) y, dest, wts, (const bf16 *) shared, (const bf16 *) residual, \
               norm_w, (bf16 *) out, (bf16 *) out_norm, k, d, eps, jib::warm_for(T))
    if (nv <= 128) JIB_CN(128, 1);            // the same (threads, values per thread) choice as jib_rmsnorm
    else if (nv <= 256) JIB_CN(256, 1);
    else if (nv <= 1024) JIB_CN(256, 4);
    else if (nv <= 2048) JIB_CN(512, 4);
    else return JIB_E_ARG;
#undef JIB_CN
    return launched();
}

}  // extern "C"
