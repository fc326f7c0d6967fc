// Sampling on the device from the top-k candidates: top-k / top-p / min-p truncation, temperature, and one draw per row
// from a uniform number supplied by the host.
//
// Reference: the candidates of the device top-k ("presample", src/llama-execute-decode.cpp:132-154) go to the host, where
// the sampler chain runs top_k -> top_p -> min_p -> temperature -> dist (common/sampling_local.cpp:153-209,
// src/llama-sampling.cpp:146-590).  Here the same four stages run next to the top-k kernel, so that only the chosen id
// leaves the device -- and can feed the next step without a round trip.  The random stream stays on the host: one
// uniform per row and step arrives with the step's inputs, so a request's draws depend on its seed and step only.
// Samplers that need token history or the vocabulary (penalties, DRY, grammar, logit bias, typical, XTC) stay on the host.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "jib_kernels.h"
#include "pdl.cuh"

namespace {

constexpr int SAMPLE_MAX_K = 128;

// vals/ids [n][k]: candidates sorted by value, descending (as jib_topk writes them).  params [n][5]: temperature (<= 0: take
// the best candidate), top_k (<= 0: all k), top_p (>= 1: off), min_p (<= 0: off), u in [0, 1).  One warp per row.
// Because the candidates are sorted, every truncation keeps a prefix: top-k by rank, top-p while the probability mass before
// a candidate is below top_p (softmax of the untempered logits of the top-k set), min-p while logit >= best + ln(min_p).
__global__ void __launch_bounds__(32) sample_topk_kernel(const float * __restrict__ vals, const int * __restrict__ ids,
                                                         const float * __restrict__ params, int * __restrict__ out, int k) {
    PDL_TRIGGER_TOP();
    pdl_wait();      // inputs come from earlier kernels; nothing is written before this point
    __shared__ float e[SAMPLE_MAX_K];
    const int row = blockIdx.x, lane = threadIdx.x;
    const float * v = vals + (size_t) row * k;
    const float * p = params + (size_t) row * 5;
    const float temp = p[0], top_p = p[2], min_p = p[3], u = p[4];
    if (temp <= 0.f) {
        if (lane == 0) out[row] = ids[(size_t) row * k];
        return;
    }
    int kk = p[1] > 0.f ? min(k, (int) p[1]) : k;
    const float m = v[0];
    float part = 0.f;
    for (int j = lane; j < kk; j += 32) {
        const float x = __expf(v[j] - m);
        e[j] = x;
        part += x;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    __syncwarp();
    if (lane == 0) {
        const float total = part;
        const float thr = min_p > 0.f ? m + __logf(min_p) : -FLT_MAX;
        // prefix that survives top-p and min-p (the first candidate always does)
        int n_keep = 1;
        float cum = e[0];
        for (int j = 1; j < kk; ++j) {
            if (top_p < 1.f && cum / total >= top_p) break;
            if (v[j] < thr) break;
            cum += e[j];
            n_keep = j + 1;
        }
        // tempered weights of the kept prefix and the draw
        const float inv_t = 1.f / temp;
        float total2 = 0.f;
        for (int j = 0; j < n_keep; ++j) {
            const float w = __expf((v[j] - m) * inv_t);
            e[j] = w;
            total2 += w;
        }
        const float target = u * total2;
        int pick = n_keep - 1;
        float cdf = 0.f;
        for (int j = 0; j < n_keep; ++j) {
            cdf += e[j];
            if (cdf > target) { pick = j; break; }
        }
        out[row] = ids[(size_t) row * k + pick];
    }
}

}  // namespace

extern "C" JIB_EXPORT int jib_sample_topk(const float * vals, const int * ids, const float * params, int * out, int n, int k, void * stream) {
    if (n <= 0) return 0;
    if (k < 1 || k > SAMPLE_MAX_K) return JIB_E_ARG;
    JIB_LAUNCH((sample_topk_kernel), n, 32, 0, (cudaStream_t) stream, vals, ids, params, out, k);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}
