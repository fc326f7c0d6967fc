// Prefill attention in the per-head (non-absorbed) form on tcgen05 tensor cores.
//
// Decode keeps the weight-absorbed MLA form (mla_flash_tcgen05.cu): one 576-wide latent row per cached token serves all
// heads.  For a prompt chunk that form costs 3.4x the FLOPs of ordinary multi-head attention (scores over 576 dims and
// values over 512 instead of 192 and 128), so chunks expand the latent rows of their sequences once per layer
// (k_nope | v = c_kv . W_kv_b^T, a plain GEMM) and run this kernel over per-head K / V.  The reference does the same
// expansion for every batch (llm_attn_mha, src/llama-graph-attn.cpp:42-217, aclnnFusedInferAttentionScore
// ggml/src/ggml-cann/aclnn_ops.cpp:5536-5622) and never uses the absorbed form for prompts.
//
// Orientation: queries on the MMA M axis.  A CTA owns 128 consecutive query tokens of one sequence and one head:
//   S[128 q, 128 kv]  = Q[128, 192] . K[128 kv, 192]^T        A = Q (K-major), B = K tile (K-major): 3 chunks of 64 dims,
//                                                             the last one (RoPE part) shared by all heads
//   O[128 q, 128 dv] += P[128 q, 128 kv] . V[128 kv, 128 dv]   A = P (bf16, written by the softmax warps, K-major),
//                                                             B = V tile read MN-major (dv contiguous, as stored)
// One thread owns one query row of S (its TMEM lane): row max and row sum need no cross-thread traffic.  S is double
// buffered in TMEM so that Q.K^T of the next KV tile runs under the softmax of the current one; O is rescaled only when
// the running maximum grew by more than 2^8 since the last rescale (the exponent base stays behind the true maximum by
// at most that factor, which fp32 / bf16 absorb), so the correction pass is rare.
// Warp 0: TMA producer.  Warp 1: MMA issuer, owns TMEM.  Warps 2..5: softmax, P, correction, epilogue.
// Causality and sequence boundaries come from q_start / seq_lens; KV tiles below the diagonal skip the mask.
// All waits are bounded (sm100.cuh); no multicast.
#include "sm100.cuh"

#include <mutex>
#include <string.h>

#include "jib_kernels.h"
#include "pdl.cuh"
#include "timeline.cuh"

using namespace sm100;

namespace {

typedef __nv_bfloat16 bf16;

constexpr int DN = 128, DR = 64, DQK = DN + DR, DV = 128;
constexpr int QT = 128;                       // query rows per CTA
constexpr int KT = 128;                       // kv rows per tile
constexpr int CHUNK = QT * 128;               // [128 rows][64 cols] bf16 with 128-byte rows
constexpr int Q_BYTES = 3 * CHUNK, K_BYTES = 3 * CHUNK, V_BYTES = 2 * CHUNK, P_BYTES = 2 * CHUNK;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + 2 * K_BYTES + V_BYTES + P_BYTES + 256;
constexpr int TMEM_COLS = 512;                // S x2 (256) + O (128), rounded to a power of two
constexpr int NUM_THREADS = 192;
constexpr float RESCALE_LAG = 8.0f;           // log2 units the exponent base may lag behind the running maximum

struct MhaArgs {
    const int * q_start;      // [n_seqs + 1] first query row of every sequence
    const int * seq_lens;     // [n_seqs] cached tokens per sequence, this chunk included
    const int * kv_start;     // [n_seqs] first row of the sequence in the expanded K/V buffers
    bf16 * out;               // [T][H * 128]
    int * status;
    long long ldo;
    int n_seqs, T, H;
    float scale_log2e;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
mha_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                   const __grid_constant__ CUtensorMap tmPE, const MhaArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y;

    uint8_t * base = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t * q_s = base;
    uint8_t * k_s = q_s + Q_BYTES;                    // 2 stages
    uint8_t * v_s = k_s + 2 * K_BYTES;
    uint8_t * p_s = v_s + V_BYTES;
    uint64_t * bars = (uint64_t *) (p_s + P_BYTES);
    uint64_t * q_full = bars;
    uint64_t * k_full = bars + 1;                     // [2]
    uint64_t * k_empty = bars + 3;                    // [2]
    uint64_t * v_full = bars + 5;
    uint64_t * v_empty = bars + 6;
    uint64_t * s_full = bars + 7;                     // [2]
    uint64_t * s_empty = bars + 9;                    // [2]
    uint64_t * p_full = bars + 11;
    uint64_t * p_empty = bars + 12;
    uint64_t * o_done = bars + 13;
    uint32_t * tmem_slot = (uint32_t *) (bars + 14);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); }
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        mbar_init(p_full, 4);
        mbar_init(p_empty, 1);
        mbar_init(o_done, 1);
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmKV);
        prefetch_tmap(&tmPE);
    }
    // This kernel takes ALL tensor-memory columns of its SM, and tcgen05.alloc blocks until they are free.  So it asks for them
    // only after the grid before it has completed (a CTA of that grid that still had to start on this SM could never get
    // its own columns), and it lets the grid after it start only once every CTA of this one holds its columns.
    pdl_wait();                                       // q, the expanded K / V and the sequence tables
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_launch_dependents();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_S = tmem, tm_O = tmem + 2 * KT;

    // ---- which (sequence, query tile) is this CTA?  blockIdx.x walks the tiles of all sequences, last tile of a
    // sequence first (it sees the most KV tiles) ----
    int b = -1, q0 = 0, q_len = 0, tile = 0;
    {
        int x = blockIdx.x;
        for (int s = 0; s < a.n_seqs; ++s) {
            const int qs = a.q_start[s], ql = a.q_start[s + 1] - qs;
            const int nt = (ql + QT - 1) / QT;
            if (x < nt) { b = s; q0 = qs; q_len = ql; tile = nt - 1 - x; break; }
            x -= nt;
        }
    }
    int n_tiles = 0, ctx0 = 0, kv0 = 0, rows = 0;
    if (b >= 0) {
        const int S = a.seq_lens[b];
        ctx0 = S - q_len;                             // tokens cached before this chunk
        kv0 = a.kv_start[b];
        rows = min(QT, q_len - tile * QT);            // valid query rows of the tile
        const int last_lim = ctx0 + tile * QT + rows; // kv rows visible to the last valid query row
        n_tiles = rows > 0 && S > 0 ? (last_lim + KT - 1) / KT : 0;
    }
    const int row0 = q0 + tile * QT;                  // first query row (global)

    if (n_tiles > 0 && warp == 0) {
        // ================= TMA producer =================
        if (elect_one()) {
            mbar_expect_tx(q_full, Q_BYTES);
            for (int c = 0; c < 3; ++c) tma_load_2d(q_s + c * CHUNK, &tmQ, q_full, h * DQK + c * 64, row0);
            for (int kt = 0; kt < n_tiles; ++kt) {
                const int s = kt & 1;
                const int krow = kv0 + kt * KT;
                if (!mbar_wait(&k_empty[s], ((kt >> 1) & 1) ^ 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 31, kt); break; }
                uint8_t * kd = k_s + s * K_BYTES;
                mbar_expect_tx(&k_full[s], K_BYTES);
                tma_load_2d(kd, &tmKV, &k_full[s], h * (DN + DV), krow);
                tma_load_2d(kd + CHUNK, &tmKV, &k_full[s], h * (DN + DV) + 64, krow);
                tma_load_2d(kd + 2 * CHUNK, &tmPE, &k_full[s], 0, krow);
                if (!mbar_wait(v_empty, (kt & 1) ^ 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 32, kt); break; }
                mbar_expect_tx(v_full, V_BYTES);
                tma_load_2d(v_s, &tmKV, v_full, h * (DN + DV) + DN, krow);
                tma_load_2d(v_s + CHUNK, &tmKV, v_full, h * (DN + DV) + DN + 64, krow);
            }
        }
    } else if (n_tiles > 0 && warp == 1) {
        // ================= MMA issuer =================
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_bf16(QT, KT, 0, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(QT, DV, 0, 1);       // B (V) read MN-major
            const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s), v_addr = smem_u32(v_s);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 33, 0);
            auto pv = [&](int t) {
                if (!mbar_wait(p_full, t & 1) || !mbar_wait(v_full, t & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 35, t); ok = false; return; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk)
                    mma_bf16(tm_O, desc_k_sw128(p_addr + (kk >> 2) * CHUNK + (kk & 3) * 32), desc_mn_sw128(v_addr + kk * 2048, CHUNK, 1024),
                             idesc_pv, (t | kk) != 0);
                // o_done first: a softmax warp that has seen p_empty of this product must find o_done of the same product
                // complete as well, or its parity wait at the end (or before a rescale) could be answered by the phase before
                mma_commit(o_done);
                mma_commit(v_empty);
                mma_commit(p_empty);
            };
            for (int kt = 0; kt < n_tiles && ok; ++kt) {
                const int s = kt & 1;
                const uint32_t ph = (kt >> 1) & 1;
                if (!mbar_wait(&k_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 34, kt); ok = false; break; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(k_s + s * K_BYTES);
#pragma unroll
                for (int c = 0; c < 3; ++c)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        mma_bf16(tm_S + s * KT, desc_k_sw128(q_addr + c * CHUNK + kk * 32), desc_k_sw128(k_addr + c * CHUNK + kk * 32), idesc_qk,
                                 (c | kk) != 0);
                mma_commit(&k_empty[s]);
                mma_commit(&s_full[s]);
                if (kt >= 1) pv(kt - 1);
            }
            if (ok) pv(n_tiles - 1);
            if (!ok) {                                // release anyone still waiting on this thread
                mma_commit(&s_full[0]);
                mma_commit(&s_full[1]);
                mma_commit(p_empty);
                mma_commit(o_done);
            }
        }
    } else if (n_tiles > 0) {
        // ================= softmax / correction / epilogue (warps 2..5) =================
        const int qd = warp & 3;
        const int r = qd * 32 + lane;                 // query row of this thread inside the tile
        const uint32_t lane_addr = (uint32_t) (qd * 32) << 16;
        const int lim = r < rows ? ctx0 + tile * QT + r + 1 : 0;      // visible kv rows of this query row
        const int lim_first = ctx0 + tile * QT + 1;                   // ... of the tile's first row
        float m_ref = -INFINITY;                      // exponent base, log2 domain (score * scale * log2 e)
        float l_sum = 0.f;
        bool ok = true;
        for (int kt = 0; kt < n_tiles && ok; ++kt) {
            const int s = kt & 1;
            if (!mbar_wait(&s_full[s], (kt >> 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 36, kt); ok = false; }
            ok = __all_sync(0xffffffffu, ok);         // the tensor-memory loads below are warp-wide: leave as a whole warp
            if (!ok) break;
            tc_fence_after();
            const uint32_t ts = tm_S + lane_addr + s * KT;
            const bool need_mask = (kt + 1) * KT > lim_first;          // the tile reaches the diagonal (or the sequence end)
            const int vis = lim - kt * KT;            // columns [0, vis) of this tile are visible to this row
            // The row's 128 scores come out of tensor memory once, all loads in flight before one wait; the S buffer is
            // handed back to the tensor core right away (Q.K^T of the tile after the next may start).
            float x[KT];
#pragma unroll
            for (int c = 0; c < KT; c += 16) tmem_ld16(ts + c, reinterpret_cast<uint32_t (&)[16]>(x[c]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[s]);
            float mt = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < KT; ++c) { x[c] = c < vis ? x[c] * a.scale_log2e : -INFINITY; mt = fmaxf(mt, x[c]); }
            } else {
#pragma unroll
                for (int c = 0; c < KT; ++c) { x[c] *= a.scale_log2e; mt = fmaxf(mt, x[c]); }
            }
            // the exponent base follows the maximum only when it has fallen behind by more than RESCALE_LAG
            const bool grow = mt > m_ref + RESCALE_LAG || m_ref == -INFINITY;
            const float m_new = grow ? mt : m_ref;
            const bool any_grow = __any_sync(0xffffffffu, grow && kt > 0 && m_ref != -INFINITY);
            if (any_grow) {
                // O holds sums relative to the old base: wait for the products in flight, then rescale this row
                if (!mbar_wait(o_done, (kt - 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 37, kt); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
                tc_fence_after();
                const float cf = (grow && m_ref != -INFINITY) ? exp2f(m_ref - m_new) : 1.f;
                if (ok) {
#pragma unroll 1
                    for (int c = 0; c < DV; c += 16) {
                        uint32_t v[16];
                        tmem_ld16(tm_O + lane_addr + c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * cf);
                        tmem_st16(tm_O + lane_addr + c, v);
                    }
                    tmem_st_wait();
                }
                l_sum *= cf;
            } else if (grow && m_ref != -INFINITY) {
                l_sum *= exp2f(m_ref - m_new);        // kt == 0 cannot get here; kept for completeness
            }
            m_ref = m_new;
            // p = 2^(x - base) in registers (the previous P.V may still be reading the P tile), row sum
            const float base_l2 = m_ref == -INFINITY ? 0.f : m_ref;   // every x is -inf then: p = 0
            uint32_t packed[KT / 2];
#pragma unroll
            for (int c = 0; c < KT; c += 2) {
                const float p0 = exp2f(x[c] - base_l2), p1 = exp2f(x[c + 1] - base_l2);
                l_sum += p0 + p1;
                const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                packed[c >> 1] = *(const uint32_t *) &pk;
            }
            // the previous P.V must have read P before it is overwritten
            if (kt > 0 && !mbar_wait(p_empty, (kt - 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 38, kt); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            // P (bf16) into the swizzled K-major tile: 8 kv columns = one 16-byte unit of row r in chunk c / 64
#pragma unroll
            for (int c = 0; c < KT; c += 8) {
                uint8_t * prow = p_s + (c >> 6) * CHUNK + r * 128;
                const int u0 = (c & 63) >> 3;         // 16-byte unit index inside the 128-byte row
                *(uint4 *) (prow + ((u0 ^ (r & 7)) << 4)) = make_uint4(packed[c / 2], packed[c / 2 + 1], packed[c / 2 + 2], packed[c / 2 + 3]);
            }
            fence_proxy_async();                      // P stores -> visible to the tensor core's async-proxy reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // ---- epilogue: O / l -> bf16 rows ----
        if (ok && !mbar_wait(o_done, (n_tiles - 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 39, 0); ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (ok) {
            // tcgen05.ld is a warp-wide instruction (.sync.aligned): all 32 lanes execute it, also in a tile whose valid
            // rows end inside this warp; only the stores are predicated per row.  (Executed under a per-lane condition it
            // never completes.)
            const bool valid = r < rows;
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            bf16 * dst = a.out + (size_t) (row0 + (valid ? r : 0)) * a.ldo + (size_t) h * DV;
#pragma unroll 1
            for (int c = 0; c < DV; c += 16) {
                uint32_t v[16];
                tmem_ld16(tm_O + lane_addr + c, v);
                tmem_ld_wait();
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
                    o[j >> 1] = *(const uint32_t *) &pk;
                }
                if (valid) {
                    *(uint4 *) (dst + c) = make_uint4(o[0], o[1], o[2], o[3]);
                    *(uint4 *) (dst + c + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- latent rows of the sequences of a batch, gathered from the paged cache into one contiguous buffer ---------------------
// lat [total][row] <- cache[block_tables[b][s / bs] * bs + s % bs][row] for s < seq_lens[b]; kv_start[b] = first row of
// sequence b (exclusive prefix of seq_lens).  grid (ceil(max rows / 8), 1): every CTA walks the sequence table itself.
__global__ void __launch_bounds__(256) kv_gather_kernel(const bf16 * __restrict__ cache, const int * __restrict__ block_tables, int max_blocks,
                                                        const int * __restrict__ seq_lens, int n_seqs, int block_size, int row_elems,
                                                        long long n_slots, bf16 * __restrict__ lat, int * __restrict__ kv_start, int total_cap) {
    PDL_TRIGGER_TOP();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.x * 8 + warp;              // global row of the gathered buffer this warp copies
    int b = -1, s = 0, acc = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int S = seq_lens[i];
        if (blockIdx.x == 0 && threadIdx.x == 0) kv_start[i] = acc;
        if (b < 0 && g < acc + S) { b = i; s = g - acc; }
        acc += S;
    }
    if (b < 0 || g >= total_cap) return;
    const int blk = block_tables[(size_t) b * max_blocks + s / block_size];
    const long long slot = (long long) blk * block_size + s % block_size;
    if (slot < 0 || slot >= n_slots) return;
    const uint4 * src = (const uint4 *) (cache + (size_t) slot * row_elems);
    uint4 * dst = (uint4 *) (lat + (size_t) g * row_elems);
    for (int i = lane; i < row_elems / 8; i += 32) dst[i] = src[i];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn) p;
    });
    return fn;
}

// bf16 matrix [rows][cols], row stride in elements; box {64 cols, 128 rows}; 128-byte swizzle; rows past the end read zero
int map_2d(CUtensorMap * out, const void * ptr, long long rows, long long cols, long long row_stride) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return JIB_E_DRIVER;
    if (((uintptr_t) ptr & 15) || (row_stride * 2) % 16) return JIB_E_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t) cols, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) row_stride * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0 : JIB_E_TENSORMAP;
}

}  // namespace

extern "C" {

// Gathers the latent rows of all sequences of the batch (seq_lens[b] rows each, in sequence order) from the paged cache
// layer into lat [total_cap][row_elems] and writes the first row of every sequence to kv_start [n_seqs].
JIB_EXPORT int jib_kv_gather(const void * cache, long long n_slots, const int * block_tables, int max_blocks, const int * seq_lens,
                             int n_seqs, int block_size, int row_elems, void * lat, int * kv_start, int total_cap, void * stream) {
    if (n_seqs <= 0 || total_cap <= 0) return 0;
    if (row_elems % 8 || block_size <= 0) return JIB_E_ARG;
    JIB_LAUNCH((kv_gather_kernel), (total_cap + 7) / 8, 256, 0, (cudaStream_t) stream, (const bf16 *) cache, block_tables, max_blocks, seq_lens,
               n_seqs, block_size, row_elems, n_slots, (bf16 *) lat, kv_start, total_cap);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

// Causal multi-head attention of a prompt chunk.  q [T][H][192] (RoPE applied to the last 64 dims), row stride q_stride;
// kv [total][H][256] = k_nope | v per head; kpe [total][64] with row stride kpe_stride (the RoPE part of the keys, shared by
// the heads); out [T][H * 128] bf16, row stride ldo.  Sequence b owns query rows q_start[b]..q_start[b+1] (the LAST such rows
// of its seq_lens[b] cached tokens) and K/V rows kv_start[b].. ; n_q_tiles >= sum_b ceil(q_len_b / 128).
JIB_EXPORT int jib_mha_prefill(const void * q, long long q_stride, const void * kv, const void * kpe, long long kpe_stride, long long total,
                               const int * q_start, const int * seq_lens, const int * kv_start, int n_seqs, int T, int H, float scale,
                               int n_q_tiles, void * out, long long ldo, int * status, void * stream_) {
    cudaStream_t stream = (cudaStream_t) stream_;
    if (T <= 0 || n_seqs <= 0 || n_q_tiles <= 0) return 0;
    if (ldo % 8 || ((uintptr_t) out & 15) || total <= 0) return JIB_E_ALIGN;
    CUtensorMap mq, mkv, mpe;
    int rc = map_2d(&mq, q, T, (long long) H * DQK, q_stride);
    if (rc) return rc;
    rc = map_2d(&mkv, kv, total, (long long) H * (DN + DV), (long long) H * (DN + DV));
    if (rc) return rc;
    rc = map_2d(&mpe, kpe, total, DR, kpe_stride);
    if (rc) return rc;
    MhaArgs a;
    a.q_start = q_start; a.seq_lens = seq_lens; a.kv_start = kv_start; a.out = (bf16 *) out; a.status = status; a.ldo = ldo;
    a.n_seqs = n_seqs; a.T = T; a.H = H;
    a.scale_log2e = scale * 1.4426950408889634f;
    static std::atomic<unsigned char> attr_done[jib::MAX_DEVICES];
    if (!jib::ensure_dyn_smem(mha_prefill_kernel, SMEM_BYTES, attr_done)) return JIB_E_LAUNCH;
    JIB_LAUNCH((mha_prefill_kernel), dim3(n_q_tiles, H), NUM_THREADS, SMEM_BYTES, stream, mq, mkv, mpe, a);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

}  // extern "C"
