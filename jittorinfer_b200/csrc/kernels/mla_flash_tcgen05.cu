// Weight-absorbed MLA attention on tcgen05 tensor cores, reading the paged latent cache by TMA.
//
// Reference: llm_attn_mla (src/llama-graph-attn.cpp:219-342) = 4 matmuls + softmax with the [S, T*H] score
// matrix and a transposed latent copy in HBM.  Here the whole thing is one flash-style kernel with a
// split-KV variant for decode; scores and probabilities never leave the SM.
//
// Orientation (transposed, so that 16 heads x 1..2 tokens are enough to use 128-lane MMAs):
//   S^T[kv 128, NQ]   = Lat[kv 128, 576] . Q^T[576, NQ]        A = latent tile (K-major), B = Q (K-major)
//   O^T[512,   NQ]   += Lat^T[512, kv 128] . P^T[kv 128, NQ]    A = the SAME latent tile read MN-major, B = P (K-major)
// with NQ = QT tokens x 16 heads query columns.  One latent tile therefore feeds both products from one copy
// in shared memory — the reason the reference's transposed duplicate of c_kv is not needed.
//
// CTA = (token group, kv split, head group of 16).  Warp 0: TMA producer (two 64-row boxes per 64-dim chunk,
// one per KV block).  Warp 1: MMA issuer, owns TMEM.  Warps 2..5: softmax over the 128 kv lanes of S^T
// (cross-lane max by shuffles), P^T written to shared memory in the swizzled K-major layout, running-max
// correction of O^T in TMEM (tcgen05.ld / .st), final normalisation and store.
// TMEM: S^T NQ columns + O^T 4 x NQ columns.  Shared memory: Q (9 chunks), P^T, a ring of latent "pair" slots
// (two adjacent 64-dim chunks = one 128-dim MMA M tile) and two slots for the rope chunk.
// All waits are bounded (see sm100.cuh); no multicast.
#include "sm100.cuh"

#include <mutex>
#include <string.h>

#include "jib_kernels.h"
#include "pdl.cuh"
#include "timeline.cuh"

using namespace sm100;

namespace {

typedef __nv_bfloat16 bf16;

constexpr int R = 512, DR = 64, D = R + DR;
constexpr int KV_TILE = 128;
constexpr int BLK = 64;                 // KV block size (tokens) the kernel is built for
constexpr int CHUNK_BYTES = KV_TILE * 128;          // [128 kv][64 dims] bf16, 128-byte rows
constexpr int PAIR_BYTES = 2 * CHUNK_BYTES;
constexpr int N_LAT_PAIRS = R / 128;                // 4 M tiles of 128 dims
constexpr int NUM_THREADS = 192;

template <int QT>
struct FCfg {
    static constexpr int NQ = QT * 16;
    static constexpr int NPAIR = QT == 1 ? 5 : 4;   // latent pair slots in flight
    static constexpr int Q_BYTES = (D / 64) * NQ * 128;
    static constexpr int P_BYTES = 2 * NQ * 128;    // two [NQ][64 kv] swizzled blocks
    static constexpr int RING_BYTES = NPAIR * PAIR_BYTES + 2 * CHUNK_BYTES;
    static constexpr int RED_BYTES = 4 * NQ * 4;    // cross-warp max exchange
    static constexpr int SMEM_BYTES = 1024 + RING_BYTES + Q_BYTES + P_BYTES + RED_BYTES + 512;
    static constexpr int TMEM_COLS = 5 * NQ <= 128 ? 128 : 256;
};

struct FlashArgs {
    const int * block_tables;
    const int * seq_lens;
    const int * q_start;
    float * part_o;       // [T][n_splits][H][R]
    float * part_ml;      // [T][n_splits][H][2]
    bf16 * o_lat;         // [T][H][R]
    int * status;
    int max_blocks, n_seqs, T, H, n_splits, n_blocks;
    float scale_log2e;
};

__device__ __forceinline__ int find_seq(const int * q_start, int n_seqs, int t) {
    int lo = 0, hi = n_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (q_start[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

template <int QT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
mla_flash_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, const FlashArgs a) {
    using C = FCfg<QT>;
    constexpr int NQ = C::NQ;
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * QT, sp = blockIdx.y, hg = blockIdx.z;

    uint8_t * base = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t * ring = base;                                    // NPAIR pair slots, then 2 rope slots
    uint8_t * rope_ring = ring + C::NPAIR * PAIR_BYTES;
    uint8_t * q_s = rope_ring + 2 * CHUNK_BYTES;              // 9 chunks [NQ][64]
    uint8_t * p_s = q_s + C::Q_BYTES;                         // 2 blocks [NQ][64 kv]
    float * red = (float *) (p_s + C::P_BYTES);               // [4 warps][NQ]
    uint64_t * bars = (uint64_t *) ((uint8_t *) red + C::RED_BYTES);
    uint64_t * lat_full = bars;                               // [NPAIR]
    uint64_t * lat_free = bars + C::NPAIR;                    // [NPAIR]
    uint64_t * rope_full = bars + 2 * C::NPAIR;               // [2]
    uint64_t * rope_free = rope_full + 2;                     // [2]
    uint64_t * q_full = rope_free + 2;
    uint64_t * s_ready = q_full + 1;
    uint64_t * p_ready = s_ready + 1;
    uint64_t * o_ready = p_ready + 1;
    uint32_t * tmem_slot = (uint32_t *) (o_ready + 1);

    // ---- work description: up to QT distinct sequences among this CTA's tokens ("passes") ----
    // pass j covers the tokens of the group that belong to sequence pass_seq[j]; a column of another sequence is
    // masked (limit 0) in that pass, so its running state and its O^T column stay untouched.
    int pass_seq[QT], pass_k0[QT], pass_k1[QT];
    int lim[QT][QT];                      // lim[pass][token]: visible kv positions of that token in that pass
    int n_pass = 0;
    {
        int prev = -1;
#pragma unroll
        for (int j = 0; j < QT; ++j) {
            const int t = t0 + j;
            if (t >= a.T) break;
            const int b = find_seq(a.q_start, a.n_seqs, t);
            const int q0 = a.q_start[b], q1 = a.q_start[b + 1];
            const int S = a.seq_lens[b];
            const int n_kv = (t < q1 && S > 0) ? S - (q1 - q0) + (t - q0) + 1 : 0;
            if (b != prev) {
                pass_seq[n_pass] = b;
#pragma unroll
                for (int jj = 0; jj < QT; ++jj) lim[n_pass][jj] = 0;
                ++n_pass;
                prev = b;
            }
            lim[n_pass - 1][j] = n_kv;
        }
        for (int p = 0; p < n_pass; ++p) {
            int mx = 0;
#pragma unroll
            for (int jj = 0; jj < QT; ++jj) mx = max(mx, lim[p][jj]);
            int chunk = (mx + a.n_splits - 1) / a.n_splits;
            chunk = (chunk + KV_TILE - 1) / KV_TILE * KV_TILE;
            if (chunk < KV_TILE) chunk = KV_TILE;
            pass_k0[p] = sp * chunk;
            pass_k1[p] = min(mx, pass_k0[p] + chunk);
        }
    }
    int total_tiles = 0;
    for (int p = 0; p < n_pass; ++p) total_tiles += pass_k1[p] > pass_k0[p] ? (pass_k1[p] - pass_k0[p] + KV_TILE - 1) / KV_TILE : 0;

    JIB_KS(2, 0);
    if (total_tiles == 0) {
        pdl_wait();
        // nothing visible for this (group, split): publish an empty partial / zero output and leave
        const int wr = threadIdx.x;
        for (int idx = wr; idx < QT * 16; idx += NUM_THREADS) {
            const int j = idx / 16, h = hg * 16 + (idx & 15), t = t0 + j;
            if (t >= a.T || h >= a.H) continue;
            if (a.n_splits > 1) {
                const size_t pidx = ((size_t) t * a.n_splits + sp) * a.H + h;
                a.part_ml[pidx * 2] = -INFINITY;
                a.part_ml[pidx * 2 + 1] = 0.f;
            } else {
                bf16 * po = a.o_lat + ((size_t) t * a.H + h) * R;
                for (int i = 0; i < R; ++i) po[i] = __float2bfloat16(0.f);
            }
        }
        return;
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::NPAIR; ++i) { mbar_init(&lat_full[i], 1); mbar_init(&lat_free[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&rope_full[i], 1); mbar_init(&rope_free[i], 1); }
        mbar_init(q_full, 1);
        mbar_init(s_ready, 1);
        mbar_init(p_ready, 4);
        mbar_init(o_ready, 1);
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmKV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    PDL_TRIGGER_TOP();      // only now: the next grid may start once every CTA of this one holds its tensor-memory columns
    const uint32_t tmem = *tmem_slot;
    pdl_wait();                                 // q, the latent cache rows written this step, and all outputs
    JIB_KS(2, 1);
    const uint32_t tm_S = tmem;                 // NQ columns
    const uint32_t tm_O = tmem + NQ;            // 4 x NQ columns

    if (warp == 0) {
        // ================= TMA producer =================
        if (elect_one()) {
            mbar_expect_tx(q_full, C::Q_BYTES);
            for (int c = 0; c < D / 64; ++c) tma_load_3d(q_s + c * NQ * 128, &tmQ, q_full, c * 64, hg * 16, t0);
            int it = 0;                            // global tile counter (ring phases run across passes)
            bool ok = true;
            for (int p = 0; p < n_pass && ok; ++p) {
                const int * bt = a.block_tables + (size_t) pass_seq[p] * a.max_blocks;
                for (int kb = pass_k0[p]; kb < pass_k1[p] && ok; kb += KV_TILE, ++it) {
                    int blk0 = bt[kb / BLK];
                    int blk1 = (kb / BLK + 1 < a.max_blocks) ? bt[kb / BLK + 1] : blk0;
                    blk0 = min(max(blk0, 0), a.n_blocks - 1);        // rows past the sequence end are masked later
                    blk1 = min(max(blk1, 0), a.n_blocks - 1);
                    // rope chunk first (the QK product needs all nine chunks, PV only the latent pairs)
                    {
                        const int s = it & 1;
                        const uint32_t ph = (it >> 1) & 1;
                        if (!mbar_wait(&rope_free[s], ph ^ 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 21, it); ok = false; break; }
                        uint8_t * dst = rope_ring + s * CHUNK_BYTES;
                        mbar_expect_tx(&rope_full[s], CHUNK_BYTES);
                        tma_load_2d(dst, &tmKV, &rope_full[s], R, blk0 * BLK);
                        tma_load_2d(dst + CHUNK_BYTES / 2, &tmKV, &rope_full[s], R, blk1 * BLK);
                    }
                    for (int m = 0; m < N_LAT_PAIRS && ok; ++m) {
                        const int u = it * N_LAT_PAIRS + m;              // use counter of the pair ring
                        const int s = u % C::NPAIR;
                        const uint32_t ph = (u / C::NPAIR) & 1;
                        if (!mbar_wait(&lat_free[s], ph ^ 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 22, it); ok = false; break; }
                        uint8_t * dst = ring + s * PAIR_BYTES;
                        mbar_expect_tx(&lat_full[s], PAIR_BYTES);
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int x = (2 * m + half) * 64;
                            tma_load_2d(dst + half * CHUNK_BYTES, &tmKV, &lat_full[s], x, blk0 * BLK);
                            tma_load_2d(dst + half * CHUNK_BYTES + CHUNK_BYTES / 2, &tmKV, &lat_full[s], x, blk1 * BLK);
                        }
                    }
                }
            }
            PDL_TRIGGER_LATE();      // every load of this CTA is in flight
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_bf16(128, NQ, 0, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(128, NQ, 1, 0);      // A (latent) read MN-major
            bool ok = mbar_wait(q_full, 0);
            if (!ok) jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 23, 0);
            const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
            for (int it = 0; it < total_tiles && ok; ++it) {
                // ---- S^T = Lat . Q^T over 9 chunks of 64 dims ----
                for (int m = 0; m < N_LAT_PAIRS && ok; ++m) {
                    const int u = it * N_LAT_PAIRS + m;
                    const int s = u % C::NPAIR;
                    if (!mbar_wait(&lat_full[s], (u / C::NPAIR) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 24, it); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(ring + s * PAIR_BYTES);
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            mma_bf16(tm_S, desc_k_sw128(a_addr + half * CHUNK_BYTES + kk * 32),
                                     desc_k_sw128(q_addr + (2 * m + half) * NQ * 128 + kk * 32), idesc_qk, (m | half | kk) != 0);
                }
                if (!ok) break;
                {
                    const int s = it & 1;
                    if (!mbar_wait(&rope_full[s], (it >> 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 25, it); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(rope_ring + s * CHUNK_BYTES);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        mma_bf16(tm_S, desc_k_sw128(a_addr + kk * 32), desc_k_sw128(q_addr + 8 * NQ * 128 + kk * 32), idesc_qk, true);
                    mma_commit(&rope_free[s]);
                }
                mma_commit(s_ready);
                // ---- O^T += Lat^T . P^T ----
                if (!mbar_wait(p_ready, it & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 26, it); ok = false; break; }
                tc_fence_after();
                for (int m = 0; m < N_LAT_PAIRS; ++m) {
                    const int u = it * N_LAT_PAIRS + m;
                    const int s = u % C::NPAIR;
                    const uint32_t a_addr = smem_u32(ring + s * PAIR_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KV_TILE / 16; ++kk)
                        mma_bf16(tm_O + m * NQ, desc_mn_sw128(a_addr + kk * 2048, CHUNK_BYTES, 1024),
                                 desc_k_sw128(p_addr + (kk >> 2) * NQ * 128 + (kk & 3) * 32), idesc_pv, (it | kk) != 0);
                    mma_commit(&lat_free[s]);
                }
                mma_commit(o_ready);
            }
            if (!ok) {           // release anyone still waiting on this thread
                mma_commit(s_ready);
                mma_commit(o_ready);
            }
        }
    } else {
        // ================= softmax / correction / epilogue (warps 2..5) =================
        const int qd = warp & 3;                      // TMEM lane quarter of this warp
        const int row = qd * 32 + lane;               // kv lane (softmax) and output dim inside a 128-dim tile (epilogue)
        const uint32_t lane_addr = (uint32_t) (qd * 32) << 16;
        float m_run[NQ], l_part[NQ];
#pragma unroll
        for (int c = 0; c < NQ; ++c) { m_run[c] = -INFINITY; l_part[c] = 0.f; }
        bool ok = true;
        int it = 0;
        for (int p = 0; p < n_pass && ok; ++p) {
            for (int kb = pass_k0[p]; kb < pass_k1[p] && ok; kb += KV_TILE, ++it) {
                if (!mbar_wait(s_ready, it & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 27, it); ok = false; break; }
                tc_fence_after();
                if (it == 0) JIB_KS_T(2, 4, 64);
                float s[NQ];
#pragma unroll
                for (int c = 0; c < NQ; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(tm_S + lane_addr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) s[c + j] = __uint_as_float(v[j]);
                }
                const int pos = kb + row;
                // tile max per column over the 128 kv lanes
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    const bool vis = pos < lim[p][c >> 4];
                    float v = vis ? s[c] : -INFINITY;
                    s[c] = v;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
                    if (lane == 0) red[qd * NQ + c] = v;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                float corr[NQ];
                bool any_corr = false;
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    const float mt = fmaxf(fmaxf(red[c], red[NQ + c]), fmaxf(red[2 * NQ + c], red[3 * NQ + c]));
                    const float m_new = fmaxf(m_run[c], mt);
                    const float cf = (m_new == -INFINITY) ? 1.f : exp2f((m_run[c] - m_new) * a.scale_log2e);
                    corr[c] = cf;
                    any_corr |= cf != 1.f;
                    const float pv = (s[c] == -INFINITY) ? 0.f : exp2f((s[c] - m_new) * a.scale_log2e);
                    l_part[c] = l_part[c] * cf + pv;
                    m_run[c] = m_new;
                    // P^T[c][row] (bf16) into the swizzled K-major block
                    const int blk = row >> 6, kcol = row & 63;
                    const uint32_t off = blk * (NQ * 128) + c * 128 + ((((kcol * 2) >> 4) ^ (c & 7)) << 4) + ((kcol * 2) & 15);
                    *(bf16 *) (p_s + off) = __float2bfloat16(pv);
                }
                // running-max correction of O^T (previous PV products must have landed)
                if (it > 0) {
                    if (!mbar_wait(o_ready, (it - 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 28, it); ok = false; }
                    tc_fence_after();
                    if (any_corr && ok) {
#pragma unroll 1
                        for (int m = 0; m < N_LAT_PAIRS; ++m)
#pragma unroll
                            for (int c = 0; c < NQ; c += 16) {
                                uint32_t v[16];
                                tmem_ld16(tm_O + lane_addr + m * NQ + c, v);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr[c + j]);
                                tmem_st16(tm_O + lane_addr + m * NQ + c, v);
                            }
                        tmem_st_wait();
                    }
                }
                fence_proxy_async();          // P^T stores -> visible to the tensor core's async-proxy reads
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready);
                asm volatile("bar.sync 1, 128;" ::: "memory");   // red[] reuse in the next tile
            }
        }
        // ---- epilogue ----
        if (ok && !mbar_wait(o_ready, (total_tiles - 1) & 1)) { jib_report(a.status, JIB_ERR_WAIT_TIMEOUT, 29, 0); ok = false; }
        tc_fence_after();
        // l per column = sum over the 128 kv lanes
        float l_tot[NQ];
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
            float v = l_part[c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[qd * NQ + c] = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int c = 0; c < NQ; ++c) l_tot[c] = red[c] + red[NQ + c] + red[2 * NQ + c] + red[3 * NQ + c];
        if (ok) {
#pragma unroll 1
            for (int m = 0; m < N_LAT_PAIRS; ++m) {
                const int dim = m * 128 + row;
#pragma unroll
                for (int c0 = 0; c0 < NQ; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tm_O + lane_addr + m * NQ + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int c = c0 + j;
                        const int t = t0 + (c >> 4), h = hg * 16 + (c & 15);
                        if (t >= a.T || h >= a.H) continue;
                        const float o = __uint_as_float(v[j]);
                        if (a.n_splits > 1) {
                            a.part_o[(((size_t) t * a.n_splits + sp) * a.H + h) * R + dim] = o;
                        } else {
                            const float inv = l_tot[c] > 0.f ? 1.f / l_tot[c] : 0.f;
                            a.o_lat[((size_t) t * a.H + h) * R + dim] = __float2bfloat16(o * inv);
                        }
                    }
                }
            }
            if (a.n_splits > 1 && row < NQ) {
                // one thread per column publishes (m, l); m is kept in score units * scale (natural-log domain)
                const int c = row;
                const int t = t0 + (c >> 4), h = hg * 16 + (c & 15);
                if (t < a.T && h < a.H) {
                    const size_t pidx = ((size_t) t * a.n_splits + sp) * a.H + h;
                    a.part_ml[pidx * 2] = m_run[c] == -INFINITY ? -INFINITY : m_run[c] * a.scale_log2e * 0.6931471805599453f;
                    a.part_ml[pidx * 2 + 1] = l_tot[c];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, C::TMEM_COLS);
    JIB_KS(2, 9);
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

template <int QT>
int launch_flash(const CUtensorMap & mq, const CUtensorMap & mkv, const FlashArgs & a, dim3 grid, cudaStream_t stream) {
    using C = FCfg<QT>;
    static std::atomic<unsigned char> attr_done[jib::MAX_DEVICES];
    if (!jib::ensure_dyn_smem(mla_flash_kernel<QT>, C::SMEM_BYTES, attr_done)) return JIB_E_LAUNCH;
    JIB_LAUNCH((mla_flash_kernel<QT>), grid, NUM_THREADS, C::SMEM_BYTES, stream, mq, mkv, a);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}

}  // namespace

JIB_TL_DEFINE_SETTER(flash)

// q [T][H][576] bf16, cache [n_blocks*64][576] bf16 (one layer), o_lat [T][H][512] bf16.
// qt: query tokens per CTA (1 for decode batches, 2 for prompt chunks).  n_splits > 1 writes partials that
// jib_mla_combine merges.  Only block_size 64, r 512, dr 64.
extern "C" JIB_EXPORT int jib_mla_flash(const void * q, const void * cache, long long n_slots, const int * block_tables, int max_blocks,
                                        const int * seq_lens, const int * q_start, int n_seqs, int T, int H, float scale, int n_splits,
                                        int qt, float * part_o, float * part_ml, void * o_lat, int * status, void * stream_) {
    cudaStream_t stream = (cudaStream_t) stream_;
    if (T <= 0) return 0;
    if (n_splits < 1 || (qt != 1 && qt != 2) || n_slots % BLK) return JIB_E_ARG;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return JIB_E_DRIVER;
    if (((uintptr_t) q & 15) || ((uintptr_t) cache & 15)) return JIB_E_ALIGN;
    CUtensorMap mq, mkv;
    {
        cuuint64_t dims[3] = {(cuuint64_t) D, (cuuint64_t) H, (cuuint64_t) T};
        cuuint64_t strides[2] = {(cuuint64_t) D * 2, (cuuint64_t) H * D * 2};
        cuuint32_t box[3] = {64, 16, (cuuint32_t) qt};
        cuuint32_t estr[3] = {1, 1, 1};
        if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return JIB_E_TENSORMAP;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t) D, (cuuint64_t) n_slots};
        cuuint64_t strides[1] = {(cuuint64_t) D * 2};
        cuuint32_t box[2] = {64, BLK};
        cuuint32_t estr[2] = {1, 1};
        if (fn(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(cache), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return JIB_E_TENSORMAP;
    }
    FlashArgs a;
    a.block_tables = block_tables; a.seq_lens = seq_lens; a.q_start = q_start; a.part_o = part_o; a.part_ml = part_ml;
    a.o_lat = (bf16 *) o_lat; a.status = status; a.max_blocks = max_blocks; a.n_seqs = n_seqs; a.T = T; a.H = H;
    a.n_splits = n_splits; a.n_blocks = (int) (n_slots / BLK);
    a.scale_log2e = scale * 1.4426950408889634f;
    dim3 grid((T + qt - 1) / qt, n_splits, (H + 15) / 16);
    return qt == 1 ? launch_flash<1>(mq, mkv, a, grid, stream) : launch_flash<2>(mq, mkv, a, grid, stream);
}
