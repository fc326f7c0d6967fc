// C ABI of libjib200_kernels.so: every launcher takes raw device pointers and a CUDA stream, returns
// 0 on success or a negative JIB_E_* code, and never allocates or synchronises.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define JIB_EXPORT __attribute__((visibility("default")))

enum {
    JIB_E_ARG = -1,         // unsupported shape / argument
    JIB_E_ALIGN = -2,       // pointer or stride not 16-byte aligned (TMA requirement)
    JIB_E_DRIVER = -3,      // cuTensorMapEncodeTiled entry point unavailable
    JIB_E_TENSORMAP = -4,   // tensor-map encode failed
    JIB_E_LAUNCH = -5,      // kernel launch failed
    JIB_E_SCRATCH = -6,     // scratch / counter buffer too small for the requested split
};

#ifdef __cplusplus
extern "C" {
#endif

// Y[b][t][n] = sum_k X[b][t][k] * W[b][n][k]  (bf16 in, fp32 accumulate), optional second weight
// (w2: out = silu(X W^T) * (X W2^T)), optional residual add, optional expert-grouped rows.
typedef struct jib_gemm_desc {
    const void * x;            // bf16 activations
    const void * w;            // bf16 weights [batch][N][K]
    const void * w2;           // NULL, or second weight of the gated pair (same layout as w)
    void * out;
    const void * residual;     // NULL or [rows][N] added in the epilogue
    const int * seg;           // NULL, or device int[batch+1]: rows of expert b are [seg[b], seg[b+1]) of x / out
    void * scratch;            // split-K partials (fp32), may be NULL (then no split)
    int * counters;            // split-K tile counters, zero-initialised once; the kernel leaves them zero
    int * status;              // 4 ints, see sm100.cuh; may be NULL
    long long x_row_stride, x_batch_stride;   // elements
    long long w_row_stride, w_batch_stride;
    long long ldo, out_batch_stride, ldr, res_batch_stride;
    long long x_rows_total;    // grouped: total rows of x (all experts)
    size_t scratch_bytes;
    int n_counters;
    int T, N, K, batch;        // grouped: T = upper bound of rows of one expert
    int max_rows;              // grouped: tighter bound of rows per expert if known (else 0)
    int active_hint;           // grouped: expected number of non-empty experts (split-K heuristic), else 0
    int out_f32, res_f32;
    int splits;                // 0 = choose
    int bn;                    // 0 = choose; token-tile width 16/32/64/128/256
    int sm_count;
    int ar_site;               // fused all-reduce: call-site index (see comm_fused.cu)
    const void * ar;           // NULL, or a JibArCtx: the epilogue sums the tile over all ranks through peer memory
    const void * out_row_ptr;  // NULL, or device array [rows] of bf16 row addresses (may be peer memory): row i of the result is
                               // stored there instead of out + i * ldo (a NULL entry drops the row)
    const void * ag_flags;     // NULL, or device unsigned[ag_world]: rows [s*ag_rows, (s+1)*ag_rows) of x are valid once
    const void * ag_epoch;     //   ag_flags[s] == *ag_epoch (all-gather fused into the activation loads)
    int ag_rows, ag_world;
    int ar_rs_rows;            // with ar: > 0 = reduce-scatter by token rows (row i delivered to rank i / ar_rs_rows only)
    const int * src_token;     // grouped, small batches: x is NOT expert-sorted but holds the src_rows token rows themselves; every
    int src_rows;              //   non-empty expert multiplies all of them (src_rows <= the token tile) and result row i (in the
                               //   expert-sorted order that seg describes) is the accumulator column src_token[i]: the gather of
                               //   token rows into sorted order is never materialised
    const int * expert_list;   // grouped: NULL, or device int[n_slots]: the launch covers only these experts (entries < 0 are unused
    int n_slots;               //   slots); n_slots <= batch.  For batches that hit few experts: most of the grid would exit at once
    int list_tiles;            // 1: expert_list entries are (token tile << 16 | expert) pairs (jib_moe_tile_list, built for this bn):
                               //   the launch covers exactly the token tiles that exist instead of T / bn tiles for every expert
    int pdl_flags;             // grouped, two launches back to back over one segment table: 1 on the first (it lets its dependents
                               //   start only once the table is known to be complete), 2 on the second (it may read the table and
                               //   request weights before the first launch has finished); 0 otherwise
} jib_gemm_desc;

JIB_EXPORT int jib_gemm_bf16(const jib_gemm_desc * d, void * stream);

// ---- sampling (sampling.cu) ---------------------------------------------------------------------
// One id per row from the row's top-k candidates (vals / ids [n][k], sorted by value, descending; k <= 128).
// params [n][5] fp32: temperature (<= 0: best candidate), top_k (<= 0: all), top_p (>= 1: off), min_p (<= 0: off), u in [0, 1).
JIB_EXPORT int jib_sample_topk(const float * vals, const int * ids, const float * params, int * out, int n, int k, void * stream);

// Block-quantised checkpoint data (ggml types Q4_0 .. Q8_K) -> bf16, at load time (dequant.cu).
JIB_EXPORT int jib_dequantize_bf16(unsigned ggml_type, const void * src, unsigned long long n_elements, void * dst, void * stream);

// ---- memory-bound kernels (elementwise.cu) ----------------------------------------------------
JIB_EXPORT int jib_embed_gather(const void * table, const int * ids, void * out, int T, int d, int n_vocab, void * stream);
JIB_EXPORT int jib_rmsnorm(const void * x, const void * residual, const float * w, void * out_norm, void * out_sum, int T, int d,
                           long long x_stride, float eps, void * stream);
// q_out: where the rotated RoPE part of token 0, head 0 goes; token t, head h at q_out + t * qo_row + h * qo_head (elements):
// into the absorbed-query buffer [T][H][r + dr] at offset r, or in place into q at offset dn.
JIB_EXPORT int jib_mla_qkv_post(const void * q, long long q_stride, const void * ckv, long long ckv_stride, const float * kv_norm_w,
                                float eps, const float * rope_table, const int * positions, const int * slot_mapping, void * cache,
                                void * q_out, long long qo_row, long long qo_head, int T, int H, int dn, int dr, int r, int max_pos,
                                long long n_slots, int * status, void * stream);
JIB_EXPORT int jib_argmax(const float * logits, int * out, int n, int V, void * stream);
JIB_EXPORT int jib_topk(const float * logits, float * vals, int * ids, int n, int V, int k, void * stream);
JIB_EXPORT int jib_kv_block_copy(void * cache, long long layer_stride_elems, int n_layers, const int * src, const int * dst, int n,
                                 int block_elems, void * stream);
JIB_EXPORT int jib_gather_rows(const void * x, const int * src_row, void * out, int rows, int d, int n_src, void * stream);

// ---- MoE routing (moe.cu) ---------------------------------------------------------------------
// logits: fp32 scratch [T][E] (router outputs, kept for inspection).  ids / wts have k + n_shared columns: the last
// n_shared columns name the shared experts (ids E, E+1, ...; weight 1) so that they run in the grouped GEMMs.
JIB_EXPORT int jib_moe_gate(const void * g, const float * w_router, const float * bias, float * logits, int * ids, float * wts, int T,
                            int d, int E, int k, int n_group, int topk_group, float scale, int norm, int sigmoid, int n_shared,
                            int group_top2, void * stream);
// jib_moe_gate + jib_moe_permute (over the k + n_shared id columns) in one launch, for T <= 64.  counter: one device int that is
// zero between launches.  norm_w != NULL: the rows of g are RMS-normalised first (as jib_rmsnorm would) and stored to g_out.
JIB_EXPORT int jib_moe_route_fused(const void * g, const float * w_router, const float * bias, float * logits, int * ids, float * wts,
                                   int * seg, int * src_token, int * dest, int * counter, int T, int d, int E, int k, int n_group,
                                   int topk_group, float scale, int norm, int sigmoid, int n_shared, int group_top2, int expert_base,
                                   int E_local, const float * norm_w, float eps, void * g_out, void * stream);
// Stable counting sort of the (token, k) pairs by local expert. dest[t*k+j] = sorted row or -1 (not local).
// seg has room for 2 * E_local + 1 ints: the E_local + 1 segment offsets, then the list of the experts that have rows (in
// order, -1 after the last): what jib_gemm_desc.expert_list takes.  (jib_moe_route_fused writes the same; the multi-CTA
// sort for large batches writes the offsets only.)
JIB_EXPORT int jib_moe_permute(const int * ids, int T, int k, int expert_base, int E_local, int * seg, int * src_token, int * dest,
                               void * stream);
// (expert, token tile) work list of a grouped launch with token-tile width bn: out[i] = tile << 16 | expert for every tile of
// every expert that has rows, in expert order, -1 up to cap.  cap >= rows / bn + E_local always suffices.
JIB_EXPORT int jib_moe_tile_list(const int * seg, int E_local, int bn, int * out, int cap, void * stream);
JIB_EXPORT int jib_moe_permute_multi(const int * ids, int T, int k, int expert_base, int E_local, int * seg, int * src_token, int * dest,
                                     int * tmp, void * stream);
JIB_EXPORT int jib_moe_combine(const void * y, const int * dest, const float * wts, const void * shared, const void * residual,
                               void * out, int T, int k, int d, void * stream);
// The same followed by RMSNorm(out) * norm_w (fp32 weights, as jib_rmsnorm) in one launch; bitwise the two-launch results.
JIB_EXPORT int jib_moe_combine_norm(const void * y, const int * dest, const float * wts, const void * shared, const void * residual,
                                    const float * norm_w, void * out, void * out_norm, int T, int k, int d, float eps, void * stream);

// ---- attention (mla_attention.cu) -------------------------------------------------------------
// Split-KV absorbed MLA over the paged latent cache. q [T][H][r+dr] bf16; o_lat [T][H][r] bf16.
// part_o [T][n_splits][H][r] fp32 and part_ml [T][n_splits][H][2] fp32 are scratch.
JIB_EXPORT int jib_mla_attention(const void * q, const void * cache, const int * block_tables, int max_blocks, const int * seq_lens,
                                 const int * q_start, int n_seqs, int T, int H, int r, int dr, int block_size, float scale,
                                 int n_splits, float * part_o, float * part_ml, void * o_lat, void * stream);

JIB_EXPORT int jib_mla_combine(const float * part_o, const float * part_ml, int n_splits, int T, int H, int r, void * o_lat,
                               void * stream);
// tcgen05 flash MLA (mla_flash_tcgen05.cu): r = 512, dr = 64, block size 64 only; qt = query tokens per CTA (1 or 2).
JIB_EXPORT int jib_mla_flash(const void * q, const void * cache, long long n_slots, const int * block_tables, int max_blocks,
                             const int * seq_lens, const int * q_start, int n_seqs, int T, int H, float scale, int n_splits, int qt,
                             float * part_o, float * part_ml, void * o_lat, int * status, void * stream);

// ---- prefill attention in the per-head form (mha_prefill_tcgen05.cu): head dims 128 + 64 (keys), 128 (values) ---------------
// jib_kv_gather: lat [total_cap][row_elems] <- the cached latent rows of every sequence, in sequence order; kv_start [n_seqs].
JIB_EXPORT int jib_kv_gather(const void * cache, long long n_slots, const int * block_tables, int max_blocks, const int * seq_lens,
                             int n_seqs, int block_size, int row_elems, void * lat, int * kv_start, int total_cap, void * stream);
// q [T][H][192] (RoPE applied), kv [total][H][256] = k_nope | v, kpe [total][64] (row stride kpe_stride), out [T][H * 128].
JIB_EXPORT int jib_mha_prefill(const void * q, long long q_stride, const void * kv, const void * kpe, long long kpe_stride, long long total,
                               const int * q_start, const int * seq_lens, const int * kv_start, int n_seqs, int T, int H, float scale,
                               int n_q_tiles, void * out, long long ldo, int * status, void * stream);

// ---- expert-parallel all-to-all over peer memory (ep_alltoall.cu); ctx is a JibEpCtx (ep_alltoall.h) ---------
JIB_EXPORT int jib_ep_plan(const int * ids, int T, int k, const struct JibEpCtx * ctx, int site, int * seg, int * pair_dst, void * stream);
JIB_EXPORT int jib_ep_push(const void * x, const int * pair_dst, int T, int k, const struct JibEpCtx * ctx, int site, const int * seg,
                           int * done_counter, void * row_ptr, void * stream);
JIB_EXPORT int jib_ep_combine(const float * wts, const int * pair_dst, const void * shared, const void * residual, void * out, int T,
                              int k, const struct JibEpCtx * ctx, int site, void * stream);

#ifdef __cplusplus
}
#endif
