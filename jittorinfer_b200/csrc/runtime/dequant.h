// Expansion of block-quantised ggml tensor data (Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q2_K Q3_K Q4_K Q5_K Q6_K Q8_K) to fp32 or bf16 on
// the host, split over threads by block range.  This is the load-time path of quantised checkpoints: the device stores
// bf16.  The reference expands the same formats in ggml/src/ggml-quants.c (formats: ggml/src/ggml-common.h:160-365).
#pragma once

#include <cstdint>

namespace jib {

// Elements / bytes of one block of a ggml type; 0 for a type this file does not expand.
uint64_t quant_block_elems(uint32_t ggml_type);
uint64_t quant_block_bytes(uint32_t ggml_type);

// Expands n_elements (a multiple of the block size) from src to dst (float, or bf16 bit patterns when dst_bf16).
// n_threads <= 0: one thread per 4 M elements, at most the hardware concurrency.
// Returns 0, -1 (type not handled) or -2 (n_elements is not a whole number of blocks).
int dequantize(uint32_t ggml_type, const void * src, uint64_t n_elements, void * dst, bool dst_bf16, int n_threads);

// The same expansion through the per-element layout function shared with device code; for cross-checking only.
int dequantize_elementwise(uint32_t ggml_type, const void * src, uint64_t n_elements, float * dst);

}  // namespace jib
