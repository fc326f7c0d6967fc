// Expansion of block-quantised checkpoint tensors to bf16 on the device: the quantised bytes cross PCIe (a quarter to a
// half of the bf16 size) and the expansion runs at memory speed instead of on host cores.  Load-time only.
//
// Each thread produces eight consecutive elements (one 16-byte store); eight divides every block size, so the eight
// elements share a block.  The value of an element comes from jib_quant_elem (include/jib_quant_layout.h), the function the
// host library verifies against its block expanders, so the bit layouts are not restated here.
// The reference expands quantised rows on its device only inside get_rows (ggml/src/ggml-cann/kernels/get_row_q4_0.cpp,
// get_row_q8_0.cpp) and keeps Q4_0 / Q8_0 weights quantised for its matmul.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "jib_kernels.h"
#include "jib_quant_layout.h"

namespace {

__global__ void __launch_bounds__(256) dequant_bf16_kernel(uint32_t type, uint32_t elems, uint32_t bytes, const uint8_t * __restrict__ src,
                                                           uint64_t n_groups, __nv_bfloat16 * __restrict__ dst) {
    const uint64_t g = (uint64_t) blockIdx.x * blockDim.x + threadIdx.x;          // group of eight elements
    if (g >= n_groups) return;
    const uint64_t first = g * 8;
    const uint8_t * blk = src + (first / elems) * bytes;
    const int e0 = (int) (first % elems);
    __align__(16) __nv_bfloat16 out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __float2bfloat16_rn(jib_quant_elem(type, blk, e0 + i));
    *reinterpret_cast<uint4 *>(dst + first) = *reinterpret_cast<const uint4 *>(out);
}

}  // namespace

// src: n_elements / block_elems blocks of `ggml_type`; dst: n_elements bf16, 16-byte aligned.
// Returns 0, JIB_E_ARG (type not handled, partial block, misaligned dst, too large) or JIB_E_LAUNCH.
extern "C" JIB_EXPORT int jib_dequantize_bf16(unsigned ggml_type, const void * src, unsigned long long n_elements, void * dst,
                                              void * stream) {
    uint32_t elems = 0, bytes = 0;
    if (!jib_quant_traits(ggml_type, &elems, &bytes)) return JIB_E_ARG;
    if (n_elements % elems) return JIB_E_ARG;
    if (((uintptr_t) dst & 15) != 0) return JIB_E_ARG;
    if (n_elements == 0) return 0;
    const uint64_t n_groups = n_elements / 8;
    const uint64_t n_blocks = (n_groups + 255) / 256;
    if (n_blocks > 0x7FFFFFFFull) return JIB_E_ARG;
    dequant_bf16_kernel<<<(unsigned) n_blocks, 256, 0, (cudaStream_t) stream>>>(ggml_type, elems, bytes, (const uint8_t *) src, n_groups,
                                                                                (__nv_bfloat16 *) dst);
    return cudaGetLastError() == cudaSuccess ? 0 : JIB_E_LAUNCH;
}
