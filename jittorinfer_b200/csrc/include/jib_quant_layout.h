// Value of one element of a block-quantised ggml tensor, as a function of (type, block bytes, element index), usable from
// host and device code alike.  The host library checks it against its per-block expanders (runtime/dequant.cpp) on random
// blocks, so a device kernel that calls it inherits a layout that has been verified without a GPU.
//
// Layouts (ggml/src/ggml-common.h:160-365 in the reference): see the table at the top of runtime/dequant.cpp.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#    define JIB_HD __host__ __device__ __forceinline__
#else
#    define JIB_HD inline
#endif

// Elements and bytes per block; false for a type that is not handled.
JIB_HD bool jib_quant_traits(uint32_t type, uint32_t * elems, uint32_t * bytes) {
    switch (type) {
        case 2:  *elems = 32;  *bytes = 18;  return true;   // Q4_0
        case 3:  *elems = 32;  *bytes = 20;  return true;   // Q4_1
        case 6:  *elems = 32;  *bytes = 22;  return true;   // Q5_0
        case 7:  *elems = 32;  *bytes = 24;  return true;   // Q5_1
        case 8:  *elems = 32;  *bytes = 34;  return true;   // Q8_0
        case 10: *elems = 256; *bytes = 84;  return true;   // Q2_K
        case 11: *elems = 256; *bytes = 110; return true;   // Q3_K
        case 12: *elems = 256; *bytes = 144; return true;   // Q4_K
        case 13: *elems = 256; *bytes = 176; return true;   // Q5_K
        case 14: *elems = 256; *bytes = 210; return true;   // Q6_K
        case 15: *elems = 256; *bytes = 292; return true;   // Q8_K
        default: *elems = 0;   *bytes = 0;   return false;
    }
}

JIB_HD float jib_bits_to_float(uint32_t bits) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(bits);
#else
    float f;
    memcpy(&f, &bits, 4);
    return f;
#endif
}

// IEEE half (two little-endian bytes) -> float, subnormals included.
JIB_HD float jib_half_bytes_to_float(const uint8_t * p) {
    const uint32_t h = (uint32_t) p[0] | ((uint32_t) p[1] << 8);
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return jib_bits_to_float(sign);
        int shift = 0;
        while ((man & 0x400u) == 0) { man <<= 1; ++shift; }
        return jib_bits_to_float(sign | ((uint32_t) (113 - shift) << 23) | ((man & 0x3FFu) << 13));
    }
    if (exp == 31) return jib_bits_to_float(sign | 0x7F800000u | (man << 13));
    return jib_bits_to_float(sign | ((exp + 112) << 23) | (man << 13));
}

JIB_HD int jib_nibble32(const uint8_t * qs, int e) { return e < 16 ? (qs[e] & 0x0F) : (qs[e - 16] >> 4); }

JIB_HD uint32_t jib_word_le(const uint8_t * p) {
    return (uint32_t) p[0] | ((uint32_t) p[1] << 8) | ((uint32_t) p[2] << 16) | ((uint32_t) p[3] << 24);
}

// Six-bit (scale, min) pair i of the 12 packed bytes of Q4_K / Q5_K.
JIB_HD void jib_k4_scale_min(const uint8_t * p, int i, int * sc, int * mn) {
    if (i < 4) {
        *sc = p[i] & 63;
        *mn = p[4 + i] & 63;
    } else {
        *sc = (p[4 + i] & 0x0F) | ((p[i - 4] >> 6) << 4);
        *mn = (p[4 + i] >> 4) | ((p[i] >> 6) << 4);
    }
}

// Element e (0 <= e < block elements) of block b of the given type.  Unknown type: 0.
JIB_HD float jib_quant_elem(uint32_t type, const uint8_t * b, int e) {
    switch (type) {
        case 2: return jib_half_bytes_to_float(b) * (float) (jib_nibble32(b + 2, e) - 8);
        case 3: return jib_half_bytes_to_float(b) * (float) jib_nibble32(b + 4, e) + jib_half_bytes_to_float(b + 2);
        case 6: {
            const int hi = (int) ((jib_word_le(b + 2) >> e) & 1u) << 4;
            return jib_half_bytes_to_float(b) * (float) ((jib_nibble32(b + 6, e) | hi) - 16);
        }
        case 7: {
            const int hi = (int) ((jib_word_le(b + 4) >> e) & 1u) << 4;
            return jib_half_bytes_to_float(b) * (float) (jib_nibble32(b + 8, e) | hi) + jib_half_bytes_to_float(b + 2);
        }
        case 8: return jib_half_bytes_to_float(b) * (float) (int8_t) b[2 + e];
        case 10: {
            const int h = e >> 7, j = (e >> 5) & 3, l = e & 31;
            const uint8_t sc = b[8 * h + 2 * j + (l >> 4)];
            const int q = (b[16 + 32 * h + l] >> (2 * j)) & 3;
            return jib_half_bytes_to_float(b + 80) * (float) (sc & 0x0F) * (float) q - jib_half_bytes_to_float(b + 82) * (float) (sc >> 4);
        }
        case 11: {
            const int h = e >> 7, j = (e >> 5) & 3, l = e & 31;
            const int i = 8 * h + 2 * j + (l >> 4);
            const uint8_t * packed = b + 96;
            const int low = i < 8 ? (packed[i] & 0x0F) : (packed[i - 8] >> 4);
            const int top = (packed[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
            int q = (b[32 + 32 * h + l] >> (2 * j)) & 3;
            if (((b[l] >> (4 * h + j)) & 1) == 0) q -= 4;
            return jib_half_bytes_to_float(b + 108) * (float) ((low | (top << 4)) - 32) * (float) q;
        }
        case 12: {
            const int sub = e >> 5, l = e & 31, c = sub >> 1;
            int sc, mn;
            jib_k4_scale_min(b + 4, sub, &sc, &mn);
            const uint8_t v = b[16 + 32 * c + l];
            const int q = (sub & 1) ? (v >> 4) : (v & 0x0F);
            return jib_half_bytes_to_float(b) * (float) sc * (float) q - jib_half_bytes_to_float(b + 2) * (float) mn;
        }
        case 13: {
            const int sub = e >> 5, l = e & 31, c = sub >> 1;
            int sc, mn;
            jib_k4_scale_min(b + 4, sub, &sc, &mn);
            const uint8_t v = b[48 + 32 * c + l];
            int q = (sub & 1) ? (v >> 4) : (v & 0x0F);
            q |= ((b[16 + l] >> sub) & 1) << 4;
            return jib_half_bytes_to_float(b) * (float) sc * (float) q - jib_half_bytes_to_float(b + 2) * (float) mn;
        }
        case 14: {
            const int h = e >> 7, g = (e >> 5) & 3, l = e & 31;
            const uint8_t lo = b[64 * h + 32 * (g & 1) + l];
            const int low4 = (g & 2) ? (lo >> 4) : (lo & 0x0F);
            const int top2 = (b[128 + 32 * h + l] >> (2 * g)) & 3;
            const int8_t sc = (int8_t) b[192 + 8 * h + 2 * g + (l >> 4)];
            return jib_half_bytes_to_float(b + 208) * (float) sc * (float) ((low4 | (top2 << 4)) - 32);
        }
        case 15: return jib_bits_to_float(jib_word_le(b)) * (float) (int8_t) b[4 + e];
        default: return 0.0f;
    }
}
