// Host-side expansion of block-quantised ggml tensor data; see dequant.h.
//
// Every expander writes one block of floats from one block of bytes and addresses both by computed index (element e of
// the block <- which byte, which bits, which scale), so the layouts can be read off the code:
//
//   32-element types   element e < 16 is the low nibble of byte e, element e >= 16 the high nibble of byte e - 16; the
//                      fifth bit of Q5_x is bit e of a 32-bit word.
//   256-element types  Q2_K / Q3_K: element e = 128 h + 32 j + l is bits 2j..2j+1 of byte 32 h + l, scale 8 h + 2 j + l/16;
//                      Q4_K / Q5_K: element e = 64 c + 32 t + l is nibble t of byte 32 c + l, scale 2 c + t;
//                      Q6_K: element e = 128 h + 32 g + l has its low four bits in nibble g/2 of byte 64 h + 32 (g%2) + l,
//                      its top two bits at 2g of byte 32 h + l of the second array, scale 8 h + 2 g + l/16.
#include "dequant.h"

#include "jib_quant_layout.h"

#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

namespace jib {
namespace {

inline float half_to_float(const uint8_t * p) {
    const uint32_t h = (uint32_t) p[0] | ((uint32_t) p[1] << 8);
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {                                       // subnormal half: renormalise
            int shift = 0;
            while ((man & 0x400u) == 0) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((uint32_t) (113 - shift) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t) ((u >> 16) | 0x40u);       // NaN stays NaN
    u += 0x7FFFu + ((u >> 16) & 1u);                                                   // round to nearest even
    return (uint16_t) (u >> 16);
}

inline uint32_t word_le(const uint8_t * p) {
    return (uint32_t) p[0] | ((uint32_t) p[1] << 8) | ((uint32_t) p[2] << 16) | ((uint32_t) p[3] << 24);
}

inline int nibble(const uint8_t * qs, int e) { return e < 16 ? (qs[e] & 0x0F) : (qs[e - 16] >> 4); }

void expand_q4_0(const uint8_t * b, float * y) {
    const float d = half_to_float(b);
    for (int e = 0; e < 32; ++e) y[e] = d * (float) (nibble(b + 2, e) - 8);
}
void expand_q4_1(const uint8_t * b, float * y) {
    const float d = half_to_float(b), m = half_to_float(b + 2);
    for (int e = 0; e < 32; ++e) y[e] = d * (float) nibble(b + 4, e) + m;
}
void expand_q5_0(const uint8_t * b, float * y) {
    const float d = half_to_float(b);
    const uint32_t hi = word_le(b + 2);
    for (int e = 0; e < 32; ++e) y[e] = d * (float) ((nibble(b + 6, e) | (int) (((hi >> e) & 1u) << 4)) - 16);
}
void expand_q5_1(const uint8_t * b, float * y) {
    const float d = half_to_float(b), m = half_to_float(b + 2);
    const uint32_t hi = word_le(b + 4);
    for (int e = 0; e < 32; ++e) y[e] = d * (float) (nibble(b + 8, e) | (int) (((hi >> e) & 1u) << 4)) + m;
}
void expand_q8_0(const uint8_t * b, float * y) {
    const float d = half_to_float(b);
    for (int e = 0; e < 32; ++e) y[e] = d * (float) (int8_t) b[2 + e];
}

void expand_q2_k(const uint8_t * b, float * y) {
    const uint8_t * scales = b, * qs = b + 16;
    const float d = half_to_float(b + 80), dmin = half_to_float(b + 82);
    for (int e = 0; e < 256; ++e) {
        const int h = e >> 7, j = (e >> 5) & 3, l = e & 31;
        const uint8_t sc = scales[8 * h + 2 * j + (l >> 4)];
        const int q = (qs[32 * h + l] >> (2 * j)) & 3;
        y[e] = d * (float) (sc & 0x0F) * (float) q - dmin * (float) (sc >> 4);
    }
}

void expand_q3_k(const uint8_t * b, float * y) {
    const uint8_t * hmask = b, * qs = b + 32, * packed = b + 96;
    const float d = half_to_float(b + 108);
    int scale[16];
    for (int i = 0; i < 16; ++i) {
        const int low = i < 8 ? (packed[i] & 0x0F) : (packed[i - 8] >> 4);
        const int top = (packed[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
        scale[i] = (low | (top << 4)) - 32;
    }
    for (int e = 0; e < 256; ++e) {
        const int h = e >> 7, j = (e >> 5) & 3, l = e & 31;
        int q = (qs[32 * h + l] >> (2 * j)) & 3;
        if (((hmask[l] >> (4 * h + j)) & 1) == 0) q -= 4;
        y[e] = d * (float) scale[8 * h + 2 * j + (l >> 4)] * (float) q;
    }
}

// Six-bit scales and mins of Q4_K / Q5_K: entries 0..3 sit in the low six bits of bytes 0..3 (scales) and 4..7 (mins);
// entries 4..7 have their low four bits in bytes 8..11 and their top two bits in the spare bits of bytes 0..7.
inline void k4_scale_min(const uint8_t * p, int i, int * sc, int * mn) {
    if (i < 4) {
        *sc = p[i] & 63;
        *mn = p[4 + i] & 63;
    } else {
        *sc = (p[4 + i] & 0x0F) | ((p[i - 4] >> 6) << 4);
        *mn = (p[4 + i] >> 4) | ((p[i] >> 6) << 4);
    }
}

void expand_q4_k(const uint8_t * b, float * y) {
    const float d = half_to_float(b), dmin = half_to_float(b + 2);
    const uint8_t * qs = b + 16;
    for (int sub = 0; sub < 8; ++sub) {
        int sc, mn;
        k4_scale_min(b + 4, sub, &sc, &mn);
        const float ds = d * (float) sc, ms = dmin * (float) mn;
        const int c = sub >> 1, t = sub & 1;
        for (int l = 0; l < 32; ++l) {
            const int q = t ? (qs[32 * c + l] >> 4) : (qs[32 * c + l] & 0x0F);
            y[32 * sub + l] = ds * (float) q - ms;
        }
    }
}

void expand_q5_k(const uint8_t * b, float * y) {
    const float d = half_to_float(b), dmin = half_to_float(b + 2);
    const uint8_t * qh = b + 16, * qs = b + 48;
    for (int sub = 0; sub < 8; ++sub) {
        int sc, mn;
        k4_scale_min(b + 4, sub, &sc, &mn);
        const float ds = d * (float) sc, ms = dmin * (float) mn;
        const int c = sub >> 1, t = sub & 1;
        for (int l = 0; l < 32; ++l) {
            int q = t ? (qs[32 * c + l] >> 4) : (qs[32 * c + l] & 0x0F);
            q |= ((qh[l] >> sub) & 1) << 4;
            y[32 * sub + l] = ds * (float) q - ms;
        }
    }
}

void expand_q6_k(const uint8_t * b, float * y) {
    const uint8_t * ql = b, * qh = b + 128;
    const int8_t * scales = (const int8_t *) (b + 192);
    const float d = half_to_float(b + 208);
    for (int e = 0; e < 256; ++e) {
        const int h = e >> 7, g = (e >> 5) & 3, l = e & 31;
        const uint8_t lo = ql[64 * h + 32 * (g & 1) + l];
        const int low4 = (g & 2) ? (lo >> 4) : (lo & 0x0F);
        const int top2 = (qh[32 * h + l] >> (2 * g)) & 3;
        y[e] = d * (float) scales[8 * h + 2 * g + (l >> 4)] * (float) ((low4 | (top2 << 4)) - 32);
    }
}

void expand_q8_k(const uint8_t * b, float * y) {
    float d;
    memcpy(&d, b, 4);
    for (int e = 0; e < 256; ++e) y[e] = d * (float) (int8_t) b[4 + e];
}

struct Traits {
    uint32_t type;
    uint32_t elems, bytes;
    void (*expand)(const uint8_t *, float *);
};
const Traits kTraits[] = {
    {2, 32, 18, expand_q4_0},    {3, 32, 20, expand_q4_1},    {6, 32, 22, expand_q5_0},    {7, 32, 24, expand_q5_1},
    {8, 32, 34, expand_q8_0},    {10, 256, 84, expand_q2_k},  {11, 256, 110, expand_q3_k}, {12, 256, 144, expand_q4_k},
    {13, 256, 176, expand_q5_k}, {14, 256, 210, expand_q6_k}, {15, 256, 292, expand_q8_k},
};
const Traits * find(uint32_t t) {
    for (const Traits & x : kTraits) if (x.type == t) return &x;
    return nullptr;
}

void run_range(const Traits * tr, const uint8_t * src, uint64_t b0, uint64_t b1, void * dst, bool bf16) {
    float tmp[256];
    for (uint64_t blk = b0; blk < b1; ++blk) {
        const uint8_t * p = src + blk * tr->bytes;
        if (!bf16) {
            tr->expand(p, (float *) dst + blk * tr->elems);
        } else {
            tr->expand(p, tmp);
            uint16_t * o = (uint16_t *) dst + blk * tr->elems;
            for (uint32_t e = 0; e < tr->elems; ++e) o[e] = float_to_bf16(tmp[e]);
        }
    }
}

}  // namespace

uint64_t quant_block_elems(uint32_t t) { const Traits * x = find(t); return x ? x->elems : 0; }
uint64_t quant_block_bytes(uint32_t t) { const Traits * x = find(t); return x ? x->bytes : 0; }

// One element at a time through the layout function that device code shares (include/jib_quant_layout.h): slow, exists so
// that the function can be checked against the block expanders above.
int dequantize_elementwise(uint32_t ggml_type, const void * src, uint64_t n_elements, float * dst) {
    uint32_t elems = 0, bytes = 0;
    if (!jib_quant_traits(ggml_type, &elems, &bytes)) return -1;
    if (n_elements % elems) return -2;
    const uint8_t * p = (const uint8_t *) src;
    for (uint64_t i = 0; i < n_elements; ++i) dst[i] = jib_quant_elem(ggml_type, p + (i / elems) * bytes, (int) (i % elems));
    return 0;
}

int dequantize(uint32_t ggml_type, const void * src, uint64_t n_elements, void * dst, bool dst_bf16, int n_threads) {
    const Traits * tr = find(ggml_type);
    if (tr == nullptr) return -1;
    if (n_elements % tr->elems) return -2;
    const uint64_t n_blocks = n_elements / tr->elems;
    if (n_blocks == 0) return 0;
    if (n_threads <= 0) {
        const uint64_t want = (n_elements + (4u << 20) - 1) / (4u << 20);
        const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
        n_threads = (int) std::min<uint64_t>(want, hw);
    }
    n_threads = (int) std::min<uint64_t>((uint64_t) std::max(1, n_threads), n_blocks);
    if (n_threads == 1) {
        run_range(tr, (const uint8_t *) src, 0, n_blocks, dst, dst_bf16);
        return 0;
    }
    std::vector<std::thread> pool;
    const uint64_t per = (n_blocks + n_threads - 1) / n_threads;
    for (int t = 0; t < n_threads; ++t) {
        const uint64_t b0 = per * t, b1 = std::min(n_blocks, b0 + per);
        if (b0 >= b1) break;
        pool.emplace_back(run_range, tr, (const uint8_t *) src, b0, b1, dst, dst_bf16);
    }
    for (std::thread & th : pool) th.join();
    return 0;
}

}  // namespace jib
