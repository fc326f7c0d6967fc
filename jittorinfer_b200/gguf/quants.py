"""Block-quantised ggml tensor types: byte layouts, vectorised de-quantisers and plain quantisers.

A checkpoint quantised with any of the classic (``Q4_0 Q4_1 Q5_0 Q5_1 Q8_0``) or K-family (``Q2_K .. Q6_K``, ``Q8_K``)
types loads here: the bytes of a rank's shard are expanded to fp32 on the host (natively when the runtime library is
there, ``csrc/runtime/dequant.cpp``; with the numpy code below otherwise) and stored on the device as bf16, the dtype
every GEMM kernel of this package consumes.  The reference keeps Q4_0 / Q8_0 quantised on its device and sends every
other quantised type to its CPU backend (ggml/src/ggml-cann/ggml-cann.cpp:490-1380 for the two device layouts; the
formats themselves: ggml/src/ggml-common.h:160-365, expansion ggml/src/ggml-quants.c:263-375, 771-805, 1141-1187,
1379-1410, 1610-1645, 1837-1866).  The codebook types (``IQ*``, ``TQ*``) are not handled.

Every de-quantiser takes ``blocks``: uint8 ``[n_blocks, block_bytes]`` and returns float32 ``[n_blocks, block_elems]``.
The quantisers are simple round-to-nearest encoders (no error-weighted search): they exist so that files of every type
can be written for tests and tools, not to compete with an offline quantiser.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import numpy as np

# ggml_type numbering
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 = 2, 3, 6, 7, 8
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_K = 10, 11, 12, 13, 14, 15

# type -> (elements per block, bytes per block)
TRAITS: Dict[int, Tuple[int, int]] = {
    Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
    Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), Q8_K: (256, 292),
}
NAMES = {Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q8_0: "Q8_0", Q2_K: "Q2_K", Q3_K: "Q3_K",
         Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", Q8_K: "Q8_K"}


def _f16(b: np.ndarray) -> np.ndarray:
    """uint8 [n, 2] (little endian half) -> float32 [n, 1]."""
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def _nibbles(qs: np.ndarray) -> np.ndarray:
    """uint8 [n, m] -> uint8 [n, 2m]: all low nibbles, then all high nibbles (the order of the 32-element types)."""
    return np.concatenate([qs & 0x0F, qs >> 4], axis=1)


def _bits32(qh: np.ndarray) -> np.ndarray:
    """uint8 [n, 4] (little-endian word) -> uint8 [n, 32]: bit i of the word."""
    w = np.ascontiguousarray(qh).view("<u4")                       # [n, 1]
    return ((w >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)


# ---- 32-element types ---------------------------------------------------------------------------------------------------
def dq_q4_0(b):
    return (_nibbles(b[:, 2:18]).astype(np.float32) - 8.0) * _f16(b[:, 0:2])


def dq_q4_1(b):
    return _nibbles(b[:, 4:20]).astype(np.float32) * _f16(b[:, 0:2]) + _f16(b[:, 2:4])


def dq_q5_0(b):
    q = _nibbles(b[:, 6:22]) | (_bits32(b[:, 2:6]) << 4)
    return (q.astype(np.float32) - 16.0) * _f16(b[:, 0:2])


def dq_q5_1(b):
    q = _nibbles(b[:, 8:24]) | (_bits32(b[:, 4:8]) << 4)
    return q.astype(np.float32) * _f16(b[:, 0:2]) + _f16(b[:, 2:4])


def dq_q8_0(b):
    return b[:, 2:34].view(np.int8).astype(np.float32) * _f16(b[:, 0:2])


# ---- 256-element super-blocks -------------------------------------------------------------------------------------------
_SHIFT4 = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)


def _crumbs(qs: np.ndarray) -> np.ndarray:
    """uint8 [n, 64] -> uint8 [n, 2, 4, 32]: element (h, j, l) = bits 2j..2j+1 of byte 32h + l (Q2_K / Q3_K order)."""
    return (qs.reshape(-1, 2, 1, 32) >> _SHIFT4) & 3


def dq_q2_k(b):
    n = b.shape[0]
    sc = b[:, 0:16].reshape(n, 2, 4, 2, 1)                         # scale byte of (h, j, 16-element half)
    v = _crumbs(b[:, 16:80]).reshape(n, 2, 4, 2, 16).astype(np.float32)
    d, dmin = _f16(b[:, 80:82]).reshape(n, 1, 1, 1, 1), _f16(b[:, 82:84]).reshape(n, 1, 1, 1, 1)
    return (d * (sc & 0x0F).astype(np.float32) * v - dmin * (sc >> 4).astype(np.float32)).reshape(n, 256)


def _q3_scales(s: np.ndarray) -> np.ndarray:
    """12 packed bytes -> 16 six-bit scales (bytes 0..7: low four bits of scales 0..7 | 8..15; bytes 8..11: two bits each
    of scales b, 4+b, 8+b, 12+b)."""
    out = np.concatenate([s[:, 0:8] & 0x0F, s[:, 0:8] >> 4], axis=1)
    t = s[:, 8:12]
    top = np.concatenate([t & 3, (t >> 2) & 3, (t >> 4) & 3, t >> 6], axis=1)
    return out | (top << 4)


def dq_q3_k(b):
    n = b.shape[0]
    hm = b[:, 0:32]
    plane = (hm.reshape(n, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 8, 1)) & 1       # [n, bit 4h+j, l]
    v = _crumbs(b[:, 32:96]).astype(np.int16) - 4 * (1 - plane.reshape(n, 2, 4, 32).astype(np.int16))
    sc = _q3_scales(b[:, 96:108]).astype(np.int16) - 32
    d = _f16(b[:, 108:110]).reshape(n, 1, 1, 1, 1)
    y = d * sc.reshape(n, 2, 4, 2, 1).astype(np.float32) * v.reshape(n, 2, 4, 2, 16).astype(np.float32)
    return y.reshape(n, 256)


def _k4_scales(s: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """12 packed bytes -> (8 six-bit scales, 8 six-bit mins) of Q4_K / Q5_K."""
    sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)], axis=1)
    mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=1)
    return sc, mn


def dq_q4_k(b):
    n = b.shape[0]
    sc, mn = _k4_scales(b[:, 4:16])
    qs = b[:, 16:144].reshape(n, 4, 32)
    v = np.stack([qs & 0x0F, qs >> 4], axis=2).astype(np.float32)                              # [n, 4, 2, 32]
    d, dmin = _f16(b[:, 0:2]).reshape(n, 1, 1, 1), _f16(b[:, 2:4]).reshape(n, 1, 1, 1)
    y = d * sc.reshape(n, 4, 2, 1).astype(np.float32) * v - dmin * mn.reshape(n, 4, 2, 1).astype(np.float32)
    return y.reshape(n, 256)


def dq_q5_k(b):
    n = b.shape[0]
    sc, mn = _k4_scales(b[:, 4:16])
    qh = b[:, 16:48]
    high = (qh.reshape(n, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 8, 1)) & 1        # bit 2c + (0 low | 1 high)
    qs = b[:, 48:176].reshape(n, 4, 32)
    v = (np.stack([qs & 0x0F, qs >> 4], axis=2) | (high.reshape(n, 4, 2, 32) << 4)).astype(np.float32)
    d, dmin = _f16(b[:, 0:2]).reshape(n, 1, 1, 1), _f16(b[:, 2:4]).reshape(n, 1, 1, 1)
    y = d * sc.reshape(n, 4, 2, 1).astype(np.float32) * v - dmin * mn.reshape(n, 4, 2, 1).astype(np.float32)
    return y.reshape(n, 256)


def dq_q6_k(b):
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 2, 32)                          # (h, first | second 32 bytes, l)
    low = np.concatenate([ql & 0x0F, ql >> 4], axis=2)             # [n, 2, 4, 32]: groups 0, 1 low nibbles; 2, 3 high
    top = (b[:, 128:192].reshape(n, 2, 1, 32) >> _SHIFT4) & 3
    q = (low | (top << 4)).astype(np.int16) - 32
    sc = b[:, 192:208].view(np.int8).reshape(n, 2, 4, 2, 1).astype(np.float32)
    d = _f16(b[:, 208:210]).reshape(n, 1, 1, 1, 1)
    return (d * sc * q.reshape(n, 2, 4, 2, 16).astype(np.float32)).reshape(n, 256)


def dq_q8_k(b):
    d = np.ascontiguousarray(b[:, 0:4]).view("<f4")
    return b[:, 4:260].view(np.int8).astype(np.float32) * d


DEQUANT: Dict[int, Callable[[np.ndarray], np.ndarray]] = {
    Q4_0: dq_q4_0, Q4_1: dq_q4_1, Q5_0: dq_q5_0, Q5_1: dq_q5_1, Q8_0: dq_q8_0,
    Q2_K: dq_q2_k, Q3_K: dq_q3_k, Q4_K: dq_q4_k, Q5_K: dq_q5_k, Q6_K: dq_q6_k, Q8_K: dq_q8_k,
}


def dequantize(ggml_type: int, raw, n_elements: int) -> np.ndarray:
    """Raw bytes of ``n_elements`` elements of ``ggml_type`` -> float32 [n_elements] (numpy implementation)."""
    blk, bsz = TRAITS[ggml_type]
    if n_elements % blk:
        raise ValueError(f"{NAMES[ggml_type]}: element count {n_elements} is not a multiple of {blk}")
    blocks = np.frombuffer(raw, dtype=np.uint8, count=n_elements // blk * bsz).reshape(-1, bsz)
    out = np.empty((blocks.shape[0], blk), dtype=np.float32)
    step = max(1, (1 << 22) // blk)                                # bounded temporaries: 4 M elements at a time
    for i in range(0, blocks.shape[0], step):
        out[i:i + step] = DEQUANT[ggml_type](blocks[i:i + step])
    return out.reshape(-1)


# ---- quantisers (round to nearest) --------------------------------------------------------------------------------------
def _half_bytes(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x.astype(np.float16).reshape(-1, 1)).view(np.uint8)               # [n, 2]


def _as_f16(x: np.ndarray) -> np.ndarray:
    """The value a half-precision field will hold (the codes are chosen against the stored scale, not the exact one)."""
    return x.astype(np.float16).astype(np.float32)


def _safe_inv(x: np.ndarray) -> np.ndarray:
    return np.where(x != 0, 1.0 / np.where(x != 0, x, 1.0), 0.0).astype(np.float32)


def _pack_nibbles(q: np.ndarray) -> np.ndarray:
    """uint8 [n, 2m] (low halves first) -> [n, m]."""
    m = q.shape[1] // 2
    return q[:, :m] | (q[:, m:] << 4)


def _pack_bits32(bits: np.ndarray) -> np.ndarray:
    w = (bits.astype(np.uint32) << np.arange(32, dtype=np.uint32)).sum(axis=1, dtype=np.uint32)
    return np.ascontiguousarray(w.astype("<u4").reshape(-1, 1)).view(np.uint8)                    # [n, 4]


def _affine(x: np.ndarray, levels: int):
    """Per row: (step, offset >= 0) of x ~ step * q - offset with q in 0..levels."""
    lo = np.minimum(x.min(axis=1, keepdims=True), 0.0)
    hi = np.maximum(x.max(axis=1, keepdims=True), 0.0)
    return (hi - lo) / levels, -lo


def q_q4_1(x):
    d, off = _affine(x, 15)
    d, m = _as_f16(d), _as_f16(-off)
    q = np.clip(np.rint((x - m) * _safe_inv(d)), 0, 15).astype(np.uint8)
    return np.concatenate([_half_bytes(d), _half_bytes(m), _pack_nibbles(q)], axis=1)


def q_q5_0(x):
    idx = np.abs(x).argmax(axis=1)
    d = _as_f16(x[np.arange(x.shape[0]), idx].reshape(-1, 1) / -16.0)
    q = np.clip(np.rint(x * _safe_inv(d)) + 16, 0, 31).astype(np.uint8)
    return np.concatenate([_half_bytes(d), _pack_bits32(q >> 4), _pack_nibbles(q & 0x0F)], axis=1)


def q_q5_1(x):
    d, off = _affine(x, 31)
    d, m = _as_f16(d), _as_f16(-off)
    q = np.clip(np.rint((x - m) * _safe_inv(d)), 0, 31).astype(np.uint8)
    return np.concatenate([_half_bytes(d), _half_bytes(m), _pack_bits32(q >> 4), _pack_nibbles(q & 0x0F)], axis=1)


def _pack_crumbs(v: np.ndarray) -> np.ndarray:
    """uint8 [n, 2, 4, 32] with values 0..3 -> [n, 64] (inverse of ``_crumbs``)."""
    return (v << _SHIFT4).sum(axis=2, dtype=np.uint8).reshape(-1, 64)


def _two_level(step: np.ndarray, levels: int):
    """Sub-block steps [n, s] -> (super scale [n, 1] as stored in half precision, integer codes 0..levels [n, s])."""
    d = _as_f16(step.max(axis=1, keepdims=True) / levels)
    return d, np.clip(np.rint(step * _safe_inv(d)), 0, levels).astype(np.uint8)


def q_q2_k(x):
    n = x.shape[0]
    sub = x.reshape(n * 16, 16)
    step, off = _affine(sub, 3)
    d, sc = _two_level(step.reshape(n, 16), 15)
    dmin, mn = _two_level(off.reshape(n, 16), 15)
    eff_d = (d * sc).reshape(n * 16, 1)
    eff_m = (dmin * mn).reshape(n * 16, 1)
    q = np.clip(np.rint((sub + eff_m) * _safe_inv(eff_d)), 0, 3).astype(np.uint8)
    return np.concatenate([sc | (mn << 4), _pack_crumbs(q.reshape(n, 2, 4, 32)), _half_bytes(d), _half_bytes(dmin)], axis=1)


def q_q3_k(x):
    n = x.shape[0]
    sub = x.reshape(n * 16, 16)
    idx = np.abs(sub).argmax(axis=1)
    step = (sub[np.arange(n * 16), idx] / -4.0).reshape(n, 16)                 # signed: the largest magnitude maps to -4
    d = _as_f16(np.abs(step).max(axis=1, keepdims=True) / 31.0)
    sc = np.clip(np.rint(step * _safe_inv(d)), -32, 31).astype(np.int16)
    eff = (d * sc).reshape(n * 16, 1)
    q = (np.clip(np.rint(sub * _safe_inv(eff)), -4, 3).astype(np.int16) + 4).astype(np.uint8).reshape(n, 2, 4, 32)   # 0..7
    plane = (q >> 2).reshape(n, 8, 32)                                         # bit 4h+j of hmask byte l
    hmask = (plane << np.arange(8, dtype=np.uint8).reshape(1, 8, 1)).sum(axis=1, dtype=np.uint8)
    u = (sc + 32).astype(np.uint8)                                             # six bits each
    lo = (u[:, 0:8] & 0x0F) | ((u[:, 8:16] & 0x0F) << 4)
    t = u >> 4
    hi = t[:, 0:4] | (t[:, 4:8] << 2) | (t[:, 8:12] << 4) | (t[:, 12:16] << 6)
    return np.concatenate([hmask, _pack_crumbs(q & 3), lo, hi, _half_bytes(d)], axis=1)


def _pack_k4_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    a = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    b = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    c = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return np.concatenate([a, b, c], axis=1)


def _q45_k(x, levels):
    n = x.shape[0]
    sub = x.reshape(n * 8, 32)
    step, off = _affine(sub, levels)
    d, sc = _two_level(step.reshape(n, 8), 63)
    dmin, mn = _two_level(off.reshape(n, 8), 63)
    eff_d, eff_m = (d * sc).reshape(n * 8, 1), (dmin * mn).reshape(n * 8, 1)
    q = np.clip(np.rint((sub + eff_m) * _safe_inv(eff_d)), 0, levels).astype(np.uint8).reshape(n, 4, 2, 32)
    return d, dmin, sc, mn, q


def q_q4_k(x):
    d, dmin, sc, mn, q = _q45_k(x, 15)
    qs = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(-1, 128)
    return np.concatenate([_half_bytes(d), _half_bytes(dmin), _pack_k4_scales(sc, mn), qs], axis=1)


def q_q5_k(x):
    d, dmin, sc, mn, q = _q45_k(x, 31)
    n = q.shape[0]
    qs = ((q[:, :, 0, :] & 0x0F) | ((q[:, :, 1, :] & 0x0F) << 4)).reshape(n, 128)
    high = (q >> 4).reshape(n, 8, 32)
    qh = (high << np.arange(8, dtype=np.uint8).reshape(1, 8, 1)).sum(axis=1, dtype=np.uint8)
    return np.concatenate([_half_bytes(d), _half_bytes(dmin), _pack_k4_scales(sc, mn), qh, qs], axis=1)


def q_q6_k(x):
    n = x.shape[0]
    sub = x.reshape(n * 16, 16)
    idx = np.abs(sub).argmax(axis=1)
    step = (sub[np.arange(n * 16), idx] / -32.0).reshape(n, 16)
    d = _as_f16(np.abs(step).max(axis=1, keepdims=True) / 127.0)
    sc = np.clip(np.rint(step * _safe_inv(d)), -128, 127).astype(np.int8)
    eff = (d * sc.astype(np.float32)).reshape(n * 16, 1)
    q = (np.clip(np.rint(sub * _safe_inv(eff)), -32, 31).astype(np.int16) + 32).astype(np.uint8).reshape(n, 2, 4, 32)   # 0..63
    low = q & 0x0F
    ql = (low[:, :, 0:2, :] | (low[:, :, 2:4, :] << 4)).reshape(n, 128)
    qh = ((q >> 4) << _SHIFT4).sum(axis=2, dtype=np.uint8).reshape(n, 64)
    return np.concatenate([ql, qh, sc.view(np.uint8), _half_bytes(d)], axis=1)


def q_q8_k(x):
    idx = np.abs(x).argmax(axis=1)
    d = (x[np.arange(x.shape[0]), idx].reshape(-1, 1) / -128.0).astype(np.float32)
    q = np.clip(np.rint(x * _safe_inv(d)), -128, 127).astype(np.int8)
    sums = q.reshape(-1, 16, 16).astype(np.int16).sum(axis=2, dtype=np.int16)
    return np.concatenate([np.ascontiguousarray(d.astype("<f4")).view(np.uint8), q.view(np.uint8),
                           np.ascontiguousarray(sums.astype("<i2")).view(np.uint8)], axis=1)


def _q_q4_0(x):
    from .format import quantize_q4_0
    return quantize_q4_0(x).reshape(-1, 18)


def _q_q8_0(x):
    from .format import quantize_q8_0
    return quantize_q8_0(x).reshape(-1, 34)


QUANT: Dict[int, Callable[[np.ndarray], np.ndarray]] = {
    Q4_0: _q_q4_0, Q4_1: q_q4_1, Q5_0: q_q5_0, Q5_1: q_q5_1, Q8_0: _q_q8_0,
    Q2_K: q_q2_k, Q3_K: q_q3_k, Q4_K: q_q4_k, Q5_K: q_q5_k, Q6_K: q_q6_k, Q8_K: q_q8_k,
}


def quantize(ggml_type: int, x: np.ndarray) -> np.ndarray:
    """float array whose size is a multiple of the block size -> raw bytes (uint8, 1-D)."""
    blk, bsz = TRAITS[ggml_type]
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if x.size % blk:
        raise ValueError(f"{NAMES[ggml_type]}: element count {x.size} is not a multiple of {blk}")
    out = QUANT[ggml_type](x.reshape(-1, blk))
    assert out.shape[1] == bsz, (NAMES[ggml_type], out.shape)
    return np.ascontiguousarray(out, dtype=np.uint8).reshape(-1)


# ---- load path: bytes of a shard -> torch tensor ------------------------------------------------------------------------
_native = None


def _native_lib():
    """The runtime library's ``jib_dequantize`` (threads over block ranges, writes fp32 or bf16), or False."""
    global _native
    if _native is None:
        try:
            import ctypes as C

            from ..runtime.native_rt import lib
            L = lib()
            L.jib_dequantize.restype = C.c_int
            L.jib_dequantize.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_int]
            _native = L
        except Exception:
            _native = False
    return _native


def dequantize_torch(ggml_type: int, blocks: np.ndarray, dtype=None, native: bool = True):
    """``blocks``: uint8 array whose last axis is one block (any leading shape, may be a strided view of the file mapping)
    -> 1-D torch tensor of ``dtype`` (float32 or bfloat16) with ``n_blocks * block_elems`` elements."""
    import torch
    dtype = dtype or torch.float32
    blk, bsz = TRAITS[ggml_type]
    assert blocks.dtype == np.uint8 and blocks.shape[-1] == bsz
    flat = np.ascontiguousarray(blocks).reshape(-1, bsz)            # copies only when the shard is strided in the file
    n = flat.shape[0] * blk
    L = _native_lib() if native and dtype in (torch.float32, torch.bfloat16) else False
    if L:
        out = torch.empty(n, dtype=dtype)
        rc = L.jib_dequantize(ggml_type, flat.ctypes.data, n, out.data_ptr(), int(dtype == torch.bfloat16), 0)
        if rc != 0:
            raise ValueError(f"jib_dequantize({NAMES[ggml_type]}) failed with {rc}")
        return out
    return torch.from_numpy(dequantize(ggml_type, flat, n)).to(dtype)


def dequantize_on_device(ggml_type: int, blocks: np.ndarray, device):
    """As ``dequantize_torch`` with the expansion on ``device``: the quantised bytes cross PCIe (a quarter to a half of the
    bf16 size), a kernel writes bf16 there.  Returns a 1-D bf16 tensor on ``device``."""
    import warnings

    import torch

    from ..ops import native
    blk, bsz = TRAITS[ggml_type]
    assert blocks.dtype == np.uint8 and blocks.shape[-1] == bsz
    flat = np.ascontiguousarray(blocks).reshape(-1)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")                            # read-only mapping
        raw = torch.from_numpy(flat).to(device, non_blocking=False)
    return native.dequantize_bf16(raw, ggml_type, flat.size // bsz * blk)
