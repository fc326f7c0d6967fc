"""GGUF v3 container constants and block-quant codecs.

Layout facts (reference: ggml/include/gguf.h:41-46, ggml/src/gguf.cpp): little-endian; header =
magic "GGUF", u32 version, u64 tensor count, u64 kv count; strings are u64 length + bytes;
tensor data starts at the next multiple of ``general.alignment`` (default 32) and each tensor
offset is aligned likewise.  ``ne[0]`` is the contiguous axis, so a row-major ``[out][in]``
weight is stored with dims ``(in, out)``.
"""
from __future__ import annotations

import numpy as np

GGUF_MAGIC = b"GGUF"
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32

# metadata value types
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)

SCALAR_FMT = {
    T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
    T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d",
}
SCALAR_NP = {
    T_U8: np.uint8, T_I8: np.int8, T_U16: np.uint16, T_I16: np.int16, T_U32: np.uint32, T_I32: np.int32,
    T_F32: np.float32, T_BOOL: np.bool_, T_U64: np.uint64, T_I64: np.int64, T_F64: np.float64,
}
TYPE_BY_NAME = {
    "u8": T_U8, "i8": T_I8, "u16": T_U16, "i16": T_I16, "u32": T_U32, "i32": T_I32, "f32": T_F32,
    "bool": T_BOOL, "str": T_STR, "u64": T_U64, "i64": T_I64, "f64": T_F64,
}

# tensor element types (ggml_type numbering)
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_BF16 = 0, 1, 2, 8, 30
GGML_I8, GGML_I16, GGML_I32 = 24, 25, 26
GGML_Q4_1, GGML_Q5_0, GGML_Q5_1 = 3, 6, 7
GGML_Q2_K, GGML_Q3_K, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K, GGML_Q8_K = 10, 11, 12, 13, 14, 15

# (block elements, block bytes)
TYPE_TRAITS = {
    GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34),
    GGML_I8: (1, 1), GGML_I16: (1, 2), GGML_I32: (1, 4),
    GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24),
    GGML_Q2_K: (256, 84), GGML_Q3_K: (256, 110), GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_Q6_K: (256, 210),
    GGML_Q8_K: (256, 292),
}
QUANTIZED = frozenset(t for t, (blk, _) in TYPE_TRAITS.items() if blk > 1)
TYPE_NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_BF16: "BF16", GGML_Q4_0: "Q4_0", GGML_Q8_0: "Q8_0",
              GGML_I8: "I8", GGML_I16: "I16", GGML_I32: "I32", GGML_Q4_1: "Q4_1", GGML_Q5_0: "Q5_0", GGML_Q5_1: "Q5_1",
              GGML_Q2_K: "Q2_K", GGML_Q3_K: "Q3_K", GGML_Q4_K: "Q4_K", GGML_Q5_K: "Q5_K", GGML_Q6_K: "Q6_K", GGML_Q8_K: "Q8_K"}


def align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def tensor_nbytes(ggml_type: int, n_elements: int) -> int:
    blk, bsz = TYPE_TRAITS[ggml_type]
    if n_elements % blk:
        raise ValueError(f"element count {n_elements} is not a multiple of block size {blk}")
    return n_elements // blk * bsz


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """fp32 [.., 32k] -> raw Q8_0 bytes (fp16 scale + 32 int8 per block)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1, keepdims=True)
    d = amax / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0)
    q = np.rint(x * inv).astype(np.int8)
    out = np.empty((x.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def dequantize_q8_0(raw: np.ndarray, n: int) -> np.ndarray:
    raw = np.frombuffer(raw, dtype=np.uint8, count=n // 32 * 34).reshape(-1, 34)
    d = raw[:, :2].copy().view(np.float16).astype(np.float32)
    q = raw[:, 2:].view(np.int8).astype(np.float32)
    return (q * d).reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """fp32 -> raw Q4_0 bytes: fp16 scale, then 16 bytes holding elements i (low nibble) and i+16 (high)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(x).argmax(axis=1)
    mx = x[np.arange(x.shape[0]), idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0)[:, None]
    q = np.clip(np.floor(x * inv + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((x.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def dequantize_q4_0(raw: np.ndarray, n: int) -> np.ndarray:
    raw = np.frombuffer(raw, dtype=np.uint8, count=n // 32 * 18).reshape(-1, 18)
    d = raw[:, :2].copy().view(np.float16).astype(np.float32)
    qs = raw[:, 2:]
    lo = (qs & 0x0F).astype(np.int8) - 8
    hi = (qs >> 4).astype(np.int8) - 8
    q = np.concatenate([lo, hi], axis=1).astype(np.float32)
    return (q * d).reshape(-1)
