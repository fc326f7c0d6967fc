"""Python face of the native byte-level BPE tokenizer (csrc/runtime/tokenizer.cpp).

Built from the ``tokenizer.ggml.*`` keys of a GGUF file, as the reference's ``llama_vocab::load``
does (src/llama-vocab.cpp:427-530); only ``model = gpt2`` with the ``deepseek-llm`` pre-tokenizer
is served, like the reference (src/llama-vocab.cpp:440, 483, 861).
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Dict, List, Sequence

import numpy as np

from .runtime import native_rt


def _sig(L):
    if getattr(L, "_tok_sig", False):
        return
    cpp, i32p, vp = C.POINTER(C.c_char_p), C.POINTER(C.c_int32), C.c_void_p
    L.jib_tok_create.restype = vp
    L.jib_tok_create.argtypes = [cpp, i32p, i32p, C.c_int, cpp, i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    L.jib_tok_destroy.restype, L.jib_tok_destroy.argtypes = None, [vp]
    L.jib_tok_encode.restype, L.jib_tok_encode.argtypes = C.c_int, [vp, C.c_char_p, C.c_int, C.c_int, C.c_int, i32p, C.c_int]
    L.jib_tok_piece.restype, L.jib_tok_piece.argtypes = C.c_int, [vp, C.c_int32, C.c_int, C.c_char_p, C.c_int]
    L.jib_tok_decode.restype, L.jib_tok_decode.argtypes = C.c_int, [vp, i32p, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int]
    for n in ("is_eog",):
        getattr(L, "jib_tok_" + n).restype, getattr(L, "jib_tok_" + n).argtypes = C.c_int, [vp, C.c_int32]
    for n in ("n_tokens", "bos", "eos", "eot"):
        getattr(L, "jib_tok_" + n).restype, getattr(L, "jib_tok_" + n).argtypes = C.c_int, [vp]
    L.jib_utf8_incomplete_tail.restype, L.jib_utf8_incomplete_tail.argtypes = C.c_int, [C.c_char_p, C.c_int]
    L._tok_sig = True


class Tokenizer:
    def __init__(self, tokens: Sequence[str], token_types: Sequence[int], merges: Sequence[str], bos: int = 11, eos: int = 11,
                 eot: int = -1, add_bos: bool = False, add_eos: bool = False):
        self._L = native_rt.lib()
        _sig(self._L)
        tb = [t.encode("utf-8") for t in tokens]
        mb = [m.encode("utf-8") for m in merges]
        ta = (C.c_char_p * len(tb))(*tb)
        ma = (C.c_char_p * max(1, len(mb)))(*mb) if mb else (C.c_char_p * 1)()
        tl = np.array([len(b) for b in tb], dtype=np.int32)
        ml = np.array([len(b) for b in mb] or [0], dtype=np.int32)
        ty = np.ascontiguousarray(token_types, dtype=np.int32) if len(token_types) else np.ones(len(tb), dtype=np.int32)
        i32p = C.POINTER(C.c_int32)
        self._h = self._L.jib_tok_create(ta, tl.ctypes.data_as(i32p), ty.ctypes.data_as(i32p), len(tb), ma, ml.ctypes.data_as(i32p),
                                         len(mb), bos, eos, eot, int(add_bos), int(add_eos))
        self.n_tokens = len(tb)

    @classmethod
    def from_gguf_kv(cls, kv: Dict[str, Any]) -> "Tokenizer":
        model = kv.get("tokenizer.ggml.model", "gpt2")
        pre = kv.get("tokenizer.ggml.pre", "deepseek-llm")
        if model != "gpt2" or pre != "deepseek-llm":
            raise ValueError(f"unsupported tokenizer {model!r}/{pre!r}: only gpt2 BPE with the deepseek-llm pre-tokenizer is served")
        toks = kv["tokenizer.ggml.tokens"]
        types = kv.get("tokenizer.ggml.token_type", [])
        return cls(toks, list(types), kv.get("tokenizer.ggml.merges", []), int(kv.get("tokenizer.ggml.bos_token_id", 11)),
                   int(kv.get("tokenizer.ggml.eos_token_id", 11)), int(kv.get("tokenizer.ggml.eot_token_id", -1)),
                   bool(kv.get("tokenizer.ggml.add_bos_token", False)), bool(kv.get("tokenizer.ggml.add_eos_token", False)))

    def __del__(self):
        try:
            if self._h:
                self._L.jib_tok_destroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def bos(self): return self._L.jib_tok_bos(self._h)
    @property
    def eos(self): return self._L.jib_tok_eos(self._h)
    @property
    def eot(self): return self._L.jib_tok_eot(self._h)
    def is_eog(self, tid: int) -> bool: return bool(self._L.jib_tok_is_eog(self._h, tid))

    def token_table(self):
        """(bytes of every token with control tokens as b"", end-of-generation ids, eos id): what a grammar sampler needs."""
        t = getattr(self, "_token_table", None)
        if t is None:
            pieces = [self.piece_bytes(i, special=False) for i in range(self.n_tokens)]
            eog = [i for i in range(self.n_tokens) if self.is_eog(i)]
            t = self._token_table = (pieces, eog, self.eos)
        return t

    def encode(self, text: str, add_special: bool = True, parse_special: bool = True) -> List[int]:
        b = text.encode("utf-8")
        cap = len(b) + 8
        out = np.empty(cap, dtype=np.int32)
        n = self._L.jib_tok_encode(self._h, b, len(b), int(add_special), int(parse_special), out.ctypes.data_as(C.POINTER(C.c_int32)), cap)
        return out[:n].tolist()

    def piece_bytes(self, tid: int, special: bool = False) -> bytes:
        buf = C.create_string_buffer(256)
        n = self._L.jib_tok_piece(self._h, tid, int(special), buf, 256)
        if n > 256:
            buf = C.create_string_buffer(n)
            self._L.jib_tok_piece(self._h, tid, int(special), buf, n)
        return buf.raw[:n]

    def decode_bytes(self, ids: Sequence[int], remove_special: bool = False, unparse_special: bool = False) -> bytes:
        a = np.ascontiguousarray(ids, dtype=np.int32)
        cap = 16 * max(1, len(a)) + 64
        buf = C.create_string_buffer(cap)
        n = self._L.jib_tok_decode(self._h, a.ctypes.data_as(C.POINTER(C.c_int32)), len(a), int(remove_special), int(unparse_special), buf, cap)
        if n > cap:
            buf = C.create_string_buffer(n)
            self._L.jib_tok_decode(self._h, a.ctypes.data_as(C.POINTER(C.c_int32)), len(a), int(remove_special), int(unparse_special), buf, n)
        return buf.raw[:n]

    def decode(self, ids: Sequence[int], **kw) -> str:
        return self.decode_bytes(ids, **kw).decode("utf-8", errors="replace")

    def incomplete_utf8_tail(self, b: bytes) -> int:
        return self._L.jib_utf8_incomplete_tail(b, len(b))
