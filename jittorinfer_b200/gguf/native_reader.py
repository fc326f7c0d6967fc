"""GGUF reader backed by the C++ parser (``csrc/runtime/gguf.cpp``): header, key/values and the tensor table are parsed
natively over a read-only mapping and tensor data is handed out as pointers into it, so a tensor-parallel rank touches
only the bytes of its own shard.  Same interface as :class:`jittorinfer_b200.gguf.io.GGUFReader` (``kv``, ``tensors``,
``tensor``, ``tensor_slice``, ``raw``); select it for model loading with ``JITTORINFER_GGUF=native``.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Any, Dict

import numpy as np

from .io import GGUFReader, TensorInfo


def _lib():
    from ..runtime.native_rt import lib
    L = lib()
    if not getattr(L, "_gguf_bound", False):
        vp = C.c_void_p
        L.jib_gguf_open.restype, L.jib_gguf_open.argtypes = vp, [C.c_char_p, C.c_int, C.c_char_p, C.c_int]
        L.jib_gguf_close.restype, L.jib_gguf_close.argtypes = None, [vp]
        L.jib_gguf_version.restype, L.jib_gguf_version.argtypes = C.c_int, [vp]
        L.jib_gguf_alignment.restype, L.jib_gguf_alignment.argtypes = C.c_int, [vp]
        L.jib_gguf_n_tensors.restype, L.jib_gguf_n_tensors.argtypes = C.c_int64, [vp]
        L.jib_gguf_tensor_info.restype = C.c_int
        L.jib_gguf_tensor_info.argtypes = [vp, C.c_int64, C.c_char_p, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32),
                                           C.POINTER(C.c_uint64), C.POINTER(vp)]
        L.jib_gguf_kv_json.restype, L.jib_gguf_kv_json.argtypes = C.c_int64, [vp, C.c_char_p, C.c_int64]
        L._gguf_bound = True
    return L


class NativeGGUFReader(GGUFReader):
    def __init__(self, path: str, populate: bool = False):
        from ..utils import fault
        fault.check("gguf_read")
        self.path = path
        self._L = _lib()
        err = C.create_string_buffer(512)
        self._h = self._L.jib_gguf_open(path.encode(), int(populate), err, 512)
        if not self._h:
            raise ValueError(f"{path}: {err.value.decode(errors='replace')}")
        self.version = self._L.jib_gguf_version(self._h)
        self.alignment = self._L.jib_gguf_alignment(self._h)
        n = self._L.jib_gguf_kv_json(self._h, None, 0)
        buf = C.create_string_buffer(n)
        self._L.jib_gguf_kv_json(self._h, buf, n)
        self.kv: Dict[str, Any] = json.loads(buf.raw[:n].decode("utf-8", errors="replace"))
        self.kv_types: Dict[str, int] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._ptr: Dict[str, int] = {}
        name = C.create_string_buffer(512)
        ne = (C.c_uint64 * 8)()
        gt, nb, data = C.c_uint32(), C.c_uint64(), C.c_void_p()
        for i in range(self._L.jib_gguf_n_tensors(self._h)):
            nd = self._L.jib_gguf_tensor_info(self._h, i, name, 512, ne, C.byref(gt), C.byref(nb), C.byref(data))
            nm = name.value.decode()
            shape = tuple(int(ne[d]) for d in reversed(range(nd)))
            self.tensors[nm] = TensorInfo(nm, shape, int(gt.value), 0, int(nb.value))
            self._ptr[nm] = int(data.value)

    def close(self):
        if getattr(self, "_h", None):
            self._L.jib_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def raw(self, name: str) -> np.ndarray:
        ti = self.tensors[name]
        # The array (and every tensor made from it) keeps this reader alive: the mapping is released only when the last
        # view is gone -- on the CPU a float32 tensor "moved" to the CPU is still a view of the file.
        buf = (C.c_uint8 * ti.nbytes).from_address(self._ptr[name])
        buf._owner = self
        arr = np.frombuffer(buf, dtype=np.uint8)
        arr.flags.writeable = False
        return arr
