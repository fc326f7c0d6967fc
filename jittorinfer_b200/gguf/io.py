"""GGUF reader (mmap, zero-copy tensor views) and writer.

The reader plays the role of ``llama_model_loader`` (src/llama-model-loader.cpp:488-541: header + KV
parse, tensor table, mmap of the data section) and of its per-rank "tensor viewers"
(823-869, 1440-1473): :meth:`GGUFReader.tensor_slice` returns a strided view of one shard of a
tensor straight from the mapping, so a TP/EP rank only ever touches its own bytes.
The writer has no counterpart in the reference (it never writes GGUF); it exists to emit the
random-init test and benchmark models.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import format as F


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]       # torch order (outermost first) = reversed ggml ne
    ggml_type: int
    offset: int                  # relative to data section
    nbytes: int

    @property
    def n_elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


# ----------------------------------------------------------------------------------------------
class GGUFWriter:
    def __init__(self, path: str, alignment: int = F.DEFAULT_ALIGNMENT):
        self.path = path
        self.alignment = alignment
        self.kv: List[Tuple[str, int, Any, Optional[int]]] = []
        self.tensors: List[Tuple[str, Tuple[int, ...], int, bytes]] = []

    # -- metadata ---------------------------------------------------------------------------
    def add(self, key: str, value: Any, vtype: Optional[str] = None):
        """``value`` may be a python scalar/str/list, or a ``(type_name, value)`` pair."""
        if isinstance(value, tuple) and len(value) == 2 and isinstance(value[0], str) and value[0] in F.TYPE_BY_NAME:
            vtype, value = value
        if isinstance(value, (list, tuple, np.ndarray)):
            if vtype is None:
                if len(value) and isinstance(value[0], str):
                    et = F.T_STR
                elif len(value) and isinstance(value[0], float):
                    et = F.T_F32
                else:
                    et = F.T_I32
            else:
                et = F.TYPE_BY_NAME[vtype]
            self.kv.append((key, F.T_ARR, list(value), et))
            return
        if vtype is None:
            if isinstance(value, bool):
                t = F.T_BOOL
            elif isinstance(value, str):
                t = F.T_STR
            elif isinstance(value, float):
                t = F.T_F32
            else:
                t = F.T_U32
        else:
            t = F.TYPE_BY_NAME[vtype]
        self.kv.append((key, t, value, None))

    def add_typed(self, key: str, value: Any, t: int, et: Optional[int] = None):
        """A key with its GGUF value type (and element type, for arrays) given as numbers: what a reader reports."""
        if t == F.T_ARR:
            if et is None:
                raise ValueError(f"{key}: an array needs its element type")
            value = [x.item() if isinstance(x, np.generic) else x for x in value]
        elif isinstance(value, np.generic):
            value = value.item()
        self.kv.append((key, t, value, et))

    def add_dict(self, d: Dict[str, Any]):
        for k, v in d.items():
            self.add(k, v)

    # -- tensors ----------------------------------------------------------------------------
    def add_tensor(self, name: str, array, ggml_type: Optional[int] = None):
        """``array``: numpy array (f32/f16) or torch tensor (f32/f16/bf16), torch-order shape."""
        try:
            import torch
            is_torch = isinstance(array, torch.Tensor)
        except Exception:  # pragma: no cover
            is_torch = False
        if is_torch:
            t = array.detach().cpu().contiguous()
            shape = tuple(t.shape)
            if ggml_type is None:
                ggml_type = {torch.float32: F.GGML_F32, torch.float16: F.GGML_F16, torch.bfloat16: F.GGML_BF16}[t.dtype]
            if ggml_type == F.GGML_BF16:
                raw = t.to(torch.bfloat16).view(torch.int16).numpy().tobytes()
            elif ggml_type == F.GGML_F16:
                raw = t.to(torch.float16).numpy().tobytes()
            elif ggml_type == F.GGML_F32:
                raw = t.to(torch.float32).numpy().tobytes()
            elif ggml_type in F.QUANTIZED:
                raw = self._quantize(name, ggml_type, t.to(torch.float32).numpy())
            else:
                raise ValueError(f"cannot write ggml type {ggml_type}")
        else:
            a = np.ascontiguousarray(array)
            shape = tuple(a.shape)
            if ggml_type is None:
                ggml_type = {np.dtype(np.float32): F.GGML_F32, np.dtype(np.float16): F.GGML_F16}[a.dtype]
            if ggml_type in F.QUANTIZED:
                raw = self._quantize(name, ggml_type, a.astype(np.float32))
            else:
                raw = a.tobytes()
        self.tensors.append((name, shape, ggml_type, raw))

    def add_tensor_lazy(self, name: str, shape, ggml_type: int, producer):
        """Registers a tensor whose bytes ``producer()`` returns only when the file is written, so that a checkpoint larger
        than host memory can be converted one tensor at a time.  ``producer`` returns what ``add_tensor`` accepts."""
        shape = tuple(int(x) for x in shape)
        n = 1
        for x in shape:
            n *= x
        self.tensors.append((name, shape, ggml_type, _LazyBytes(self, name, shape, ggml_type, producer,
                                                                  F.tensor_nbytes(ggml_type, n))))

    def add_tensor_bytes(self, name: str, shape, ggml_type: int, producer):
        """Like ``add_tensor_lazy`` for data that is already encoded: ``producer()`` returns the tensor's bytes."""
        self.add_tensor_lazy(name, shape, ggml_type, producer)
        self.tensors[-1][3].encoded = True

    @staticmethod
    def _quantize(name: str, ggml_type: int, x: np.ndarray) -> bytes:
        from . import quants
        blk = F.TYPE_TRAITS[ggml_type][0]
        if x.ndim == 0 or x.shape[-1] % blk:
            raise ValueError(f"tensor {name}: rows of {x.shape[-1] if x.ndim else 1} elements do not hold whole "
                             f"{F.TYPE_NAMES[ggml_type]} blocks of {blk}")
        return quants.quantize(ggml_type, x).tobytes()

    # -- serialisation ----------------------------------------------------------------------
    @staticmethod
    def _s(b: bytearray, s: str):
        e = s.encode("utf-8")
        b += struct.pack("<Q", len(e)) + e

    def _value(self, b: bytearray, t: int, v: Any, et: Optional[int]):
        if t == F.T_STR:
            self._s(b, v)
        elif t == F.T_ARR:
            b += struct.pack("<IQ", et, len(v))
            if et == F.T_STR:
                for s in v:
                    self._s(b, s)
            else:
                b += np.asarray(v, dtype=F.SCALAR_NP[et]).tobytes()
        else:
            b += struct.pack(F.SCALAR_FMT[t], v)

    def write(self):
        b = bytearray()
        kv = list(self.kv)
        if not any(k == "general.alignment" for k, *_ in kv):
            kv.append(("general.alignment", F.T_U32, self.alignment, None))
        b += F.GGUF_MAGIC + struct.pack("<IQQ", F.GGUF_VERSION, len(self.tensors), len(kv))
        for key, t, v, et in kv:
            self._s(b, key)
            b += struct.pack("<I", t)
            self._value(b, t, v, et)
        off = 0
        offsets = []
        for name, shape, gt, raw in self.tensors:
            self._s(b, name)
            ne = tuple(reversed(shape))
            b += struct.pack("<I", len(ne)) + struct.pack(f"<{len(ne)}Q", *ne) + struct.pack("<IQ", gt, off)
            offsets.append(off)
            off = F.align_up(off + len(raw), self.alignment)
        pad = F.align_up(len(b), self.alignment) - len(b)
        b += b"\0" * pad
        with open(self.path, "wb") as f:
            f.write(b)
            pos = 0
            for (name, shape, gt, raw), o in zip(self.tensors, offsets):
                if o > pos:
                    f.write(b"\0" * (o - pos))
                    pos = o
                data = raw.get() if isinstance(raw, _LazyBytes) else raw
                f.write(data)
                pos += len(data)
            end = F.align_up(pos, self.alignment)
            if end > pos:
                f.write(b"\0" * (end - pos))


class _LazyBytes:
    """Stand-in for the bytes of a tensor that is produced at write time; knows its length for the offset table."""

    def __init__(self, writer, name, shape, ggml_type, producer, nbytes):
        self.writer, self.name, self.shape, self.ggml_type, self.producer, self.nbytes = writer, name, shape, ggml_type, producer, nbytes

    def __len__(self):
        return self.nbytes

    encoded = False

    def get(self) -> bytes:
        if self.encoded:
            raw = bytes(self.producer())
            if len(raw) != self.nbytes:
                raise ValueError(f"tensor {self.name}: produced {len(raw)} bytes, announced {self.nbytes}")
            return raw
        tmp = GGUFWriter.__new__(GGUFWriter)
        tmp.tensors = []
        tmp.add_tensor(self.name, self.producer(), self.ggml_type)
        _, shape, _, raw = tmp.tensors[0]
        if tuple(shape) != self.shape or len(raw) != self.nbytes:
            raise ValueError(f"tensor {self.name}: produced shape {tuple(shape)} ({len(raw)} bytes), announced {self.shape} "
                             f"({self.nbytes} bytes)")
        return raw


# ----------------------------------------------------------------------------------------------
class GGUFReader:
    """Parses header/KV/tensor table and maps the file; tensors are views of the mapping."""

    def __init__(self, path: str, populate: bool = False):
        from ..utils import fault
        fault.check("gguf_read")
        self.path = path
        with open(path, "rb") as f:          # the mapping keeps its own descriptor: the file object is not needed after it
            size = os.fstat(f.fileno()).st_size
            flags = mmap.MAP_PRIVATE | (getattr(mmap, "MAP_POPULATE", 0) if populate else 0)
            self._mm = mmap.mmap(f.fileno(), size, flags=flags, prot=mmap.PROT_READ)
        self._buf = memoryview(self._mm)
        self.kv: Dict[str, Any] = {}
        self.kv_types: Dict[str, int] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._parse()

    def close(self):
        self._buf.release()
        try:
            self._mm.close()
        except BufferError:   # views still alive; the mapping is released with them
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- parsing ----------------------------------------------------------------------------
    def _parse(self):
        buf = self._buf
        if bytes(buf[:4]) != F.GGUF_MAGIC:
            raise ValueError(f"{self.path}: not a GGUF file")
        self.version, = struct.unpack_from("<I", buf, 4)
        if self.version < 2 or self.version > 3:
            raise ValueError(f"{self.path}: unsupported GGUF version {self.version}")
        n_tensors, n_kv = struct.unpack_from("<QQ", buf, 8)
        pos = 24

        last_elem_type = [0]

        def rd_str(p):
            n, = struct.unpack_from("<Q", buf, p)
            return bytes(buf[p + 8:p + 8 + n]).decode("utf-8", errors="replace"), p + 8 + n

        def rd_val(t, p):
            if t == F.T_STR:
                return rd_str(p)
            if t == F.T_ARR:
                et, n = struct.unpack_from("<IQ", buf, p)
                p += 12
                last_elem_type[0] = et
                if et == F.T_STR:
                    out = []
                    for _ in range(n):
                        s, p = rd_str(p)
                        out.append(s)
                    return out, p
                dt = np.dtype(F.SCALAR_NP[et])
                arr = np.frombuffer(buf, dtype=dt, count=n, offset=p)
                return arr, p + n * dt.itemsize
            fmt = F.SCALAR_FMT[t]
            v, = struct.unpack_from(fmt, buf, p)
            return v, p + struct.calcsize(fmt)

        self.kv_elem_types: Dict[str, int] = {}
        for _ in range(n_kv):
            key, pos = rd_str(pos)
            t, = struct.unpack_from("<I", buf, pos)
            pos += 4
            v, pos = rd_val(t, pos)
            self.kv[key] = v
            self.kv_types[key] = t
            if t == F.T_ARR:
                self.kv_elem_types[key] = last_elem_type[0]
        self.alignment = int(self.kv.get("general.alignment", F.DEFAULT_ALIGNMENT))
        for _ in range(n_tensors):
            name, pos = rd_str(pos)
            nd, = struct.unpack_from("<I", buf, pos)
            pos += 4
            ne = struct.unpack_from(f"<{nd}Q", buf, pos)
            pos += 8 * nd
            gt, off = struct.unpack_from("<IQ", buf, pos)
            pos += 12
            shape = tuple(int(x) for x in reversed(ne))
            n = 1
            for s in shape:
                n *= s
            if gt not in F.TYPE_TRAITS:
                raise ValueError(f"tensor {name}: unsupported ggml type {gt}")
            self.tensors[name] = TensorInfo(name, shape, gt, int(off), F.tensor_nbytes(gt, n))
        self.data_offset = F.align_up(pos, self.alignment)
        end = len(buf)
        for ti in self.tensors.values():
            if self.data_offset + ti.offset + ti.nbytes > end:
                raise ValueError(f"tensor {ti.name} runs past the end of the file")

    # -- access -----------------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        ti = self.tensors[name]
        return np.frombuffer(self._buf, dtype=np.uint8, count=ti.nbytes, offset=self.data_offset + ti.offset)

    def tensor(self, name: str):
        """Whole tensor as a torch tensor.  f32/f16/bf16 are zero-copy views of the mapping."""
        return self.tensor_slice(name)

    def tensor_slice(self, name: str, dim: int = 0, index: int = 0, count: int = 1):
        """Shard ``index`` of ``count`` equal parts along torch dim ``dim`` (view, no copy)."""
        import torch
        import warnings
        ti = self.tensors[name]
        raw = self.raw(name)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # read-only mapping: torch warns about non-writable buffers
            if ti.ggml_type == F.GGML_F32:
                t = torch.from_numpy(raw.view(np.float32)).view(ti.shape)
            elif ti.ggml_type == F.GGML_F16:
                t = torch.from_numpy(raw.view(np.float16)).view(ti.shape)
            elif ti.ggml_type == F.GGML_BF16:
                t = torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16).view(ti.shape)
            elif ti.ggml_type in F.QUANTIZED:
                t, count = self._dequant_shard(ti, raw, dim, index, count)
            elif ti.ggml_type == F.GGML_I32:
                t = torch.from_numpy(raw.view(np.int32)).view(ti.shape)
            else:
                raise ValueError(f"tensor {name}: cannot materialise ggml type {ti.ggml_type}")
        if count > 1:
            n = t.shape[dim]
            if n % count:
                raise ValueError(f"tensor {name}: dim {dim} of size {n} not divisible by {count}")
            step = n // count
            t = t.narrow(dim, index * step, step)
        return t

    # dtype of tensors expanded from a block-quantised type: float32, or bfloat16 when the loader stores bf16 on the device
    # anyway (halves the host memory and the bytes sent to the device)
    quant_out_dtype = None
    # a CUDA device: the quantised bytes of a shard are sent there and expanded to bf16 by a kernel (ops/native.py:
    # dequantize_bf16); tensors of quantised types then come back as device tensors
    quant_device = None

    def _dequant_shard(self, ti: TensorInfo, raw: np.ndarray, dim: int, index: int, count: int):
        """Expands shard ``index`` of ``count`` along ``dim`` of a block-quantised tensor, touching only that shard's blocks
        when the cut falls on block boundaries.  Returns (tensor, parts still to cut by the caller)."""
        from . import quants
        blk, bsz = F.TYPE_TRAITS[ti.ggml_type]
        shape = tuple(ti.shape)
        if not shape or shape[-1] % blk:
            raise ValueError(f"tensor {ti.name}: rows of {shape[-1] if shape else 1} elements do not hold whole "
                             f"{F.TYPE_NAMES[ti.ggml_type]} blocks")
        blocks = raw.reshape(shape[:-1] + (shape[-1] // blk, bsz))
        out_shape = list(shape)
        if count > 1:
            d = dim % len(shape)
            n = shape[d]
            if n % count:
                raise ValueError(f"tensor {ti.name}: dim {dim} of size {n} not divisible by {count}")
            step = n // count
            if d < len(shape) - 1:
                blocks = blocks[(slice(None),) * d + (slice(index * step, (index + 1) * step),)]
                out_shape[d], count = step, 1
            elif step % blk == 0:
                blocks = blocks[..., index * step // blk:(index + 1) * step // blk, :]
                out_shape[d], count = step, 1
        if self.quant_device is not None:
            t = quants.dequantize_on_device(ti.ggml_type, blocks, self.quant_device)
        else:
            t = quants.dequantize_torch(ti.ggml_type, blocks, self.quant_out_dtype)
        return t.view(out_shape), count

    def describe(self) -> str:
        lines = [f"GGUF v{self.version} {self.path}: {len(self.kv)} kv, {len(self.tensors)} tensors"]
        for ti in self.tensors.values():
            lines.append(f"  {ti.name:40s} {F.TYPE_NAMES[ti.ggml_type]:5s} {list(ti.shape)}")
        return "\n".join(lines)
