"""Re-encode the tensors of a GGUF file in another element type, keeping every key.

    python -m jittorinfer_b200.gguf.requant in.gguf out.gguf --type bf16       # expand once, load fast ever after
    python -m jittorinfer_b200.gguf.requant in.gguf out.gguf --type q8_0

A block-quantised checkpoint is expanded on every load (``gguf/quants.py``); a bf16 copy loads as a plain view of the file.
The other direction makes a smaller file for transport.  Tensors are streamed one at a time.  The type of each tensor is
chosen as the converter chooses it (``convert_hf.pick_type``): one-dimensional tensors, biases and the router stay f32, rows
that do not hold whole blocks fall back to Q8_0 / f16.  (The reference has no such tool; upstream ``llama-quantize`` plays
this role for its users.)
"""
from __future__ import annotations

import argparse
from typing import Callable, Optional

import torch

from . import format as F
from .convert_hf import OUT_TYPES, pick_type
from .io import GGUFReader, GGUFWriter


def requantize(src: str, dst: str, out_type: str, progress: Optional[Callable[[str], None]] = None) -> int:
    """Returns the number of tensors whose type changed."""
    if out_type.lower() not in OUT_TYPES:
        raise ValueError(f"output type {out_type!r}: one of {sorted(OUT_TYPES)}")
    gt = OUT_TYPES[out_type.lower()]
    changed = 0
    with GGUFReader(src) as rd:
        w = GGUFWriter(dst, alignment=rd.alignment)
        for k, v in rd.kv.items():
            if k == "general.alignment":
                continue
            w.add_typed(k, v, rd.kv_types[k], rd.kv_elem_types.get(k))
        for name, ti in rd.tensors.items():
            keep = ti.ggml_type in (F.GGML_I8, F.GGML_I16, F.GGML_I32)
            new = ti.ggml_type if keep else pick_type(name, tuple(ti.shape), gt)
            changed += int(new != ti.ggml_type)

            def raw(n=name):
                if progress is not None:
                    progress(n)
                return rd.raw(n).tobytes()

            def expanded(n=name):
                if progress is not None:
                    progress(n)
                return rd.tensor(n).to(torch.float32)
            if new == ti.ggml_type:
                w.add_tensor_bytes(name, ti.shape, ti.ggml_type, raw)                 # bytes as they are
            else:
                w.add_tensor_lazy(name, ti.shape, new, expanded)
        w.write()
    return changed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--type", required=True, help=", ".join(sorted(OUT_TYPES)))
    ap.add_argument("-q", "--quiet", action="store_true")
    a = ap.parse_args(argv)
    n = requantize(a.src, a.dst, a.type, None if a.quiet else (lambda s: print(s, flush=True)))
    print(f"wrote {a.dst}: {n} tensors re-encoded as {a.type}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
