"""Dump of the op graph of one forward pass (or of one layer of it) as Graphviz ``dot`` text.

The reference prints and writes ``llama_graph_deepseek2_ge_<il>.dot`` for the layer named by ``LLAMA_PRINT_LAYER``
while it builds the persistent decode graph (src/llama-context-load-utils.cpp:154-162).  There is no graph IR here -- the
model is a PyTorch module graph -- so the dump is recorded from an eager forward pass: every call of the ``ops``
front-end becomes a node (op name, operand and result shapes); an edge joins a node to the earlier node whose result
tensor (or a view of it) it reads.  Layers are told apart through ``DeepSeek2Model.tensor_hook``, which fires after
each block.

    with GraphDump(model) as g:
        engine.step()
    open("layer3.dot", "w").write(g.to_dot(layer=3))

``LLAMA_PRINT_LAYER=<il>`` makes the engine do this for its first step and write ``jittorinfer_graph_<il>.dot`` into the
working directory (``dump_on_first_step``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..ops.profile import OPS


# operands that an op writes in place (positional index): they count as results of the node as well
IN_PLACE = {"mla_qkv_post": (7, 8), "q_absorb": (2,), "kv_block_copy": (0,)}


def _tensors(x) -> List[torch.Tensor]:
    if isinstance(x, torch.Tensor):
        return [x]
    if isinstance(x, (tuple, list)):
        return [t for y in x for t in _tensors(y)]
    return []


def _key(t: torch.Tensor) -> int:
    try:
        return t.untyped_storage().data_ptr()
    except RuntimeError:
        return id(t)


class GraphDump:
    def __init__(self, model=None):
        self.model = model
        self.nodes: List[Dict] = []             # {"id", "op", "layer", "in": [shapes], "out": [shapes]}
        self.edges: List[tuple] = []            # (producer id, consumer id)
        self._producer: Dict[int, int] = {}     # storage -> node id that wrote it last
        self._saved = []
        self._layer = 0
        self._depth = 0

    def _wrap(self, name, fn):
        def wrapped(*args, **kwargs):
            if self._depth:
                return fn(*args, **kwargs)
            self._depth += 1
            try:
                out = fn(*args, **kwargs)
            finally:
                self._depth -= 1
            ins = [t for t in _tensors(list(args) + list(kwargs.values())) if t.dim() > 0]
            outs = _tensors(out)
            nid = len(self.nodes)
            self.nodes.append({"id": nid, "op": name, "layer": self._layer,
                               "in": ["x".join(map(str, t.shape)) for t in ins],
                               "out": ["x".join(map(str, t.shape)) for t in outs]})
            seen = set()
            for t in ins:
                p = self._producer.get(_key(t))
                if p is not None and p != nid and p not in seen:
                    seen.add(p)
                    self.edges.append((p, nid))
            written = [args[i] for i in IN_PLACE.get(name, ()) if i < len(args) and isinstance(args[i], torch.Tensor)]
            for t in outs + written:
                self._producer[_key(t)] = nid
            return out
        return wrapped

    def _hook(self, name: str, t: torch.Tensor) -> None:
        if name.endswith(".ffn_out"):
            self._layer += 1                     # the ops that follow belong to the next block (or to the output head)
        if self._prev_hook is not None:
            self._prev_hook(name, t)

    def __enter__(self):
        from .. import ops
        for n in OPS:
            fn = getattr(ops, n, None)
            if fn is not None:
                self._saved.append((n, fn))
                setattr(ops, n, self._wrap(n, fn))
        self._prev_hook = getattr(self.model, "tensor_hook", None) if self.model is not None else None
        if self.model is not None:
            self.model.tensor_hook = self._hook
        return self

    def __exit__(self, *exc):
        from .. import ops
        for n, fn in self._saved:
            setattr(ops, n, fn)
        self._saved.clear()
        if self.model is not None:
            self.model.tensor_hook = self._prev_hook
        return False

    def to_dot(self, layer: Optional[int] = None) -> str:
        keep = {n["id"] for n in self.nodes if layer is None or n["layer"] == layer}
        lines = ["digraph forward {", "  rankdir=TB;", "  node [shape=box, fontname=monospace, fontsize=10];"]
        for n in self.nodes:
            if n["id"] not in keep:
                continue
            label = f"{n['op']}\\nin: {', '.join(n['in'][:4])}\\nout: {', '.join(n['out'][:2])}"
            lines.append(f"  n{n['id']} [label=\"{label}\"];")
        ext = set()
        for a, b in self.edges:
            if b in keep and a in keep:
                lines.append(f"  n{a} -> n{b};")
            elif b in keep and a not in ext:      # input that comes from another layer
                ext.add(a)
                src = self.nodes[a]
                lines.append(f"  n{a} [label=\"{src['op']} (blk {src['layer']})\", style=dashed];")
                lines.append(f"  n{a} -> n{b};")
            elif b in keep:
                lines.append(f"  n{a} -> n{b};")
        lines.append("}")
        return "\n".join(lines) + "\n"


def requested_layer() -> Optional[int]:
    v = os.environ.get("LLAMA_PRINT_LAYER", "")
    try:
        return int(v) if v != "" else None
    except ValueError:
        return None


def dump_on_first_step(engine, layer: int, directory: str = ".") -> None:
    """Arms ``engine`` so that its next step with tokens runs eagerly under a ``GraphDump`` and writes the layer's dot file."""
    inner = engine.step

    def step_once():
        engine.step = inner                      # one shot
        if not engine.has_work():
            engine.step = step_once              # nothing to record yet: stay armed
            return inner()
        with GraphDump(engine.model) as g:
            ev = inner()
        path = os.path.join(directory, f"jittorinfer_graph_{layer}.dot")
        text = g.to_dot(layer)
        with open(path, "w") as f:
            f.write(text)
        print(text)
        engine.graph_dump = g
        return ev

    engine.step = step_once
