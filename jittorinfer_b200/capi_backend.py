"""Python side of ``libllama.so`` (the ``llama.h`` C API).

The C++ library owns the API objects, the GGUF metadata, the tokenizer, the samplers and the KV block
tables; this module owns what lives on the GPU: the weights (``load_model``), the paged latent cache
(``create_context``) and the forward pass (``forward``).  Every function takes and returns plain
integers so that the bridge needs no object marshalling: buffers are passed as addresses of memory the
C++ side keeps alive for the duration of the call.

Reference counterparts: model load ``src/llama-model-load-utils.cpp:13-153``, context creation
``src/llama-context-load-utils.cpp:32-190``, the compute step of ``llama_decode_impl``
(``src/llama-execute-decode.cpp:209-290``) including the device top-k "presample" (132-154), and the
data-parallel ``llama_empty_run`` (367-394).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict

import numpy as np
import torch

from . import ops
from .models.deepseek2 import ForwardBatch

_models: Dict[int, "_Model"] = {}
_contexts: Dict[int, "_Context"] = {}
_next_handle = 1


def _handle() -> int:
    global _next_handle
    _next_handle += 1
    return _next_handle


def _i32(addr: int, n: int) -> np.ndarray:
    return np.ctypeslib.as_array(C.cast(addr, C.POINTER(C.c_int32)), shape=(n,)) if n else np.empty(0, np.int32)


class _Model:
    def __init__(self, model, device, world, rank, data_parallel):
        self.model, self.device, self.world, self.rank, self.data_parallel = model, device, world, rank, data_parallel


class _Context:
    def __init__(self, m: _Model, n_blocks: int, block_size: int, presample: int, n_ctx: int, rope: dict):
        self.m = m
        self._rope_changed = _rope_overrides(m.model, rope)
        hp = m.model.hp
        dtype = m.model.dtype
        self.block_size = block_size
        self.presample = presample
        if getattr(m.model, "split", False):
            from .runtime.engine import SplitCache
            self.cache = SplitCache(m.model.layer_dev, n_blocks * block_size, hp.kv_row, dtype, block_size)
        else:
            self.cache = torch.zeros(hp.n_layer, n_blocks * block_size, hp.kv_row, dtype=dtype, device=m.device)
        if n_ctx > m.model.max_positions or self._rope_changed:
            lo, hi = hp.yarn_corr_dims()
            m.model.max_positions = max(n_ctx, m.model.max_positions)
            n_ctx = m.model.max_positions
            m.model.rope_table = ops.ref.yarn_table(n_ctx, hp.qk_rope_head_dim, hp.rope_freq_base, hp.freq_scale, hp.ext_factor,
                                                    hp.rope_attn, lo, hi, device=m.device)


def _rope_overrides(model, rope: dict) -> bool:
    """llama_context_params.rope_freq_base / rope_freq_scale / yarn_attn_factor / yarn_orig_ctx / rope_scaling_type: values
    that differ from "keep the model's" replace the hyper-parameters (the attention scale follows: it depends on the
    frequency scale through the YaRN magnitude factor).  The model object is shared by the contexts made from it."""
    import dataclasses
    hp, ch = model.hp, {}
    if rope.get("freq_base", 0) > 0 and rope["freq_base"] != hp.rope_freq_base:
        ch["rope_freq_base"] = float(rope["freq_base"])
    st = int(rope.get("scaling_type", -1))
    if st == 0 and hp.rope_scaling_type != "none":
        ch["rope_scaling_type"] = "none"
    elif st == 2 and hp.rope_scaling_type != "yarn":
        ch["rope_scaling_type"] = "yarn"
    if rope.get("freq_scale", 0) > 0 and abs(1.0 / rope["freq_scale"] - hp.rope_scaling_factor) > 1e-9:
        ch["rope_scaling_factor"] = 1.0 / float(rope["freq_scale"])
    if rope.get("attn_factor", 0) > 0 and rope["attn_factor"] != 1.0 and rope["attn_factor"] != hp.rope_attn_factor:
        ch["rope_attn_factor"] = float(rope["attn_factor"])
    if rope.get("orig_ctx", 0) > 0 and rope["orig_ctx"] != hp.rope_orig_ctx:
        ch["rope_orig_ctx"] = int(rope["orig_ctx"])
    if not ch:
        return False
    model.hp = dataclasses.replace(hp, **ch)
    return True


def load_model(path: str, use_gpu: int, main_gpu: int, tp_id: int, num_parallel: int, expert_parallel: int,
               check_tensors: int, data_parallel: int, layer_split: str = "", kv_overrides: str = "{}") -> int:
    from .runtime.factory import build_model
    on_gpu = bool(use_gpu) and torch.cuda.is_available()
    if on_gpu:
        dev_index = int(os.environ.get("LOCAL_RANK", tp_id if num_parallel > 1 else main_gpu))
        device = torch.device("cuda", dev_index)
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")
    if num_parallel > 1 and not torch.distributed.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.distributed.init_process_group("nccl" if on_gpu else "gloo", rank=tp_id, world_size=num_parallel)
    layer_devices, tensor_split = None, None
    if layer_split and on_gpu and num_parallel == 1 and torch.cuda.device_count() > 1:
        n = torch.cuda.device_count()
        if layer_split != "even":
            tensor_split = [float(x) for x in layer_split.split(",")][:n]
            if sum(tensor_split) <= 0:
                tensor_split = None
        layer_devices = [torch.device("cuda", (main_gpu + i) % n) for i in range(n)]
    model = build_model(gguf_path=path, device=device, dtype=torch.bfloat16 if on_gpu else torch.float32, world=num_parallel,
                        rank=tp_id, expert_parallel=bool(expert_parallel), layer_devices=layer_devices, tensor_split=tensor_split,
                        kv_overrides=__import__("json").loads(kv_overrides or "{}"), check_tensors=bool(check_tensors))
    h = _handle()
    _models[h] = _Model(model, device, num_parallel, tp_id, bool(data_parallel))
    return h


def free_model(h: int) -> int:
    _models.pop(h, None)
    return 0


def create_context(mh: int, n_blocks: int, block_size: int, presample: int, n_ctx: int, rope: str = "{}") -> int:
    h = _handle()
    _contexts[h] = _Context(_models[mh], n_blocks, block_size, presample, n_ctx, __import__("json").loads(rope or "{}"))
    return h


def free_context(h: int) -> int:
    _contexts.pop(h, None)
    return 0


def copy_blocks(ch: int, addr: int, n: int) -> int:
    """Device copies of whole cache blocks: ``n`` (src, dst) pairs (copy-on-write and defragmentation)."""
    c = _contexts[ch]
    pairs = torch.from_numpy(_i32(addr, 2 * n).reshape(n, 2).copy())
    if not isinstance(c.cache, torch.Tensor):
        c.cache.copy_blocks(pairs[:, 0].numpy(), pairs[:, 1].numpy())
        return 0
    src = pairs[:, 0].contiguous().to(c.m.device)
    dst = pairs[:, 1].contiguous().to(c.m.device)
    ops.kv_block_copy(c.cache, src, dst, c.block_size)
    return 0


def forward(ch: int, addr: int, T: int, B: int, max_blocks: int, n_out: int, max_q: int, out_addr: int, idx_addr: int,
            sync_all: int) -> int:
    """One forward chunk.  The int32 buffer at ``addr`` is
    ``[tokens T | positions T | slot_mapping T | out_rows n_out | seq_lens B | q_start B+1 | block_tables B*max_blocks]``.
    Writes ``n_out`` rows to ``out_addr`` (fp32 logits, or the top-k values with ids to ``idx_addr`` as int64)."""
    c = _contexts[ch]
    dev = c.m.device
    n = 3 * T + n_out + B + B + 1 + B * max_blocks
    host = torch.from_numpy(_i32(addr, n).copy())
    d = host.to(dev, non_blocking=False)
    o = 0

    def take(k):
        nonlocal o
        v = d[o:o + k]
        o += k
        return v

    tokens, positions, slots, out_rows = take(T), take(T), take(T), take(n_out)
    seq_lens, q_start = take(B), take(B + 1)
    tables = take(B * max_blocks).view(B, max_blocks)
    batch = ForwardBatch(tokens, positions, slots, tables, seq_lens, q_start, out_rows, max_q_len=max_q)
    logits = c.m.model.forward(batch, c.cache)
    if n_out:
        if c.presample > 0:
            k = min(c.presample, logits.shape[1])
            if logits.is_cuda:
                with torch.cuda.device(logits.device):       # a layer-split model ends on its last GPU
                    vals, ids = ops.topk_logits(logits.contiguous(), k)
            else:
                vals, ids = ops.topk_logits(logits.contiguous(), k)
            v_host = np.ctypeslib.as_array(C.cast(out_addr, C.POINTER(C.c_float)), shape=(n_out, k))
            i_host = np.ctypeslib.as_array(C.cast(idx_addr, C.POINTER(C.c_int64)), shape=(n_out, k))
            torch.from_numpy(v_host).copy_(vals.float().cpu())
            torch.from_numpy(i_host).copy_(ids.long().cpu())
        else:
            V = logits.shape[1]
            v_host = np.ctypeslib.as_array(C.cast(out_addr, C.POINTER(C.c_float)), shape=(n_out, V))
            torch.from_numpy(v_host).copy_(logits.float().cpu())
    if dev.type == "cuda":
        ops.nat().check_status(dev)
    return _sync_token_count(c, T) if sync_all else T


def _sync_token_count(c: _Context, T: int) -> int:
    """Data-parallel bookkeeping: the number of tokens all ranks processed in this step."""
    if c.m.world <= 1 or not torch.distributed.is_initialized():
        return T
    t = torch.tensor([T], dtype=torch.int64, device=c.m.device if c.m.device.type == "cuda" else "cpu")
    torch.distributed.all_reduce(t)
    return int(t.item())


def empty_run(ch: int) -> int:
    """A rank without work joins the other ranks' step (their collectives need every rank)."""
    c = _contexts[ch]
    return _sync_token_count(c, 0)


def synchronize(ch: int) -> int:
    c = _contexts[ch]
    if c.m.device.type == "cuda":
        torch.cuda.synchronize(c.m.device)
    return 0
