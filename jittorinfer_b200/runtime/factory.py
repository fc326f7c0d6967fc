"""Engine construction: model source (GGUF file or random init) + parallel layout -> LLMEngine.

Counterpart of ``common_init_from_params`` (common/common_local.cpp:121-209: model load, then
context creation) for this runtime.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..models.deepseek2 import DeepSeek2Model
from ..models.hparams import DeepSeek2HParams
from ..models.weights import ShardSpec, iter_gguf, iter_random
from .engine import EngineConfig, LLMEngine


def build_model(hp: Optional[DeepSeek2HParams] = None, gguf_path: Optional[str] = None, device="cuda",
                dtype: torch.dtype = torch.bfloat16, world: int = 1, rank: int = 0, expert_parallel: bool = True,
                comm=None, seed: int = 0, std: float = 0.02, max_positions: int = 8192, fast_random: bool = True,
                dp_attention: bool = False, ep_max_tokens: int = 256, layer_devices=None,
                tensor_split=None, kv_overrides=None, check_tensors: bool = False) -> DeepSeek2Model:
    """``dp_attention``: attention data-parallel (every rank serves its own requests), routed experts sharded over the
    ranks and reached through the all-to-all dispatcher; ``ep_max_tokens`` bounds the tokens of one rank per step."""
    dp_attention = dp_attention and world > 1
    spec = ShardSpec(rank, world, (expert_parallel or dp_attention) and world > 1, dp_attention)
    if gguf_path is not None:
        import os
        if os.environ.get("JITTORINFER_GGUF", "").lower() == "native":
            from ..gguf.native_reader import NativeGGUFReader as GGUFReader      # C++ parser + mapping
        else:
            from ..gguf.io import GGUFReader
        reader = GGUFReader(gguf_path)
        if dtype == torch.bfloat16 and torch.device(device).type == "cuda":
            reader.quant_out_dtype = torch.bfloat16      # block-quantised tensors are expanded straight to the stored dtype
            if os.environ.get("JITTORINFER_DEVICE_DEQUANT", "1") != "0" and layer_devices is None:
                reader.quant_device = torch.device(device)   # ... on the device: the quantised bytes cross PCIe, not the bf16
        if kv_overrides:                 # metadata overrides (llama_model_params.kv_overrides)
            reader.kv.update(kv_overrides)
        hp = DeepSeek2HParams.from_gguf_kv(reader.kv, reader.tensors)
        weights = iter_gguf(reader, hp, spec)
        if check_tensors:                # llama_model_params.check_tensors / the YAML key of the same name
            from ..models.weights import checked
            weights = checked(weights)
    else:
        assert hp is not None
        dev = torch.device(device)
        weights = iter_random(hp, spec=spec, seed=seed, std=std, dtype=dtype if dev.type == "cuda" else torch.float32,
                              device=dev, fast=fast_random and dev.type == "cuda")
    ep = None
    if dp_attention:
        from ..parallel.ep import make_ep_dispatcher
        ep = make_ep_dispatcher(torch.device(device), world, rank, hp.n_expert, hp.n_embd, hp.n_expert_used,
                                hp.n_layer - hp.n_layer_dense_lead, max_tokens=ep_max_tokens)
    elif world > 1 and comm is None:
        from ..parallel.comm import make_communicator
        comm = make_communicator(torch.device(device), world, rank, hp.n_embd, hp.n_layer)
    if layer_devices is not None and len(layer_devices) != hp.n_layer:
        from ..models.deepseek2 import assign_layers
        layer_devices = assign_layers(hp.n_layer, layer_devices, tensor_split)   # a device list: contiguous layer ranges
    return DeepSeek2Model(hp, weights, dtype=dtype, device=device, spec=spec, comm=comm, max_positions=max_positions, ep=ep,
                          layer_devices=layer_devices)


def kv_tokens_for_budget(total_bytes: int, free_bytes: int, utilization: float, n_layer: int, kv_row: int, elem_bytes: int,
                         block_size: int = 64, reserve_bytes: int = 2 << 30) -> int:
    """Tokens of latent cache that fit when the process may occupy ``utilization`` of the device.

    ``free_bytes`` is what the device reports after the weights are resident; ``reserve_bytes`` is held back for
    activations, workspaces and captured graphs.  One cached token costs ``n_layer * kv_row * elem_bytes`` (DeepSeek-V2:
    60 x 576 x 2 = 69 KB).  The result is a whole number of blocks, 0 if nothing fits."""
    used = total_bytes - free_bytes
    budget = int(total_bytes * utilization) - used - reserve_bytes
    per_token = n_layer * kv_row * elem_bytes
    if budget <= 0 or per_token <= 0:
        return 0
    return budget // per_token // block_size * block_size


def build_engine(hp: Optional[DeepSeek2HParams] = None, gguf_path: Optional[str] = None, device="cuda",
                 dtype: torch.dtype = torch.bfloat16, world: int = 1, rank: int = 0, n_parallel: int = 8,
                 n_ctx_slot: int = 2048, n_batch: int = 2048, seed: int = 0, graph_buckets: Sequence[int] = (1, 2, 4, 8),
                 cuda_graphs: bool = True, expert_parallel: bool = True, comm=None, n_ctx: Optional[int] = None,
                 dp_attention: bool = False, ep_max_tokens: int = 256, layer_devices=None, tensor_split=None,
                 gpu_memory_utilization: Optional[float] = None, check_tensors: bool = False, **engine_kw) -> LLMEngine:
    """``gpu_memory_utilization`` (with ``n_ctx`` None or 0): size the latent cache from the memory left after the weights
    are loaded, so that the process fills that share of the GPU."""
    if dp_attention and world > 1:
        n_batch = min(n_batch, ep_max_tokens)          # a step's tokens must fit the dispatcher's buffers
    model = build_model(hp, gguf_path, device, dtype, world, rank, expert_parallel, comm, seed,
                        max_positions=max(n_ctx_slot, 64), dp_attention=dp_attention, ep_max_tokens=ep_max_tokens,
                        layer_devices=layer_devices, tensor_split=tensor_split, check_tensors=check_tensors)
    dev = torch.device(device)
    if not n_ctx and gpu_memory_utilization and dev.type == "cuda":
        free, total = torch.cuda.mem_get_info(dev)
        elem = torch.empty(0, dtype=dtype).element_size()
        fit = kv_tokens_for_budget(total, free, gpu_memory_utilization, model.hp.n_layer, model.hp.kv_row, elem)
        if fit < n_ctx_slot:
            raise RuntimeError(f"only {fit} cache tokens fit at gpu_memory_utilization={gpu_memory_utilization}; "
                               f"one sequence needs {n_ctx_slot}")
        n_ctx = fit
    cfg = EngineConfig(n_ctx=n_ctx or n_ctx_slot * n_parallel, n_batch=n_batch, n_parallel=n_parallel, n_ctx_slot=n_ctx_slot,
                       graph_buckets=tuple(graph_buckets), cuda_graphs=cuda_graphs, **engine_kw)
    return LLMEngine(model, cfg)
