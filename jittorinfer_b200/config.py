"""YAML server / model configuration with the reference's key set.

The reference reads one YAML file into ``common_params`` (common/common_local.h:206-343; the keys
and defaults are listed in 159-203) and its servers take only ``--config/-c``
(examples/server/server.cpp:1575-1595).  The same files load here unchanged.  Keys that configure
the Ascend back end (``enable_ge``, ``enable_cann_flash_attention``, ``n_threads`` ...) are accepted
and mapped onto what they mean for this engine or ignored with a note; new keys select the B200
specifics (``tp_size``, ``ep_size``, ``kv_block_size``, ``gpu_memory_utilization``,
``max_num_seqs``, ``cuda_graph_buckets``).  ``CUDA_VISIBLE_DEVICES`` plays the role of
``ASCEND_RT_VISIBLE_DEVICES``.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional, Tuple

import yaml

log = logging.getLogger("jittorinfer_b200.config")

SPLIT_MODES = ("LLAMA_SPLIT_MODE_NONE", "LLAMA_SPLIT_MODE_LAYER", "LLAMA_SPLIT_MODE_ROW")
REASONING_FORMATS = ("COMMON_REASONING_FORMAT_NONE", "COMMON_REASONING_FORMAT_DEEPSEEK")

# accepted for file compatibility; they tune the reference's CPU/NPU back ends and have no effect here
IGNORED_KEYS = {"n_threads", "n_threads_batch", "use_mlock", "offload_input", "n_gpu_layers",
                "enable_cann_flash_attention", "enable_fused_moe", "reranking", "no_perf"}


@dataclass
class ServerConfig:
    # ---- reference keys (common/common_local.h:211-336) ----
    main_gpu: int = 0
    split_mode: str = "LLAMA_SPLIT_MODE_LAYER"
    use_mmap: bool = True
    check_tensors: bool = False        # verify that every weight is finite while loading
    enable_mla: bool = True            # always true here: the latent cache is the only KV layout
    enable_ge: bool = True             # maps to cuda_graphs (persistent compiled decode graph)
    presample_count: int = 64          # device top-k width handed to the host sampler chain; -1 = full logits
    display_chat: bool = False
    n_predict: int = -1
    n_ctx: int = 16384
    n_batch: int = 2048
    n_keep: int = 0
    n_parallel: int = 8
    model: str = ""
    model_alias: str = ""
    special: bool = False
    cont_batching: bool = True
    port: int = 8080
    n_threads_http: int = -1
    hostname: str = "127.0.0.1"
    chat_template: str = ""
    defrag_thold: float = -1.0
    reasoning_format: str = "COMMON_REASONING_FORMAT_DEEPSEEK"
    # ---- additions for this engine ----
    tp_size: int = 1
    ep_size: int = 1
    kv_block_size: int = 64
    gpu_memory_utilization: float = 0.9
    kv_cache_auto: bool = False        # size the latent cache from the memory left after the weights (gpu_memory_utilization
                                       # of the device) instead of n_ctx
    max_seq_len: int = 0               # per-sequence token limit; 0 = n_ctx / slots as in the reference
    max_num_seqs: Optional[int] = None
    cuda_graph_buckets: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64)
    layer_split_gpus: int = 0          # split_mode LAYER: consecutive layer ranges on this many GPUs of one process;
                                       # 0 = as many as the weights need (1 when they fit on main_gpu)
    tensor_split: Tuple[float, ...] = ()   # relative share of layers per GPU (reference key; empty = even)
    attention_dp: bool = False         # ep_size ranks each serve their own requests (attention data-parallel), routed experts
                                       # sharded over them and reached through the all-to-all dispatcher
    ep_max_tokens: int = 256           # attention_dp: most tokens one rank schedules per step (sizes the dispatch buffers)
    mixed_prompt_budget: int = 0       # most prompt tokens per step while requests are generating (0 = n_batch)
    device_sampling: bool = False      # sample on the device when a request needs only top-k / top-p / min-p / temperature
    run_ahead: bool = False            # greedy requests: launch decode step k+1 before the ids of step k reach the host
    enforce_response_format: bool = True   # chat response_format (json_object / json_schema) constrains sampling with a grammar
    random_init: str = ""              # preset name ("lite", "v2", "tiny"): serve random weights instead of a GGUF file
    ignored: Dict[str, Any] = field(default_factory=dict)

    @property
    def world_size(self) -> int:
        return max(self.tp_size, self.ep_size)

    @property
    def cuda_graphs(self) -> bool:
        return bool(self.enable_ge)

    @property
    def slots(self) -> int:
        return self.max_num_seqs or self.n_parallel

    def validate(self) -> None:
        if self.split_mode not in SPLIT_MODES:
            raise ValueError(f"split_mode must be one of {SPLIT_MODES}")
        if self.reasoning_format not in REASONING_FORMATS:
            raise ValueError(f"reasoning_format must be one of {REASONING_FORMATS}")
        if self.tp_size not in (1, 2, 4, 8) or self.ep_size not in (1, 2, 4, 8):
            raise ValueError("tp_size / ep_size must be 1, 2, 4 or 8")       # reference: llama-model.cpp:467-476
        if self.ep_size > 1 and self.tp_size > 1 and self.ep_size != self.tp_size:
            raise ValueError("expert parallelism shares the tensor-parallel group: ep_size must equal tp_size")
        if self.attention_dp and (self.ep_size < 2 or self.tp_size > 1):
            raise ValueError("attention_dp needs ep_size >= 2 and tp_size == 1 (attention is replicated, not sharded)")
        if self.kv_block_size != 64:
            raise ValueError("kv_block_size must be 64 (the attention kernels are built for 64-token blocks)")
        if not (0.05 <= self.gpu_memory_utilization <= 0.98):
            raise ValueError("gpu_memory_utilization must be in [0.05, 0.98]")
        if self.n_parallel < 1 or self.n_batch < 1 or self.n_ctx < self.kv_block_size:
            raise ValueError("n_parallel, n_batch must be >= 1 and n_ctx >= kv_block_size")


def load_yaml(path: Optional[str]) -> ServerConfig:
    """Missing file -> defaults, as the reference does (common/common_local.h:206-210)."""
    cfg = ServerConfig()
    if not path:
        return cfg
    try:
        with open(path) as f:
            data = yaml.safe_load(f) or {}
    except FileNotFoundError:
        log.warning("config %s not found: using defaults", path)
        return cfg
    known = {f.name for f in fields(ServerConfig)} - {"ignored"}
    for k, v in data.items():
        if k in known:
            if k == "cuda_graph_buckets":
                v = tuple(int(x) for x in v)
            if k == "tensor_split":
                v = tuple(float(x) for x in (v or ()))
            if k == "n_parallel":
                v = int(v)          # the reference clamps to 32 (cell bitset); block tables have no such limit
            setattr(cfg, k, v)
        elif k in IGNORED_KEYS:
            cfg.ignored[k] = v
        else:
            log.warning("unknown config key %r ignored", k)
            cfg.ignored[k] = v
    if cfg.split_mode == "LLAMA_SPLIT_MODE_ROW" and cfg.tp_size == 1 and "tp_size" not in data:
        log.info("split_mode ROW without tp_size: set tp_size/ep_size to shard the model over GPUs")
    if cfg.n_batch < 64:
        # the reference's graph-engine configuration sets n_batch to its padded decode width (e.g. 16); here n_batch is
        # the token budget of a step, i.e. the prompt chunk size
        log.warning("n_batch %d: prompts will be processed %d tokens per step; 512-2048 is the useful range here", cfg.n_batch, cfg.n_batch)
    cfg.validate()
    return cfg
