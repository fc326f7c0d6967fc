"""Tensor table, sharding plan, random initialisation and GGUF load for DeepSeek-V2 weights.

Tensor names and shapes are the GGUF ones the reference creates in ``llama_model::load_tensors``
(src/llama-model.cpp:744-867; name table src/llama-arch.cpp:903-927).  The per-tensor shard rule
mirrors the reference's ``llm_split_method`` choices (src/llama-model.cpp:309-322, 761-866):

* by head: ``attn_q`` / ``attn_q_b`` / ``attn_kv_b`` (output rows), ``attn_output`` (input columns)
* dense FFN and shared experts: gate/up by output rows, down by input columns
* routed experts: on the expert axis under expert parallelism, else on the ``n_ff_exp`` axis
* replicated: norms, ``attn_q_a``, ``attn_kv_a_mqa``, router, token embedding, ``output``

A rank only ever materialises its own shard: the GGUF path slices the mmap view, the random path
generates each tensor from a (seed, tensor-name, outer-index) stream so that every rank's shard is
bit-identical to the corresponding slice of the single-GPU tensor.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Tuple

import torch

from .hparams import DeepSeek2HParams


@dataclass(frozen=True)
class ShardSpec:
    tp_rank: int = 0
    tp_size: int = 1
    expert_parallel: bool = False     # routed experts split on the expert axis over the tp group
    dp_attention: bool = False        # attention / dense / shared experts replicated (every rank has its own tokens);
                                      # only the routed experts are sharded, on the expert axis

    @property
    def sharded(self) -> bool:
        return self.tp_size > 1


def tensor_table(hp: DeepSeek2HParams) -> Dict[str, Tuple[int, ...]]:
    """name -> full (unsharded) torch-order shape."""
    d, H = hp.n_embd, hp.n_head
    t: Dict[str, Tuple[int, ...]] = {"token_embd.weight": (hp.n_vocab, d)}
    for il in range(hp.n_layer):
        p = f"blk.{il}."
        t[p + "attn_norm.weight"] = (d,)
        if hp.is_lite:
            t[p + "attn_q.weight"] = (H * hp.qk_head_dim, d)
        else:
            t[p + "attn_q_a.weight"] = (hp.q_lora_rank, d)
            t[p + "attn_q_a_norm.weight"] = (hp.q_lora_rank,)
            t[p + "attn_q_b.weight"] = (H * hp.qk_head_dim, hp.q_lora_rank)
        t[p + "attn_kv_a_mqa.weight"] = (hp.kv_row, d)
        t[p + "attn_kv_a_norm.weight"] = (hp.kv_lora_rank,)
        t[p + "attn_kv_b.weight"] = (H * (hp.qk_nope_head_dim + hp.v_head_dim), hp.kv_lora_rank)
        t[p + "attn_output.weight"] = (d, H * hp.v_head_dim)
        t[p + "ffn_norm.weight"] = (d,)
        if il < hp.n_layer_dense_lead:
            t[p + "ffn_gate.weight"] = (hp.n_ff, d)
            t[p + "ffn_up.weight"] = (hp.n_ff, d)
            t[p + "ffn_down.weight"] = (d, hp.n_ff)
        else:
            t[p + "ffn_gate_inp.weight"] = (hp.n_expert, d)
            if hp.router_bias:
                t[p + "exp_probs_b.bias"] = (hp.n_expert,)
            t[p + "ffn_gate_exps.weight"] = (hp.n_expert, hp.n_ff_exp, d)
            t[p + "ffn_up_exps.weight"] = (hp.n_expert, hp.n_ff_exp, d)
            t[p + "ffn_down_exps.weight"] = (hp.n_expert, d, hp.n_ff_exp)
            if hp.n_expert_shared:
                fs = hp.n_ff_exp * hp.n_expert_shared
                t[p + "ffn_gate_shexp.weight"] = (fs, d)
                t[p + "ffn_up_shexp.weight"] = (fs, d)
                t[p + "ffn_down_shexp.weight"] = (d, fs)
    t["output_norm.weight"] = (d,)
    t["output.weight"] = (hp.n_vocab, d)
    return t


def shard_dim(name: str, spec: ShardSpec) -> Optional[int]:
    """Torch dim along which ``name`` is split across the TP group (None = replicated)."""
    if not spec.sharded:
        return None
    base = name.split(".")[-2] if name.startswith("blk.") else name
    if spec.dp_attention:
        return 0 if base in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps") else None
    if base in ("attn_q", "attn_q_b", "attn_kv_b", "ffn_gate", "ffn_up", "ffn_gate_shexp", "ffn_up_shexp"):
        return 0
    if base in ("attn_output", "ffn_down", "ffn_down_shexp"):
        return 1
    if base in ("ffn_gate_exps", "ffn_up_exps"):
        return 0 if spec.expert_parallel else 1
    if base == "ffn_down_exps":
        return 0 if spec.expert_parallel else 2
    return None


def local_shape(name: str, shape: Tuple[int, ...], spec: ShardSpec) -> Tuple[int, ...]:
    dim = shard_dim(name, spec)
    if dim is None:
        return shape
    if shape[dim] % spec.tp_size:
        raise ValueError(f"{name}: dim {dim} ({shape[dim]}) is not divisible by tp_size {spec.tp_size}")
    s = list(shape)
    s[dim] //= spec.tp_size
    return tuple(s)


def _stream_seed(seed: int, name: str, outer: int) -> int:
    h = hashlib.blake2b(f"{seed}:{name}:{outer}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, shape: Tuple[int, ...], spec: ShardSpec, seed: int, std: float,
                  dtype: torch.dtype, device) -> torch.Tensor:
    """Shard of a N(0, std) tensor (norm gammas: 1 + N(0, std)); identical across shardings.

    Values are drawn on the CPU generator one outer slice at a time (3-D expert tensors: per expert;
    2-D: whole matrix) so that device and world size never change the numbers.
    """
    dim = shard_dim(name, spec)
    is_norm = name.endswith("_norm.weight")
    gen = torch.Generator(device="cpu")

    def draw(outer: int, shp) -> torch.Tensor:
        gen.manual_seed(_stream_seed(seed, name, outer))
        x = torch.randn(shp, generator=gen, dtype=torch.float32) * std
        return x + 1.0 if is_norm else x

    if len(shape) == 3:
        E = shape[0]
        if dim == 0:
            step = E // spec.tp_size
            experts = range(spec.tp_rank * step, (spec.tp_rank + 1) * step)
        else:
            experts = range(E)
        parts = []
        for e in experts:
            x = draw(e, shape[1:])
            if dim in (1, 2):
                n = shape[dim] // spec.tp_size
                x = x.narrow(dim - 1, spec.tp_rank * n, n)
            parts.append(x.to(dtype).to(device))
        return torch.stack(parts, 0)
    x = draw(0, shape)
    if dim is not None:
        n = shape[dim] // spec.tp_size
        x = x.narrow(dim, spec.tp_rank * n, n)
    return x.to(dtype).contiguous().to(device)


def fast_random_tensor(name: str, shape: Tuple[int, ...], spec: ShardSpec, seed: int, std: float,
                       dtype: torch.dtype, device) -> torch.Tensor:
    """Device-side generation for benchmark-sized models (values depend on the sharding)."""
    shp = local_shape(name, shape, spec)
    gen = torch.Generator(device=device)
    gen.manual_seed(_stream_seed(seed, name, spec.tp_rank if shard_dim(name, spec) is not None else 0))
    x = torch.empty(shp, dtype=dtype, device=device)
    x.normal_(0.0, std, generator=gen)
    if name.endswith("_norm.weight"):
        x += 1.0
    return x


def iter_random(hp: DeepSeek2HParams, spec: ShardSpec = ShardSpec(), seed: int = 0, std: float = 0.02,
                dtype: torch.dtype = torch.float32, device="cpu", fast: bool = False
                ) -> Iterator[Tuple[str, torch.Tensor]]:
    fn = fast_random_tensor if fast else random_tensor
    for name, shape in tensor_table(hp).items():
        yield name, fn(name, shape, spec, seed, std, dtype, device)


def random_weights(hp: DeepSeek2HParams, **kw) -> Dict[str, torch.Tensor]:
    return dict(iter_random(hp, **kw))


def write_random_gguf(path: str, hp: DeepSeek2HParams, seed: int = 0, std: float = 0.02,
                      dtype: torch.dtype = torch.float32, vocab: bool = True, quant: Optional[int] = None) -> None:
    """Emit a random-init GGUF with the reference's key/tensor layout (and a byte-level toy vocab).

    ``quant``: a block-quantised ggml type for the matrices.  As offline quantisers do, a matrix whose rows do not hold
    whole blocks of that type falls back to Q8_0 (or stays in ``dtype``), and norms and router weights stay f32."""
    from ..gguf import format as F
    from ..gguf.io import GGUFWriter

    def pick(name: str, t: torch.Tensor):
        if quant is None or "ffn_gate_inp" in name:
            return None
        for cand in (quant, F.GGML_Q8_0):
            if t.shape[-1] % F.TYPE_TRAITS[cand][0] == 0:
                return cand
        return None
    w = GGUFWriter(path)
    w.add_dict(hp.to_gguf_kv())
    if vocab:
        from ..utils.toy_vocab import toy_vocab_kv
        w.add_dict(toy_vocab_kv(hp.n_vocab, hp.bos_id, hp.eos_id))
    for name, t in iter_random(hp, seed=seed, std=std, dtype=torch.float32):
        if t.dim() == 1:
            w.add_tensor(name, t)                      # norms stay f32, as in real checkpoints
        elif pick(name, t) is not None:
            w.add_tensor(name, t, pick(name, t))
        else:
            w.add_tensor(name, t.to(dtype))
    w.write()


def iter_gguf(reader, hp: DeepSeek2HParams, spec: ShardSpec = ShardSpec()) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, CPU shard view) for every tensor of the model; checks names and shapes."""
    table = tensor_table(hp)
    seen = 0
    for name, shape in table.items():
        if name not in reader.tensors:
            if name == "output.weight" and "token_embd.weight" in reader.tensors:
                yield name, reader.tensor("token_embd.weight")      # tied embeddings
                continue
            raise KeyError(f"GGUF is missing tensor {name}")
        ti = reader.tensors[name]
        if tuple(ti.shape) != tuple(shape):
            raise ValueError(f"{name}: GGUF shape {ti.shape} != expected {shape}")
        dim = shard_dim(name, spec)
        seen += 1
        if dim is None:
            yield name, reader.tensor(name)
        else:
            yield name, reader.tensor_slice(name, dim, spec.tp_rank, spec.tp_size)
    extra = [n for n in reader.tensors if n not in table and not n.endswith("exp_probs_b.bias")]
    if extra:
        raise ValueError(f"GGUF has {len(extra)} tensors the model does not use, e.g. {extra[:3]}")


def checked(weights: Iterator[Tuple[str, torch.Tensor]]) -> Iterator[Tuple[str, torch.Tensor]]:
    """Passes the tensors on after verifying that every floating-point value is finite -- what the reference's
    ``check_tensors`` asks of its loader (src/llama-model-loader.cpp:924-1167 validates each tensor's data while reading).
    A truncated download or a bad conversion shows as NaN / Inf long before it shows in the output text."""
    for name, t in weights:
        if t.is_floating_point():
            bad = int((~torch.isfinite(t)).sum())
            if bad:
                raise ValueError(f"tensor {name}: {bad} of {t.numel()} values are NaN or infinite")
        yield name, t


class StagedUploader:
    """Host -> device copies of large checkpoint tensors through a ring of pinned staging buffers.

    A tensor that is a view of the GGUF mapping is pageable memory: a plain ``.to(device)`` makes the driver stage it
    synchronously in small pieces.  Here the file pages are copied into one of ``n_buffers`` pinned buffers (this is what
    actually reads the file) while the previous buffer's asynchronous copy to the device is still in flight, so disk /
    page-cache reads overlap the PCIe transfer.  The reference does the same with four 1 MiB buffers
    (``load_all_data``, src/llama-model-loader.cpp:924-1167); at 50+ GB/s of PCIe a chunk of tens of MiB is needed to
    amortise the per-copy cost.  Dtype conversion happens on the device after the raw bytes have arrived.
    """

    def __init__(self, device, chunk_bytes: int = 64 << 20, n_buffers: int = 3, min_bytes: int = 256 << 20):
        self.device = torch.device(device)
        self.chunk_bytes, self.min_bytes = int(chunk_bytes), int(min_bytes)
        cuda = self.device.type == "cuda"
        self.bufs = [torch.empty(self.chunk_bytes, dtype=torch.uint8, pin_memory=cuda) for _ in range(n_buffers)]
        self.events = [torch.cuda.Event() if cuda else None for _ in range(n_buffers)]
        self.n_chunks = 0

    def upload(self, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``t``: a CPU tensor.  Returns it on the device (converted to ``dtype`` there when given)."""
        if t.device.type != "cpu" or t.numel() * t.element_size() < self.min_bytes:
            return t.to(device=self.device, dtype=dtype or t.dtype).contiguous()
        if self.device.type == "cuda" and self.device.index is not None and torch.cuda.current_device() != self.device.index:
            with torch.cuda.device(self.device):             # events and copies must share the target device's stream
                return self.upload(t, dtype)
        src = t.contiguous().view(-1).view(torch.uint8)
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        dst = out.view(-1).view(torch.uint8)
        n, k = src.numel(), 0
        for off in range(0, n, self.chunk_bytes):
            m = min(self.chunk_bytes, n - off)
            i = k % len(self.bufs)
            if self.events[i] is not None and k >= len(self.bufs):
                self.events[i].synchronize()                 # the device copy that last used this buffer has finished
            self.bufs[i][:m].copy_(src[off:off + m])         # file pages -> pinned memory
            dst[off:off + m].copy_(self.bufs[i][:m], non_blocking=True)
            if self.events[i] is not None:
                self.events[i].record()
            k += 1
        self.n_chunks += k
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return out.to(dtype) if dtype is not None and dtype != out.dtype else out
