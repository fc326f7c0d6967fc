"""DeepSeek-V2 family hyper-parameters.

The reference keeps these in ``llama_hparams`` (src/llama-hparams.h:27-153) filled from
GGUF keys in ``llama_model::load_hparams`` (src/llama-model.cpp:1047-1250).  Here they are
one dataclass that can be built from GGUF metadata, from a named preset, or by hand, and
that can be written back as GGUF metadata (the reference never writes GGUF).

Unlike the reference, "Lite" (no q-LoRA) is keyed on ``q_lora_rank == 0`` / tensor
presence, not on ``n_layer == 27`` (src/llama-model.cpp:1184).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict, replace
from typing import Any, Dict

ARCH = "deepseek2"


@dataclass
class DeepSeek2HParams:
    n_vocab: int = 102400
    n_embd: int = 2048
    n_layer: int = 27
    n_head: int = 16
    n_layer_dense_lead: int = 1
    n_ff: int = 10944                 # dense FFN inner size
    n_ff_exp: int = 1408              # per routed expert inner size
    n_expert: int = 64
    n_expert_used: int = 6
    n_expert_shared: int = 2
    expert_weights_scale: float = 1.0
    expert_weights_norm: bool = False
    expert_gating_func: str = "softmax"   # or "sigmoid"
    group_score_top2: bool = False        # group-limited routing scores a group by its two best experts (V3) instead of its best (V2)
    router_bias: bool = False             # per-expert selection bias (blk.N.exp_probs_b.bias; DeepSeek-V3-shaped checkpoints)
    n_group: int = 1                  # group-limited routing (DeepSeek-V2: 8)
    topk_group: int = 1               # groups kept per token (DeepSeek-V2: 3)
    q_lora_rank: int = 0              # 0 => dense q projection ("Lite")
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    rms_eps: float = 1e-6
    rope_freq_base: float = 10000.0
    rope_scaling_type: str = "yarn"   # "none" | "yarn"
    rope_scaling_factor: float = 40.0
    rope_orig_ctx: int = 4096
    rope_yarn_log_mul: float = 0.0707
    rope_attn_factor: float = 1.0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    n_ctx_train: int = 163840
    bos_id: int = 100000
    eos_id: int = 100001

    # ---- derived -------------------------------------------------------------------
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def kv_row(self) -> int:
        """Width of one cached latent row: compressed kv + rotated shared key."""
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def is_lite(self) -> bool:
        return self.q_lora_rank == 0

    @property
    def freq_scale(self) -> float:
        return 1.0 / self.rope_scaling_factor if self.rope_scaling_type == "yarn" else 1.0

    @property
    def ext_factor(self) -> float:
        return 1.0 if self.rope_scaling_type == "yarn" else 0.0

    @property
    def mscale(self) -> float:
        # src/llama-graph-deepseek2.cpp:123-125
        return self.rope_attn_factor * (1.0 + self.rope_yarn_log_mul * math.log(1.0 / self.freq_scale))

    @property
    def kq_scale(self) -> float:
        return self.mscale * self.mscale / math.sqrt(self.qk_head_dim)

    @property
    def rope_attn(self) -> float:
        """Magnitude factor handed to RoPE so that YaRN's own (1+0.1 ln(1/s)) cancels."""
        return 1.0 / (1.0 + 0.1 * math.log(1.0 / self.freq_scale))

    def yarn_corr_dims(self):
        dr = self.qk_rope_head_dim

        def corr(b):
            return dr * math.log(self.rope_orig_ctx / (b * 2.0 * math.pi)) / (2.0 * math.log(self.rope_freq_base))

        lo = max(0.0, math.floor(corr(self.yarn_beta_fast)))
        hi = min(dr - 1.0, math.ceil(corr(self.yarn_beta_slow)))
        return lo, hi

    def n_params(self) -> int:
        d, H = self.n_embd, self.n_head
        attn = d * self.kv_row + self.kv_lora_rank * H * (self.qk_nope_head_dim + self.v_head_dim) + H * self.v_head_dim * d
        if self.is_lite:
            attn += d * H * self.qk_head_dim
        else:
            attn += d * self.q_lora_rank + self.q_lora_rank * H * self.qk_head_dim
        dense = 3 * d * self.n_ff
        moe = 3 * d * self.n_ff_exp * (self.n_expert + self.n_expert_shared) + d * self.n_expert
        nl_moe = self.n_layer - self.n_layer_dense_lead
        return 2 * self.n_vocab * d + self.n_layer * attn + self.n_layer_dense_lead * dense + nl_moe * moe

    def replace(self, **kw) -> "DeepSeek2HParams":
        return replace(self, **kw)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    # ---- GGUF metadata -----------------------------------------------------------
    def to_gguf_kv(self) -> Dict[str, Any]:
        a = ARCH
        kv = {
            "general.architecture": a,
            "general.name": "deepseek2-random-init",
            f"{a}.context_length": ("u32", self.n_ctx_train),
            f"{a}.embedding_length": ("u32", self.n_embd),
            f"{a}.block_count": ("u32", self.n_layer),
            f"{a}.feed_forward_length": ("u32", self.n_ff),
            f"{a}.attention.head_count": ("u32", self.n_head),
            f"{a}.attention.head_count_kv": ("u32", self.n_head),
            f"{a}.attention.key_length": ("u32", self.qk_head_dim),
            f"{a}.attention.value_length": ("u32", self.v_head_dim),
            f"{a}.attention.layer_norm_rms_epsilon": ("f32", self.rms_eps),
            f"{a}.attention.kv_lora_rank": ("u32", self.kv_lora_rank),
            f"{a}.rope.dimension_count": ("u32", self.qk_rope_head_dim),
            f"{a}.rope.freq_base": ("f32", self.rope_freq_base),
            f"{a}.leading_dense_block_count": ("u32", self.n_layer_dense_lead),
            f"{a}.expert_count": ("u32", self.n_expert),
            f"{a}.expert_used_count": ("u32", self.n_expert_used),
            f"{a}.expert_shared_count": ("u32", self.n_expert_shared),
            f"{a}.expert_feed_forward_length": ("u32", self.n_ff_exp),
            f"{a}.expert_weights_scale": ("f32", self.expert_weights_scale),
            f"{a}.expert_weights_norm": ("bool", self.expert_weights_norm),
            f"{a}.expert_gating_func": ("u32", 1 if self.expert_gating_func == "softmax" else 2),
            f"{a}.expert_group_count": ("u32", self.n_group),
            f"{a}.expert_group_used_count": ("u32", self.topk_group),
            f"{a}.vocab_size": ("u32", self.n_vocab),
            "tokenizer.ggml.bos_token_id": ("u32", self.bos_id),
            "tokenizer.ggml.eos_token_id": ("u32", self.eos_id),
        }
        if self.q_lora_rank:
            kv[f"{a}.attention.q_lora_rank"] = ("u32", self.q_lora_rank)
        if self.rope_scaling_type == "yarn":
            kv[f"{a}.rope.scaling.type"] = "yarn"
            kv[f"{a}.rope.scaling.factor"] = ("f32", self.rope_scaling_factor)
            kv[f"{a}.rope.scaling.original_context_length"] = ("u32", self.rope_orig_ctx)
            kv[f"{a}.rope.scaling.yarn_log_multiplier"] = ("f32", self.rope_yarn_log_mul)
        return kv

    @classmethod
    def from_gguf_kv(cls, kv: Dict[str, Any], tensor_names=None) -> "DeepSeek2HParams":
        a = kv.get("general.architecture", ARCH)
        if a != ARCH:
            raise ValueError(f"unsupported architecture {a!r}: only {ARCH!r} is served")

        def g(key, default=None):
            return kv.get(f"{a}.{key}", default)

        hp = cls()
        hp.n_ctx_train = int(g("context_length", hp.n_ctx_train))
        hp.n_embd = int(g("embedding_length"))
        hp.n_layer = int(g("block_count"))
        hp.n_ff = int(g("feed_forward_length", 0))
        hp.n_head = int(g("attention.head_count"))
        key_len = int(g("attention.key_length"))
        hp.v_head_dim = int(g("attention.value_length"))
        hp.qk_rope_head_dim = int(g("rope.dimension_count"))
        hp.qk_nope_head_dim = key_len - hp.qk_rope_head_dim
        hp.rms_eps = float(g("attention.layer_norm_rms_epsilon", 1e-6))
        hp.kv_lora_rank = int(g("attention.kv_lora_rank"))
        hp.q_lora_rank = int(g("attention.q_lora_rank", 0))
        if tensor_names is not None and "blk.0.attn_q.weight" in tensor_names:
            hp.q_lora_rank = 0
        hp.rope_freq_base = float(g("rope.freq_base", 10000.0))
        hp.n_layer_dense_lead = int(g("leading_dense_block_count", 0))
        hp.n_expert = int(g("expert_count", 0))
        hp.n_expert_used = int(g("expert_used_count", 0))
        hp.n_expert_shared = int(g("expert_shared_count", 0))
        hp.n_ff_exp = int(g("expert_feed_forward_length", 0))
        hp.expert_weights_scale = float(g("expert_weights_scale", 1.0))
        hp.expert_weights_norm = bool(g("expert_weights_norm", False))
        gf = int(g("expert_gating_func", 1))
        hp.expert_gating_func = "sigmoid" if gf == 2 else "softmax"
        hp.group_score_top2 = gf == 2          # DeepSeek-V3 routing: sigmoid scores, groups ranked by their two best experts
        hp.n_group = int(g("expert_group_count", 1))
        hp.topk_group = int(g("expert_group_used_count", 1))
        st = g("rope.scaling.type", "none")
        hp.rope_scaling_type = "yarn" if st == "yarn" else "none"
        hp.rope_scaling_factor = float(g("rope.scaling.factor", 1.0))
        hp.rope_orig_ctx = int(g("rope.scaling.original_context_length", hp.n_ctx_train))
        hp.rope_yarn_log_mul = float(g("rope.scaling.yarn_log_multiplier", 0.0))
        hp.rope_attn_factor = float(g("rope.scaling.attn_factor", 1.0))
        hp.yarn_beta_fast = float(g("rope.scaling.yarn_beta_fast", hp.yarn_beta_fast))
        hp.yarn_beta_slow = float(g("rope.scaling.yarn_beta_slow", hp.yarn_beta_slow))
        nv = g("vocab_size")
        if nv is None:
            toks = kv.get("tokenizer.ggml.tokens")
            nv = len(toks) if toks is not None else hp.n_vocab
        hp.n_vocab = int(nv)
        hp.bos_id = int(kv.get("tokenizer.ggml.bos_token_id", 11))
        hp.eos_id = int(kv.get("tokenizer.ggml.eos_token_id", 11))
        if tensor_names is not None:
            hp.router_bias = any(str(n).endswith("exp_probs_b.bias") for n in tensor_names)
        return hp


def preset(name: str) -> DeepSeek2HParams:
    """Named shapes used by the tests and benchmarks."""
    name = name.lower().replace("_", "-")
    if name in ("tiny", "tiny-deepseek2"):
        # 2 layers (dense, then MoE), plain top-2 softmax gating, no q-LoRA.
        return DeepSeek2HParams(
            n_vocab=1024, n_embd=256, n_layer=2, n_head=4, n_layer_dense_lead=1, n_ff=512, n_ff_exp=128,
            n_expert=8, n_expert_used=2, n_expert_shared=1, q_lora_rank=0, kv_lora_rank=64,
            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_ctx_train=4096,
            rope_scaling_type="yarn", rope_scaling_factor=40.0, rope_orig_ctx=4096, bos_id=0, eos_id=1)
    if name in ("tiny-v2", "tiny-qlora"):
        # like tiny but with the q-LoRA branch and group-limited routing, to cover the V2 code paths
        return DeepSeek2HParams(
            n_vocab=1024, n_embd=256, n_layer=3, n_head=4, n_layer_dense_lead=1, n_ff=512, n_ff_exp=128,
            n_expert=16, n_expert_used=4, n_expert_shared=2, q_lora_rank=96, kv_lora_rank=64,
            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_ctx_train=4096,
            n_group=4, topk_group=2, expert_weights_scale=4.0, bos_id=0, eos_id=1)
    if name in ("lite", "deepseek-v2-lite", "v2-lite"):
        return DeepSeek2HParams()
    if name in ("lite-2l",):
        # DeepSeek-V2-Lite's layer shapes (hidden 2048, 16 heads, latent 512 + 64, 64 experts top-6 + 2 shared) with three
        # layers (one dense, two MoE) and a small vocabulary: what the GPU tests run the benchmarked kernels on
        return DeepSeek2HParams(n_layer=3, n_vocab=4096)
    if name in ("v2-2l",):
        # DeepSeek-V2's shapes where they select kernels (hidden 5120, q-LoRA 1536, latent 512 + 64, 160 experts in 8 groups
        # of which 3 are eligible, top-6, weight scale 16), cut down where only size follows (32 heads, expert width 512,
        # two layers, small vocabulary) so that a test can hold it next to an fp32 oracle
        return DeepSeek2HParams(
            n_vocab=4096, n_embd=5120, n_layer=2, n_head=32, n_ff=4096, n_ff_exp=512, n_expert=160, n_expert_used=6,
            n_expert_shared=2, expert_weights_scale=16.0, n_group=8, topk_group=3, q_lora_rank=1536)
    if name in ("v2", "deepseek-v2"):
        return DeepSeek2HParams(
            n_embd=5120, n_layer=60, n_head=128, n_ff=12288, n_ff_exp=1536, n_expert=160, n_expert_used=6,
            n_expert_shared=2, expert_weights_scale=16.0, n_group=8, topk_group=3, q_lora_rank=1536)
    if name in ("tiny-v3",):
        # the DeepSeek-V3-shaped code paths at toy size: sigmoid gating with a selection bias, renormalised weights,
        # group-limited routing, two leading dense layers, q-LoRA
        return DeepSeek2HParams(
            n_vocab=1024, n_embd=256, n_layer=4, n_head=4, n_layer_dense_lead=2, n_ff=512, n_ff_exp=128,
            n_expert=16, n_expert_used=4, n_expert_shared=1, q_lora_rank=96, kv_lora_rank=64,
            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_ctx_train=4096,
            n_group=4, topk_group=2, expert_weights_scale=2.5, expert_weights_norm=True, expert_gating_func="sigmoid",
            router_bias=True, group_score_top2=True, bos_id=0, eos_id=1)
    if name in ("v3", "deepseek-v3"):
        # DeepSeek-V3 / R1 shape (671B): the reference recognises it by layer count (src/llama-model.cpp:1203-1215).
        # 1.3 TB of bf16 weights: shape only, for sizing and for checkpoints sharded over more memory than one node has.
        return DeepSeek2HParams(
            n_vocab=129280, n_embd=7168, n_layer=61, n_head=128, n_layer_dense_lead=3, n_ff=18432, n_ff_exp=2048,
            n_expert=256, n_expert_used=8, n_expert_shared=1, expert_weights_scale=2.5, expert_weights_norm=True,
            expert_gating_func="sigmoid", router_bias=True, group_score_top2=True, n_group=8, topk_group=4, q_lora_rank=1536,
            n_ctx_train=163840, rope_orig_ctx=4096)
    raise KeyError(name)
