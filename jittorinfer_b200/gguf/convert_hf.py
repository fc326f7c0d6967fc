"""Hugging Face checkpoint directory -> GGUF in the key / tensor layout this package (and the reference) serves.

    python -m jittorinfer_b200.gguf.convert_hf /data/DeepSeek-V2-Lite-Chat out.gguf --type bf16
    python -m jittorinfer_b200.gguf.convert_hf /data/DeepSeek-V2-Chat out.gguf --type Q8_0

Reads ``config.json`` (the original DeepSeek layout with ``rope_theta`` / ``rope_scaling`` as well as the newer
``rope_parameters`` layout), the ``*.safetensors`` shards (through their index when there is one) and ``tokenizer.json``.
Tensors are streamed: one tensor (for the routed experts: the stack of one layer's experts) is resident at a time, so the
236B checkpoint converts on a host with far less memory than the model.

The reference ships no converter -- its GGUF files come from upstream tooling -- but it fixes what the file must contain:
the ``deepseek2.*`` keys it reads (src/llama-model.cpp:1047-1250), the tensor names (src/llama-arch.cpp:903-927) with the
routed experts stacked as ``ffn_{gate,up,down}_exps`` [n_expert, rows, cols], and a ``gpt2`` / ``deepseek-llm`` vocabulary
(src/llama-vocab.cpp:440-483).  Two keys beyond those, ``expert_group_count`` and ``expert_group_used_count``, carry the
group-limited routing of the 236B model, which this package implements and the reference ignores.
"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..models.hparams import DeepSeek2HParams
from . import format as F

OUT_TYPES = {"f32": F.GGML_F32, "f16": F.GGML_F16, "bf16": F.GGML_BF16}
OUT_TYPES.update({name.lower(): t for t, name in F.TYPE_NAMES.items() if t in F.QUANTIZED and name != "Q8_K"})


# ---- hyper-parameters ---------------------------------------------------------------------------------------------------
def hparams_from_hf_config(cfg: Dict[str, Any]) -> DeepSeek2HParams:
    mt = cfg.get("model_type", "")
    if mt not in ("deepseek_v2", "deepseek_v3"):
        raise ValueError(f"model_type {mt!r}: only deepseek_v2 / deepseek_v3 checkpoints convert to the deepseek2 layout")
    hp = DeepSeek2HParams()
    hp.n_vocab = int(cfg["vocab_size"])
    hp.n_embd = int(cfg["hidden_size"])
    hp.n_layer = int(cfg["num_hidden_layers"])
    hp.n_head = int(cfg["num_attention_heads"])
    if int(cfg.get("num_key_value_heads") or hp.n_head) != hp.n_head:
        raise ValueError("num_key_value_heads differs from num_attention_heads: not a multi-head latent attention checkpoint")
    hp.n_ff = int(cfg["intermediate_size"])
    hp.n_ff_exp = int(cfg.get("moe_intermediate_size") or 0)
    hp.n_expert = int(cfg.get("n_routed_experts") or 0)
    hp.n_expert_used = int(cfg.get("num_experts_per_tok") or 0)
    hp.n_expert_shared = int(cfg.get("n_shared_experts") or 0)
    hp.n_layer_dense_lead = int(cfg.get("first_k_dense_replace") or 0) if hp.n_expert else hp.n_layer
    if hp.n_expert and int(cfg.get("moe_layer_freq") or 1) != 1:
        raise ValueError("moe_layer_freq != 1: the deepseek2 layout has dense blocks only at the front")
    hp.expert_weights_scale = float(cfg.get("routed_scaling_factor") or 1.0)
    hp.expert_weights_norm = bool(cfg.get("norm_topk_prob") or False)
    v3 = mt == "deepseek_v3"                # sigmoid scores, bias-corrected group-limited choice: implied by the model type
    sigmoid = cfg.get("scoring_func", "sigmoid" if v3 else "softmax") == "sigmoid"
    hp.expert_gating_func = "sigmoid" if sigmoid else "softmax"
    hp.group_score_top2 = sigmoid
    method = cfg.get("topk_method") or ("noaux_tc" if v3 else "greedy")
    if method in ("group_limited_greedy", "noaux_tc"):
        hp.n_group, hp.topk_group = int(cfg.get("n_group") or 1), int(cfg.get("topk_group") or 1)
    else:
        hp.n_group = hp.topk_group = 1
    hp.q_lora_rank = int(cfg.get("q_lora_rank") or 0)
    hp.kv_lora_rank = int(cfg["kv_lora_rank"])
    hp.qk_nope_head_dim = int(cfg["qk_nope_head_dim"])
    hp.qk_rope_head_dim = int(cfg["qk_rope_head_dim"])
    hp.v_head_dim = int(cfg["v_head_dim"])
    hp.rms_eps = float(cfg.get("rms_norm_eps", 1e-6))
    hp.n_ctx_train = int(cfg.get("max_position_embeddings", 4096))
    rope = dict(cfg.get("rope_parameters") or {})
    scaling = dict(cfg.get("rope_scaling") or {})
    hp.rope_freq_base = float(rope.get("rope_theta", cfg.get("rope_theta", 10000.0)))
    kind = scaling.get("type") or scaling.get("rope_type") or rope.get("rope_type") or "default"
    src = scaling if scaling else rope
    if kind == "yarn":
        hp.rope_scaling_type = "yarn"
        hp.rope_scaling_factor = float(src.get("factor", 1.0))
        hp.rope_orig_ctx = int(src.get("original_max_position_embeddings", hp.n_ctx_train))
        hp.rope_yarn_log_mul = 0.1 * float(src.get("mscale_all_dim") or 0.0)
        hp.yarn_beta_fast = float(src.get("beta_fast", 32.0))
        hp.yarn_beta_slow = float(src.get("beta_slow", 1.0))
    elif kind in ("default", "none", None):
        hp.rope_scaling_type, hp.rope_scaling_factor, hp.rope_yarn_log_mul = "none", 1.0, 0.0
        hp.rope_orig_ctx = hp.n_ctx_train
    else:
        raise ValueError(f"rope scaling {kind!r} is not one the deepseek2 graph implements (none, yarn)")

    def first(v, default):
        if isinstance(v, (list, tuple)):
            v = v[0] if v else None
        return int(v) if v is not None else default
    hp.bos_id, hp.eos_id = first(cfg.get("bos_token_id"), 0), first(cfg.get("eos_token_id"), 1)
    hp.router_bias = False
    return hp


# ---- tensors ------------------------------------------------------------------------------------------------------------
_LAYER = {
    "input_layernorm.weight": "attn_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.q_a_proj.weight": "attn_q_a.weight",
    "self_attn.q_a_layernorm.weight": "attn_q_a_norm.weight",
    "self_attn.q_b_proj.weight": "attn_q_b.weight",
    "self_attn.kv_a_proj_with_mqa.weight": "attn_kv_a_mqa.weight",
    "self_attn.kv_a_layernorm.weight": "attn_kv_a_norm.weight",
    "self_attn.kv_b_proj.weight": "attn_kv_b.weight",
    "self_attn.o_proj.weight": "attn_output.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
    "mlp.gate.weight": "ffn_gate_inp.weight",
    "mlp.gate.e_score_correction_bias": "exp_probs_b.bias",
    "mlp.shared_experts.gate_proj.weight": "ffn_gate_shexp.weight",
    "mlp.shared_experts.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_experts.down_proj.weight": "ffn_down_shexp.weight",
}
_TOP = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
_EXPERT = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$")
_FUSED = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(gate_up_proj|down_proj)$")
_PLAIN = re.compile(r"^model\.layers\.(\d+)\.(.+)$")


class Checkpoint:
    """The tensors of a checkpoint directory by name, loaded one at a time from whichever shard holds them."""

    def __init__(self, directory: str):
        from safetensors import safe_open
        self._open = safe_open
        self.directory = directory
        index = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.where: Dict[str, str] = dict(json.load(f)["weight_map"])
        else:
            files = sorted(fn for fn in os.listdir(directory) if fn.endswith(".safetensors"))
            if not files:
                raise FileNotFoundError(f"{directory}: no .safetensors file")
            self.where = {}
            for fn in files:
                with safe_open(os.path.join(directory, fn), "pt") as f:
                    for k in f.keys():
                        self.where[k] = fn
        self._handles: Dict[str, Any] = {}

    def names(self) -> List[str]:
        return list(self.where)

    def _file(self, fn: str):
        if fn not in self._handles:
            if len(self._handles) >= 8:                          # a bounded number of mappings open at once
                self._handles.pop(next(iter(self._handles))).__exit__(None, None, None)
            self._handles[fn] = self._open(os.path.join(self.directory, fn), "pt").__enter__()
        return self._handles[fn]

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._file(self.where[name]).get_slice(name).get_shape())

    def get(self, name: str) -> torch.Tensor:
        return self._file(self.where[name]).get_tensor(name)

    def close(self):
        for h in self._handles.values():
            h.__exit__(None, None, None)
        self._handles.clear()


def plan_tensors(ck: Checkpoint, hp: DeepSeek2HParams) -> Dict[str, Tuple[Tuple[int, ...], Callable[[], torch.Tensor]]]:
    """GGUF name -> (shape, producer).  Routed experts of a layer are stacked; multi-token-prediction layers beyond
    ``num_hidden_layers`` and rotary caches are dropped; anything else that has no place is an error."""
    plan: Dict[str, Tuple[Tuple[int, ...], Callable[[], torch.Tensor]]] = {}
    experts: Dict[Tuple[int, str], Dict[int, str]] = {}
    unknown = []
    for name in ck.names():
        if name.endswith("rotary_emb.inv_freq"):
            continue
        if name in _TOP:
            plan[_TOP[name]] = (ck.shape(name), (lambda n=name: ck.get(n)))
            continue
        m = _EXPERT.match(name)
        if m:
            il, ie, kind = int(m.group(1)), int(m.group(2)), m.group(3)
            if il < hp.n_layer:
                experts.setdefault((il, kind), {})[ie] = name
            continue
        m = _FUSED.match(name)
        if m:
            il, kind = int(m.group(1)), m.group(2)
            if il >= hp.n_layer:
                continue
            e, r, c = ck.shape(name)
            if kind == "down_proj":
                plan[f"blk.{il}.ffn_down_exps.weight"] = ((e, r, c), (lambda n=name: ck.get(n)))
            else:                                                # rows: gate, then up
                plan[f"blk.{il}.ffn_gate_exps.weight"] = ((e, r // 2, c), (lambda n=name, h=r // 2: ck.get(n)[:, :h].contiguous()))
                plan[f"blk.{il}.ffn_up_exps.weight"] = ((e, r // 2, c), (lambda n=name, h=r // 2: ck.get(n)[:, h:].contiguous()))
            continue
        m = _PLAIN.match(name)
        if m and m.group(2) in _LAYER:
            il = int(m.group(1))
            if il < hp.n_layer:
                plan[f"blk.{il}.{_LAYER[m.group(2)]}"] = (ck.shape(name), (lambda n=name: ck.get(n)))
            continue
        if m and int(m.group(1)) >= hp.n_layer:
            continue                                             # multi-token-prediction head of DeepSeek-V3
        unknown.append(name)
    if unknown:
        raise ValueError(f"{len(unknown)} checkpoint tensors have no place in the deepseek2 layout, e.g. {unknown[:4]}")
    for (il, kind), by_id in experts.items():
        if sorted(by_id) != list(range(hp.n_expert)):
            raise ValueError(f"layer {il}: {kind}_proj of {len(by_id)} experts found, {hp.n_expert} expected")
        r, c = ck.shape(by_id[0])
        names = [by_id[i] for i in range(hp.n_expert)]
        plan[f"blk.{il}.ffn_{kind}_exps.weight"] = ((hp.n_expert, r, c), (lambda ns=names: torch.stack([ck.get(n) for n in ns])))
    if "output.weight" not in plan and "token_embd.weight" in plan:          # tied embeddings
        plan["output.weight"] = plan["token_embd.weight"]
    return plan


# ---- vocabulary ---------------------------------------------------------------------------------------------------------
def _token_text(v) -> Optional[str]:
    if isinstance(v, dict):
        v = v.get("content")
    return v if isinstance(v, str) else None


def vocab_kv_from_hf(directory: str, hp: DeepSeek2HParams) -> Dict[str, Any]:
    """``tokenizer.json`` (+ ``tokenizer_config.json``) -> the ``tokenizer.*`` keys.  Token strings stay in the byte-level
    alphabet they already use; ids the tokenizer does not define up to ``vocab_size`` become unused padding entries."""
    with open(os.path.join(directory, "tokenizer.json"), encoding="utf-8") as f:
        tj = json.load(f)
    model = tj.get("model", {})
    if model.get("type") != "BPE":
        raise ValueError(f"tokenizer model {model.get('type')!r}: the deepseek2 vocabulary is byte-level BPE")
    n = hp.n_vocab
    tokens: List[Optional[str]] = [None] * n
    types = [1] * n
    for tok, i in model["vocab"].items():
        if i >= n:
            raise ValueError(f"token id {i} is outside vocab_size {n}")
        tokens[i] = tok
    for a in tj.get("added_tokens", []):
        i = int(a["id"])
        if i >= n:
            raise ValueError(f"added token id {i} is outside vocab_size {n}")
        tokens[i] = a["content"]
        types[i] = 3 if a.get("special") else 4
    for i in range(n):
        if tokens[i] is None:
            tokens[i], types[i] = f"[PAD{i}]", 5
    merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
    kv: Dict[str, Any] = {
        "tokenizer.ggml.model": "gpt2",
        "tokenizer.ggml.pre": "deepseek-llm",
        "tokenizer.ggml.tokens": tokens,
        "tokenizer.ggml.token_type": ("i32", types),
        "tokenizer.ggml.merges": merges,
    }
    tc: Dict[str, Any] = {}
    p = os.path.join(directory, "tokenizer_config.json")
    if os.path.exists(p):
        with open(p, encoding="utf-8") as f:
            tc = json.load(f)
    index = {t: i for i, t in enumerate(tokens)}
    for key, field in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("pad_token", "padding_token_id"),
                       ("unk_token", "unknown_token_id")):
        text = _token_text(tc.get(key))
        if text is not None and text in index:
            kv[f"tokenizer.ggml.{field}"] = ("u32", index[text])
    kv["tokenizer.ggml.add_bos_token"] = bool(tc.get("add_bos_token", True))
    kv["tokenizer.ggml.add_eos_token"] = bool(tc.get("add_eos_token", False))
    if isinstance(tc.get("chat_template"), str):
        kv["tokenizer.chat_template"] = tc["chat_template"]
    return kv


# ---- conversion ---------------------------------------------------------------------------------------------------------
def pick_type(name: str, shape: Tuple[int, ...], out_type: int) -> int:
    """Norms, biases and the router stay f32 (they are small and the router decides which experts run); a matrix whose rows
    do not hold whole blocks of a quantised ``out_type`` falls back to Q8_0, then to f16."""
    if len(shape) < 2 or name.endswith("ffn_gate_inp.weight") or name.endswith(".bias"):
        return F.GGML_F32
    for cand in (out_type, F.GGML_Q8_0, F.GGML_F16):
        if shape[-1] % F.TYPE_TRAITS[cand][0] == 0:
            return cand
    return F.GGML_F32


def convert(hf_dir: str, out_path: str, out_type: str = "bf16", toy_vocab: bool = False, name: Optional[str] = None,
            progress: Optional[Callable[[str], None]] = None) -> DeepSeek2HParams:
    from ..models.weights import tensor_table
    from .io import GGUFWriter
    if out_type.lower() not in OUT_TYPES:
        raise ValueError(f"output type {out_type!r}: one of {sorted(OUT_TYPES)}")
    gt = OUT_TYPES[out_type.lower()]
    with open(os.path.join(hf_dir, "config.json")) as f:
        cfg = json.load(f)
    hp = hparams_from_hf_config(cfg)
    ck = Checkpoint(hf_dir)
    try:
        plan = plan_tensors(ck, hp)
        hp.router_bias = any(n.endswith("exp_probs_b.bias") for n in plan)
        table = tensor_table(hp)
        missing = [n for n in table if n not in plan]
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors of the architecture, e.g. {missing[:4]}")
        for n, shape in table.items():
            if tuple(plan[n][0]) != tuple(shape):
                raise ValueError(f"{n}: checkpoint shape {tuple(plan[n][0])}, architecture says {tuple(shape)}")
        w = GGUFWriter(out_path)
        kv = hp.to_gguf_kv()
        kv["general.name"] = name or os.path.basename(os.path.normpath(hf_dir))
        if hp.rope_scaling_type == "yarn":
            kv["deepseek2.rope.scaling.yarn_beta_fast"] = ("f32", hp.yarn_beta_fast)
            kv["deepseek2.rope.scaling.yarn_beta_slow"] = ("f32", hp.yarn_beta_slow)
        w.add_dict(kv)
        if toy_vocab:
            from ..utils.toy_vocab import toy_vocab_kv
            w.add_dict(toy_vocab_kv(hp.n_vocab, hp.bos_id, hp.eos_id))
        else:
            vk = vocab_kv_from_hf(hf_dir, hp)
            w.add_dict(vk)

        def producer(n, fn):
            def run():
                if progress is not None:
                    progress(n)
                return fn().to(torch.float32)
            return run
        for n, shape in table.items():
            w.add_tensor_lazy(n, shape, pick_type(n, tuple(shape), gt), producer(n, plan[n][1]))
        w.write()
    finally:
        ck.close()
    return hp


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("hf_dir")
    ap.add_argument("out")
    ap.add_argument("--type", default="bf16", help="f32, f16, bf16 or a block-quantised type: " +
                    ", ".join(sorted(k for k in OUT_TYPES if k not in ("f32", "f16", "bf16"))))
    ap.add_argument("--toy-vocab", action="store_true", help="write a byte-level stand-in vocabulary (no tokenizer.json needed)")
    ap.add_argument("--name", default=None)
    ap.add_argument("-q", "--quiet", action="store_true")
    a = ap.parse_args(argv)
    hp = convert(a.hf_dir, a.out, a.type, a.toy_vocab, a.name, None if a.quiet else (lambda n: print(n, flush=True)))
    print(f"wrote {a.out}: {hp.n_layer} layers, {hp.n_params() / 1e9:.2f} B parameters, type {a.type}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
