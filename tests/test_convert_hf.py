"""Checkpoint conversion from the Hugging Face layout, checked against third-party implementations: the ``transformers``
DeepseekV2 model for the forward pass (an implementation written independently of this package and of the reference) and the
``tokenizers`` library for the vocabulary and pre-tokeniser."""
import json
import os

import pytest
import torch


def _library():
    """The third-party model classes, imported on first use (collection stays cheap and free of side effects)."""
    pytest.importorskip("transformers")
    pytest.importorskip("safetensors")
    try:
        from transformers import DeepseekV2Config, DeepseekV2ForCausalLM
    except Exception:                                           # pragma: no cover
        pytest.skip("this transformers release has no DeepseekV2 model")
    return DeepseekV2Config, DeepseekV2ForCausalLM


from jittorinfer_b200.gguf import format as F
from jittorinfer_b200.gguf.convert_hf import convert, hparams_from_hf_config, vocab_kv_from_hf
from jittorinfer_b200.gguf.io import GGUFReader
from jittorinfer_b200.models.hparams import DeepSeek2HParams
from jittorinfer_b200.models.oracle import OracleModel
from jittorinfer_b200.models.weights import iter_gguf

LITE = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
            first_k_dense_replace=1, kv_lora_rank=64, q_lora_rank=None, n_routed_experts=8, n_shared_experts=2,
            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, num_experts_per_tok=3, moe_intermediate_size=128,
            routed_scaling_factor=1.0, topk_method="greedy", max_position_embeddings=512, bos_token_id=0, eos_token_id=1)
# the 236B model's structure in small: low-rank queries, group-limited routing, scaled expert weights, YaRN far past the
# original context.  mscale == mscale_all_dim -> the library applies no magnitude correction; the tiny value makes the
# softmax-scale correction of the original model (which the library omits and this package applies) vanish as well.
V2 = dict(vocab_size=512, hidden_size=256, intermediate_size=384, num_hidden_layers=3, num_attention_heads=4,
          first_k_dense_replace=1, kv_lora_rank=64, q_lora_rank=48, n_routed_experts=16, n_shared_experts=1,
          qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=48, num_experts_per_tok=4, moe_intermediate_size=96,
          routed_scaling_factor=16.0, topk_method="group_limited_greedy", n_group=4, topk_group=2,
          max_position_embeddings=2560, bos_token_id=0, eos_token_id=1,
          rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 40.0, "original_max_position_embeddings": 64,
                           "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 1e-9, "mscale_all_dim": 1e-9})


def make_hf(tmp_path, kw, seed):
    DeepseekV2Config, DeepseekV2ForCausalLM = _library()
    torch.manual_seed(seed)
    model = DeepseekV2ForCausalLM(DeepseekV2Config(**kw)).eval()
    d = str(tmp_path / "hf")
    model.save_pretrained(d, safe_serialization=True)
    for mod in model.modules():                                 # the release at hand reads an attribute its constructor never sets
        if type(mod).__name__ == "DeepseekV2Moe" and not hasattr(mod, "num_experts"):
            mod.num_experts = model.config.n_routed_experts
    return model, d


def oracle_from(path):
    rd = GGUFReader(path)
    hp = DeepSeek2HParams.from_gguf_kv(rd.kv, rd.tensors)
    w = {k: v.to(torch.float32) for k, v in iter_gguf(rd, hp)}
    return hp, OracleModel(hp, w), rd


def test_lite_checkpoint_matches_the_library_model(tmp_path):
    model, d = make_hf(tmp_path, LITE, 0)
    out = str(tmp_path / "m.gguf")
    hp = convert(d, out, "f32", toy_vocab=True)
    assert (hp.q_lora_rank, hp.n_expert, hp.n_expert_used, hp.n_expert_shared, hp.rope_scaling_type) == (0, 8, 3, 2, "none")
    ids = torch.tensor([[5, 17, 200, 33, 7, 450, 2, 99, 311, 64, 12, 12, 400]])
    with torch.no_grad():
        ref = model(ids).logits[0]
    hp2, oracle, rd = oracle_from(out)
    assert abs(hp2.rms_eps - hp.rms_eps) < 1e-12 and hp2.__class__(**dict(hp2.__dict__, rms_eps=hp.rms_eps)) == hp   # f32 key
    assert rd.tensors["blk.1.ffn_gate_exps.weight"].shape == (8, 128, 256)        # per-expert matrices stacked
    assert rd.tensors["blk.1.ffn_gate_inp.weight"].ggml_type == F.GGML_F32
    got = oracle.forward(ids[0])
    assert (got - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
    rd.close()
    # the serving engine on the converted file generates what the library generates
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    eng = build_engine(None, gguf_path=out, device="cpu", dtype=torch.float32, n_parallel=2, n_ctx_slot=64, cuda_graphs=False)
    mine = eng.generate([ids[0].tolist()], SamplingParams(ignore_eos=True), max_new_tokens=8)[0]
    with torch.no_grad():
        theirs = model.generate(ids, max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)[0, ids.shape[1]:].tolist()
    assert mine == theirs


def test_v2_structure_with_yarn_and_group_routing_matches_the_library_model(tmp_path):
    model, d = make_hf(tmp_path, V2, 1)
    out = str(tmp_path / "m.gguf")
    hp = convert(d, out, "f32", toy_vocab=True)
    assert (hp.q_lora_rank, hp.n_group, hp.topk_group, hp.expert_weights_scale) == (48, 4, 2, 16.0)
    assert (hp.rope_scaling_type, hp.rope_scaling_factor, hp.rope_orig_ctx) == ("yarn", 40.0, 64)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(2, 512, (1, 200), generator=g)          # three times the original context
    with torch.no_grad():
        ref = model(ids).logits[0]
    _, oracle, rd = oracle_from(out)
    got = oracle.forward(ids[0])
    assert (got - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
    # the routing restriction is live in this comparison: without it other experts would be picked
    hp_free = DeepSeek2HParams.from_gguf_kv(rd.kv, rd.tensors)
    hp_free.n_group = hp_free.topk_group = 1
    w = {k: v.to(torch.float32) for k, v in iter_gguf(rd, hp_free)}
    free = OracleModel(hp_free, w).forward(ids[0])
    assert (free - ref).abs().max().item() > 1e-3
    rd.close()


def test_quantised_output_and_fallback_types(tmp_path):
    model, d = make_hf(tmp_path, LITE, 3)
    out = str(tmp_path / "q.gguf")
    seen = []
    convert(d, out, "q4_k", toy_vocab=True, progress=seen.append)
    rd = GGUFReader(out)
    kinds = {n: ti.ggml_type for n, ti in rd.tensors.items()}
    assert kinds["blk.0.attn_q.weight"] == F.GGML_Q4_K                # rows of 256
    assert kinds["blk.1.ffn_down_exps.weight"] == F.GGML_Q8_0         # rows of 128: no whole super-block
    assert kinds["blk.0.attn_norm.weight"] == F.GGML_F32 and kinds["blk.1.ffn_gate_inp.weight"] == F.GGML_F32
    assert seen == list(rd.tensors)                                    # streamed in file order, one producer call each
    rd.close()
    ids = torch.tensor([[9, 8, 7, 300, 301, 302, 5, 5]])
    with torch.no_grad():
        ref = model(ids).logits[0]
    _, oracle, rd = oracle_from(out)
    got = oracle.forward(ids[0])
    rel = ((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
    assert 0 < rel < 0.3                                               # four-bit weights: close, not equal
    out8 = str(tmp_path / "q8.gguf")                                   # (a mapped file is never rewritten in place)
    convert(d, out8, "q8_0", toy_vocab=True)
    rd.close()
    _, oracle, rd = oracle_from(out8)
    rel8 = ((oracle.forward(ids[0]) - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
    assert 0 < rel8 < 0.03 and rel8 < rel
    rd.close()
    with pytest.raises(ValueError):
        convert(d, str(tmp_path / "none.gguf"), "q9_z", toy_vocab=True)


def test_original_config_layout_and_errors(tmp_path):
    cfg = dict(model_type="deepseek_v2", vocab_size=102400, hidden_size=5120, intermediate_size=12288, num_hidden_layers=60,
               num_attention_heads=128, num_key_value_heads=128, moe_intermediate_size=1536, n_routed_experts=160,
               num_experts_per_tok=6, n_shared_experts=2, first_k_dense_replace=1, routed_scaling_factor=16.0,
               norm_topk_prob=False, scoring_func="softmax", topk_method="group_limited_greedy", n_group=8, topk_group=3,
               q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rms_norm_eps=1e-6,
               max_position_embeddings=163840, rope_theta=10000, bos_token_id=100000, eos_token_id=100001,
               rope_scaling={"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096, "beta_fast": 32,
                             "beta_slow": 1, "mscale": 0.707, "mscale_all_dim": 0.707})
    hp = hparams_from_hf_config(cfg)
    from jittorinfer_b200.models.hparams import preset
    ref = preset("v2")
    for f in ("n_vocab", "n_embd", "n_layer", "n_head", "n_ff", "n_ff_exp", "n_expert", "n_expert_used", "n_expert_shared",
              "n_layer_dense_lead", "expert_weights_scale", "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim",
              "qk_rope_head_dim", "v_head_dim", "rope_scaling_type", "rope_scaling_factor", "rope_orig_ctx", "n_group",
              "topk_group"):
        assert getattr(hp, f) == getattr(ref, f), f
    assert abs(hp.rope_yarn_log_mul - 0.0707) < 1e-9 and (hp.bos_id, hp.eos_id) == (100000, 100001)
    with pytest.raises(ValueError):
        hparams_from_hf_config(dict(cfg, model_type="llama"))
    with pytest.raises(ValueError):
        hparams_from_hf_config(dict(cfg, rope_scaling={"type": "linear", "factor": 2}))
    with pytest.raises(ValueError):
        hparams_from_hf_config(dict(cfg, num_key_value_heads=8))
    with pytest.raises(ValueError):
        hparams_from_hf_config(dict(cfg, moe_layer_freq=2))
    lite = hparams_from_hf_config(dict(cfg, q_lora_rank=None, topk_method="greedy", n_group=1, topk_group=1, moe_layer_freq=1,
                                       num_hidden_layers=27, ep_size=1, aux_loss_alpha=0.001, seq_aux=True))
    assert lite.q_lora_rank == 0 and lite.is_lite and (lite.n_group, lite.topk_group) == (1, 1)


def test_missing_and_foreign_tensors_are_reported(tmp_path):
    _, d = make_hf(tmp_path, LITE, 4)
    from safetensors.torch import load_file, save_file
    p = os.path.join(d, "model.safetensors")
    sd = {k: v.clone() for k, v in load_file(p).items()}           # own memory: the file is rewritten below
    extra = dict(sd)
    extra["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)          # dropped silently
    extra["model.layers.3.mlp.gate.weight"] = torch.ones(8, 256)                   # a layer past num_hidden_layers: dropped
    save_file(extra, p)
    convert(d, str(tmp_path / "ok.gguf"), "f16", toy_vocab=True)
    extra["model.vision_tower.weight"] = torch.ones(4, 4)
    save_file(extra, p)
    with pytest.raises(ValueError, match="no place"):
        convert(d, str(tmp_path / "bad.gguf"), "f16", toy_vocab=True)
    lacking = {k: v for k, v in sd.items() if k != "model.layers.1.mlp.experts.5.up_proj.weight"}
    save_file(lacking, p)
    with pytest.raises(ValueError, match="experts"):
        convert(d, str(tmp_path / "bad.gguf"), "f16", toy_vocab=True)
    lacking = {k: v for k, v in sd.items() if k != "model.layers.2.self_attn.o_proj.weight"}
    save_file(lacking, p)
    with pytest.raises(ValueError, match="lacks"):
        convert(d, str(tmp_path / "bad.gguf"), "f16", toy_vocab=True)
    tied = {k: v for k, v in sd.items() if k != "lm_head.weight"}                  # tied embeddings: the head is the table
    save_file(tied, p)
    convert(d, str(tmp_path / "tied.gguf"), "f32", toy_vocab=True)
    rd = GGUFReader(str(tmp_path / "tied.gguf"))
    assert torch.equal(rd.tensor("output.weight"), rd.tensor("token_embd.weight"))
    rd.close()


# The pre-tokeniser rules of the deepseek-llm vocabulary as regular expressions for the ``tokenizers`` library; the letter
# class is cut down to Basic Latin .. Latin Extended-B, which is what the sample texts below use.
RULES = ["[\r\n]", "\\s?[A-Za-zµÀ-ÖØ-öø-ƺ]+", "\\s?[!-/:-~！-／：-～‘-‟　-。]+", "\\s+$", "[一-龥ࠀ-一가-퟿]+", "\\p{N}+"]
CORPUS = [
    "The quick brown fox jumps over the lazy dog. The dog sleeps; the fox runs!",
    "Größe, naïve façade, Ærøskøbing and Ångström are Latin words with diacritics.",
    "def main(argc, argv):\n    return 0 if argc == 1 else len(argv) * 3.14159\n",
    "深度求索发布了新的模型。今天天气很好，我们去公园散步。",
    "한국어 문장도 몇 개 넣어 둔다. 모델은 2024년 5월에 공개되었다.",
    "Numbers: 1234567890, 42, 3.5e10, 100%, $9.99, 2024-05-06T07:08:09Z",
    "tabs\tand  double  spaces   and trailing space \n\nnew paragraphs\r\nwindows line ends",
] * 4
SAMPLES = [
    "Hello world", " leading space", "trailing space ", "two  spaces", "line\nbreak\n\nparagraph", "tab\tseparated",
    "The fox, the dog; and the 3 cats!", "naïve façade in Ærøskøbing", "x = y * 3.14159 + argv[0]",
    "深度求索的模型在2024年发布。", "한국어와 English mixed 123", "100% of $9.99", "a", "", "   ", "\n", "ends with newline\n",
    "punctuation!!! ??? ... --- ___", "CamelCaseWordsAndUPPERCASE", "mixed中文and英文text", "12345678901234567890",
    "quotes ‘single’ “double” and　ideographic space",
]


def test_vocabulary_conversion_agrees_with_the_tokenizers_library(tmp_path):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, models, pre_tokenizers, trainers
    bos, eos = "<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>"
    tok = tk.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(r), "isolated") for r in RULES] +
                                                [pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=[bos, eos], show_progress=False,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS, trainer)
    tok.add_tokens(["<tool_call>"])                              # an added token that is not special
    d = tmp_path / "hf"
    d.mkdir()
    tok.save(str(d / "tokenizer.json"))
    json.dump({"bos_token": {"content": bos}, "eos_token": eos, "add_bos_token": True, "add_eos_token": False,
               "chat_template": "{% for m in messages %}{{ m['content'] }}{% endfor %}"}, open(d / "tokenizer_config.json", "w"))
    n_defined = tok.get_vocab_size(with_added_tokens=True)
    hp = DeepSeek2HParams()
    hp.n_vocab = n_defined + 9                                   # the embedding table is padded past the tokenizer
    kv = vocab_kv_from_hf(str(d), hp)
    tokens, types = kv["tokenizer.ggml.tokens"], kv["tokenizer.ggml.token_type"][1]
    assert len(tokens) == hp.n_vocab and tokens[-1].startswith("[PAD") and types[-1] == 5
    assert kv["tokenizer.ggml.bos_token_id"] == ("u32", tok.token_to_id(bos)) and kv["tokenizer.ggml.eos_token_id"] == ("u32", tok.token_to_id(eos))
    assert types[tok.token_to_id(bos)] == 3 and types[tok.token_to_id("<tool_call>")] == 4
    assert kv["tokenizer.chat_template"].startswith("{% for")
    flat = {k: (v[1] if isinstance(v, tuple) else v) for k, v in kv.items()}
    from jittorinfer_b200.tokenizer import Tokenizer
    mine = Tokenizer.from_gguf_kv(flat)
    assert len(json.load(open(d / "tokenizer.json"))["model"]["merges"]) > 100
    for text in SAMPLES + CORPUS[:7]:
        theirs = tok.encode(text, add_special_tokens=False).ids
        got = mine.encode(text, add_special=False, parse_special=False)
        assert got == theirs, (text, [tokens[i] for i in got], [tokens[i] for i in theirs])
        assert mine.decode(got) == text
    assert mine.encode("x", add_special=True)[0] == tok.token_to_id(bos)
    special = mine.encode(f"a{eos}b<tool_call>", add_special=False, parse_special=True)
    assert tok.token_to_id(eos) in special and tok.token_to_id("<tool_call>") in special


def test_v3_structure_matches_the_library_model(tmp_path):
    """Sigmoid scores, bias-corrected group-limited choice (groups ranked by their two best experts), normalised and scaled
    weights, and the softmax-scale correction of YaRN (mscale_all_dim = 1: scale x (1 + 0.1 ln 40)^2), which the library's V3
    model applies like the original model does."""
    try:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    except Exception:                                           # pragma: no cover
        pytest.skip("this transformers release has no DeepseekV3 model")
    cfg = DeepseekV3Config(vocab_size=512, hidden_size=256, intermediate_size=384, num_hidden_layers=3, num_attention_heads=4,
                           num_key_value_heads=4, first_k_dense_replace=1, kv_lora_rank=64, q_lora_rank=48, n_routed_experts=16,
                           n_shared_experts=1, qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=48, num_experts_per_tok=4,
                           moe_intermediate_size=96, routed_scaling_factor=2.5, n_group=4, topk_group=2, norm_topk_prob=True,
                           max_position_embeddings=2560, bos_token_id=0, eos_token_id=1,
                           rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 40.0,
                                            "original_max_position_embeddings": 64, "beta_fast": 32.0, "beta_slow": 1.0,
                                            "mscale": 1.0, "mscale_all_dim": 1.0})
    torch.manual_seed(7)
    model = DeepseekV3ForCausalLM(cfg).eval()
    with torch.no_grad():
        for mod in model.modules():
            if hasattr(mod, "e_score_correction_bias"):
                mod.e_score_correction_bias.copy_(torch.randn_like(mod.e_score_correction_bias) * 0.1)
    d = str(tmp_path / "hf")
    model.save_pretrained(d, safe_serialization=True)
    out = str(tmp_path / "m.gguf")
    hp = convert(d, out, "f32", toy_vocab=True)
    assert (hp.expert_gating_func, hp.group_score_top2, hp.router_bias, hp.expert_weights_norm) == ("sigmoid", True, True, True)
    assert (hp.n_group, hp.topk_group, hp.expert_weights_scale) == (4, 2, 2.5) and abs(hp.rope_yarn_log_mul - 0.1) < 1e-12
    ids = torch.randint(2, 512, (1, 160), generator=torch.Generator().manual_seed(8))
    with torch.no_grad():
        ref = model(ids).logits[0]
    _, oracle, rd = oracle_from(out)
    assert "blk.1.exp_probs_b.bias" in rd.tensors
    got = oracle.forward(ids[0])
    assert (got - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
    rd.close()
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    eng = build_engine(None, gguf_path=out, device="cpu", dtype=torch.float32, n_parallel=2, n_ctx_slot=256, cuda_graphs=False)
    prompt = ids[0, :70].tolist()                               # past the original context of 64
    mine = eng.generate([prompt], SamplingParams(ignore_eos=True), max_new_tokens=6)[0]
    with torch.no_grad():
        theirs = model.generate(ids[:, :70], max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, 70:].tolist()
    assert mine == theirs


@pytest.mark.gpu
def test_gpu_engine_on_a_converted_checkpoint_follows_the_library_model(tmp_path):
    """bf16 kernels against the library's fp32 model: the first tokens of a greedy continuation agree and the logits of the
    prompt's last position agree to bf16 resolution (read through the engine's top-k log-probabilities)."""
    model, d = make_hf(tmp_path, LITE, 0)
    out = str(tmp_path / "m.gguf")
    convert(d, out, "bf16", toy_vocab=True)
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    ids = torch.tensor([[5, 17, 200, 33, 7, 450, 2, 99, 311, 64, 12, 12, 400]])
    eng = build_engine(None, gguf_path=out, device="cuda", n_parallel=2, n_ctx_slot=64, cuda_graphs=False)
    mine = eng.generate([ids[0].tolist()], SamplingParams(ignore_eos=True), max_new_tokens=4)[0]
    with torch.no_grad():
        theirs = model.generate(ids, max_new_tokens=4, do_sample=False, eos_token_id=None, pad_token_id=0)[0, ids.shape[1]:].tolist()
        ref = model(ids).logits[0, -1]
    assert mine[0] == theirs[0] or ref[mine[0]] > ref.max() - 0.05         # bf16 may swap a near tie
    assert sum(a == b for a, b in zip(mine, theirs)) >= 2
