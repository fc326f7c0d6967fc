"""GGUF writer/reader round trip, shard views and hparams mapping."""
import numpy as np
import torch

from jittorinfer_b200.gguf import format as F
from jittorinfer_b200.gguf.io import GGUFReader, GGUFWriter
from jittorinfer_b200.models.hparams import DeepSeek2HParams, preset
from jittorinfer_b200.models.weights import ShardSpec, iter_gguf, iter_random, random_weights, tensor_table, write_random_gguf


def test_roundtrip_types_and_alignment(tmp_path):
    p = str(tmp_path / "t.gguf")
    w = GGUFWriter(p)
    w.add("general.architecture", "deepseek2")
    w.add("x.u32", ("u32", 7))
    w.add("x.f32", 1.5)
    w.add("x.flag", True)
    w.add("x.strs", ["a", "bc", "é"])
    w.add("x.ints", [1, 2, 3])
    a = torch.randn(3, 64)
    w.add_tensor("a.f32", a)
    w.add_tensor("a.bf16", a.bfloat16())
    w.add_tensor("a.f16", a.half())
    w.add_tensor("a.q8", a, F.GGML_Q8_0)
    w.add_tensor("a.q4", a, F.GGML_Q4_0)
    w.write()
    r = GGUFReader(p)
    assert r.kv["x.u32"] == 7 and r.kv["x.f32"] == 1.5 and r.kv["x.flag"] is True
    assert r.kv["x.strs"] == ["a", "bc", "é"] and list(r.kv["x.ints"]) == [1, 2, 3]
    assert torch.equal(r.tensor("a.f32"), a) and torch.equal(r.tensor("a.bf16"), a.bfloat16())
    assert torch.equal(r.tensor("a.f16"), a.half())
    assert (r.tensor("a.q8") - a).abs().max() < 0.03 and (r.tensor("a.q4") - a).abs().max() < 0.5
    for ti in r.tensors.values():
        assert (r.data_offset + ti.offset) % 32 == 0
    assert torch.equal(r.tensor_slice("a.f32", 1, 1, 2), a[:, 32:])


def test_random_gguf_loads_back_and_shards_agree(tmp_path):
    hp = preset("tiny-v2")
    p = str(tmp_path / "m.gguf")
    write_random_gguf(p, hp, seed=0)
    r = GGUFReader(p)
    hp2 = DeepSeek2HParams.from_gguf_kv(r.kv, r.tensors)
    for k in ("n_embd", "n_layer", "n_head", "q_lora_rank", "kv_lora_rank", "n_expert", "n_group", "topk_group", "n_vocab"):
        assert getattr(hp, k) == getattr(hp2, k), k
    full = dict(iter_gguf(r, hp2))
    ref = random_weights(hp, seed=0)
    assert set(full) == set(tensor_table(hp)) and all(torch.equal(full[k].float(), ref[k]) for k in ref)
    for ep in (False, True):
        for rank in range(2):
            spec = ShardSpec(rank, 2, ep)
            from_file = dict(iter_gguf(r, hp2, spec))
            from_rng = dict(iter_random(hp, spec=spec, seed=0))
            assert all(torch.equal(from_file[k].float(), from_rng[k]) for k in from_rng)
    e = full["blk.1.ffn_gate_exps.weight"]
    assert torch.equal(dict(iter_gguf(r, hp2, ShardSpec(1, 2, True)))["blk.1.ffn_gate_exps.weight"], e[e.shape[0] // 2:])
