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


def test_native_reader_matches_python_reader(tmp_path, monkeypatch):
    """The C++ parser sees the same key/values, tensor table and bytes as the Python one, and a model loaded through it
    produces the same logits."""
    import numpy as np
    import torch
    from jittorinfer_b200.gguf.io import GGUFReader
    from jittorinfer_b200.gguf.native_reader import NativeGGUFReader
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import write_random_gguf
    p = str(tmp_path / "m.gguf")
    write_random_gguf(p, preset("tiny"), seed=3, dtype=torch.bfloat16)
    py, nat = GGUFReader(p), NativeGGUFReader(p)
    assert nat.version == py.version and nat.alignment == py.alignment
    assert set(nat.kv) == set(py.kv)
    for k, v in py.kv.items():
        w = nat.kv[k]
        if isinstance(v, np.ndarray):
            assert list(v.tolist()) == w, k
        elif isinstance(v, float):
            assert abs(v - w) <= 1e-6 * max(1.0, abs(v)), k
        else:
            assert v == w, k
    assert list(nat.tensors) == list(py.tensors)
    for name, ti in py.tensors.items():
        tn = nat.tensors[name]
        assert (tn.shape, tn.ggml_type, tn.nbytes) == (ti.shape, ti.ggml_type, ti.nbytes)
        assert np.array_equal(nat.raw(name), py.raw(name)), name
    a = nat.tensor_slice("blk.1.ffn_gate_exps.weight", 0, 1, 2)
    b = py.tensor_slice("blk.1.ffn_gate_exps.weight", 0, 1, 2)
    assert torch.equal(a, b)
    with __import__("pytest").raises(ValueError):
        NativeGGUFReader(str(tmp_path / "missing.gguf"))
    from jittorinfer_b200.runtime.factory import build_model
    m_py = build_model(gguf_path=p, device="cpu", dtype=torch.float32)
    monkeypatch.setenv("JITTORINFER_GGUF", "native")
    m_nat = build_model(gguf_path=p, device="cpu", dtype=torch.float32)
    assert torch.equal(m_py.layers[1].w_gate_exps, m_nat.layers[1].w_gate_exps) and torch.equal(m_py.tok_embd, m_nat.tok_embd)
    # on the CPU the float32 weights are views of the mapping: it must outlive the reader object that created it
    import gc
    del nat, py
    gc.collect()
    from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    outs = [LLMEngine(m, EngineConfig(n_ctx=256, n_batch=32, n_parallel=1)).generate([[1, 2, 3, 4]], SamplingParams(ignore_eos=True), 4)
            for m in (m_py, m_nat)]
    assert outs[0] == outs[1]


def test_staged_uploader_chunks_and_converts():
    import torch
    from jittorinfer_b200.models.weights import StagedUploader
    up = StagedUploader("cpu", chunk_bytes=1000, n_buffers=2, min_bytes=1)
    t = torch.randn(37, 53)                                   # 7844 bytes -> 8 chunks, the last one partial
    out = up.upload(t)
    assert torch.equal(out, t) and up.n_chunks == 8
    half = up.upload(t.half(), dtype=torch.bfloat16)
    assert half.dtype == torch.bfloat16 and torch.equal(half, t.half().to(torch.bfloat16))
    small = StagedUploader("cpu", min_bytes=1 << 20)
    assert torch.equal(small.upload(t), t) and small.n_chunks == 0      # below the threshold: plain copy


def test_check_tensors_rejects_a_file_with_non_finite_weights(tmp_path):
    """``check_tensors`` (model parameter of the C API, key of the YAML files) verifies every weight while loading."""
    import pytest
    from jittorinfer_b200.config import ServerConfig, load_yaml
    from jittorinfer_b200.gguf.io import GGUFReader, GGUFWriter
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.runtime.factory import build_model
    good, bad = str(tmp_path / "good.gguf"), str(tmp_path / "bad.gguf")
    write_random_gguf(good, preset("tiny"), seed=2)
    with GGUFReader(good) as rd:
        w = GGUFWriter(bad)
        for k, v in rd.kv.items():
            if k != "general.alignment":
                w.add_typed(k, v, rd.kv_types[k], rd.kv_elem_types.get(k))
        for name in rd.tensors:
            t = rd.tensor(name).clone()
            if name == "blk.1.ffn_up_exps.weight":
                t[3, 5, 7] = float("nan")
                t[0, 0, 0] = float("inf")
            w.add_tensor(name, t)
        w.write()
    build_model(gguf_path=good, device="cpu", dtype=torch.float32, check_tensors=True)
    build_model(gguf_path=bad, device="cpu", dtype=torch.float32)                       # not asked: loads
    with pytest.raises(ValueError, match="blk.1.ffn_up_exps.weight: 2 of"):
        build_model(gguf_path=bad, device="cpu", dtype=torch.float32, check_tensors=True)
    y = tmp_path / "c.yaml"
    y.write_text("model: x.gguf\ncheck_tensors: true\nuse_mlock: true\n")
    cfg = load_yaml(str(y))
    assert cfg.check_tensors is True and "use_mlock" in cfg.ignored and ServerConfig().check_tensors is False
