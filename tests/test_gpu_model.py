"""Native bf16 model + engine on the GPU vs the fp32 oracle and vs the PyTorch-op baseline."""
import pytest
import torch

from jittorinfer_b200 import ops
from jittorinfer_b200.models.deepseek2 import DeepSeek2Model, ForwardBatch
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.oracle import OracleModel
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
from jittorinfer_b200.runtime.sampling import SamplingParams

pytestmark = pytest.mark.gpu


def _batch(toks, n_past, dev, bs=64):
    T = len(toks)
    S = n_past + T
    nb = (S + bs - 1) // bs
    bt = torch.arange(1, 1 + nb).int()[None]
    pos = torch.arange(n_past, S).int()
    slots = (bt[0][(pos // bs).long()] * bs + pos % bs).int()
    return ForwardBatch(tokens=torch.tensor(toks).int().to(dev), positions=pos.to(dev), slot_mapping=slots.to(dev),
                        block_tables=bt.to(dev), seq_lens=torch.tensor([S]).int().to(dev),
                        q_start=torch.tensor([0, T]).int().to(dev), out_rows=torch.arange(T).int().to(dev), max_q_len=T,
                        attn_meta={"total_kv": S, "n_q_tiles": (T + 127) // 128})


def rows_close(a, b, scale, frac=0.8):
    """bf16 activations can flip a near-tie in expert routing for a few tokens; all other rows must be tight."""
    err = (a - b).abs().amax(dim=-1)
    ok = (err < 0.06 * scale).float().mean().item()
    assert ok >= frac, f"only {ok:.2f} of rows within tolerance; worst {err.max().item():.3f} vs scale {scale:.3f}"


@pytest.mark.parametrize("name", ["tiny", "tiny-v2"])
def test_native_logits_match_oracle(name):
    hp = preset(name)
    w = random_weights(hp, seed=0, std=0.05)
    wq = {k: v.bfloat16().float() for k, v in w.items()}        # oracle sees the same bf16-rounded weights
    o = OracleModel(hp, wq)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(hp.n_layer, 6 * 64, hp.kv_row, dtype=torch.bfloat16, device="cuda")
    toks = torch.randint(0, hp.n_vocab, (70,), generator=torch.Generator().manual_seed(2)).tolist()
    l_ref = o.forward(torch.tensor(toks))
    l_nat = m.forward(_batch(toks, 0, "cuda"), cache).cpu()
    ops.nat().check_status()
    scale = l_ref.abs().max().item()
    rows_close(l_nat, l_ref, scale)
    nxt = [5, 9, 700, 31, 2, 64]                 # a second chunk on top of the cached prefix
    l_ref2 = o.forward(torch.tensor(nxt))
    l_nat2 = m.forward(_batch(nxt, 70, "cuda"), cache).cpu()
    rows_close(l_nat2, l_ref2, scale, frac=0.6)
    # the PyTorch-op baseline on the same device agrees as well
    ops.set_force_torch(True)
    try:
        cache2 = torch.zeros_like(cache)
        l_t = m.forward(_batch(toks, 0, "cuda"), cache2).cpu()
    finally:
        ops.set_force_torch(False)
    rows_close(l_t, l_ref, scale)


def test_engine_cuda_graphs_equal_eager_and_track_oracle():
    hp = preset("tiny")
    w = random_weights(hp, seed=0, std=0.05)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16, device="cuda")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (32, 70, 5)]
    outs = {}
    for graphs in (True, False):
        eng = LLMEngine(m, EngineConfig(n_ctx=2048, n_batch=48, n_parallel=4, cuda_graphs=graphs, graph_buckets=(1, 2, 4)))
        outs[graphs] = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=24)
        if graphs:
            assert eng.stats["graph_steps"] > 20 and eng.launches > 0
    ops.nat().check_status()
    assert outs[True] == outs[False]
    o = OracleModel(hp, {k: v.bfloat16().float() for k, v in w.items()})
    agree = sum(a == b for p, out in zip(prompts, outs[True]) for a, b in zip(out, o.generate(p, 24)))
    assert agree >= 36      # bf16 vs fp32: greedy paths may split late, never early


def _row_rel_err(a, b):
    """Per row: largest logit error relative to the row's largest reference logit."""
    return ((a - b).abs().amax(dim=-1) / b.abs().amax(dim=-1).clamp_min(1e-6))


@pytest.mark.parametrize("name", ["lite-2l", "v2-2l"])
def test_real_shapes_logits_match_oracle_and_take_the_tensor_core_paths(name):
    """DeepSeek-V2-Lite / DeepSeek-V2 layer shapes (the benchmarked kernels: tcgen05 flash-MLA over the 576-wide latent rows,
    K = 2048 / 5120 GEMMs, 64 / 160-expert gating, grouped expert GEMMs) against the fp32 oracle, on logits: a 70-token prompt
    chunk, a chunked continuation, then 8 sequences decoding under CUDA graphs.  Rows whose routing flipped on a near-tie
    (bf16 activations against fp32) may exceed the tolerance; they are counted and bounded separately."""
    hp = preset(name)
    w = random_weights(hp, seed=0, std=0.02)
    o = OracleModel(hp, {k: v.bfloat16().float() for k, v in w.items()})
    m = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16, device="cuda")
    nat = ops.nat()
    n0 = dict(nat.launches_by_name)
    cache = torch.zeros(hp.n_layer, 8 * 64, hp.kv_row, dtype=torch.bfloat16, device="cuda")
    toks = torch.randint(0, hp.n_vocab, (70,), generator=torch.Generator().manual_seed(2)).tolist()
    l_ref = o.forward(torch.tensor(toks))
    l_nat = m.forward(_batch(toks, 0, "cuda"), cache).float().cpu()
    nxt = torch.randint(0, hp.n_vocab, (9,), generator=torch.Generator().manual_seed(3)).tolist()
    l_ref2 = o.forward(torch.tensor(nxt))
    l_nat2 = m.forward(_batch(nxt, 70, "cuda"), cache).float().cpu()
    nat.check_status()
    err = torch.cat([_row_rel_err(l_nat, l_ref), _row_rel_err(l_nat2, l_ref2)])
    # bf16 activations through every GEMM of the stack put the typical row at ~1.3e-2 of its largest logit (measured);
    # 3e-2 bounds the ordinary rows, rows beyond it are the ones whose expert choice flipped on a near-tie
    # With 160 experts whose outputs are scaled by 16 (v2-2l) more rows sit on a routing near-tie and a flip moves a row
    # further: measured 0.91 of the rows within 3e-2, median 1.7e-2, worst 0.36.
    tol, frac, med = (3e-2, 0.95, 2e-2) if name == "lite-2l" else (4e-2, 0.88, 2.5e-2)
    tight = (err <= tol).float().mean().item()
    flipped = int((err > tol).sum())
    print(f"{name}: rows within {tol}: {tight:.3f}; median row error {err.median().item():.4f}; rows beyond (routing flips): {flipped}; "
          f"worst {err.max().item():.3f}")
    assert tight >= frac, f"{name}: only {tight:.3f} of rows within {tol} (worst {err.max().item():.3f})"
    assert err.median().item() <= med
    assert err.max().item() < 0.5                              # a flipped expert moves a row, it does not destroy it
    # arg-max agreement where the reference's margin is not a near-tie
    top2 = l_ref.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * l_ref.abs().amax(dim=-1)
    clear &= err[:l_ref.shape[0]] <= tol                                        # a row whose routing flipped may also change its arg-max
    assert bool((l_nat.argmax(-1)[clear] == l_ref.argmax(-1)[clear]).all())
    ran = {k: nat.launches_by_name.get(k, 0) - n0.get(k, 0) for k in ("mla_flash", "mha_prefill", "mla_attention", "gemm_grouped", "moe_gate")}
    # tcgen05 attention, not the SIMT fallback: the 70-token chunk in the per-head form, the 9-token one in the absorbed form
    assert ran["mha_prefill"] == hp.n_layer and ran["mla_flash"] == hp.n_layer and ran["mla_attention"] == 0, ran
    assert ran["gemm_grouped"] >= 4 and ran["moe_gate"] >= 2, ran
    # 8 sequences decoding under CUDA graphs: tokens against the oracle's greedy continuation
    eng = LLMEngine(m, EngineConfig(n_ctx=8 * 256, n_batch=256, n_parallel=8, graph_buckets=(1, 2, 4, 8)))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (70, 33, 8, 100, 64, 65, 17, 5)]
    n1 = nat.launches_by_name.get("mla_flash", 0)
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=6)
    nat.check_status()
    assert eng.stats["graph_steps"] >= 5 and nat.launches_by_name.get("mla_flash", 0) > n1
    ref = [o.generate(p, 6) for p in prompts[:3]]
    first = sum(int(a[0] == b[0]) for a, b in zip(outs, ref))
    agree = sum(int(x == y) for a, b in zip(outs, ref) for x, y in zip(a, b))
    print(f"{name}: {agree}/18 greedy tokens equal the oracle's over 3 sequences (first tokens: {first}/3)")
    # (v2-2l: a routing flip in a prompt's last row changes that sequence's continuation from its first token on)
    assert (first == 3 and agree >= 12) if name == "lite-2l" else (first >= 2 and agree >= 9)


def test_layer_split_over_two_gpus_equals_one_gpu():
    """Layer-split serving (consecutive layer ranges on consecutive GPUs of one process, activations hopping between them): the
    same tokens as the model on one GPU, eager steps on both devices (every kernel sets its per-device launch attributes)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    hp = preset("lite-2l")
    w = random_weights(hp, seed=0, std=0.02)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (40, 70, 9)]
    outs = []
    for devices in (None, [torch.device("cuda", 0), torch.device("cuda", 1), torch.device("cuda", 1)]):
        m = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16, device="cuda:0", layer_devices=devices)
        eng = LLMEngine(m, EngineConfig(n_ctx=2048, n_batch=64, n_parallel=4, graph_buckets=(1, 2, 4)))
        outs.append(eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=10))
        for d in range(2):
            torch.cuda.synchronize(d)
        ops.nat().check_status()
        del eng, m
    assert outs[0] == outs[1]


def test_quantised_file_expanded_on_the_device_serves_the_same_tokens(tmp_path, monkeypatch):
    """A Q4_K / Q8_0 file: blocks sent to the GPU and expanded there (the default) against blocks expanded on the host and
    uploaded as bf16.  Same bf16 weights either way, so the same tokens."""
    from jittorinfer_b200.gguf import format as F
    from jittorinfer_b200.models.weights import write_random_gguf
    from jittorinfer_b200.runtime.factory import build_engine
    hp = preset("tiny")
    path = str(tmp_path / "q.gguf")
    write_random_gguf(path, hp, seed=0, std=0.05, quant=F.GGML_Q4_K)
    prompts = [list(range(3, 40)), [7, 9, 400, 12]]
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("JITTORINFER_DEVICE_DEQUANT", flag)
        eng = build_engine(None, gguf_path=path, device="cuda", n_parallel=2, n_ctx_slot=128, graph_buckets=(1, 2))
        outs.append(eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=8))
        del eng
    assert outs[0] == outs[1], outs
