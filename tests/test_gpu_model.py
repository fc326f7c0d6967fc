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
                        q_start=torch.tensor([0, T]).int().to(dev), out_rows=torch.arange(T).int().to(dev), max_q_len=T)


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
