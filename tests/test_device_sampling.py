"""Sampling on the device (ops.sample_topk + the engine's "sample" mode), on the CPU reference ops.

The CUDA kernel implements the same arithmetic; its numerics test compares it with this reference on the GPU."""
import math

import numpy as np
import pytest
import torch

from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.ops import reference as ref
from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
from jittorinfer_b200.runtime.sampling import HostSampler, SamplingParams, device_samplable


def _expected(v, temp, top_k, top_p, min_p):
    """Probabilities of the chain top_k -> top_p -> min_p -> temperature over candidates sorted descending (float64)."""
    k = len(v)
    kk = min(k, top_k) if top_k > 0 else k
    e = np.exp(v[:kk] - v[0])
    before = (np.cumsum(e) - e) / e.sum()
    keep = np.ones(kk, dtype=bool)
    if top_p < 1:
        keep &= before < top_p
    if min_p > 0:
        keep &= v[:kk] >= v[0] + math.log(min_p)
    keep[0] = True
    n = int(np.argmin(keep)) if not keep.all() else kk
    w = np.exp((v[:n] - v[0]) / temp)
    return w / w.sum()


@pytest.mark.parametrize("temp,top_k,top_p,min_p", [(0.8, 40, 0.95, 0.05), (1.5, 0, 1.0, 0.0), (0.5, 8, 0.6, 0.0), (1.0, 0, 1.0, 0.2)])
def test_draws_follow_the_truncated_tempered_distribution(temp, top_k, top_p, min_p):
    g = torch.Generator().manual_seed(5)
    k, n = 64, 40000
    v = torch.sort(torch.randn(k, generator=g) * 2.0, descending=True).values
    ids = torch.randperm(5000, generator=g)[:k].int()
    u = torch.rand(n, generator=g)
    params = torch.tensor([temp, top_k, top_p, min_p, 0.0]).repeat(n, 1)
    params[:, 4] = u
    out = ref.sample_topk(v[None].expand(n, k).contiguous(), ids[None].expand(n, k).contiguous(), params)
    want = _expected(v.double().numpy(), temp, top_k, top_p, min_p)
    pos = {int(t): i for i, t in enumerate(ids.tolist())}
    counts = np.bincount([pos[int(t)] for t in out.tolist()], minlength=k)
    assert counts[len(want):].sum() == 0                                  # nothing outside the kept prefix
    freq = counts[:len(want)] / n
    assert np.abs(freq - want).max() < 4 * np.sqrt(want.max() / n) + 1e-3
    # greedy rows and u at the edges
    edge = torch.tensor([[0.0, 40, 0.9, 0.0, 0.7], [temp, top_k, top_p, min_p, 0.0], [temp, top_k, top_p, min_p, 0.999999]])
    o = ref.sample_topk(v[None].expand(3, k).contiguous(), ids[None].expand(3, k).contiguous(), edge)
    assert int(o[0]) == int(ids[0]) and int(o[1]) == int(ids[0]) and pos[int(o[2])] == len(want) - 1


def test_same_distribution_as_the_host_chain():
    """The numpy chain (HostSampler) and the device form agree on which candidates survive and on their probabilities."""
    g = torch.Generator().manual_seed(9)
    v = torch.sort(torch.randn(64, generator=g) * 2.5, descending=True).values.double().numpy()
    ids = np.arange(100, 164)
    p = SamplingParams(temperature=0.9, top_k=20, top_p=0.8, min_p=0.02, seed=1)
    hs = HostSampler(p)
    n = 20000
    host = np.bincount([hs.sample(v, ids) - 100 for _ in range(n)], minlength=64) / n
    want = _expected(v, 0.9, 20, 0.8, 0.02)
    assert (host[len(want):] == 0).all() and np.abs(host[:len(want)] - want).max() < 0.015


def _engine(hp, w, **kw):
    return LLMEngine(DeepSeek2Model(hp, w.items(), dtype=torch.float32),
                     EngineConfig(n_ctx=2048, n_batch=64, n_parallel=4, n_ctx_slot=256, device_sampling=True, **kw))


def test_engine_device_sampling_is_seeded_and_independent_of_run_ahead():
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (12, 40, 7)]
    sp = [SamplingParams(temperature=1.1, top_k=30, top_p=0.9, min_p=0.01, seed=10 + i, ignore_eos=True, max_tokens=14 - 3 * i)
          for i in range(3)]
    assert all(device_samplable(p) for p in sp) and not device_samplable(SamplingParams(temperature=0.8, repeat_penalty=1.1))

    def run(**kw):
        eng = _engine(hp, w, **kw)
        ids = [eng.add_request(p, s) for p, s in zip(prompts, sp)]
        greedy = eng.add_request(prompts[0], SamplingParams(ignore_eos=True, max_tokens=9))
        while eng.has_work():
            eng.step()
        assert all(eng.requests[i].dev is not None and eng.requests[i].sampler is None for i in ids)
        return [eng.requests[i].output for i in ids], eng.requests[greedy].output, eng

    a, ga, e1 = run()
    b, gb, e2 = run(run_ahead=True)
    assert a == b and ga == gb and [len(o) for o in a] == [14, 11, 8]
    assert e2.stats.get("run_ahead_steps", 0) >= 5                       # sampled requests run ahead too
    from jittorinfer_b200.models.oracle import OracleModel
    assert ga == OracleModel(hp, w).generate(prompts[0], 9)              # the greedy neighbour is untouched
    assert any(x != y for x, y in zip(a[0], OracleModel(hp, w).generate(prompts[0], 14)))      # and sampling does sample
    # another seed, another text; the same seed, the same text
    eng = _engine(hp, w)
    r1 = eng.generate([prompts[0]], SamplingParams(temperature=1.1, top_k=30, top_p=0.9, min_p=0.01, seed=10, ignore_eos=True), max_new_tokens=14)
    r2 = eng.generate([prompts[0]], SamplingParams(temperature=1.1, top_k=30, top_p=0.9, min_p=0.01, seed=99, ignore_eos=True), max_new_tokens=14)
    assert r1[0] == a[0] and r2[0] != r1[0]


def test_device_sampled_request_next_to_a_host_chain_request():
    """A request that needs the host chain (repeat penalty) turns the step into a candidates-to-host step; the
    device-samplable neighbour then draws on the host with the same arithmetic and the same random stream."""
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    g = torch.Generator().manual_seed(4)
    p1, p2 = (torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (15, 22))
    s_dev = SamplingParams(temperature=0.9, top_k=25, top_p=0.95, min_p=0.0, seed=5, ignore_eos=True, max_tokens=12)
    alone = _engine(hp, w).generate([p1], s_dev)[0]
    eng = _engine(hp, w)
    a = eng.add_request(p1, s_dev)
    b = eng.add_request(p2, SamplingParams(temperature=0.7, repeat_penalty=1.2, seed=8, ignore_eos=True, max_tokens=12))
    while eng.has_work():
        eng.step()
    assert eng.requests[b].sampler is not None and len(eng.requests[b].output) == 12
    assert eng.requests[a].output == alone


def test_unseeded_sampled_requests_get_the_same_seed_on_every_sharded_rank():
    """Tensor/expert-parallel ranks sample independently over identical logits: without a request seed the engine derives
    one from the request id, which advances alike on all ranks -- two engines standing in for two ranks draw the same
    tokens; an unsharded engine leaves the seed to chance."""
    import types
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    prompt = list(range(5, 25))
    outs = []
    for _ in range(2):
        eng = _engine(hp, w)
        eng.model.spec = types.SimpleNamespace(sharded=True, dp_attention=False, tp_size=2, tp_rank=0, expert_parallel=True)
        rid = eng.add_request(prompt, SamplingParams(temperature=1.3, top_k=50, ignore_eos=True, max_tokens=10))
        assert eng.requests[rid].params.seed is not None
        while eng.has_work():
            eng.step()
        outs.append(eng.requests[rid].output)
    assert outs[0] == outs[1] and len(outs[0]) == 10
    plain = _engine(hp, w)
    rid = plain.add_request(prompt, SamplingParams(temperature=1.3, ignore_eos=True, max_tokens=2))
    assert plain.requests[rid].params.seed is None
