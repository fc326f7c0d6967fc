"""fp32 oracle self-consistency and the module graph + engine against it (CPU)."""
import pytest
import torch

from jittorinfer_b200.models.deepseek2 import DeepSeek2Model, ForwardBatch
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.oracle import OracleModel, gate_topk
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
from jittorinfer_b200.runtime.sampling import SamplingParams


def _batch(toks, n_past, bs=64, first_block=1):
    T = len(toks)
    S = n_past + T
    nb = (S + bs - 1) // bs
    bt = torch.arange(first_block, first_block + nb).int()[None]
    pos = torch.arange(n_past, S).int()
    slots = (bt[0][(pos // bs).long()] * bs + pos % bs).int()
    return ForwardBatch(tokens=torch.tensor(toks).int(), positions=pos, slot_mapping=slots, block_tables=bt,
                        seq_lens=torch.tensor([S]).int(), q_start=torch.tensor([0, T]).int(),
                        out_rows=torch.arange(T).int(), max_q_len=T)


def test_absorbed_equals_naive():
    for name in ("tiny", "tiny-v2"):
        hp = preset(name)
        w = random_weights(hp, seed=0)
        toks = torch.randint(0, hp.n_vocab, (20,), generator=torch.Generator().manual_seed(1))
        a = OracleModel(hp, w, absorbed=True).forward(toks)
        b = OracleModel(hp, w, absorbed=False).forward(toks)
        assert (a - b).abs().max() < 1e-4


def test_model_matches_oracle_prefill_and_decode():
    for name in ("tiny", "tiny-v2"):
        hp = preset(name)
        w = random_weights(hp, seed=0)
        o = OracleModel(hp, w)
        m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
        cache = torch.zeros(hp.n_layer, 6 * 64, hp.kv_row)
        toks = torch.randint(0, hp.n_vocab, (70,), generator=torch.Generator().manual_seed(2)).tolist()
        assert (m.forward(_batch(toks, 0), cache) - o.forward(torch.tensor(toks))).abs().max() < 1e-4
        assert (m.forward(_batch([5, 9], 70), cache) - o.forward(torch.tensor([5, 9]))).abs().max() < 1e-4


def test_group_limited_routing_restricts_groups():
    hp = preset("tiny-v2")
    logits = torch.randn(50, hp.n_expert, generator=torch.Generator().manual_seed(3))
    ids, w = gate_topk(hp, logits)
    groups = ids // (hp.n_expert // hp.n_group)
    assert all(len(set(g.tolist())) <= hp.topk_group for g in groups)
    assert torch.all(w > 0)


def test_engine_greedy_matches_oracle_token_by_token():
    """32 random prompt ids, 32 greedy tokens, continuous batching + chunked prefill on."""
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=2048, n_batch=48, n_parallel=4))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (32, 70, 5, 100, 17)]
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=32)
    o = OracleModel(hp, w)
    for p, out in zip(prompts, outs):
        assert out == o.generate(p, 32)
    assert eng.kv.check()
    assert eng.sched.stats()["finished"] == 5


def test_engine_sampling_modes_run():
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    eng = LLMEngine(DeepSeek2Model(hp, w.items(), dtype=torch.float32), EngineConfig(n_ctx=1024, n_batch=64, n_parallel=2))
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, min_p=0.02, repeat_penalty=1.1, seed=3, max_tokens=12, ignore_eos=True)
    a = eng.generate([[1, 2, 3, 4]], sp)
    b = eng.generate([[1, 2, 3, 4]], sp)
    assert a == b and len(a[0]) == 12          # same seed -> same tokens
    c = eng.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.8, seed=4, max_tokens=12, ignore_eos=True))
    assert len(c[0]) == 12


def test_layer_split_matches_oracle():
    """Layer ranges on different devices (two spellings of the CPU stand in for two GPUs): per-device cache tensors,
    per-device copies of the step inputs, activations hopping between ranges."""
    from jittorinfer_b200.models.deepseek2 import assign_layers
    assert assign_layers(4, ["a", "b"]) == ["a", "a", "b", "b"]
    assert assign_layers(5, ["a", "b"], [3, 1]) == ["a", "a", "a", "a", "b"]
    assert assign_layers(3, ["a", "b", "c"], None) == ["a", "b", "c"]
    hp = preset("tiny-v2")
    w = random_weights(hp, seed=0)
    devs = assign_layers(hp.n_layer, [torch.device("cpu"), torch.device("cpu", 0)])
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32, layer_devices=devs)
    assert m.split and len({str(d) for d in m.layer_dev}) == 2
    eng = LLMEngine(m, EngineConfig(n_ctx=1024, n_batch=32, n_parallel=2))
    assert len(eng.kv_cache.by_dev) == 2
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (50, 9)]
    ref = [OracleModel(hp, w).generate(p, 8) for p in prompts]
    assert eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=8) == ref


def test_yarn_rope_nmse_on_the_reference_cases():
    """The reference's only op-level check with a threshold (tests/ops/test_ops_speed.cpp:1125-1178, NMSE <= 1e-7 at
    :361): YaRN RoPE with the DeepSeek-V2 decode parameters -- n_dims 64, adjacent pairs, n_ctx_orig 4096, freq_scale
    1/40, ext_factor 1, attn_factor 1/(1 + 0.1 ln 40) -- on shapes {64,1,16}, {64,16,16}, {64,16,64}, {64,16,128}
    (head dim, heads, tokens).  Here the table-driven rotation is compared with a scalar float64 restatement of the
    per-element formula (theta_extrap = pos * base^(-2i/d), ramp mix with the correction range, magnitude scale)."""
    import math
    from jittorinfer_b200.ops import reference as ref
    hp = preset("lite")
    n_dims, base, n_orig, fs, ext = 64, hp.rope_freq_base, 4096, 0.025, 1.0
    attn = 1.0 / (1.0 + 0.1 * math.log(40.0))
    assert abs(attn - 0.730520) < 1e-6

    def corr_dim(n_rot):
        return n_dims * math.log(n_orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))
    lo, hi = max(0.0, math.floor(corr_dim(32.0))), min(n_dims - 1.0, math.ceil(corr_dim(1.0)))
    assert (lo, hi) == tuple(hp.yarn_corr_dims())
    for heads, tokens in ((1, 16), (16, 16), (16, 64), (16, 128)):
        g = torch.Generator().manual_seed(heads * 1000 + tokens)
        x = torch.randn(tokens, heads, n_dims, generator=g, dtype=torch.float64)
        pos = torch.randint(0, 8192, (tokens,), generator=g)
        table = ref.yarn_table(8192, n_dims, base, fs, ext, attn, lo, hi)
        got = ref._rope(x.float(), table[pos]).double()
        want = torch.empty_like(x)
        mscale = attn * (1.0 + 0.1 * math.log(1.0 / fs))
        for t in range(tokens):
            for i in range(n_dims // 2):
                te = float(pos[t]) * base ** (-2.0 * i / n_dims)
                ramp = 1.0 - min(1.0, max(0.0, (i - lo) / max(0.001, hi - lo)))
                theta = fs * te * (1.0 - ramp * ext) + te * ramp * ext
                c, s = math.cos(theta) * mscale, math.sin(theta) * mscale
                x0, x1 = x[t, :, 2 * i], x[t, :, 2 * i + 1]
                want[t, :, 2 * i], want[t, :, 2 * i + 1] = x0 * c - x1 * s, x0 * s + x1 * c
        nmse = float(((got - want) ** 2).sum() / (want ** 2).sum())
        assert nmse <= 1e-7, (heads, tokens, nmse)


def test_v3_shaped_paths_match_oracle(tmp_path):
    """Sigmoid gating with a selection bias, renormalised weights, group-limited routing and two leading dense layers
    (the DeepSeek-V3-shaped branch of the architecture): module graph and engine against the oracle, also through a GGUF
    round trip (the bias tensors switch the branch on)."""
    from jittorinfer_b200.models.weights import write_random_gguf
    from jittorinfer_b200.runtime.factory import build_engine
    hp = preset("tiny-v3")
    assert hp.router_bias and preset("v3").n_expert == 256
    w = random_weights(hp, seed=0, std=0.05)
    assert "blk.2.exp_probs_b.bias" in w and "blk.1.exp_probs_b.bias" not in w
    o = OracleModel(hp, w)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    cache = torch.zeros(hp.n_layer, 4 * 64, hp.kv_row)
    toks = torch.randint(0, hp.n_vocab, (40,), generator=torch.Generator().manual_seed(7)).tolist()
    assert (m.forward(_batch(toks, 0), cache) - o.forward(torch.tensor(toks))).abs().max() < 1e-4
    p = str(tmp_path / "v3.gguf")
    write_random_gguf(p, hp, seed=0, std=0.05)
    eng = build_engine(None, gguf_path=p, device="cpu", dtype=torch.float32, n_parallel=2, n_ctx_slot=256, n_batch=32)
    assert eng.hp.router_bias and eng.hp.expert_gating_func == "sigmoid" and eng.hp.n_layer_dense_lead == 2
    assert eng.generate([toks], SamplingParams(ignore_eos=True), max_new_tokens=8) == [OracleModel(hp, w).generate(toks, 8)]


def test_tensor_hook_sees_every_block_output():
    hp = preset("tiny-v2")
    w = random_weights(hp, seed=0)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    seen = {}
    m.tensor_hook = lambda name, t: seen.__setitem__(name, tuple(t.shape))
    cache = torch.zeros(hp.n_layer, 2 * 64, hp.kv_row)
    logits = m.forward(_batch([1, 2, 3, 4, 5], 0), cache)
    names = [f"blk.{il}.{k}" for il in range(hp.n_layer) for k in ("attn_out", "ffn_inp", "ffn_out")] + ["result_norm", "result_output"]
    assert list(seen) == names
    assert seen["blk.0.ffn_out"] == (5, hp.n_embd) and seen["result_output"] == tuple(logits.shape)
    m.tensor_hook = None
    assert torch.equal(m.forward(_batch([1, 2, 3, 4, 5], 0), cache), logits)


def test_engine_under_kv_pressure_preempts_and_still_matches_oracle():
    """More requests than the cache can hold at once, with defragmentation on: sequences are preempted (youngest first),
    recomputed later, blocks are compacted -- and every request still produces exactly the oracle's tokens."""
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    # 10 blocks of 64 tokens for 6 slots of up to 256 tokens: at most two or three long sequences fit together
    eng = LLMEngine(m, EngineConfig(n_ctx=640, n_batch=96, n_parallel=6, n_ctx_slot=256, defrag_thold=0.05))
    g = torch.Generator().manual_seed(11)
    lens = (150, 90, 170, 40, 120, 60, 200, 30)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in lens]
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=24)
    o = OracleModel(hp, w)
    assert outs == [o.generate(p, 24) for p in prompts]
    st = eng.sched.stats()
    assert st["preemptions"] >= 1 and st["finished"] == len(prompts)
    assert eng.kv.check() and eng.kv.used_blocks <= eng.kv.n_blocks


def test_poisoned_free_blocks_never_reach_the_logits(monkeypatch):
    """JITTORINFER_KV_POISON=1: blocks are filled with NaN when their last reference goes away and every step's logits are
    checked.  Preemption, recomputation, shared prefixes, cancellation and defragmentation must still give the oracle's
    tokens; a block table that names a freed block (made by hand here) must be caught."""
    monkeypatch.setenv("JITTORINFER_KV_POISON", "1")
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=640, n_batch=96, n_parallel=6, n_ctx_slot=256, defrag_thold=0.05))
    g = torch.Generator().manual_seed(12)
    shared = torch.randint(0, hp.n_vocab, (70,), generator=g).tolist()                     # a prefix that several requests share
    lens = (150, 90, 40, 120, 60, 30)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in lens] + [shared + [5, 6], shared + [7]]
    victim = eng.add_request(torch.randint(0, hp.n_vocab, (100,), generator=g).tolist(), SamplingParams(ignore_eos=True, max_tokens=50))
    eng.step()
    eng.cancel(victim)                                                                      # frees blocks in mid-flight
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=20)
    o = OracleModel(hp, w)
    assert outs == [o.generate(p, 20) for p in prompts]
    assert eng.stats["poisoned_blocks"] > 0 and eng.kv.check()
    assert eng.sched.stats()["preemptions"] >= 1

    # negative control: a sequence whose table points at a freed (poisoned) block
    rid = eng.add_request(prompts[0][:80], SamplingParams(ignore_eos=True, max_tokens=8))
    eng.step()
    free_poisoned = [b for b in range(eng.kv.n_blocks) if eng.kv.refcount(b) == 0]
    assert free_poisoned
    eng.kv_cache[:, free_poisoned[0] * 64:(free_poisoned[0] + 1) * 64] = float("nan")     # as the engine leaves a freed block
    real = eng.sched.step

    def stale(arrays):
        info = real(arrays)
        eng.io.h["block_tables"][0] = free_poisoned[0]              # first block of the first scheduled sequence
        return info
    eng.sched.step = stale
    with pytest.raises(RuntimeError, match="poisoned"):
        eng.step()
    eng.sched.step = real
    eng.cancel(rid)


def test_expected_active_experts_hint():
    """Split-K hint of the grouped GEMMs: expected distinct local experts under uniform routing (merged shared experts
    always count)."""
    from jittorinfer_b200.ops.native import expected_active_experts as f
    assert f(8, 6, 20, 160) == 6            # V2, 8 ranks, 8 tokens: 20 * (1 - (1 - 6/160)^8) = 5.3
    assert f(8, 8, 66, 64) == 37            # Lite with the two shared experts merged: 2 + 64 * (1 - (1 - 6/64)^8) = 36.9
    assert f(1, 8, 66, 64) == 8 and f(1, 6, 160, 160) == 6
    assert f(2048, 6, 20, 160) == 20 and f(64, 6, 20, 160) == 19


def _run_ahead_engine(hp, w, **kw):
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    return LLMEngine(m, EngineConfig(n_ctx=2048, n_batch=64, n_parallel=4, n_ctx_slot=256, run_ahead=True, **kw))


def test_run_ahead_decoding_matches_the_oracle():
    """The engine launches decode step k + 1 before it has read the ids of step k (greedy requests): same tokens as the
    oracle for requests of different lengths (they leave the batch at different steps), with a request that joins in
    mid-stream, one that is cancelled while a step is in flight, and an end-of-sequence stop."""
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    o = OracleModel(hp, w)
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (9, 33, 70, 5)]
    news = (20, 7, 13, 1)
    eng = _run_ahead_engine(hp, w)
    ids = [eng.add_request(p, SamplingParams(ignore_eos=True, max_tokens=n)) for p, n in zip(prompts, news)]
    late = None
    victim = eng.add_request(prompts[0][:6], SamplingParams(ignore_eos=True, max_tokens=40))      # waits for a free slot
    n_calls = 0
    while eng.has_work():
        eng.step()
        n_calls += 1
        if n_calls == 6:
            late = eng.add_request(prompts[1][:12], SamplingParams(ignore_eos=True, max_tokens=9))
        if n_calls == 14:
            eng.cancel(victim)
        assert n_calls < 400
    for rid, p, n in zip(ids, prompts, news):
        assert eng.requests[rid].output == o.generate(p, n), (rid, n)
        assert eng.requests[rid].finish_reason == "length"
    assert eng.requests[late].output == o.generate(prompts[1][:12], 9)
    v = eng.requests[victim]
    assert v.finish_reason == "cancelled" and v.output == o.generate(prompts[0][:6], 40)[:len(v.output)]
    assert eng.stats.get("run_ahead_steps", 0) >= 10 and eng.kv.check()

    # end of sequence: declare a token that the model is known to produce mid-way the end-of-sequence token
    ref = o.generate(prompts[2], 13)
    eos = ref[6]
    stop_at = ref.index(eos)
    hp2 = hp.replace(eos_id=eos)
    eng2 = _run_ahead_engine(hp2, w)
    a = eng2.add_request(prompts[2], SamplingParams(max_tokens=13))
    b = eng2.add_request(prompts[0], SamplingParams(ignore_eos=True, max_tokens=20))
    while eng2.has_work():
        eng2.step()
    assert eng2.requests[a].output == ref[:stop_at + 1] and eng2.requests[a].finish_reason == "stop"
    assert eng2.requests[b].output == o.generate(prompts[0], 20)
    # the slot that ended early can be reused with its cached prefix
    c = eng2.add_request(prompts[2], SamplingParams(ignore_eos=True, max_tokens=5))
    while eng2.has_work():
        eng2.step()
    assert eng2.requests[c].output == ref[:5] and eng2.kv.check()
    # the synchronous engine gives the same events, one step earlier
    eng3 = LLMEngine(DeepSeek2Model(hp, w.items(), dtype=torch.float32), EngineConfig(n_ctx=2048, n_batch=64, n_parallel=4, n_ctx_slot=256))
    assert eng3.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=6) == \
        _run_ahead_engine(hp, w).generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=6)


def test_run_ahead_under_kv_pressure_and_with_a_host_sampler(tmp_path, monkeypatch):
    """Scarce blocks (preemption possible) and a request whose sampler runs on the host both make the engine read the ids
    before it plans the next step; outputs stay those of the oracle, and the step trace covers the run-ahead calls."""
    from jittorinfer_b200.utils.trace import Tracer
    monkeypatch.setenv("JITTORINFER_TRACE", str(tmp_path / "t.jsonl"))
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    o = OracleModel(hp, w)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=640, n_batch=96, n_parallel=6, n_ctx_slot=256, defrag_thold=0.05, run_ahead=True))
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (150, 90, 170, 40, 120, 60, 200, 30)]
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=24)
    assert outs == [o.generate(p, 24) for p in prompts]
    assert eng.sched.stats()["preemptions"] >= 1 and eng.kv.check()
    # a sampled (non-greedy) request next to a greedy one: the greedy one is unaffected
    a = eng.add_request(prompts[3], SamplingParams(ignore_eos=True, max_tokens=10))
    b = eng.add_request(prompts[5], SamplingParams(ignore_eos=True, max_tokens=10, temperature=0.9, seed=3))
    while eng.has_work():
        eng.step()
    assert eng.requests[a].output == o.generate(prompts[3], 10) and len(eng.requests[b].output) == 10
    ahead_before = eng.stats.get("run_ahead_steps", 0)
    assert eng.generate(prompts[3:5], SamplingParams(ignore_eos=True), max_new_tokens=12) == [o.generate(p, 12) for p in prompts[3:5]]
    assert eng.stats["run_ahead_steps"] >= ahead_before + 8          # with room in the cache the engine runs ahead again
    eng.tracer.close()
    recs = Tracer.read(str(tmp_path / "t.jsonl"))
    steps = [r for r in recs if r["kind"] == "step"]
    assert len(steps) == eng.stats["steps"] and any(r["mode"] == "ahead" for r in steps)
    assert sum(r["finished"] for r in recs if r["kind"] in ("step", "collect")) == len(prompts) + 4


def test_prefix_blocks_are_shared_across_slots(monkeypatch):
    """Requests whose prompts start like the tokens another slot already holds (a common system prompt) start from that
    slot's full blocks by reference: fewer prompt tokens are evaluated, the outputs are still the oracle's, also while the
    donor keeps generating and after it has gone; poisoning of freed blocks is on to catch any use of a released block."""
    monkeypatch.setenv("JITTORINFER_KV_POISON", "1")
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    o = OracleModel(hp, w)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=4096, n_batch=256, n_parallel=4, n_ctx_slot=512))
    g = torch.Generator().manual_seed(31)
    system = torch.randint(0, hp.n_vocab, (150,), generator=g).tolist()          # two full blocks + 22 tokens
    tails = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (9, 17, 30)]
    first = eng.add_request(system + tails[0], SamplingParams(ignore_eos=True, max_tokens=30))
    eng.step()                                                                   # the donor's prompt is in the cache now
    before = eng.sched.stats()["prompt_tokens"]
    second = eng.add_request(system + tails[1], SamplingParams(ignore_eos=True, max_tokens=12))
    third = eng.add_request(system[:140] + tails[2], SamplingParams(ignore_eos=True, max_tokens=12))
    while eng.has_work():
        eng.step()
    st = eng.sched.stats()
    assert st["prefix_shared"] == 2
    assert st["prompt_tokens"] - before == (150 + 17 - 128) + (140 + 30 - 128)   # only what lies beyond the shared blocks
    assert eng.requests[first].output == o.generate(system + tails[0], 30)
    assert eng.requests[second].output == o.generate(system + tails[1], 12)
    assert eng.requests[third].output == o.generate(system[:140] + tails[2], 12)
    assert eng.kv.check()
    # the donor's slot is reused by an unrelated prompt (its blocks lose one reference each); a sharer's cache still serves
    other = torch.randint(0, hp.n_vocab, (200,), generator=g).tolist()
    outs = eng.generate([other, other[:50], system + tails[1] + [1, 2, 3]], SamplingParams(ignore_eos=True), max_new_tokens=8)
    assert outs == [o.generate(p, 8) for p in (other, other[:50], system + tails[1] + [1, 2, 3])]
    assert eng.kv.check() and eng.stats["poisoned_blocks"] >= 0


@pytest.mark.parametrize("seed", range(6))
def test_random_serving_scenarios_match_the_oracle(seed, monkeypatch):
    """Seeded random scenarios -- slots, cache size (some small enough to preempt), prompts that share prefixes, token
    limits, arrivals spread over steps, run-ahead on or freed-block poisoning on: every request's tokens are the oracle's."""
    import random
    rng = random.Random(seed)
    run_ahead = seed % 2 == 0
    if not run_ahead:
        monkeypatch.setenv("JITTORINFER_KV_POISON", "1")
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    o = OracleModel(hp, w)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    n_slots = rng.choice([2, 3, 4])
    eng = LLMEngine(m, EngineConfig(n_ctx=rng.choice([512, 768, 2048]), n_batch=rng.choice([48, 128]), n_parallel=n_slots, n_ctx_slot=320,
                                    defrag_thold=rng.choice([-1.0, 0.05]), run_ahead=run_ahead))
    base = [rng.randrange(hp.n_vocab) for _ in range(200)]
    reqs = []
    for _ in range(rng.randint(4, 7)):
        if rng.random() < 0.5:
            prompt = base[:rng.choice([64, 130, 190])] + [rng.randrange(hp.n_vocab) for _ in range(rng.randint(1, 30))]
        else:
            prompt = [rng.randrange(hp.n_vocab) for _ in range(rng.randint(1, 150))]
        reqs.append((rng.randint(0, 10), prompt, rng.randint(1, 18)))
    ids, step = {}, 0
    while step < 12 or eng.has_work():
        for i, (when, prompt, n_new) in enumerate(reqs):
            if when == step:
                ids[i] = eng.add_request(prompt, SamplingParams(ignore_eos=True, max_tokens=n_new))
        eng.step()
        step += 1
        assert step < 2000
    for i, (_, prompt, n_new) in enumerate(reqs):
        st = eng.requests[ids[i]]
        assert st.output == o.generate(prompt, n_new), (seed, i)
        assert st.finish_reason == "length"
    assert eng.kv.check()


def test_logprobs_of_generated_tokens_match_the_oracle():
    """params.logprobs: per generated token its log-probability and the most likely alternatives, from the device top-k
    and the row's log-normaliser; compared with log_softmax of the oracle's logits."""
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    o = OracleModel(hp, w)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=1024, n_batch=64, n_parallel=2, n_ctx_slot=256, run_ahead=True))
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, hp.n_vocab, (19,), generator=g).tolist()
    a = eng.add_request(prompt, SamplingParams(ignore_eos=True, max_tokens=6, logprobs=True, top_logprobs=3))
    b = eng.add_request(prompt[:7], SamplingParams(ignore_eos=True, max_tokens=6))                  # a neighbour without
    while eng.has_work():
        eng.step()
    st = eng.requests[a]
    assert st.output == o.generate(prompt, 6) and eng.requests[b].logprobs == [] and len(st.logprobs) == 6
    o.reset()
    seq = list(prompt)
    for n, (tok, lp, alts) in enumerate(st.logprobs):
        o.reset()
        ref = torch.log_softmax(o.forward(torch.tensor(seq))[-1].double(), -1)
        assert tok == st.output[n] == int(ref.argmax())
        assert abs(lp - float(ref[tok])) < 1e-4
        top = torch.topk(ref, 3)
        assert [t for t, _ in alts] == top.indices.tolist()
        assert all(abs(x - float(y)) < 1e-4 for (_, x), y in zip(alts, top.values))
        seq.append(tok)
