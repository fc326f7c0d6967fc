"""Expert parallelism with data-parallel attention: each rank decodes its own prompt, routed experts are reached
through the all-to-all dispatcher, and every rank must reproduce the single-rank oracle on its own tokens.

CPU: 2 gloo ranks, fp32, library all-to-all.  GPU (needs >= 2 devices): library all-to-all and the fused
peer-memory kernels, bf16.  One rank finishes early and keeps joining the collectives without tokens.
"""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPT_LENS = (20, 70, 33, 5)
N_NEW = (10, 6, 8, 3)            # ranks generate different numbers of tokens: the others keep stepping idle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompts(hp):
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in PROMPT_LENS]


def _worker(rank, world, port, backend, comm_impl, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), JITTORINFER_COMM=comm_impl, NCCL_NVLS_ENABLE="0")
    try:
        from jittorinfer_b200.models.deepseek2 import DeepSeek2Model, ForwardBatch
        from jittorinfer_b200.models.hparams import preset
        from jittorinfer_b200.models.weights import ShardSpec, iter_random
        from jittorinfer_b200.parallel.ep import make_ep_dispatcher
        gpu = backend == "nccl"
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        if gpu:
            torch.cuda.set_device(dev)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=dev)
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
        hp = preset("tiny-v2")
        spec = ShardSpec(rank, world, expert_parallel=True, dp_attention=True)
        n_moe = hp.n_layer - hp.n_layer_dense_lead
        ep = make_ep_dispatcher(dev, world, rank, hp.n_expert, hp.n_embd, hp.n_expert_used, n_moe, max_tokens=96)
        dtype = torch.bfloat16 if gpu else torch.float32
        model = DeepSeek2Model(hp, iter_random(hp, spec=spec, seed=0, std=0.05), dtype=dtype, device=dev, spec=spec, ep=ep)
        cache = torch.zeros(hp.n_layer, 4 * 64, hp.kv_row, dtype=dtype, device=dev)
        prompt, n_new = _prompts(hp)[rank], N_NEW[rank]
        steps = max(N_NEW[:world])

        def batch(toks, n_past):
            T = len(toks)
            S = n_past + T
            nb = (S + 63) // 64
            bt = torch.arange(1, 1 + nb, dtype=torch.int32)[None]
            pos = torch.arange(n_past, S, dtype=torch.int32)
            slots = (bt[0][(pos // 64).long()] * 64 + pos % 64).int()
            mk = lambda t: t.to(dev)
            return ForwardBatch(mk(torch.tensor(toks, dtype=torch.int32)), mk(pos), mk(slots), mk(bt), mk(torch.tensor([S], dtype=torch.int32)),
                                mk(torch.tensor([0, T], dtype=torch.int32)), mk(torch.tensor([T - 1], dtype=torch.int32)), max_q_len=T)

        out, n_past, toks = [], 0, prompt
        for step in range(steps):
            if len(out) < n_new:
                logits = model.forward(batch(toks, n_past), cache)
                n_past += len(toks)
                toks = [int(logits[0].argmax())]
                out.append(toks[0])
            else:
                model.forward(None, None)               # no tokens of my own: serve my experts to the others
        if gpu:
            torch.cuda.synchronize()
            from jittorinfer_b200.ops import native
            native.check_status()
        q.put((rank, out, ep.n_collectives, ep.fused))
        dist.barrier()
        ep.close()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "ERROR: " + traceback.format_exc(), 0, False))
        raise


def _engine_worker(rank, world, port, backend, comm_impl, q):
    """Every rank serves its own requests through its own scheduler; the engines step together."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), JITTORINFER_COMM=comm_impl, NCCL_NVLS_ENABLE="0")
    try:
        from jittorinfer_b200.models.hparams import preset
        from jittorinfer_b200.runtime.sampling import SamplingParams
        gpu = backend == "nccl"
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        if gpu:
            torch.cuda.set_device(dev)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=dev)
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
        hp = preset("tiny-v2")
        from jittorinfer_b200.runtime.factory import build_model
        from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
        model = build_model(hp, device=dev, dtype=torch.bfloat16 if gpu else torch.float32, world=world, rank=rank, std=0.05,
                            max_positions=256, dp_attention=True, ep_max_tokens=64, fast_random=False)
        eng = LLMEngine(model, EngineConfig(n_ctx=512, n_batch=48, n_parallel=2, graph_buckets=(1, 2), cuda_graphs=gpu))
        eng.warmup()
        prompts = _prompts(hp)
        mine = [prompts[i] for i in range(len(prompts)) if i % world == rank]          # rank 0: prompts 0, 2; rank 1: 1, 3
        news = [N_NEW[i] for i in range(len(prompts)) if i % world == rank]
        ids = [eng.add_request(p, SamplingParams(ignore_eos=True, max_tokens=n)) for p, n in zip(mine, news)]
        steps = eng.run_until_all_idle()
        outs = [eng.requests[i].output for i in ids]
        if gpu:
            torch.cuda.synchronize()
            from jittorinfer_b200.ops import native
            native.check_status()
        q.put((rank, outs, steps, eng.stats.get("idle_steps", 0), eng.stats["graph_steps"]))
        dist.barrier()
        model.ep.close()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "ERROR: " + traceback.format_exc(), 0, 0, 0))
        raise


def _run(world, backend, comm_impl, timeout=180, target=None):
    target = target or _worker
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, backend, comm_impl, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=timeout) for _ in range(world)]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():          # only ever our own children, by handle
                p.terminate()
    for r in res:
        assert not isinstance(r[1], str), r[1]
    return sorted(res)


def _oracle(world, bf16_weights):
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.oracle import OracleModel
    from jittorinfer_b200.models.weights import random_weights
    hp = preset("tiny-v2")
    w = random_weights(hp, seed=0, std=0.05)
    if bf16_weights:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    o = OracleModel(hp, w)
    return [o.generate(p, n) for p, n in list(zip(_prompts(hp), N_NEW))[:world]]


def test_dp_attention_ep_two_cpu_ranks_match_oracle():
    res = _run(2, "gloo", "nccl")
    ref = _oracle(2, False)
    assert [r[1] for r in res] == ref
    assert res[0][2] > 0 and not res[0][3]


def test_dp_engines_step_together_cpu():
    res = _run(2, "gloo", "nccl", target=_engine_worker)
    ref = _oracle(4, False)
    assert res[0][1] == [ref[0], ref[2]] and res[1][1] == [ref[1], ref[3]]
    assert res[0][2] == res[1][2]                      # both ranks left the loop at the same step
    assert res[0][3] + res[1][3] > 0                   # the rank that finished first kept stepping idle


def _agree(got, ref):
    # bf16 can flip an arg-max between near-equal logits; from then on the sequences differ legitimately
    n = 0
    for a, b in zip(got, ref):
        if a != b:
            break
        n += 1
    return n


@pytest.mark.gpu
@pytest.mark.parametrize("comm_impl", ["nccl", "fused"])
def test_dp_attention_ep_two_gpus(comm_impl):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, "nccl", comm_impl)
    ref = _oracle(2, True)
    assert res[0][3] == (comm_impl == "fused")
    for r, want in zip(res, ref):
        assert _agree(r[1], want) >= min(4, len(want)), (r[1], want)


@pytest.mark.gpu
def test_dp_engines_fused_graphs_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, "nccl", "fused", target=_engine_worker)
    ref = _oracle(4, True)
    want = [[ref[0], ref[2]], [ref[1], ref[3]]]
    for r, w in zip(res, want):
        for got, exp in zip(r[1], w):
            assert len(got) == len(exp) and _agree(got, exp) >= min(3, len(exp)), (got, exp)
    assert res[0][2] == res[1][2] and res[0][4] > 0    # same step count; decode steps were graph replays


@pytest.mark.gpu
def test_dp_attention_ep_fused_equals_library_two_gpus():
    """Same kernels for the experts, different transport: the sampled tokens must be identical."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    a = _run(2, "nccl", "nccl")
    b = _run(2, "nccl", "fused")
    assert [r[1] for r in a] == [r[1] for r in b]
