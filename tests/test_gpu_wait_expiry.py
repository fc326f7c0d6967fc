"""A device-side wait that runs out: the kernel returns, the status words say which wait, the next launch works.

The in-kernel collectives wait for flags that other ranks write.  Every such wait is bounded; this file makes one run out
on purpose, on ONE GPU and without any fault: a two-"rank" context is built whose peer buffers are ordinary local
allocations, and nothing ever plays rank 1, so the flag rank 0 waits for is never set.  The poll limit is a field of the
context (a few thousand polls here, about a millisecond).  Nothing traps, hangs or is killed: the kernel gives up,
records {wait timeout, site}, finishes, and the host reads that (``ops.native.check_status`` / the engine's per-step
status read).  A second part plays the missing rank from the host -- its partial and its flag are written before the
launch -- and checks the reduced result, which shows the same launch path completing normally.
(Reference: a blocking HcclAllReduce plus stream synchronisation, ggml/src/ggml-cann/aclnn_ops.cpp:522-536: a silent peer
blocks it for good.)
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_TILES = 64


def _ar_ctx(native, world=2, max_rows=16, d=512, n_sites=2, spin_limit=3000):
    from jittorinfer_b200.parallel.comm import ArCtx
    ws = native.workspace(torch.device(DEV, torch.cuda.current_device()))
    keep = {"recv": [torch.zeros(2 * world * max_rows * d, dtype=torch.float32, device=DEV) for _ in range(world)],
            "flags": [torch.zeros(n_sites * world * MAX_TILES, dtype=torch.int32, device=DEV) for _ in range(world)],
            "epoch": torch.ones(1, dtype=torch.int32, device=DEV)}
    ctx = ArCtx()
    for i in range(world):
        ctx.recv[i] = keep["recv"][i].data_ptr()
        ctx.flags[i] = keep["flags"][i].data_ptr()
    ctx.epoch, ctx.status = keep["epoch"].data_ptr(), ws.status.data_ptr()
    ctx.world, ctx.rank, ctx.n_sites, ctx.max_rows, ctx.d_max, ctx.max_tiles = world, 0, n_sites, max_rows, d, MAX_TILES
    ctx.spin_limit = spin_limit
    return ctx, keep


def _oneshot(native):
    L = native.load()
    from jittorinfer_b200.parallel.comm import ArCtx
    vp = C.c_void_p
    L.jib_allreduce_oneshot.restype = C.c_int
    L.jib_allreduce_oneshot.argtypes = [vp, C.c_int, vp, vp, C.c_int, C.c_int, C.POINTER(ArCtx), C.c_int, vp]
    return L.jib_allreduce_oneshot


def test_all_reduce_wait_for_a_silent_peer_runs_out_and_is_reported():
    from jittorinfer_b200.ops import native
    native.load()
    native.check_status()
    ctx, keep = _ar_ctx(native)
    stream = torch.cuda.current_stream().cuda_stream
    T, d = 8, 512
    x = torch.randn(T, d, device=DEV)
    out = torch.zeros(T, d, dtype=torch.bfloat16, device=DEV)
    # stand-alone one-shot all-reduce: rank 1 never signals
    assert _oneshot(native)(x.data_ptr(), 1, None, out.data_ptr(), T, d, C.byref(ctx), 0, stream) == 0
    torch.cuda.synchronize()                                    # the kernel returned by itself
    with pytest.raises(RuntimeError, match="wait timeout at site 41"):      # 40 + the source rank that stayed silent
        native.check_status()
    native.check_status()                                       # the status words were cleared by the report
    # the same wait inside the GEMM epilogue
    xb, w = torch.randn(T, 256, device=DEV).bfloat16(), (torch.randn(d, 256, device=DEV) * 0.05).bfloat16()
    native.gemm(xb, w, ar=ctx, ar_site=1)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="wait timeout at site 41"):
        native.check_status()
    # an ordinary launch afterwards is unaffected
    y = native.gemm(xb, w)
    torch.cuda.synchronize()
    ref = xb.float() @ w.float().T
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    native.check_status()


def test_all_reduce_completes_when_the_host_plays_the_peer():
    from jittorinfer_b200.ops import native
    native.load()
    ctx, keep = _ar_ctx(native, spin_limit=0)                   # the default limit
    stream = torch.cuda.current_stream().cuda_stream
    T, d, site, world, max_rows = 8, 512, 0, 2, 16
    x = torch.randn(T, d, device=DEV)
    peer = torch.randn(T, d, device=DEV)
    res = torch.randn(T, d, device=DEV).bfloat16()
    # rank 1's part, written ahead of time: its partial rows in slot [1] of rank 0's receive buffer (parity half of
    # site 0 at an odd epoch with an even site count = 0) and its flag for every tile of this launch
    recv0 = keep["recv"][0].view(2, world, max_rows, d)
    recv0[0, 1, :T] = peer
    flags0 = keep["flags"][0].view(2, world, MAX_TILES)
    flags0[site, 1, :] = 1                                      # == the epoch
    out = torch.zeros(T, d, dtype=torch.bfloat16, device=DEV)
    assert _oneshot(native)(x.data_ptr(), 1, res.data_ptr(), out.data_ptr(), T, d, C.byref(ctx), site, stream) == 0
    torch.cuda.synchronize()
    native.check_status()
    want = (x + peer + res.float())
    assert (out.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_expert_parallel_plan_wait_runs_out_and_is_reported():
    from jittorinfer_b200.ops import native
    from jittorinfer_b200.parallel.ep import EpCtx
    L = native.load()
    native.check_status()
    ws = native.workspace(torch.device(DEV, torch.cuda.current_device()))
    world, E_local, d, n_sites, max_rows, max_pairs = 2, 4, 256, 2, 64, 64
    E = E_local * world
    keep = {"xrecv": [torch.zeros(2 * max_rows * d, dtype=torch.bfloat16, device=DEV) for _ in range(world)],
            "meta": [torch.zeros(2 * max_rows, dtype=torch.int32, device=DEV) for _ in range(world)],
            "counts": [torch.zeros(2 * world * E, dtype=torch.int32, device=DEV) for _ in range(world)],
            "yret": [torch.zeros(2 * max_pairs * d, dtype=torch.bfloat16, device=DEV) for _ in range(world)],
            "flags": [torch.zeros(n_sites * 3 * world, dtype=torch.int32, device=DEV) for _ in range(world)],
            "epoch": torch.ones(1, dtype=torch.int32, device=DEV)}
    ctx = EpCtx()
    for i in range(world):
        for name in ("xrecv", "meta", "counts", "yret", "flags"):
            getattr(ctx, name)[i] = keep[name][i].data_ptr()
    ctx.epoch, ctx.status = keep["epoch"].data_ptr(), ws.status.data_ptr()
    ctx.world, ctx.rank, ctx.n_sites, ctx.E_local, ctx.d, ctx.max_recv_rows, ctx.max_pairs = world, 0, n_sites, E_local, d, max_rows, max_pairs
    ctx.spin_limit = 3000
    vp = C.c_void_p
    L.jib_ep_plan.restype = C.c_int
    L.jib_ep_plan.argtypes = [vp, C.c_int, C.c_int, C.POINTER(EpCtx), C.c_int, vp, vp, vp]
    T, k = 4, 2
    ids = torch.randint(0, E, (T, k), device=DEV, dtype=torch.int32)
    seg = torch.zeros(E_local + 1, dtype=torch.int32, device=DEV)
    pair_dst = torch.zeros(T * k, dtype=torch.int32, device=DEV)
    assert L.jib_ep_plan(ids.data_ptr(), T, k, C.byref(ctx), 0, seg.data_ptr(), pair_dst.data_ptr(),
                         torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="wait timeout at site 61"):      # 60 (count exchange) + source rank 1
        native.check_status()
    # with the peer silent the plan falls back to this rank's own counts: its segments cover exactly its local pairs
    local = int((ids < E_local).sum())
    assert int(seg[-1]) == local
    native.check_status()


def test_engine_discards_a_step_whose_kernels_reported_a_fault():
    """The serving loop reads the status words behind every step: a recorded code fails the step (nothing is sampled from
    it), the engine can be reset and serves again."""
    from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import random_weights
    from jittorinfer_b200.ops import native
    from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    native.load()
    hp = preset("tiny")
    w = random_weights(hp, seed=0, std=0.05)
    model = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16, device="cuda:0")
    eng = LLMEngine(model, EngineConfig(n_ctx=512, n_batch=64, n_parallel=2, graph_buckets=(1, 2)))
    prompt = list(range(1, 20))
    want = eng.generate([prompt], SamplingParams(ignore_eos=True), max_new_tokens=6)[0]
    rid = eng.add_request(prompt, SamplingParams(max_tokens=6, ignore_eos=True))
    eng.step()
    # what a kernel does when a wait runs out: code 1 (wait timeout), a site number
    native.workspace(torch.device("cuda", 0)).status.copy_(torch.tensor([1, 41, 0, 0], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="wait timeout at site 41.*step discarded"):
        eng.step()
    assert eng.stats["device_faults"] == 1
    eng.reset()
    again = eng.generate([prompt], SamplingParams(ignore_eos=True), max_new_tokens=6)[0]
    assert again == want and rid not in eng.requests
    native.check_status()
