"""Host-side fault injection, failure detection and tracing (CPU only; nothing here faults a GPU).

Failures are made on the host: an armed fault site raises or withholds, a worker process goes silent or exits, an
allocator reports no free blocks.  The checks: in-flight requests fail with 503 and the server keeps serving; memory
pressure delays but does not change the generated tokens; a silent or dead rank is detected within the timeout; the
step trace is complete and parseable.
"""
import json
import multiprocessing as mp
import os
import threading
import time
import urllib.error
import urllib.request

import pytest
import torch

from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.oracle import OracleModel
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
from jittorinfer_b200.runtime.sampling import SamplingParams
from jittorinfer_b200.utils import fault
from jittorinfer_b200.utils.trace import Tracer


@pytest.fixture(autouse=True)
def _disarm():
    fault.configure("")
    yield
    fault.configure("")


def _engine(**kw):
    hp = preset("tiny")
    w = random_weights(hp, seed=0)
    m = DeepSeek2Model(hp, w.items(), dtype=torch.float32)
    return hp, w, LLMEngine(m, EngineConfig(n_ctx=1024, n_batch=48, n_parallel=4, **kw))


def test_fault_spec_parsing_and_counts():
    fault.configure("a:2,b:1+")
    assert [fault.hit("a") for _ in range(4)] == [False, True, False, False]
    assert [fault.hit("b") for _ in range(3)] == [True, True, True]
    assert not fault.hit("c") and fault.armed("a") and not fault.armed("c")
    with pytest.raises(fault.InjectedFault):
        fault.configure("x:1")
        fault.check("x")


def test_memory_pressure_delays_but_does_not_change_tokens():
    hp, w, eng = _engine()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (40, 17)]
    ref = [OracleModel(hp, w).generate(p, 10) for p in prompts]
    fault.configure("kv_alloc:3")                       # the third step sees an allocator without free blocks
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=10)
    assert outs == ref
    assert eng.kv.check()


def test_engine_reset_after_failed_step():
    hp, w, eng = _engine()
    prompt = list(range(1, 30))
    ref = OracleModel(hp, w).generate(prompt, 6)
    eng.add_request(prompt, SamplingParams(ignore_eos=True, max_tokens=6))
    eng.step()
    fault.configure("engine_step:1")
    with pytest.raises(fault.InjectedFault):
        eng.step()
    eng.reset()
    assert not eng.has_work() and eng.kv.used_blocks == 0 and eng.stats["resets"] == 1
    assert eng.generate([prompt], SamplingParams(ignore_eos=True), max_new_tokens=6) == [ref]


def test_gguf_read_fault(tmp_path):
    from jittorinfer_b200.gguf.io import GGUFReader
    from jittorinfer_b200.models.weights import write_random_gguf
    p = str(tmp_path / "m.gguf")
    write_random_gguf(p, preset("tiny"))
    fault.configure("gguf_read:1")
    with pytest.raises(fault.InjectedFault):
        GGUFReader(p)
    assert GGUFReader(p).kv["general.architecture"] == "deepseek2"       # the next open succeeds


def test_server_fails_inflight_with_503_and_keeps_serving():
    from jittorinfer_b200.config import ServerConfig
    from jittorinfer_b200.server.app import ServerContext, serve
    from jittorinfer_b200.server.chat import ChatTemplate
    from jittorinfer_b200.server.launch import build_from_config
    cfg = ServerConfig(random_init="tiny", n_ctx=1024, n_parallel=2, n_batch=64, port=0, enable_ge=False)
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"))
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl))
    httpd = serve(ctx, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}/v1/completions"
    body = json.dumps({"prompt": "hello", "max_tokens": 6, "temperature": 0, "ignore_eos": True}).encode()

    def post():
        req = urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            return r.status, json.loads(r.read().decode())

    try:
        ok = post()
        assert ok[0] == 200
        fault.configure("engine_step:2")                 # the second step of the next request fails
        with pytest.raises(urllib.error.HTTPError) as e:
            post()
        assert e.value.code == 503 and "engine step failed" in e.value.read().decode()
        again = post()                                   # the engine was reset and serves the same answer
        assert again[0] == 200 and again[1]["choices"][0]["text"] == ok[1]["choices"][0]["text"]
        assert ctx.metrics.c["requests_failed_total"] >= 1 and eng.stats["resets"] == 1
    finally:
        httpd.shutdown()
        httpd.server_close()
        ctx.shutdown()


# ---- failure detection among processes ---------------------------------------------------------------
def _hb_worker(rank, world, port, mode, q):
    """mode: 'ok' beats until told to stop; 'silent' stops beating after 3 beats (fault site); 'exit' leaves at once."""
    import torch.distributed as dist
    from jittorinfer_b200.parallel.health import Heartbeat
    from jittorinfer_b200.utils import fault as f
    store = dist.TCPStore("127.0.0.1", port, world, is_master=False, timeout=__import__("datetime").timedelta(seconds=20))
    if mode == "silent":
        f.configure("heartbeat:3+")
    hb = Heartbeat(store, rank, world, interval=0.05, timeout=0.6).start()
    if mode == "exit":
        time.sleep(0.3)
        q.put((rank, "left"))
        os._exit(0)                                      # between steps, nothing in flight
    store.wait(["stop"])
    hb.stop()
    q.put((rank, "stopped"))


def test_heartbeat_detects_silent_and_dead_ranks():
    import datetime
    import socket
    import torch.distributed as dist
    from jittorinfer_b200.parallel.health import Heartbeat
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 4
    store = dist.TCPStore("127.0.0.1", port, world, is_master=True, timeout=datetime.timedelta(seconds=20), wait_for_workers=False)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hb_worker, args=(r, world, port, mode, q)) for r, mode in ((1, "ok"), (2, "silent"), (3, "exit"))]
    for p in procs:
        p.start()
    hb = Heartbeat(store, 0, world, interval=0.05, timeout=0.6).start()
    try:
        assert hb.wait_all_alive(30.0)                   # rendezvous: everybody published once
        assert hb.dead() == []
        deadline = time.monotonic() + 15
        gone = []
        while time.monotonic() < deadline and sorted(gone) != [2, 3]:
            time.sleep(0.1)
            gone = hb.dead()
        assert sorted(gone) == [2, 3]                    # the silent and the departed rank, not the healthy one
    finally:
        store.set("stop", "1")
        hb.stop()
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()


def test_rendezvous_timeout_when_a_rank_never_joins():
    import torch.distributed as dist
    from jittorinfer_b200.parallel.health import Heartbeat
    hb = Heartbeat(dist.HashStore(), 0, 2, interval=0.05, timeout=0.3)
    t0 = time.monotonic()
    assert not hb.wait_all_alive(0.5)                    # rank 1 never publishes
    assert time.monotonic() - t0 < 5


def test_transport_fault_and_dead_worker_stop_the_broadcast():
    import torch.distributed as dist
    from jittorinfer_b200.parallel.health import Heartbeat
    from jittorinfer_b200.server.app import ServerContext

    class _Ctx(ServerContext):
        def __init__(self):
            self.world, self.rank, self.group = 2, 0, None
            self.stop_flag = threading.Event()

    c = _Ctx()
    fault.configure("transport:1")
    with pytest.raises(fault.InjectedFault):
        c._share_tasks([])
    fault.configure("")
    c.heartbeat = Heartbeat(dist.HashStore(), 0, 2, interval=0.05, timeout=0.2)
    c.heartbeat.dead()                                   # first look starts the clock for rank 1
    time.sleep(0.4)
    with pytest.raises(RuntimeError, match="stopped responding"):
        c._share_tasks([])


# ---- tracing -----------------------------------------------------------------------------------------
def test_step_trace_is_complete(tmp_path, monkeypatch):
    path = str(tmp_path / "trace.jsonl")
    monkeypatch.setenv("JITTORINFER_TRACE", path)
    hp, w, eng = _engine()
    assert eng.tracer.enabled
    prompts = [list(range(1, 60)), list(range(5, 20))]
    outs = eng.generate(prompts, SamplingParams(ignore_eos=True), max_new_tokens=5)
    eng.tracer.close()
    recs = Tracer.read(path)
    steps = [r for r in recs if r["kind"] == "step"]
    assert len(steps) == eng.stats["steps"] and [r["step"] for r in steps] == list(range(1, len(steps) + 1))
    assert sum(r["tokens"] for r in steps) == eng.stats["tokens_in"]
    assert sum(r["outputs"] for r in steps) == sum(len(o) for o in outs)
    assert sum(r["finished"] for r in steps) == 2
    assert steps[0]["max_q"] > 1 and steps[-1]["max_q"] == 1                 # prefill chunks first, single-token steps last
    assert all(set(r["phase_ms"]) >= {"schedule", "launch", "finish"} and r["kv_used"] <= r["kv_total"] for r in steps)
    assert all(a["t_ms"] <= b["t_ms"] for a, b in zip(steps, steps[1:]))


def test_load_trace_lists_tensors(capfd, monkeypatch):
    from jittorinfer_b200.utils import trace
    monkeypatch.setattr(trace, "_LOAD", True)
    hp = preset("tiny")
    DeepSeek2Model(hp, random_weights(hp, seed=0).items(), dtype=torch.float32)
    err = capfd.readouterr().err
    assert "load_tensor: token_embd.weight" in err and "blk.1.ffn_gate_exps.weight" in err


def test_watchdog_fires_once_for_a_silent_rank():
    import torch.distributed as dist
    from jittorinfer_b200.parallel.health import Heartbeat, Watchdog
    store = dist.HashStore()
    me = Heartbeat(store, 1, 2, interval=0.05, timeout=0.3).start()
    zero = Heartbeat(store, 0, 2, interval=0.05, timeout=0.3).start()
    seen = []
    wd = Watchdog(me, [0], on_dead=seen.append, period=0.05).start()
    time.sleep(0.5)
    assert not wd.fired                                  # rank 0 is beating
    zero.stop()                                          # rank 0 goes silent
    deadline = time.monotonic() + 10
    while not wd.fired and time.monotonic() < deadline:
        time.sleep(0.05)
    assert wd.fired and seen == [[0]]
    wd.stop()
    me.stop()


def test_layer_graph_dump_as_dot(tmp_path, monkeypatch):
    """LLAMA_PRINT_LAYER=<il>: the first engine step writes the op graph of that layer (the reference writes a dot file of
    its graph-engine layer graph, src/llama-context-load-utils.cpp:154-162)."""
    import torch
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    monkeypatch.setenv("LLAMA_PRINT_LAYER", "1")
    monkeypatch.chdir(tmp_path)
    eng = build_engine(preset("tiny"), device="cpu", dtype=torch.float32, n_parallel=2, n_ctx_slot=64, n_batch=32, cuda_graphs=False)
    out = eng.generate([[3, 4, 5, 6, 7]], SamplingParams(ignore_eos=True), max_new_tokens=3)
    assert len(out[0]) == 3
    dot = (tmp_path / "jittorinfer_graph_1.dot").read_text()
    assert dot.startswith("digraph forward {") and dot.rstrip().endswith("}")
    for op in ("rmsnorm", "linear", "mla_qkv_post", "q_absorb", "mla_attention", "v_up", "moe_gate", "moe_ffn"):
        assert op in dot, op
    assert "embed_gather" not in dot.split("style=dashed")[0] or "blk 0" in dot       # layer 1 starts from layer 0's output
    assert dot.count("->") >= 8
    g = eng.graph_dump
    layers = {n["layer"] for n in g.nodes}
    assert layers == set(range(eng.hp.n_layer + 1))                                    # blocks + the output head
    # the attention chain is connected: mla_attention reads what q_absorb wrote (through q_full)
    ids = {n["id"]: n for n in g.nodes}
    assert any(ids[a]["op"] == "q_absorb" and ids[b]["op"] == "mla_attention" for a, b in g.edges) or \
        any(ids[a]["op"] == "mla_qkv_post" and ids[b]["op"] == "mla_attention" for a, b in g.edges)
