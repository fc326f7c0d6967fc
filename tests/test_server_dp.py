"""Attention data-parallel serving on 2 CPU ranks: rank 0 serves HTTP and assigns requests round robin; both ranks step
together; tokens generated on rank 1 reach the client through the per-iteration gather."""
import json
import multiprocessing as mp
import os
import socket
import sys
import time
import urllib.request

import pytest

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, master_port, http_port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(master_port), RANK=str(rank), WORLD_SIZE=str(world), JITTORINFER_COMM="nccl")
    import torch.distributed as dist
    from jittorinfer_b200.config import ServerConfig
    from jittorinfer_b200.server.app import ServerContext, serve
    from jittorinfer_b200.server.chat import ChatTemplate
    from jittorinfer_b200.server.launch import build_from_config
    dist.init_process_group("gloo", rank=rank, world_size=world)
    control = dist.new_group(backend="gloo")
    cfg = ServerConfig(random_init="tiny-v2", n_ctx=1024, n_parallel=2, n_batch=64, port=http_port, enable_ge=False, ep_size=world,
                       attention_dp=True, ep_max_tokens=64)
    cfg.validate()
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"), world=world, rank=rank)
    assert eng.dp
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl), rank=rank, world=world, control_group=control)
    if rank != 0:
        ctx.run()
        q.put((rank, eng.stats["tokens_out"], eng.stats.get("idle_steps", 0)))
        return
    httpd = serve(ctx, "127.0.0.1", http_port)
    q.put(("ready", http_port, 0))
    try:
        httpd.serve_forever()       # until GET /exit
    finally:
        ctx.shutdown()              # joins the engine thread, whose last broadcast tells the other ranks to stop
        httpd.server_close()
    q.put((rank, eng.stats["tokens_out"], eng.stats.get("idle_steps", 0)))


def _post(url, body):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return json.loads(r.read().decode())


def test_dp_server_two_cpu_ranks():
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.oracle import OracleModel
    from jittorinfer_b200.models.weights import random_weights
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    mport, hport = _free_port(), _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, mport, hport, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        assert q.get(timeout=180)[0] == "ready"
        url = f"http://127.0.0.1:{hport}"
        hp = preset("tiny-v2")
        oracle = OracleModel(hp, random_weights(hp, seed=0))
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(1, hp.n_vocab, (n,), generator=g).tolist() for n in (12, 30, 7)]
        import concurrent.futures as cf
        with cf.ThreadPoolExecutor(3) as ex:             # three requests in flight: ranks 0, 1, 0
            futs = [ex.submit(_post, url + "/v1/completions", {"prompt": p, "max_tokens": 6, "temperature": 0, "ignore_eos": True,
                                                               "return_tokens": True}) for p in prompts]
            outs = [f.result() for f in futs]
        for p, o in zip(prompts, outs):
            assert o["usage"]["completion_tokens"] == 6 and o["usage"]["prompt_tokens"] == len(p)
        toks = [o["choices"][0].get("tokens") for o in outs]
        if all(t is not None for t in toks):
            assert toks == [oracle.generate(p, 6) for p in prompts]
        try:
            urllib.request.urlopen(url + "/exit", timeout=10).read()
        except Exception:
            pass
        stats = sorted(q.get(timeout=120) for _ in range(2))
        assert stats[0][1] + stats[1][1] == 18 and stats[1][1] == 6          # rank 1 generated the second request's tokens
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()


@pytest.mark.parametrize("ep_size", [2, 1])
def test_mpi_server_launcher_two_cpu_ranks(tmp_path, ep_size):
    """The real entry point: ``python -m jittorinfer_b200.server.mpi_server --nproc 2`` spawns the ranks, rank 0 serves
    HTTP, the ranks run tensor-parallel with identical schedulers, heartbeats are on, ``GET /exit`` stops every rank.
    ``ep_size`` 2: whole experts per rank; 1: every expert's FFN columns sharded over the ranks."""
    import subprocess
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.oracle import OracleModel
    from jittorinfer_b200.models.weights import random_weights
    hport, mport = _free_port(), _free_port()
    cfg = tmp_path / "c.yaml"
    cfg.write_text(f"random_init: tiny-v2\nn_ctx: 1024\nn_parallel: 2\nn_batch: 64\nport: {hport}\nenable_ge: false\ntp_size: 2\nep_size: {ep_size}\n")
    env = dict(os.environ, JITTORINFER_COMM="nccl", JITTORINFER_HEARTBEAT_TIMEOUT="20")
    p = subprocess.Popen([sys.executable, "-m", "jittorinfer_b200.server.mpi_server", "--nproc", "2", "--master-port", str(mport),
                          "-c", str(cfg)], cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        url = f"http://127.0.0.1:{hport}"
        deadline = time.time() + 180
        while time.time() < deadline:
            try:
                if urllib.request.urlopen(url + "/health", timeout=2).status == 200:
                    break
            except Exception:
                assert p.poll() is None, p.stdout.read()[-3000:]
                time.sleep(0.5)
        hp = preset("tiny-v2")
        prompt = torch.randint(1, hp.n_vocab, (15,), generator=torch.Generator().manual_seed(9)).tolist()
        out = _post(url + "/v1/completions", {"prompt": prompt, "max_tokens": 5, "temperature": 0, "ignore_eos": True, "return_tokens": True})
        assert out["choices"][0]["tokens"] == OracleModel(hp, random_weights(hp, seed=0)).generate(prompt, 5)
        try:
            urllib.request.urlopen(url + "/exit", timeout=10).read()
        except Exception:
            pass
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()               # our own child, by handle


@pytest.mark.gpu
@pytest.mark.parametrize("dp", [False, True])
def test_mpi_server_two_gpus_serves_over_http(tmp_path, dp):
    """The multi-process server on two GPUs with the in-kernel collectives and CUDA graphs: tensor + expert parallel ranks with
    identical schedulers, or (dp) data-parallel attention with the routed experts reached through the all-to-all dispatcher.
    Several requests at once over HTTP; tokens against the fp32 oracle (bf16 weights); ``GET /exit`` stops every rank."""
    import subprocess
    import threading
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.oracle import OracleModel
    from jittorinfer_b200.models.weights import random_weights, write_random_gguf
    hport, mport = _free_port(), _free_port()
    cfg = tmp_path / "c.yaml"
    hp = preset("tiny-v2")
    gguf = tmp_path / "m.gguf"                      # a file, so that every rank and the oracle hold the same numbers
    write_random_gguf(str(gguf), hp, seed=0, std=0.05)
    cfg.write_text(f"model: {gguf}\nn_ctx: 2048\nn_parallel: 4\nn_batch: 64\nport: {hport}\nenable_ge: true\n"
                   + ("tp_size: 1\nep_size: 2\nattention_dp: true\nep_max_tokens: 64\n" if dp else "tp_size: 2\nep_size: 2\n"))
    env = dict(os.environ, JITTORINFER_COMM="fused", NCCL_NVLS_ENABLE="0", JITTORINFER_HEARTBEAT_TIMEOUT="30")
    p = subprocess.Popen([sys.executable, "-m", "jittorinfer_b200.server.mpi_server", "--nproc", "2", "--master-port", str(mport),
                          "-c", str(cfg)], cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        url = f"http://127.0.0.1:{hport}"
        deadline = time.time() + 240
        up = False
        while time.time() < deadline:
            try:
                if urllib.request.urlopen(url + "/health", timeout=2).status == 200:
                    up = True
                    break
            except Exception:
                assert p.poll() is None, p.stdout.read()[-3000:]
                time.sleep(0.5)
        assert up, "server did not come up"
        g = torch.Generator().manual_seed(9)
        prompts = [torch.randint(1, hp.n_vocab, (n,), generator=g).tolist() for n in (15, 40, 7, 22)]
        outs = [None] * len(prompts)

        def ask(i):
            outs[i] = _post(url + "/v1/completions", {"prompt": prompts[i], "max_tokens": 6, "temperature": 0, "ignore_eos": True,
                                                      "return_tokens": True})["choices"][0]["tokens"]
        ths = [threading.Thread(target=ask, args=(i,)) for i in range(len(prompts))]
        for t in ths:
            t.start()
        for t in ths:
            t.join(timeout=120)
        o = OracleModel(hp, {k: v.bfloat16().float() for k, v in random_weights(hp, seed=0, std=0.05).items()})
        for pr, got in zip(prompts, outs):
            want = o.generate(pr, 6)
            assert got is not None and len(got) == 6 and got[0] == want[0], (got, want)
            assert sum(int(a == b) for a, b in zip(got, want)) >= 3, (got, want)
        try:
            urllib.request.urlopen(url + "/exit", timeout=10).read()
        except Exception:
            pass
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()               # our own child, by handle
