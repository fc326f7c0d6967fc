#!/usr/bin/env python
"""Headline benchmark: decode output tokens/s at concurrency 1/2/4/8 (the headline value is the one at 8).

* N = 1: DeepSeek-V2-Lite (27 layers, 64 experts top-6 + 2 shared, MLA) on one B200.
* N > 1: DeepSeek-V2 (236B architecture) tensor/expert-parallel over N GPUs, layer count scaled
  as 60 * N / 8 (the full 60 layers on 8 GPUs), global batch fixed.
* every N: a `same_model` sub-record -- DeepSeek-V2 architecture with a fixed 12 layers (fits one GPU) run at TP=N
  with the same global batch: the strong-scaling curve of one model, which the headline (a different model per N,
  as the published baseline is) cannot give.

Workload (random-init bf16 weights, synthetic uniform-random token ids): C concurrent requests,
each a 1024-token prompt followed by greedy decoding with EOS ignored.  After the prompts have been
prefilled, W warm-up decode steps run untimed and then R regions of EXACTLY K engine decode steps each are timed with
CUDA events on the launching stream (barrier + synchronize on both sides, max over ranks); `ms_per_step` / `value` come
from the median region and min / max are reported beside them.  Every timed step is a full engine step through the
public API (`LLMEngine.step()`): the scheduler writes the step inputs into pinned host memory, one H2D copy, one
CUDA-graph replay of the whole model with on-device greedy sampling, one D2H copy of the sampled ids, scheduler commit.
`e2e` repeats the measurement over whole requests (`LLMEngine.generate()`: prefill + all decode steps, wall clock),
`http` drives the OpenAI-compatible server over a socket with the reference harness' workload (1 GPU), and
`graph_only_ms` is the bare graph replay time.

Weights (tens of GB) exceed the 126 MB L2, so every step streams them from HBM: no L2 flush needed.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE = {("lite", 1): 73.3, ("lite", 2): 114.43, ("lite", 4): 166.82, ("lite", 8): 249.28,
            ("v2", 1): 9.3, ("v2", 2): 15.37, ("v2", 4): 25.80, ("v2", 8): 45.69}


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed regions run (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    # The reference (JittorInfer) is a CMake/C++ project for Ascend NPUs (CANN, HCCL): it has no Python package
    # (pip: "Neither 'setup.py' nor 'pyproject.toml' found"), no CUDA backend and cannot execute on this machine.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a C++/CANN (Ascend NPU) project: not pip-installable (no setup.py/pyproject.toml), "
                      "no CUDA backend; only its published numbers (other hardware) exist"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each (fewer if the generation budget is short)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--gen-len", type=int, default=512)
    ap.add_argument("--model", default=None, help="lite | v2 | tiny (default: lite for 1 GPU, v2 otherwise)")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--ops", default="native", choices=["native", "torch"], help="torch = PyTorch/cuBLAS baseline ops")
    ap.add_argument("--sweep", action="store_true", help="kept for compatibility: the concurrency sweep is always reported")
    ap.add_argument("--no-sweep", action="store_true", help="headline concurrency only")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-same-model", action="store_true", help="skip the fixed-model strong-scaling sub-record")
    ap.add_argument("--no-http", action="store_true", help="skip the through-the-server sub-record (1 GPU only)")
    ap.add_argument("--same-model-layers", type=int, default=12)
    ap.add_argument("--experts", default=os.environ.get("JITTORINFER_BENCH_EXPERTS", "tp"), choices=["ep", "tp"],
                    help="N > 1: routed experts sharded by FFN column (tp, default: every rank holds 1 / N of every expert, so the ranks "
                         "stream the same bytes whatever the routing; measured 6-7 %% faster per step on 2 and 4 GPUs) or by expert "
                         "(ep: every rank holds E / N whole experts, the reference's layout)")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: dry run of this script's whole flow on the reference ops with --model tiny (a check of the "
                         "script, not a measurement)")
    ap.add_argument("--run-ahead", action="store_true",
                    help="launch decode step k+1 before the ids of step k reach the host (EngineConfig.run_ahead)")
    ap.add_argument("--timeline", action="store_true",
                    help="diagnostic (needs JITTORINFER_KERNELS_SO = the timeline build): report how long the fused all-reduces "
                         "wait for their peers during the timed steps; the stamps cost time, so the tokens/s of such a run is not a result")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from jittorinfer_b200 import ops
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.ops.expected import default_bandwidth, step_memory_bytes
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        new_event = lambda: torch.cuda.Event(enable_timing=True)      # noqa: E731
        synchronize = torch.cuda.synchronize
    else:
        if (args.model or "lite") != "tiny":
            raise SystemExit("--device cpu is a dry run of the script with --model tiny (one process, or gloo ranks under torchrun)")
        dev = torch.device("cpu")

        class _HostEvent:
            def record(self):
                self.t = time.perf_counter()

            def elapsed_time(self, other):
                return (other.t - self.t) * 1e3
        new_event = _HostEvent
        synchronize = lambda: None                                     # noqa: E731
    if world > 1:
        if cuda:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    if args.ops == "torch":
        ops.set_force_torch(True)

    model_name = args.model or ("lite" if world == 1 else "v2")
    hp = preset(model_name)
    if args.layers:
        hp = hp.replace(n_layer=args.layers)
    elif model_name == "v2" and world < 8:
        hp = hp.replace(n_layer=max(2, 60 * world // 8))
    C = args.concurrency
    K, W = args.steps, args.warmup
    if K < 1:
        raise SystemExit("--steps must be at least 1")
    if W + K + 4 >= args.gen_len:
        # the requested number of timed steps does not fit the configured generation length: generate longer rather than
        # refuse (one region; the JSON line's config carries the length actually used)
        args.gen_len = W + K + 8
    total_len = args.prompt_len + args.gen_len
    R = max(1, min(args.regions, (args.gen_len - W - 4) // K))
    bandwidth = default_bandwidth()

    t_start = time.time()

    def note(msg):
        if rank == 0:
            print(f"[bench +{time.time() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    def barrier():
        if world > 1:
            dist.barrier()
        synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    gen = torch.Generator().manual_seed(1234)

    def prompts(hp_, n, length=None):
        return [torch.randint(0, hp_.n_vocab, (length or args.prompt_len,), generator=gen).tolist() for _ in range(n)]

    def buckets(c):
        return tuple(b for b in (1, 2, 4, 8, 16, 32, 64) if b <= max(c, 1)) or (1,)

    def timed_decode(eng, hp_, conc: int):
        """Prefill `conc` prompts, W warm-up steps, then R regions of K timed decode steps.
        Returns (list of ms per step, one per region; kernels launched inside the regions)."""
        sp = SamplingParams(max_tokens=args.gen_len, ignore_eos=True)
        ids = [eng.add_request(p, sp) for p in prompts(hp_, conc)]
        while any(len(eng.requests[i].output) == 0 for i in ids):     # chunked prefill until every request decodes
            eng.step()
        for _ in range(W):
            eng.step()
        regions, launches = [], 0
        for _ in range(R):
            barrier()
            l0 = eng.launches
            e0, e1 = new_event(), new_event()
            e0.record()
            for _ in range(K):
                eng.step()
            e1.record()
            barrier()
            regions.append(max_over_ranks(e0.elapsed_time(e1)) / K)
            launches += eng.launches - l0
        # bare replay of the step's graph with the inputs of the last timed step still in place (all `conc` sequences live):
        # what a step costs on the device alone, without the host work between steps
        graph_ms = None
        key = (next((b for b in eng.cfg.graph_buckets if b >= conc), None), "greedy")
        if key in eng._graphs and not args.run_ahead:
            gr = eng._graphs[key][0]
            barrier()
            e0, e1 = new_event(), new_event()
            for _ in range(3):
                gr.replay()
            e0.record()
            for _ in range(16):
                gr.replay()
            e1.record()
            barrier()
            graph_ms = round(max_over_ranks(e0.elapsed_time(e1)) / 16, 4)
        for i in ids:
            eng.cancel(i)
            eng.requests.pop(i, None)
        return regions, launches, graph_ms

    def record(eng, hp_, conc: int, with_e2e: bool):
        """One concurrency: decode regions (+ whole requests through generate())."""
        regions, launches, graph_ms = timed_decode(eng, hp_, conc)
        med = statistics.median(regions)
        bound_ms = step_memory_bytes(hp_, conc, args.prompt_len + args.gen_len // 2, world) / bandwidth * 1e3
        out = {"value": round(conc * 1000.0 / med, 2), "ms_per_step": round(med, 4),
               "ms_per_step_min": round(min(regions), 4), "ms_per_step_max": round(max(regions), 4), "regions": len(regions),
               "us_per_layer": round(med * 1e3 / hp_.n_layer, 2), "membound_ms": round(bound_ms, 4),
               "fraction_of_membound": round(bound_ms / med, 3), "launches_per_step": launches // max(1, K * len(regions)),
               "gpu_launches": launches, "graph_only_ms": graph_ms}
        if with_e2e:
            ps = prompts(hp_, conc)
            h0, d0, s0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"], eng.stats["steps"]
            barrier()
            t0 = time.perf_counter()
            outs = eng.generate(ps, SamplingParams(ignore_eos=True), max_new_tokens=args.gen_len)
            barrier()
            dt = max_over_ranks(time.perf_counter() - t0)
            n_steps = eng.stats["steps"] - s0
            out["e2e"] = {"value": round(sum(len(o) for o in outs) / dt, 2), "unit": "tokens/s",
                          "h2d_bytes_per_step": (eng.stats["h2d_bytes"] - h0) // max(1, n_steps),
                          "d2h_bytes_per_step": (eng.stats["d2h_bytes"] - d0) // max(1, n_steps),
                          "what": f"LLMEngine.generate(): {conc} requests x ({args.prompt_len} prompt + {args.gen_len} generated), "
                                  f"prefill included, {n_steps} engine steps, wall clock"}
        return out

    ep_shard = args.experts == "ep"
    eng = build_engine(hp, device=dev, world=world, rank=rank, expert_parallel=ep_shard, n_parallel=C, n_ctx_slot=total_len + 64,
                       n_batch=2048, seed=0, graph_buckets=buckets(C), run_ahead=args.run_ahead)
    weight_gib = eng.model.weight_bytes() / 2**30
    note(f"model built: {weight_gib:.1f} GiB of weights on this rank")
    eng.warmup()
    note("decode graphs captured")
    tl = None
    if args.timeline:
        from jittorinfer_b200.parallel.timeline import Timeline, format_summary, summarize
        tl = Timeline(dev, capacity=1 << 22)

    sampler = ClockSampler(local).start() if rank == 0 and cuda else None
    concs = [C] if args.no_sweep else sorted({c for c in (1, 2, 4, 8) if c < C} | {C})
    by_conc = {}
    for c in concs:
        by_conc[str(c)] = record(eng, hp, c, not args.no_e2e)
        note(f"concurrency {c}: {by_conc[str(c)]['ms_per_step']:.3f} ms/step "
             f"({by_conc[str(c)]['fraction_of_membound']:.2f} of the memory bound)")
    clocks = sampler.stop() if sampler else {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["not sampled"]}
    head = by_conc[str(C)]

    timeline_summary = None
    if tl is not None:
        sm = summarize(tl.read())                  # includes prefill and warm-up steps of this measurement
        timeline_summary = {"wait_us_mean": sm.get("wait_us_mean"), "wait_us_total": sm.get("wait_us_total"), "dropped": tl.dropped(),
                            "late_us_by_source": {r: e["late_us_mean"] for r, e in sm["sources"].items()}}
        if rank == 0:
            print(format_summary(sm), file=sys.stderr, flush=True)
        tl.close()

    graph_only_ms = head.get("graph_only_ms")

    # ---- through the server (1 GPU): the reference harness' workload over HTTP ---------------------------------
    http = None
    if world == 1 and not args.no_http and not args.timeline:
        try:
            http = http_record(eng, hp, C, cuda, duration_s=6.0 if cuda else 0.5)
            note(f"http: {http['output_tokens_per_s']} tok/s through the server at {C} users")
        except Exception as e:        # the headline must not depend on a free port
            http = {"error": f"{type(e).__name__}: {e}"}

    synchronize()
    if args.ops == "native" and cuda:
        ops.nat().check_status()

    # ---- the same model at every N: DeepSeek-V2 architecture, fixed layer count, TP = N (strong scaling) ----------
    same_model = None
    if not args.no_same_model and model_name in ("lite", "v2") and not args.timeline and not args.layers:
        comm = getattr(eng.model, "comm", None)
        del eng
        if cuda:
            torch.cuda.empty_cache()
        try:       # a sub-record: whatever goes wrong here (memory for the second model, ...) must not take the headline with it
            hp2 = preset("v2").replace(n_layer=args.same_model_layers)
            eng2 = build_engine(hp2, device=dev, world=world, rank=rank, expert_parallel=ep_shard, n_parallel=C, n_ctx_slot=total_len + 64,
                                n_batch=2048, seed=0, graph_buckets=buckets(C), comm=comm)
            note(f"same_model built: {eng2.model.weight_bytes() / 2**30:.1f} GiB on this rank")
            eng2.warmup()
            rec = {}
            for c in ([C] if args.no_sweep else sorted({1, C})):
                rec[str(c)] = record(eng2, hp2, c, False)
            same_model = {"model": f"DeepSeek-V2 architecture, {hp2.n_layer} layers, random init",
                          "parallelism": (f"tp{world}+ep{world}" if ep_shard else f"tp{world}") if world > 1 else "single GPU",
                          "scaling": "strong", "global_batch": C, "value": rec[str(C)]["value"], "unit": "tokens/s", "by_concurrency": rec}
            synchronize()
            if args.ops == "native" and cuda:
                ops.nat().check_status()
            note(f"same_model: {same_model['value']} tok/s at concurrency {C}")
        except Exception as e:
            same_model = {"error": f"{type(e).__name__}: {e}"}
            note(f"same_model failed: {same_model['error']}")

    if rank == 0:
        full = (model_name == "lite" and world == 1 and hp.n_layer == 27) or (model_name == "v2" and world == 8 and hp.n_layer == 60)
        base = BASELINE.get((model_name, C)) if full else None
        par = "single GPU" if world == 1 else (f"tp{world}+ep{world} (attention heads and routed experts sharded, fused GEMM+all-reduce)" if ep_shard
                                               else f"tp{world} (attention heads and every expert's FFN columns sharded, fused GEMM+all-reduce)")
        for c, r in by_conc.items():
            b = BASELINE.get((model_name, int(c))) if full else None
            r["vs_baseline"] = round(r["value"] / b, 3) if b else None
        out = {
            "metric": f"decode output tokens/s at concurrency {C}", "value": head["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "regions": head["regions"], "ms_per_step": head["ms_per_step"],
            "ms_per_step_min": head["ms_per_step_min"], "ms_per_step_max": head["ms_per_step_max"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(head["value"] / base, 3) if base else None, "dtype": "bf16",
            "data": "synthetic (uniform-random token ids, random-init weights)", "impl": "ours", "ops": args.ops,
            "config": {"model": f"DeepSeek-V2{'-Lite' if model_name == 'lite' else ''} ({hp.n_layer} layers)" if model_name != "tiny" else "tiny",
                       "global_batch": C, "seq_len": total_len, "prompt_len": args.prompt_len, "gen_len": args.gen_len,
                       "parallelism": par, "layers": hp.n_layer, "weight_gib_per_rank": round(weight_gib, 1),
                       "scaling_note": "N = 1 runs DeepSeek-V2-Lite, N > 1 runs DeepSeek-V2 with 60 * N / 8 layers at a fixed global batch "
                                       "(per-GPU weight bytes roughly constant); tokens/s across N therefore compares different models: "
                                       "the same_model record is the strong-scaling curve of one model",
                       "l2": "weights (>= 30 GB per GPU) exceed L2; no flush needed",
                       "timed": f"{head['regions']} regions of K LLMEngine.step() decode steps (median reported): H2D step inputs + "
                                "CUDA-graph replay + D2H sampled ids"
                                + (" (one step in flight: ids are read one step late)" if args.run_ahead else "")},
            "layers": hp.n_layer, "us_per_layer": head["us_per_layer"],
            "weight_bytes_per_step": int(step_memory_bytes(hp, C, args.prompt_len + args.gen_len // 2, world)),
            "membound_ms": head["membound_ms"], "fraction_of_membound": head["fraction_of_membound"],
            "membound_bandwidth_gbs": round(bandwidth / 1e9, 1),
            "clocks": clocks, "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "graph_only_ms": graph_only_ms,
            "launches_per_step": head["launches_per_step"], "by_concurrency": by_conc,
        }
        if http is not None:
            out["http"] = http
        if same_model is not None:
            out["same_model"] = same_model
        if timeline_summary is not None:
            out["timeline"] = timeline_summary
            out["invalid_as_result"] = "run with device time stamps enabled (diagnostic)"
        print(json.dumps(out))
    note("done")
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        synchronize()
        # leave without interpreter teardown: destroying captured graphs that hold communicator state after the
        # process group is gone can block at exit
        os._exit(0)
    return 0


def http_record(eng, hp, users: int, cuda: bool, duration_s: float = 6.0):
    """Serve `eng` through the OpenAI-compatible HTTP server on a loopback port and drive it with the closed-loop load
    generator: `users` virtual users, ~5-token prompts, 110 generated tokens each (the reference harness' workload,
    script/test_benchmark.sh:8-13,72-82, shortened to a few seconds).  Tokenisation, HTTP, SSE streaming and the
    scheduler's admission are inside the measurement."""
    import socket

    from jittorinfer_b200.config import ServerConfig
    from jittorinfer_b200.server.app import ServerContext, serve
    from jittorinfer_b200.server.bench_serving import run as run_load
    from jittorinfer_b200.server.chat import ChatTemplate
    from jittorinfer_b200.tokenizer import Tokenizer
    from jittorinfer_b200.utils.toy_vocab import toy_vocab_kv
    kv = {k: (v[1] if isinstance(v, tuple) else v) for k, v in toy_vocab_kv(hp.n_vocab, hp.bos_id, hp.eos_id).items()}
    kv["tokenizer.ggml.bos_token_id"], kv["tokenizer.ggml.eos_token_id"] = hp.bos_id, hp.eos_id
    tok = Tokenizer.from_gguf_kv(kv)
    cfg = ServerConfig()
    cfg.n_parallel = eng.cfg.n_parallel
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    # the server decodes one step ahead of the sampled ids (the YAML key `run_ahead`): the HTTP and tokeniser work of a
    # step then overlaps the next step on the device (measured 1537 -> 1677 tok/s on this workload)
    prev_ahead = eng.set_run_ahead(True)
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(""))
    httpd = serve(ctx, "127.0.0.1", port, 16)             # also starts the engine thread
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        url = f"http://127.0.0.1:{port}"
        run_load(url, 0.0, users, 4, 6, 16, users, hp.n_vocab, seed=1)                    # warm-up round
        n_req = max(users, int(users * duration_s * 1.2))                                   # ~duration at >= 100 tok/s/user
        res = run_load(url, 0.0, n_req, 4, 6, 110, users, hp.n_vocab, seed=2)
    finally:
        httpd.shutdown()
        httpd.server_close()
        ctx.shutdown()
        eng.set_run_ahead(prev_ahead)
    return {"what": f"closed loop, {users} users, 4-6 token prompts, 110 generated tokens, SSE streaming over loopback HTTP "
                    "(server/app.py driven by server/bench_serving.py), engine one step ahead of the sampled ids", "requests": res["completed"], "failed": res["failed"],
            "duration_s": res["duration_s"], "output_tokens_per_s": res["output_tokens_per_s"], "ttft_ms": res["ttft_ms"],
            "inter_token_ms": res["inter_token_ms"], "errors": res["errors"]}


if __name__ == "__main__":
    sys.exit(main())
