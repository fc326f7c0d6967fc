#!/usr/bin/env python
"""Headline benchmark: decode output tokens/s at concurrency C (default 8).

* N = 1: DeepSeek-V2-Lite (27 layers, 64 experts top-6 + 2 shared, MLA) on one B200.
* N > 1: DeepSeek-V2 (236B architecture) tensor/expert-parallel over N GPUs, layer count scaled
  as 60 * N / 8 so that per-GPU work is fixed ("weak").

Workload (random-init bf16 weights, synthetic uniform-random token ids): C concurrent requests,
each a 1024-token prompt followed by greedy decoding with EOS ignored.  After the prompts have been
prefilled, W warm-up decode steps run untimed and then EXACTLY K engine decode steps are timed with
CUDA events on the launching stream (barrier + synchronize on both sides, max over ranks).  Every
timed step is a full engine step through the public API (`LLMEngine.step()`): the scheduler writes
the step inputs into pinned host memory, one H2D copy, one CUDA-graph replay of the whole model
with on-device greedy sampling, one D2H copy of the sampled ids, scheduler commit.  `value` is
C * K / time.  `e2e` repeats the measurement over whole requests (`LLMEngine.generate()`:
prefill + all decode steps, wall clock) and `graph_only_ms` is the bare graph replay time.

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
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
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
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--gen-len", type=int, default=512)
    ap.add_argument("--model", default=None, help="lite | v2 | tiny (default: lite for 1 GPU, v2 otherwise)")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--ops", default="native", choices=["native", "torch"], help="torch = PyTorch/cuBLAS baseline ops")
    ap.add_argument("--sweep", action="store_true", help="also report concurrency 1/2/4")
    ap.add_argument("--no-e2e", action="store_true")
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
        if world > 1 or (args.model or "lite") != "tiny":
            raise SystemExit("--device cpu is a single-process dry run with --model tiny")
        dev = torch.device("cpu")

        class _HostEvent:
            def record(self):
                self.t = time.perf_counter()

            def elapsed_time(self, other):
                return (other.t - self.t) * 1e3
        new_event = _HostEvent
        synchronize = lambda: None                                     # noqa: E731
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.ops == "torch":
        ops.set_force_torch(True)

    model_name = args.model or ("lite" if world == 1 else "v2")
    hp = preset(model_name)
    if args.layers:
        hp = hp.replace(n_layer=args.layers)
    elif model_name == "v2" and world < 8:
        hp = hp.replace(n_layer=max(2, 60 * world // 8))
    C = args.concurrency
    total_len = args.prompt_len + args.gen_len
    K, W = args.steps, args.warmup
    if W + K >= args.gen_len:
        raise SystemExit("steps + warmup must be smaller than --gen-len")

    t_start = time.time()

    def note(msg):
        if rank == 0:
            print(f"[bench +{time.time() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    eng = build_engine(hp, device=dev, world=world, rank=rank, n_parallel=C, n_ctx_slot=total_len + 64,
                       n_batch=2048, seed=0, graph_buckets=tuple(b for b in (1, 2, 4, 8, 16, 32, 64) if b <= max(C, 1)) or (1,),
                       run_ahead=args.run_ahead)
    g = torch.Generator().manual_seed(1234)

    def prompts(n):
        return [torch.randint(0, hp.n_vocab, (args.prompt_len,), generator=g).tolist() for _ in range(n)]

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

    def timed_decode(conc: int, k_steps: int, w_steps: int, sample_clocks: bool):
        """Prefill `conc` prompts, then time k_steps decode steps. Returns (ms_per_step, clocks, launches)."""
        sp = SamplingParams(max_tokens=args.gen_len, ignore_eos=True)
        ids = [eng.add_request(p, sp) for p in prompts(conc)]
        while any(len(eng.requests[i].output) == 0 for i in ids):     # chunked prefill until every request decodes
            eng.step()
        for _ in range(w_steps):
            eng.step()
        sampler = ClockSampler(local) if sample_clocks and rank == 0 else None
        barrier()
        if sampler:
            sampler.start()
        l0 = eng.launches
        e0, e1 = new_event(), new_event()
        e0.record()
        for _ in range(k_steps):
            eng.step()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop() if sampler else None
        launches = eng.launches - l0
        for i in ids:
            eng.cancel(i)
            eng.requests.pop(i, None)
        return ms / k_steps, clocks, launches

    note(f"model built: {eng.model.weight_bytes() / 2**30:.1f} GiB of weights on this rank")
    eng.warmup()
    note("decode graphs captured")
    tl = None
    if args.timeline:
        from jittorinfer_b200.parallel.timeline import Timeline, format_summary, summarize
        tl = Timeline(dev, capacity=1 << 22)
    ms_step, clocks, launches = timed_decode(C, K, W, True)
    note(f"timed region done: {ms_step:.3f} ms/step")
    timeline_summary = None
    if tl is not None:
        sm = summarize(tl.read())                  # includes prefill and warm-up steps of this measurement
        timeline_summary = {"wait_us_mean": sm.get("wait_us_mean"), "wait_us_total": sm.get("wait_us_total"), "dropped": tl.dropped(),
                            "late_us_by_source": {r: e["late_us_mean"] for r, e in sm["sources"].items()}}
        if rank == 0:
            print(format_summary(sm), file=sys.stderr, flush=True)
        tl.close()
    value = C * 1000.0 / ms_step

    # bare graph replay (no host work between steps): explains how much of a step is device time
    graph_only_ms = None
    key = (next(b for b in eng.cfg.graph_buckets if b >= C), "greedy")
    if key in eng._graphs:
        gr = eng._graphs[key][0]
        barrier()
        e0, e1 = new_event(), new_event()
        for _ in range(3):
            gr.replay()
        e0.record()
        for _ in range(32):
            gr.replay()
        e1.record()
        barrier()
        graph_only_ms = max_over_ranks(e0.elapsed_time(e1)) / 32

    by_conc = {}
    if args.sweep:
        for c in (1, 2, 4):
            if c < C:
                ms_c, _, _ = timed_decode(c, min(K, 64), W, False)
                by_conc[str(c)] = round(c * 1000.0 / ms_c, 2)
        by_conc[str(C)] = round(value, 2)

    e2e = None
    if not args.no_e2e:
        # whole requests through the public API: prefill + gen_len decode steps, wall clock
        ps = prompts(C)
        io_h2d0, io_d2h0, steps0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"], eng.stats["steps"]
        barrier()
        t0 = time.perf_counter()
        outs = eng.generate(ps, SamplingParams(ignore_eos=True), max_new_tokens=args.gen_len)
        barrier()
        dt = max_over_ranks(time.perf_counter() - t0)
        n_steps = eng.stats["steps"] - steps0
        e2e = {"value": round(sum(len(o) for o in outs) / dt, 2), "unit": "tokens/s",
               "h2d_bytes_per_step": (eng.stats["h2d_bytes"] - io_h2d0) // max(1, n_steps),
               "d2h_bytes_per_step": (eng.stats["d2h_bytes"] - io_d2h0) // max(1, n_steps),
               "what": f"LLMEngine.generate(): {C} requests x ({args.prompt_len} prompt + {args.gen_len} generated), "
                       f"prefill included, {n_steps} engine steps, wall clock"}
    synchronize()
    if args.ops == "native" and cuda:
        ops.nat().check_status()

    if rank == 0:
        base = BASELINE.get((model_name, C)) if (model_name == "lite" and world == 1) or (model_name == "v2" and world == 8 and hp.n_layer == 60) else None
        par = "single GPU" if world == 1 else f"tp{world}+ep{world} (attention heads and routed experts sharded, fused GEMM+all-reduce)"
        out = {
            "metric": f"decode output tokens/s at concurrency {C}", "value": round(value, 2), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / base, 3) if base else None, "dtype": "bf16",
            "data": "synthetic (uniform-random token ids, random-init weights)", "impl": "ours", "ops": args.ops,
            "config": {"model": f"DeepSeek-V2{'-Lite' if model_name == 'lite' else ''} ({hp.n_layer} layers)" if model_name != "tiny" else "tiny",
                       "global_batch": C, "seq_len": total_len, "prompt_len": args.prompt_len, "gen_len": args.gen_len,
                       "parallelism": par, "l2": "weights (>= 30 GB per GPU) exceed L2; no flush needed",
                       "timed": "K LLMEngine.step() decode steps: H2D step inputs + CUDA-graph replay + D2H sampled ids"
                                + (" (one step in flight: ids are read one step late)" if args.run_ahead else "")},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "graph_only_ms": graph_only_ms,
            "launches_per_step": launches // max(1, K),
        }
        if by_conc:
            out["by_concurrency"] = by_conc
        if timeline_summary is not None:
            out["timeline"] = timeline_summary
            out["invalid_as_result"] = "run with device time stamps enabled (diagnostic)"
        print(json.dumps(out))
    note("done")
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        # leave without interpreter teardown: destroying captured graphs that hold communicator state after the
        # process group is gone can block at exit
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
