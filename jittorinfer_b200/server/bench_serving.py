"""Load generator for the OpenAI-compatible server: open-loop Poisson arrivals, random-token prompts.

The reference measures serving throughput with an external tool (HF ``inference-benchmarker`` in throughput mode, up to
8 virtual users, ~5-token prompts, ~100 generated tokens: script/test_benchmark.sh:72-82).  This is the in-tree
equivalent, with the workload shape of a continuous-batching deployment: requests arrive as a Poisson process of
``--rate`` requests/s (``--rate 0`` = closed loop with ``--max-concurrency`` virtual users, the reference's mode), prompt
lengths are uniform in ``[--prompt-min, --prompt-max]`` random token ids, every request asks for ``--output-len`` tokens
with EOS ignored, at most ``--max-concurrency`` requests are in flight.

    python -m jittorinfer_b200.server.bench_serving --url http://127.0.0.1:8080 --rate 4 --num-requests 256 \
        --prompt-min 128 --prompt-max 4096 --output-len 256 --max-concurrency 64

Responses are streamed (SSE), so time-to-first-token and the per-token gaps are measured at the client.  One JSON
object is printed: request and token throughput, TTFT / time-per-output-token / end-to-end latency percentiles, error
count, and (when the server exposes them) the KV-cache occupancy and fragmentation read from ``/metrics``.
"""
from __future__ import annotations

import argparse
import json
import random
import threading
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class RequestResult:
    ok: bool = False
    error: str = ""
    n_prompt: int = 0
    n_out: int = 0
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    gaps: List[float] = field(default_factory=list)


def _pct(xs: List[float], p: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    return s[min(len(s) - 1, int(round(p / 100.0 * (len(s) - 1))))]


def one_request(url: str, prompt: List[int], output_len: int, timeout: float) -> RequestResult:
    r = RequestResult(n_prompt=len(prompt), t_submit=time.perf_counter())
    body = json.dumps({"prompt": prompt, "max_tokens": output_len, "temperature": 0, "ignore_eos": True, "stream": True}).encode()
    req = urllib.request.Request(url.rstrip("/") + "/v1/completions", data=body, headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as resp:
            last = None
            for raw in resp:
                line = raw.decode("utf-8", errors="replace").strip()
                if not line.startswith("data: "):
                    continue
                if line == "data: [DONE]":
                    break
                ev = json.loads(line[6:])
                if "error" in ev:
                    r.error = str(ev["error"])
                    break
                now = time.perf_counter()
                usage = ev.get("usage")
                if usage:
                    r.n_out = int(usage.get("completion_tokens", r.n_out))
                if ev.get("choices") and (ev["choices"][0].get("text") or ev["choices"][0].get("finish_reason") is None):
                    if r.t_first == 0.0:
                        r.t_first = now
                    elif last is not None:
                        r.gaps.append(now - last)
                    last = now
            r.t_done = time.perf_counter()
            if r.t_first == 0.0:
                r.t_first = r.t_done
            r.ok = not r.error
    except (urllib.error.URLError, OSError, ValueError) as e:
        r.t_done = time.perf_counter()
        r.error = f"{type(e).__name__}: {e}"
    return r


def scrape_metrics(url: str) -> Dict[str, float]:
    out: Dict[str, float] = {}
    try:
        with urllib.request.urlopen(url.rstrip("/") + "/metrics", timeout=5) as resp:
            for line in resp.read().decode().splitlines():
                if line.startswith("#") or " " not in line:
                    continue
                k, v = line.rsplit(" ", 1)
                try:
                    out[k] = float(v)
                except ValueError:
                    pass
    except (urllib.error.URLError, OSError):
        pass
    return out


def run(url: str, rate: float, num_requests: int, prompt_min: int, prompt_max: int, output_len: int, max_concurrency: int,
        n_vocab: int, seed: int = 0, timeout: float = 600.0, shared_prefix: int = 0) -> Dict[str, object]:
    """``shared_prefix`` > 0: every prompt starts with the same that many tokens (a common system prompt), followed by its
    own random tokens -- the workload in which the server's cross-request prefix sharing shows."""
    rng = random.Random(seed)
    common = [rng.randrange(1, n_vocab) for _ in range(shared_prefix)]
    prompts = [common + [rng.randrange(1, n_vocab) for _ in range(rng.randint(prompt_min, prompt_max))] for _ in range(num_requests)]
    gaps = [rng.expovariate(rate) if rate > 0 else 0.0 for _ in range(num_requests)]
    results: List[Optional[RequestResult]] = [None] * num_requests
    gate = threading.Semaphore(max_concurrency)
    kv_peak = {"used": 0.0, "frag": 0.0}
    stop_scrape = threading.Event()

    def scraper():
        while not stop_scrape.wait(0.5):
            m = scrape_metrics(url)
            kv_peak["used"] = max(kv_peak["used"], m.get("jittorinfer_kv_blocks_used_ratio", 0.0))
            kv_peak["frag"] = max(kv_peak["frag"], m.get("jittorinfer_kv_fragmentation", 0.0))

    def worker(i: int):
        try:
            results[i] = one_request(url, prompts[i], output_len, timeout)
        finally:
            gate.release()

    threading.Thread(target=scraper, daemon=True).start()
    threads = []
    t0 = time.perf_counter()
    t_next = t0
    for i in range(num_requests):
        t_next += gaps[i]
        delay = t_next - time.perf_counter()
        if delay > 0:
            time.sleep(delay)
        gate.acquire()                      # open loop up to the concurrency cap; beyond it arrivals queue at the client
        th = threading.Thread(target=worker, args=(i,), daemon=True)
        th.start()
        threads.append(th)
    for th in threads:
        th.join(timeout=timeout)
    dur = time.perf_counter() - t0
    stop_scrape.set()
    done = [r for r in results if r is not None and r.ok]
    failed = num_requests - len(done)
    ttft = [r.t_first - r.t_submit for r in done]
    e2e = [r.t_done - r.t_submit for r in done]
    tpot = [(r.t_done - r.t_first) / max(1, r.n_out - 1) for r in done if r.n_out > 1]
    itl = [g for r in done for g in r.gaps]
    out_tokens = sum(r.n_out for r in done)
    return {
        "bench": "serving", "url": url, "arrivals": f"poisson {rate}/s" if rate > 0 else f"closed loop, {max_concurrency} users",
        "requests": num_requests, "completed": len(done), "failed": failed, "duration_s": round(dur, 3),
        "prompt_len": [prompt_min, prompt_max], "shared_prefix": shared_prefix, "output_len": output_len, "max_concurrency": max_concurrency,
        "request_throughput_per_s": round(len(done) / dur, 3) if dur > 0 else 0.0,
        "output_tokens_per_s": round(out_tokens / dur, 2) if dur > 0 else 0.0,
        "total_tokens_per_s": round((out_tokens + sum(r.n_prompt for r in done)) / dur, 2) if dur > 0 else 0.0,
        "ttft_ms": {"p50": round(_pct(ttft, 50) * 1e3, 2), "p99": round(_pct(ttft, 99) * 1e3, 2)},
        "tpot_ms": {"mean": round(sum(tpot) / len(tpot) * 1e3, 3) if tpot else 0.0, "p99": round(_pct(tpot, 99) * 1e3, 3)},
        "inter_token_ms": {"p50": round(_pct(itl, 50) * 1e3, 3), "p99": round(_pct(itl, 99) * 1e3, 3)},
        "e2e_ms": {"p50": round(_pct(e2e, 50) * 1e3, 2), "p99": round(_pct(e2e, 99) * 1e3, 2)},
        "kv_peak": {"blocks_used_ratio": round(kv_peak["used"], 4), "fragmentation": round(kv_peak["frag"], 4)},
        "errors": sorted({r.error for r in results if r is not None and r.error})[:5],
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="jittorinfer_b200.server.bench_serving")
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--rate", type=float, default=4.0, help="Poisson arrival rate in requests/s; 0 = closed loop")
    ap.add_argument("--num-requests", type=int, default=128)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-concurrency", type=int, default=64)
    ap.add_argument("--n-vocab", type=int, default=102400)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--shared-prefix", type=int, default=0, help="tokens of a prompt prefix common to all requests")
    ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args(argv)
    res = run(a.url, a.rate, a.num_requests, a.prompt_min, a.prompt_max, a.output_len, a.max_concurrency, a.n_vocab, a.seed, a.timeout, a.shared_prefix)
    print(json.dumps(res))
    return 0 if res["failed"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
