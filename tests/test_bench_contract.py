"""bench.py: the whole script flow as a CPU dry run (tiny model, reference ops) and the keys of its JSON line."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
            "dtype", "data", "config", "clocks", "e2e", "gpu_launches"}


def _bench(*extra):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--device", "cpu", "--model", "tiny", "--steps", "3", "--warmup", "3",
           "--prompt-len", "8", "--gen-len", "10", "--concurrency", "2", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1                                    # exactly one JSON line on stdout
    return json.loads(lines[0])


@pytest.mark.timeout(900)
@pytest.mark.parametrize("extra", [(), ("--run-ahead", "--sweep")])
def test_bench_dry_run_prints_the_contract_line(extra):
    out = _bench(*extra)
    assert REQUIRED <= set(out)
    assert out["n_gpus"] == 1 and out["steps"] == 3 and out["warmup"] == 3 and out["higher_is_better"] is True
    assert out["value"] > 0 and abs(out["value"] - 2 * 1000.0 / out["ms_per_step"]) < 0.05 * out["value"]
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(out["config"]) and out["config"]["global_batch"] == 2
    e2e = out["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(out["clocks"])
    if "--sweep" in extra:
        assert set(out["by_concurrency"]) == {"1", "2"}


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode == 0
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["impl"] == "reference" and "unavailable" in out


@pytest.mark.timeout(900)
@pytest.mark.parametrize("experts", ["tp", "ep"])
def test_bench_dry_run_on_two_ranks(experts):
    """The multi-rank flow of the script (barriers, maximum over ranks, the same-model record that reuses the communicator, both
    expert layouts) as two gloo ranks on the CPU: rank 0 prints the one JSON line."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "bench.py"), "--gpus", "2", "--device", "cpu", "--model", "tiny", "--steps", "3",
           "--warmup", "3", "--prompt-len", "8", "--gen-len", "12", "--concurrency", "2", "--experts", experts, "--no-same-model"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=800, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert REQUIRED <= set(out) and out["n_gpus"] == 2 and out["value"] > 0
    assert out["config"]["parallelism"].startswith("tp2+ep2" if experts == "ep" else "tp2 ")
    assert set(out["by_concurrency"]) == {"1", "2"} and out["e2e"]["value"] > 0
