"""Per-op time breakdown (ops/profile.py) on the CPU reference ops."""
import json

import torch

from jittorinfer_b200 import ops
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.ops.profile import OpProfile, main, profile_engine
from jittorinfer_b200.runtime.factory import build_engine


def test_profile_covers_a_prefill_and_decode_steps_and_restores_the_ops():
    before = {n: getattr(ops, n) for n in ("linear", "rmsnorm", "moe_ffn", "mla_attention")}
    eng = build_engine(preset("tiny"), device="cpu", dtype=torch.float32, n_parallel=4, n_ctx_slot=128, n_batch=64, cuda_graphs=False)
    res = profile_engine(eng, prefill_tokens=40, decode_batch=2, decode_steps=3)
    for n, fn in before.items():
        assert getattr(ops, n) is fn                      # wrappers are gone
    pre, dec = res["prefill"], res["decode"]
    hp = eng.hp
    by = {r["op"]: r for r in pre.by_op()}
    # norms timed as ops of their own: one per attention block, one per dense FFN block (a MoE block's norm belongs to its
    # router call), the output norm
    assert by["mla_attention"]["calls"] == hp.n_layer and by["rmsnorm"]["calls"] == hp.n_layer + hp.n_layer_dense_lead + 1
    assert by["moe_ffn"]["calls"] == hp.n_layer - hp.n_layer_dense_lead
    assert any(r["op"] == "linear" and r["shapes"].startswith("40x") for r in pre.rows)
    assert abs(sum(r["share"] for r in pre.rows) - 1.0) < 1e-6 and pre.total_ms > 0 and pre.wall_ms >= pre.total_ms * 0.5
    assert {r["op"]: r for r in dec.by_op()}["mla_attention"]["calls"] == 3 * hp.n_layer
    assert "ms/call" in pre.format()


def test_leaf_mode_reports_innermost_calls_with_their_path():
    class Block:
        def run(self, x, w):
            return ops.linear(ops.rmsnorm(x, torch.ones(x.shape[1]), 1e-6)[0], w)

        def plain(self, x):
            return x + 1

    b, x, w = Block(), torch.randn(4, 8), torch.randn(8, 8)
    with OpProfile(extra=[(b, ("run", "plain"))], leaves=True) as prof:
        b.run(x, w)
        b.plain(x)
    names = sorted(r["op"] for r in prof.rows)
    assert names == ["Block.plain", "Block.run/linear", "Block.run/rmsnorm"]
    assert "run" not in b.__dict__ and b.run(x, w).shape == (4, 8)          # instance is clean again
    with OpProfile(extra=[(b, ("run",))]) as prof:                          # outermost only
        b.run(x, w)
    assert [r["op"] for r in prof.rows] == ["Block.run"]


def test_command_line_writes_json(tmp_path, capsys):
    out = tmp_path / "p.json"
    assert main(["--model", "tiny", "--device", "cpu", "--prefill", "24", "--decode-batch", "1", "--decode-steps", "1", "--json", str(out)]) == 0
    data = json.loads(out.read_text())
    assert data["prefill"]["n_calls"] > 0 and data["decode"]["by_op"]
    assert "== prefill ==" in capsys.readouterr().out


def test_expected_memory_time_tool(capsys):
    """ops/expected.py: launches of one MoE layer with their algorithmic bytes; the totals match a hand count."""
    from jittorinfer_b200.ops.expected import layer_launches, main, report
    hp = preset("lite")
    rows = layer_launches(hp, 8, 1100, 1)
    assert len(rows) == 16
    by = {k: b for k, b, _ in rows}
    assert by["GEMM q + kv_a"] == (16 * 192 + 576) * 2048 * 2
    hit = 64 * (1 - (1 - 6 / 64) ** 8)
    assert abs(by["grouped GEMM down"] - (hit + 2) * 1408 * 2048 * 2) < 1
    assert len(layer_launches(preset("v2"), 8, 1100, 8)) == 21
    text = report(hp, 8, 1100, 1, 6.5e12, measured_ms=5.0, launches=406)
    assert "one MoE layer" in text and "of the bound" in text
    assert main(["--model", "v2", "--world", "8", "--bandwidth-gbs", "6538"]) == 0
    assert "59 MoE layers" in capsys.readouterr().out


def test_expected_prefill_bounds():
    from jittorinfer_b200.ops.expected import prefill_launches, report_prefill
    hp = preset("lite")
    rows = {k: (f, b) for k, f, b, _ in prefill_launches(hp, 2048, 1)}
    assert rows["GEMM o_proj (+ residual)"][0] == 2.0 * 2048 * 2048 * 2048
    # DeepSeek head sizes: a prompt chunk runs the per-head form (K / V expanded by one GEMM); small batches and other head
    # sizes keep the absorbed form
    assert abs(rows["prompt attention (per head, causal)"][0] - 2.0 * 16 * (2048 * 2049 / 2) * (192 + 128)) < 1
    assert rows["GEMM K/V expansion (k_nope | v per head)"][0] == 2.0 * 2048 * (16 * 256) * 512
    tiny = {k: f for k, f, _, _ in prefill_launches(preset("tiny"), 128, 1)}
    assert "flash MLA (absorbed, causal)" in tiny and "GEMM q_absorb (batched per head)" in tiny
    assert abs(rows["grouped GEMM gate|up"][0] - 2.0 * 2048 * 8 * 2 * 1408 * 2048) < 1
    text = report_prefill(hp, 2048, 1, 6.5e12, 1360.0, measured_ms=55)
    assert "27 layers" in text and "of the bound" in text
