"""Build variants that can be checked without a GPU: every CUDA source cross-compiles for sm_100a both normally and with
-DJIB_BOUNDS_CHECK, and the two libraries say which one they are."""
import ctypes as C

from jittorinfer_b200 import build


def test_bounds_check_build_compiles_and_identifies_itself():
    normal = C.CDLL(build.build_kernels())
    checked = C.CDLL(build.build_kernels_bounds_check())
    assert normal.jib_bounds_check_enabled() == 0
    assert checked.jib_bounds_check_enabled() == 1
    for unit in ("elementwise", "moe"):
        assert hasattr(checked, "jib_bounds_status_" + unit)
    assert not hasattr(normal, "jib_bounds_status_moe")


def test_timeline_build_compiles_and_identifies_itself():
    """-DJIB_TIMELINE adds the device time stamps of the collective phases and the ring setters; the normal library has
    neither (the stamps compile to nothing there)."""
    normal = C.CDLL(build.build_kernels())
    timed = C.CDLL(build.build_kernels_timeline())
    assert normal.jib_timeline_enabled() == 0 and timed.jib_timeline_enabled() == 1
    for unit in ("gemm", "comm", "combine_ar"):
        assert hasattr(timed, "jib_timeline_set_" + unit) and not hasattr(normal, "jib_timeline_set_" + unit)


def test_timeline_analysis_on_synthetic_stamps():
    """Two call sites, two visits each, four ranks: rank 3 is always the last to arrive at site 1."""
    import json

    import numpy as np
    from jittorinfer_b200.parallel.timeline import STAMP_DTYPE, format_summary, summarize, to_chrome_trace
    rows, t = [], 1_000_000
    for visit in range(2):
        for site in (0, 1):
            rows.append((t, 30, site, 5, 0))                       # accumulators done
            t += 2_000
            rows.append((t, 10, site, 5, 1))                       # my partial is out (I am rank 1)
            t0 = t
            for src, lag in ((1, 100), (0, 900), (2, 1_500), (3, 6_000 if site == 1 else 1_200)):
                rows.append((t0 + lag, 11, site, 5, src))
            t = t0 + (6_300 if site == 1 else 1_800)
            rows.append((t, 12, site, 5, 1))
            t += 50_000
    stamps = np.array(rows, dtype=STAMP_DTYPE)
    assert STAMP_DTYPE.itemsize == 24
    s = summarize(stamps)
    assert s["n_stamps"] == len(rows) and set(s["sites"]) == {0, 1}
    assert abs(s["sites"][1]["wait_us_mean"] - 6.3) < 1e-6 and abs(s["sites"][0]["wait_us_mean"] - 1.8) < 1e-6
    assert s["sites"][1]["last_source"] == {3: 2} and s["sites"][0]["last_source"] == {2: 2}
    assert abs(s["sites"][0]["push_us_mean"] - 2.0) < 1e-6
    assert abs(s["sources"][3]["late_us_mean"] - (6.0 + 1.2) / 2) < 1e-6 and s["sources"][1]["arrivals"] == 4
    text = format_summary(s)
    assert "last source" in text and text.splitlines()[0].startswith(f"{len(rows)} stamps")
    ev = json.loads(to_chrome_trace(stamps, rank=1))["traceEvents"]
    assert len(ev) == len(rows) and ev[0]["name"] == "gemm_accumulators_done" and ev[1]["ts"] == 2.0
    assert summarize(stamps[:0])["sites"] == {}


def test_every_entry_point_is_exported():
    L = C.CDLL(build.build_kernels())
    for name in ("jib_gemm_bf16", "jib_gemm_bf16_noalloc", "jib_mla_flash", "jib_mla_attention", "jib_mla_combine", "jib_moe_gate",
                 "jib_moe_permute", "jib_moe_combine", "jib_rmsnorm", "jib_mla_qkv_post", "jib_embed_gather", "jib_argmax", "jib_topk",
                 "jib_kv_block_copy", "jib_gather_rows", "jib_allreduce_oneshot", "jib_allreduce_twoshot", "jib_ar_epoch_bump",
                 "jib_ep_plan", "jib_ep_push", "jib_ep_combine", "jib_symm_alloc", "jib_symm_open", "jib_allgather_rows",
                 "jib_moe_permute_multi", "jib_moe_route_fused", "jib_moe_combine_norm", "jib_moe_combine_allreduce", "jib_sample_topk"):
        assert hasattr(L, name), name


ABI_PROBE = r"""
#include <cstdio>
#include <cstddef>
#include <cuda_bf16.h>
#include "comm_fused.cuh"
#include "ep_alltoall.h"
#include "jib_kernels.h"
#define F(T, f) printf(#T "." #f " %zu\n", offsetof(T, f))
int main() {
    printf("JibArCtx %zu\n", sizeof(JibArCtx));
    F(JibArCtx, flags); F(JibArCtx, epoch); F(JibArCtx, world); F(JibArCtx, max_tiles); F(JibArCtx, recv2); F(JibArCtx, out2);
    F(JibArCtx, flags2); F(JibArCtx, max_rows2); F(JibArCtx, xg); F(JibArCtx, flags3); F(JibArCtx, ag_counter);
    printf("JibEpCtx %zu\n", sizeof(JibEpCtx));
    F(JibEpCtx, meta); F(JibEpCtx, counts); F(JibEpCtx, yret); F(JibEpCtx, flags); F(JibEpCtx, epoch); F(JibEpCtx, status);
    F(JibEpCtx, world); F(JibEpCtx, E_local); F(JibEpCtx, max_pairs);
    printf("jib_gemm_desc %zu\n", sizeof(jib_gemm_desc));
    F(jib_gemm_desc, seg); F(jib_gemm_desc, x_row_stride); F(jib_gemm_desc, x_rows_total); F(jib_gemm_desc, scratch_bytes);
    F(jib_gemm_desc, n_counters); F(jib_gemm_desc, T); F(jib_gemm_desc, splits); F(jib_gemm_desc, ar_site); F(jib_gemm_desc, ar);
    F(jib_gemm_desc, out_row_ptr); F(jib_gemm_desc, ag_flags); F(jib_gemm_desc, ag_epoch); F(jib_gemm_desc, ag_rows);
    F(jib_gemm_desc, ag_world); F(jib_gemm_desc, ar_rs_rows);
    return 0;
}
"""


def test_ctypes_structs_match_the_c_layouts(tmp_path):
    """The structs passed by pointer or by value into the CUDA library are declared twice (C header, ctypes): a host
    program prints the C sizes and offsets and they must equal the ctypes ones."""
    import os
    import subprocess
    from jittorinfer_b200.ops.native import GemmDesc
    from jittorinfer_b200.parallel.comm import ArCtx
    from jittorinfer_b200.parallel.ep import EpCtx
    src = tmp_path / "abi.cu"
    src.write_text(ABI_PROBE)
    exe = str(tmp_path / "abi")
    subprocess.run([build.nvcc_path(), "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(build.CSRC, "kernels"),
                    str(src), "-o", exe], check=True, capture_output=True)
    lines = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split("\n")
    py = {"JibArCtx": ArCtx, "JibEpCtx": EpCtx, "jib_gemm_desc": GemmDesc}
    checked = 0
    for line in filter(None, lines):
        name, val = line.split()
        if "." in name:
            t, f = name.split(".")
            assert getattr(py[t], f).offset == int(val), name
        else:
            assert C.sizeof(py[name]) == int(val), name
        checked += 1
    assert checked >= 35
