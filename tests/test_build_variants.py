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


def test_every_entry_point_is_exported():
    L = C.CDLL(build.build_kernels())
    for name in ("jib_gemm_bf16", "jib_gemm_bf16_noalloc", "jib_mla_flash", "jib_mla_attention", "jib_mla_combine", "jib_moe_gate",
                 "jib_moe_permute", "jib_moe_combine", "jib_rmsnorm", "jib_mla_qkv_post", "jib_embed_gather", "jib_argmax", "jib_topk",
                 "jib_kv_block_copy", "jib_gather_rows", "jib_allreduce_oneshot", "jib_allreduce_twoshot", "jib_ar_epoch_bump",
                 "jib_ep_plan", "jib_ep_push", "jib_ep_combine", "jib_symm_alloc", "jib_symm_open"):
        assert hasattr(L, name), name
