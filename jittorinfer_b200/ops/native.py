"""ctypes front-end of ``libjib200_kernels.so`` (the sm_100a kernels) for torch CUDA tensors.

Every wrapper passes raw device pointers and the current torch CUDA stream; outputs are allocated
with ``torch.empty`` so that the same code runs eagerly and under CUDA-graph capture.  A non-zero
return code from a launcher raises: there is no fallback to PyTorch here.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch

_lib = None
_ws: Dict[int, "Workspace"] = {}
launch_count = 0            # kernels launched through this module (bench.py reports it)
launches_by_name: Dict[str, int] = {}      # the same per launcher ("gemm", "mla_flash", ...): tests assert which path ran

# Switches for A/B measurements (each defaults to the faster path; "0" selects the separate launches).
# Expert sort over many CTAs (histogram / scan / scatter) for batches of PERMUTE_MULTI_MIN (token, expert) pairs and more.
PERMUTE_MULTI = os.environ.get("JIB_PERMUTE_MULTI", "1") == "1"
PERMUTE_MULTI_MIN = 4096
# [RMSNorm +] router logits + gating + expert sort in one launch for decode batches (<= FUSED_ROUTE_MAX_T tokens).  Off by
# default: measured on B200 the single CTA that gates and sorts after the last logit arrives costs as much as the three
# launches it replaces (profiles/decode_switches_ab_lite.md).
FUSED_ROUTE = os.environ.get("JIB_FUSED_ROUTE", "0") == "1"
# Grouped-GEMM split-K hint from the expected number of experts hit instead of all local experts.
ACTIVE_HINT_EXPECTED = os.environ.get("JIB_ACTIVE_HINT", "0") == "1"
# Expert combine fused with the RMSNorm of the next block (one launch fewer per MoE layer).
FUSED_COMBINE_NORM = os.environ.get("JIB_FUSED_COMBINE_NORM", "1") == "1"
# Decode batches: the grouped gate|up GEMM reads the token rows in place (no gather into expert order).
GROUPED_SRC = os.environ.get("JIB_GROUPED_SRC", "1") == "1"
GROUPED_SRC_MAX_T = 64
# The down-projection launch reads the segment table and requests its weights before the gate|up launch has finished.
GROUPED_PAIR = os.environ.get("JIB_GROUPED_PAIR", "1") == "1"
# Grouped launches of batches with fewer (token, expert) pairs than experts cover only the experts that have rows.
EXPERT_LIST = os.environ.get("JIB_EXPERT_LIST", "1") == "1"
# Grouped launches of prompt chunks walk a list of the (expert, token tile) pairs that exist.
TILE_LIST = os.environ.get("JIB_TILE_LIST", "1") == "1"
TILE_LIST_MIN_PAIRS = 1024
# The router launch of a decode batch also applies the RMSNorm of its input ("0": a separate norm launch before it).
ROUTE_NORM = os.environ.get("JIB_ROUTE_NORM", "1") == "1"
FUSED_ROUTE_MAX_T = 64
_route_stash: Dict[tuple, tuple] = {}       # (ids ptr, expert_base, E_local) -> (seg, src, dest) produced by the fused launch

ERRORS = {-1: "unsupported shape/argument", -2: "pointer or stride not 16-byte aligned", -3: "driver entry point missing",
          -4: "tensor map encode failed", -5: "kernel launch failed", -6: "scratch too small for requested split"}


class GemmDesc(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("x", "w", "w2", "out", "residual", "seg", "scratch", "counters", "status")] + \
               [(n, C.c_longlong) for n in ("x_row_stride", "x_batch_stride", "w_row_stride", "w_batch_stride", "ldo",
                                            "out_batch_stride", "ldr", "res_batch_stride", "x_rows_total")] + \
               [("scratch_bytes", C.c_size_t)] + \
               [(n, C.c_int) for n in ("n_counters", "T", "N", "K", "batch", "max_rows", "active_hint", "out_f32", "res_f32",
                                       "splits", "bn", "sm_count", "ar_site")] + [("ar", C.c_void_p), ("out_row_ptr", C.c_void_p), ("ag_flags", C.c_void_p),
                                                                             ("ag_epoch", C.c_void_p), ("ag_rows", C.c_int),
                                                                             ("ag_world", C.c_int), ("ar_rs_rows", C.c_int),
                                                                             ("src_token", C.c_void_p), ("src_rows", C.c_int), ("expert_list", C.c_void_p),
                                                                             ("n_slots", C.c_int), ("list_tiles", C.c_int), ("pdl_flags", C.c_int)]


def load():
    global _lib
    if _lib is not None:
        return _lib
    from .. import build
    path = os.environ.get("JITTORINFER_KERNELS_SO") or build.KERNELS_SO      # e.g. the bounds-check build
    if not os.path.exists(path):
        build.build_kernels()
    L = C.CDLL(path)
    vp, ip, fp, ll, i, f = C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_float

    def sig(name, *args):
        fn = getattr(L, name)
        fn.restype = C.c_int
        fn.argtypes = list(args)

    sig("jib_gemm_bf16", C.POINTER(GemmDesc), vp)
    sig("jib_embed_gather", vp, ip, vp, i, i, i, vp)
    sig("jib_rmsnorm", vp, vp, fp, vp, vp, i, i, ll, f, vp)
    sig("jib_mla_qkv_post", vp, ll, vp, ll, fp, f, fp, ip, ip, vp, vp, ll, ll, i, i, i, i, i, i, ll, ip, vp)
    sig("jib_kv_gather", vp, ll, ip, i, ip, i, i, i, vp, ip, i, vp)
    sig("jib_mha_prefill", vp, ll, vp, vp, ll, ll, ip, ip, ip, i, i, i, f, i, vp, ll, ip, vp)
    sig("jib_argmax", fp, ip, i, i, vp)
    sig("jib_topk", fp, fp, ip, i, i, i, vp)
    sig("jib_sample_topk", fp, ip, fp, ip, i, i, vp)
    sig("jib_kv_block_copy", vp, ll, i, ip, ip, i, i, vp)
    sig("jib_gather_rows", vp, ip, vp, i, i, i, vp)
    sig("jib_moe_gate", vp, fp, fp, fp, ip, fp, i, i, i, i, i, i, f, i, i, i, i, vp)
    sig("jib_moe_permute", ip, i, i, i, i, ip, ip, ip, vp)
    sig("jib_moe_route_fused", vp, fp, fp, fp, ip, fp, ip, ip, ip, ip, i, i, i, i, i, i, f, i, i, i, i, i, i, fp, f, vp, vp)
    sig("jib_moe_permute_multi", ip, i, i, i, i, ip, ip, ip, ip, vp)
    sig("jib_moe_tile_list", ip, i, i, ip, i, vp)
    sig("jib_moe_combine", vp, ip, fp, vp, vp, vp, i, i, i, vp)
    sig("jib_moe_combine_norm", vp, ip, fp, vp, vp, fp, vp, vp, i, i, i, f, vp)
    sig("jib_mla_attention", vp, vp, ip, i, ip, ip, i, i, i, i, i, i, f, i, fp, fp, vp, vp)
    sig("jib_mla_combine", fp, fp, i, i, i, i, vp, vp)
    sig("jib_mla_flash", vp, vp, ll, ip, i, ip, ip, i, i, i, f, i, i, fp, fp, vp, ip, vp)
    _lib = L
    return L


class Workspace:
    """Per-device scratch shared by all launches on one stream: split-K partials, tile counters
    (zero between launches by construction) and the status words kernels set when a bounded wait
    expires."""

    SCRATCH_BYTES = 96 << 20
    N_COUNTERS = 1 << 16

    def __init__(self, device: torch.device):
        self.scratch = torch.empty(self.SCRATCH_BYTES, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(self.N_COUNTERS, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.route_counter = torch.zeros(1, dtype=torch.int32, device=device)      # last-CTA detection of the fused router
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        L = load()
        if hasattr(L, "jib_bounds_check_enabled") and L.jib_bounds_check_enabled():
            with torch.cuda.device(device):          # bounds-check build: clamped indices are also reported here
                for unit in ("elementwise", "moe"):
                    fn = getattr(L, "jib_bounds_status_" + unit)
                    fn.restype, fn.argtypes = C.c_int, [C.c_void_p]
                    fn(self.status.data_ptr())


def workspace(device: torch.device) -> Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _ws.get(idx)
    if w is None:
        w = _ws[idx] = Workspace(torch.device("cuda", idx))
    return w


def check_status(device=None) -> None:
    """Raises if any kernel recorded a bounded-wait expiry or a bounds violation (synchronises)."""
    for idx, w in _ws.items():
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        st = w.status.tolist()
        if st[0] != 0:
            w.status.zero_()
            w.counters.zero_()
            names = {1: "wait timeout", 2: "index out of bounds", 3: "misaligned"}
            raise RuntimeError(f"kernel status: {names.get(st[0], st[0])} at site {st[1]} block {st[2]} extra {st[3]}")


class _RawCudaBuffer:
    """Adapter that lets torch wrap device memory it did not allocate (peer-mapped communication buffers)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor view of raw device memory (no ownership: the caller keeps the allocation alive)."""
    if dtype == torch.bfloat16:        # the array interface has no bf16: wrap as int16 and reinterpret
        return torch.as_tensor(_RawCudaBuffer(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8", torch.float16: "<f2"}[dtype]
    return torch.as_tensor(_RawCudaBuffer(ptr, shape, typestr), device=device)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ck(rc: int, what: str):
    global launch_count
    launch_count += 1
    launches_by_name[what] = launches_by_name.get(what, 0) + 1
    if rc != 0:
        raise RuntimeError(f"{what}: {ERRORS.get(rc, rc)}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---- GEMM family ---------------------------------------------------------------------------------
def gemm(x: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None, *, out: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, splits: int = 0, bn: int = 0,
         ar=None, ar_site: int = 0, ar_rs_rows: int = 0, ag=None) -> torch.Tensor:
    """out[T,N] = x[T,K] @ w[N,K]^T  (w2: silu(x w^T) * (x w2^T)) (+ residual)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(-1) == 1 and w.is_contiguous()
    T, K = x.shape
    N = w.shape[0]
    od = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty(T, N, dtype=od, device=x.device)
    ws = workspace(x.device)
    d = GemmDesc()
    d.x, d.w, d.w2, d.out, d.residual = x.data_ptr(), w.data_ptr(), _p(w2), out.data_ptr(), _p(residual)
    d.seg, d.scratch, d.counters, d.status = None, ws.scratch.data_ptr(), ws.counters.data_ptr(), ws.status.data_ptr()
    d.x_row_stride, d.x_batch_stride, d.w_row_stride, d.w_batch_stride = x.stride(0), 0, K, 0
    d.ldo, d.out_batch_stride = out.stride(0), 0
    d.ldr = residual.stride(0) if residual is not None else 0
    d.res_batch_stride, d.x_rows_total, d.scratch_bytes, d.n_counters = 0, T, ws.SCRATCH_BYTES, ws.N_COUNTERS
    d.T, d.N, d.K, d.batch, d.max_rows, d.active_hint = T, N, K, 1, 0, 0
    d.out_f32 = int(out.dtype == torch.float32)
    d.res_f32 = int(residual is not None and residual.dtype == torch.float32)
    d.splits, d.bn, d.sm_count = splits, bn, ws.sm_count
    if ar is not None:          # fused all-reduce (or, with ar_rs_rows, reduce-scatter by rows) over peer memory in the epilogue
        d.ar, d.ar_site, d.ar_rs_rows = C.addressof(ar), ar_site, ar_rs_rows
    if ag is not None:          # x is a gather buffer other ranks are still filling: (flags ptr, epoch ptr, rows per rank, world)
        d.ag_flags, d.ag_epoch, d.ag_rows, d.ag_world = ag
    _ck(load().jib_gemm_bf16(C.byref(d), _stream()), "gemm")
    return out


def gemm_batched(x_ptr: int, x_row_stride: int, x_batch_stride: int, w: torch.Tensor, out_ptr: int, ldo: int,
                 out_batch_stride: int, T: int, device, splits: int = 0) -> None:
    """Per-batch (per-head) GEMM with arbitrary element strides: out[b][t][:N] = x[b][t][:K] @ w[b]^T."""
    B, N, K = w.shape
    ws = workspace(device)
    d = GemmDesc()
    d.x, d.w, d.w2, d.out, d.residual = x_ptr, w.data_ptr(), None, out_ptr, None
    d.seg, d.scratch, d.counters, d.status = None, ws.scratch.data_ptr(), ws.counters.data_ptr(), ws.status.data_ptr()
    d.x_row_stride, d.x_batch_stride, d.w_row_stride, d.w_batch_stride = x_row_stride, x_batch_stride, K, N * K
    d.ldo, d.out_batch_stride, d.ldr, d.res_batch_stride = ldo, out_batch_stride, 0, 0
    d.x_rows_total, d.scratch_bytes, d.n_counters = T, ws.SCRATCH_BYTES, ws.N_COUNTERS
    d.T, d.N, d.K, d.batch, d.max_rows, d.active_hint = T, N, K, B, 0, 0
    d.out_f32, d.res_f32, d.splits, d.bn, d.sm_count = 0, 0, splits, 0, ws.sm_count
    _ck(load().jib_gemm_bf16(C.byref(d), _stream()), "gemm_batched")


def _seg_has_list(seg: torch.Tensor, E: int) -> bool:
    """Whether the allocation behind a segment table has room for (and, coming from ``moe_permute`` / the fused router, holds)
    the list of experts that have rows: E more ints behind the E + 1 offsets."""
    return seg.untyped_storage().nbytes() // 4 - seg.storage_offset() >= 2 * E + 1


def gemm_grouped_raw(x_ptr: int, x_rows_total: int, K: int, seg: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor],
                     max_rows: int, active_hint: int, splits: int = 0, bn: int = 0, device=None,
                     out_row_ptr: Optional[int] = None, src_token: Optional[torch.Tensor] = None, src_rows: int = 0,
                     pdl_flags: int = 0, n_slots: int = 0, tile_list: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Grouped GEMM over a raw row buffer (e.g. a peer-mapped receive buffer).  With ``out_row_ptr`` (device array of
    row addresses) every result row is stored through its pointer and nothing is returned.  With ``src_token`` the
    buffer holds the ``src_rows`` token rows unsorted and sorted result row i is computed from token ``src_token[i]``
    (``x_rows_total`` stays the number of sorted rows, i.e. rows of the result)."""
    E, N, K2 = w.shape
    assert K2 == K
    device = device or w.device
    out = None if out_row_ptr else torch.empty(x_rows_total, N, dtype=torch.bfloat16, device=device)
    ws = workspace(device)
    d = GemmDesc()
    d.x, d.w, d.w2, d.residual = x_ptr, w.data_ptr(), _p(w2), None
    d.out = out.data_ptr() if out is not None else ws.scratch.data_ptr()     # unused when rows go through pointers
    d.seg, d.scratch, d.counters, d.status = seg.data_ptr(), ws.scratch.data_ptr(), ws.counters.data_ptr(), ws.status.data_ptr()
    d.x_row_stride, d.x_batch_stride, d.w_row_stride, d.w_batch_stride = K, 0, K, N * K
    d.ldo, d.out_batch_stride, d.ldr, d.res_batch_stride = N, 0, 0, 0
    d.x_rows_total, d.scratch_bytes, d.n_counters = x_rows_total, ws.SCRATCH_BYTES, ws.N_COUNTERS
    d.T, d.N, d.K, d.batch, d.max_rows, d.active_hint = max_rows, N, K, E, max_rows, active_hint
    d.out_f32, d.res_f32, d.splits, d.bn, d.sm_count = 0, 0, splits, bn, ws.sm_count
    d.out_row_ptr = out_row_ptr
    if src_token is not None:
        d.src_token, d.src_rows = src_token.data_ptr(), src_rows
    d.pdl_flags = pdl_flags
    if tile_list is not None:    # (expert, token tile) pairs built for this bn (moe_tile_list): large batches
        assert bn > 0
        d.expert_list, d.n_slots, d.list_tiles = tile_list.data_ptr(), tile_list.numel(), 1
    elif n_slots > 0:            # seg carries the list of experts that have rows behind its E + 1 offsets (moe_permute)
        assert _seg_has_list(seg, E)
        d.expert_list, d.n_slots = seg.data_ptr() + (E + 1) * 4, n_slots
    _ck(load().jib_gemm_bf16(C.byref(d), _stream()), "gemm_grouped")
    return out


def gemm_grouped(xp: torch.Tensor, seg: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor], max_rows: int,
                 active_hint: int, splits: int = 0, pdl_flags: int = 0, n_slots: int = 0, bn: int = 0,
                 tile_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of xp are sorted by expert; expert e owns rows seg[e]:seg[e+1] and weight w[e] ([E,N,K])."""
    assert xp.stride(0) == xp.shape[1] and xp.stride(1) == 1
    return gemm_grouped_raw(xp.data_ptr(), xp.shape[0], xp.shape[1], seg, w, w2, max_rows, active_hint, splits, bn, device=xp.device,
                            pdl_flags=pdl_flags, n_slots=n_slots, tile_list=tile_list)


def linear(x, w, residual=None, out_dtype=None):
    return gemm(x, w, residual=residual, out_dtype=out_dtype)


def gateup_silu(x, wg, wu):
    return gemm(x, wg, wu)


# ---- memory-bound kernels ------------------------------------------------------------------------
def embed_gather(table, ids):
    T, d = ids.shape[0], table.shape[1]
    out = torch.empty(T, d, dtype=table.dtype, device=table.device)
    _ck(load().jib_embed_gather(table.data_ptr(), ids.data_ptr(), out.data_ptr(), T, d, table.shape[0], _stream()), "embed")
    return out


def rmsnorm(x, w, eps, residual=None):
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    T, d = x.shape
    out = torch.empty(T, d, dtype=x.dtype, device=x.device)
    summed = torch.empty(T, d, dtype=x.dtype, device=x.device) if residual is not None else None
    _ck(load().jib_rmsnorm(x.data_ptr(), _p(residual), w.data_ptr(), out.data_ptr(), _p(summed), T, d, x.stride(0),
                           float(eps), _stream()), "rmsnorm")
    return out, (summed if residual is not None else x)


def mla_qkv_post(q, ckv, kv_norm_w, eps, rope_table, positions, slot_mapping, cache, q_out, n_head, dn, dr, r):
    """``q_out`` None: the rotated RoPE part of q is written back into q (the per-head prefill form reads q as it is)."""
    T = q.shape[0]
    ws = workspace(q.device)
    if q_out is None:
        qo_ptr, qo_row, qo_head = q.data_ptr() + dn * 2, q.stride(0), dn + dr
    else:
        qo_ptr, qo_row, qo_head = q_out.data_ptr() + r * 2, n_head * (r + dr), r + dr
    _ck(load().jib_mla_qkv_post(q.data_ptr(), q.stride(0), ckv.data_ptr(), ckv.stride(0), kv_norm_w.data_ptr(), float(eps),
                                rope_table.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr(), cache.data_ptr(),
                                qo_ptr, qo_row, qo_head, T, n_head, dn, dr, r, rope_table.shape[0], cache.shape[0],
                                ws.status.data_ptr(), _stream()), "mla_qkv_post")
    return q.view(T, n_head, dn + dr)[..., :dn] if q.is_contiguous() else q.as_strided((T, n_head, dn), (q.stride(0), dn + dr, 1))


def q_absorb(q_nope, w_ukT, q_out, r):
    """q_out[t,h,:r] = q_nope[t,h,:] @ w_ukT[h]^T with w_ukT [H, r, dn]."""
    T, H, dn = q_nope.shape
    gemm_batched(q_nope.data_ptr(), q_nope.stride(0), q_nope.stride(1), w_ukT, q_out.data_ptr(), q_out.stride(0),
                 q_out.stride(1), T, q_nope.device)


def v_up(o_lat, w_uv):
    """o[t, h*dv:(h+1)*dv] = o_lat[t,h,:] @ w_uv[h]^T with w_uv [H, dv, r]."""
    T, H, r = o_lat.shape
    dv = w_uv.shape[1]
    out = torch.empty(T, H * dv, dtype=o_lat.dtype, device=o_lat.device)
    gemm_batched(o_lat.data_ptr(), o_lat.stride(0), o_lat.stride(1), w_uv, out.data_ptr(), H * dv, dv, T, o_lat.device)
    return out


def attn_splits(T: int, H: int, sm_count: int = 148) -> int:
    """Split count for the decode kernel: enough CTAs to cover the machine about twice."""
    per = max(1, T * max(1, H // 16))
    return max(1, min(32, sm_count // per))


ATTN_IMPL = os.environ.get("JITTORINFER_ATTN", "flash")      # "flash" (tcgen05) | "simt" (CUDA-core kernel)


def mla_attention(q, cache, block_tables, seq_lens, q_start, scale, r, block_size, max_q_len=None, meta=None):
    T, H, D = q.shape
    n_seqs = seq_lens.shape[0]
    prefill = (max_q_len or 1) > 1
    o = torch.empty(T, H, r, dtype=q.dtype, device=q.device)
    if ATTN_IMPL == "flash" and r == 512 and D == 576 and block_size == 64 and cache.shape[0] % 64 == 0:
        qt = 2 if prefill else 1
        n_splits = 1 if prefill else attn_splits(T, H)
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty(T, n_splits, H, r, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(T, n_splits, H, 2, dtype=torch.float32, device=q.device)
        ws = workspace(q.device)
        _ck(load().jib_mla_flash(q.data_ptr(), cache.data_ptr(), cache.shape[0], block_tables.data_ptr(), block_tables.stride(0),
                                 seq_lens.data_ptr(), q_start.data_ptr(), n_seqs, T, H, float(scale), n_splits, qt, _p(part_o),
                                 _p(part_ml), o.data_ptr(), ws.status.data_ptr(), _stream()), "mla_flash")
        if n_splits > 1:
            _ck(load().jib_mla_combine(part_o.data_ptr(), part_ml.data_ptr(), n_splits, T, H, r, o.data_ptr(), _stream()),
                "mla_combine")
        return o
    n_splits = 1 if prefill and T > 64 else attn_splits(T, H)
    if n_splits > 1:
        part_o = torch.empty(T, n_splits, H, r, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(T, n_splits, H, 2, dtype=torch.float32, device=q.device)
    else:
        part_o = part_ml = None
    _ck(load().jib_mla_attention(q.data_ptr(), cache.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
                                 seq_lens.data_ptr(), q_start.data_ptr(), n_seqs, T, H, r, D - r, block_size, float(scale),
                                 n_splits, _p(part_o), _p(part_ml), o.data_ptr(), _stream()), "mla_attention")
    return o


MHA_PREFILL = os.environ.get("JIB_MHA_PREFILL", "1") == "1"      # "0": prompt chunks use the absorbed form as well (A/B)
MHA_PREFILL_MIN_TOKENS = 64


def mha_prefill_ok(T: int, dn: int, dr: int, dv: int, r: int, block_size: int, meta) -> bool:
    """Whether a chunk of T query tokens takes the per-head prefill attention (needs the host-side totals in ``meta``)."""
    if not (MHA_PREFILL and meta is not None and T >= MHA_PREFILL_MIN_TOKENS and dn == 128 and dr == 64 and dv == 128 and r == 512):
        return False
    total, dec = meta.get("total_kv", 0), meta.get("kv_decode", 0)
    # Expanding K / V costs ~4 MFLOP per cached row and pays for itself over the many query rows of a prompt; a sequence that
    # only decodes brings one query row and its whole context.  A mixed step whose gathered rows are mostly such contexts
    # stays with the absorbed form, which reads the latent rows as they are.
    return total > 0 and dec <= total - dec


def kv_gather(cache, block_tables, seq_lens, total: int, block_size: int):
    """The cached latent rows of every sequence of the batch, in sequence order: ([total, row] bf16, first row of each
    sequence [n_seqs] int32)."""
    n_seqs = seq_lens.shape[0]
    row = cache.shape[1]
    lat = torch.empty(total, row, dtype=torch.bfloat16, device=cache.device)
    kv_start = torch.empty(n_seqs, dtype=torch.int32, device=cache.device)
    _ck(load().jib_kv_gather(cache.data_ptr(), cache.shape[0], block_tables.data_ptr(), block_tables.stride(0), seq_lens.data_ptr(),
                             n_seqs, block_size, row, lat.data_ptr(), kv_start.data_ptr(), total, _stream()), "kv_gather")
    return lat, kv_start


def mha_prefill_core(q, kv, lat, kv_start, seq_lens, q_start, scale, n_head, n_q_tiles: int):
    """The attention kernel itself: q [T, H*192], kv [total, H*256] = k_nope | v per head, lat [total, 576] (its last 64
    columns are the RoPE part of the keys, shared by the heads).  Returns [T, H*128] bf16."""
    T, total = q.shape[0], lat.shape[0]
    out = torch.empty(T, n_head * 128, dtype=torch.bfloat16, device=q.device)
    ws = workspace(q.device)
    _ck(load().jib_mha_prefill(q.data_ptr(), q.stride(0), kv.data_ptr(), lat.data_ptr() + 512 * 2, lat.shape[1], total,
                               q_start.data_ptr(), seq_lens.data_ptr(), kv_start.data_ptr(), seq_lens.shape[0], T, n_head, float(scale),
                               int(n_q_tiles), out.data_ptr(), out.stride(0), ws.status.data_ptr(), _stream()), "mha_prefill")
    return out


def mha_prefill(q, cache, w_kv_b, block_tables, seq_lens, q_start, scale, n_head, block_size, meta):
    """Causal multi-head attention of a prompt chunk in the per-head form.  q [T, H*192] (RoPE already applied in place; may
    be a strided view), cache [n_slots, 576] one layer's latent rows, w_kv_b [H*256, 512].  ``meta``: host-side totals of the
    batch, {"total_kv": sum of seq_lens, "n_q_tiles": upper bound of sum ceil(q_len / 128)}.  Returns [T, H*128] bf16."""
    lat, kv_start = kv_gather(cache, block_tables, seq_lens, int(meta["total_kv"]), block_size)
    kv = gemm(lat[:, :512], w_kv_b)                     # [total, H*256]: k_nope | v per head
    return mha_prefill_core(q, kv, lat, kv_start, seq_lens, q_start, scale, n_head, int(meta["n_q_tiles"]))


# ---- MoE -----------------------------------------------------------------------------------------
def moe_gate(g, w_router, bias, k, n_group, topk_group, scale, norm, sigmoid, n_shared=0, group_top2=False, route=None,
             pre_norm=None):
    """``route=(expert_base, E_local)``: the caller will sort these ids by local expert next (``moe_permute``); for decode
    batches both steps then run as one launch and ``moe_permute`` picks the result up.
    ``pre_norm=(weight, eps)``: ``g`` holds un-normalised rows; returns (ids, wts, rmsnorm(g) * weight), the norm done by
    the router launch itself for decode batches."""
    T, d = g.shape
    fused = FUSED_ROUTE and route is not None and T <= FUSED_ROUTE_MAX_T
    g_in = g
    g_pre = None
    if pre_norm is not None and not (fused and ROUTE_NORM):
        g, _ = rmsnorm(g, pre_norm[0], pre_norm[1])
        g_in, g_pre, pre_norm_k = g, g, None
    else:
        pre_norm_k = pre_norm
    E = w_router.shape[0]
    ids = torch.empty(T, k + n_shared, dtype=torch.int32, device=g.device)
    wts = torch.empty(T, k + n_shared, dtype=torch.float32, device=g.device)
    logits = torch.empty(T, E, dtype=torch.float32, device=g.device)
    if fused:
        expert_base, E_local = route
        n = T * (k + n_shared)
        seg = torch.empty(2 * E_local + 1, dtype=torch.int32, device=g.device)[:E_local + 1]     # + room for the list of experts hit
        src = torch.empty(n, dtype=torch.int32, device=g.device)
        dest = torch.empty(T, k + n_shared, dtype=torch.int32, device=g.device)
        assert g_in.dtype == torch.bfloat16 and g_in.is_contiguous()
        g_out = torch.empty_like(g_in) if pre_norm_k is not None else None
        _ck(load().jib_moe_route_fused(g_in.data_ptr(), w_router.data_ptr(), _p(bias), logits.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                                       seg.data_ptr(), src.data_ptr(), dest.data_ptr(), workspace(g.device).route_counter.data_ptr(),
                                       T, d, E, k, n_group, topk_group, float(scale), int(norm), int(sigmoid), n_shared,
                                       int(group_top2), expert_base, E_local, pre_norm_k[0].data_ptr() if pre_norm_k is not None else None,
                                       float(pre_norm_k[1]) if pre_norm_k is not None else 0.0, _p(g_out), _stream()), "moe_route_fused")
        _route_stash.clear()                       # at most one pending result: the sort that follows this gate
        _route_stash[(ids.data_ptr(), expert_base, E_local)] = (seg, src, dest, ids)
        return (ids, wts, g_out if g_out is not None else g_pre) if pre_norm is not None else (ids, wts)
    _ck(load().jib_moe_gate(g.data_ptr(), w_router.data_ptr(), _p(bias), logits.data_ptr(), ids.data_ptr(), wts.data_ptr(), T, d,
                            E, k, n_group, topk_group, float(scale), int(norm), int(sigmoid), n_shared, int(group_top2), _stream()), "moe_gate")
    return (ids, wts, g) if pre_norm is not None else (ids, wts)


def moe_permute(ids, expert_base, E_local):
    T, k = ids.shape
    dev = ids.device
    hit = _route_stash.pop((ids.data_ptr(), expert_base, E_local), None)
    if hit is not None and hit[3] is ids:          # the fused router launch already sorted exactly these ids
        return hit[0], hit[1], hit[2]
    seg = torch.empty(2 * E_local + 1, dtype=torch.int32, device=dev)[:E_local + 1]       # + room for the list of experts hit
    src = torch.empty(T * k, dtype=torch.int32, device=dev)
    dest = torch.empty(T, k, dtype=torch.int32, device=dev)
    if PERMUTE_MULTI and T * k >= PERMUTE_MULTI_MIN:
        # large batches (prefill): histogram / scan / stable scatter over many CTAs instead of one CTA scanning every pair
        tmp = torch.empty(((T * k + 1023) // 1024) * E_local, dtype=torch.int32, device=dev)
        _ck(load().jib_moe_permute_multi(ids.data_ptr(), T, k, expert_base, E_local, seg.data_ptr(), src.data_ptr(), dest.data_ptr(),
                                         tmp.data_ptr(), _stream()), "moe_permute_multi")
        return seg, src, dest
    _ck(load().jib_moe_permute(ids.data_ptr(), T, k, expert_base, E_local, seg.data_ptr(), src.data_ptr(), dest.data_ptr(),
                               _stream()), "moe_permute")
    return seg, src, dest


def moe_tile_list(seg, E_local: int, bn: int, n_pairs: int) -> torch.Tensor:
    """(token tile << 16 | expert) for every ``bn``-row tile of every expert that has rows, -1 padded to the bound
    n_pairs / bn + E_local (every expert can end in one partial tile)."""
    cap = n_pairs // bn + E_local
    out = torch.empty(cap, dtype=torch.int32, device=seg.device)
    _ck(load().jib_moe_tile_list(seg.data_ptr(), E_local, bn, out.data_ptr(), cap, _stream()), "moe_tile_list")
    return out


def gather_rows(x, src_row):
    R, d = src_row.shape[0], x.shape[1]
    out = torch.empty(R, d, dtype=x.dtype, device=x.device)
    _ck(load().jib_gather_rows(x.data_ptr(), src_row.data_ptr(), out.data_ptr(), R, d, x.shape[0], _stream()), "gather_rows")
    return out


def moe_combine(y, dest, wts, shared, residual, norm=None):
    """``norm=(weight, eps)``: also return rmsnorm(out) * weight from the same launch -> (out, normed)."""
    T, k = dest.shape
    d = y.shape[1]
    out = torch.empty(T, d, dtype=torch.bfloat16, device=y.device)
    if norm is not None:
        normed = torch.empty(T, d, dtype=torch.bfloat16, device=y.device)
        _ck(load().jib_moe_combine_norm(y.data_ptr(), dest.data_ptr(), wts.data_ptr(), _p(shared), _p(residual), norm[0].data_ptr(),
                                        out.data_ptr(), normed.data_ptr(), T, k, d, float(norm[1]), _stream()), "moe_combine_norm")
        return out, normed
    _ck(load().jib_moe_combine(y.data_ptr(), dest.data_ptr(), wts.data_ptr(), _p(shared), _p(residual), out.data_ptr(), T, k, d,
                               _stream()), "moe_combine")
    return out


def expected_active_experts(T: int, k: int, E_local: int, n_expert: int) -> int:
    """Expected number of distinct local experts that T tokens with k choices each out of n_expert hit (uniform routing);
    columns beyond the router's k (merged shared experts: E_local > local share of n_expert) always count."""
    always = max(0, E_local - n_expert) if E_local > n_expert else 0
    routed_local = E_local - always
    k_routed = max(1, k - always)
    p_hit = 1.0 - (1.0 - min(1.0, k_routed / max(1, n_expert))) ** T
    return max(1, min(E_local, always + int(routed_local * p_hit + 0.999)))


def moe_routed(x, ids, wts, wg, wu, wd, expert_base=0, n_expert=None):
    """Expert-sorted rows -> grouped gate|up GEMM (SiLU*mul epilogue) -> grouped down GEMM.
    Returns (y [T*k, d] in sorted order, dest [T,k])."""
    T, k = ids.shape
    E_local = wg.shape[0]
    seg, src, dest = moe_permute(ids, expert_base, E_local)
    # the two grouped launches run back to back over one segment table: the second may start on its weights early
    pair = (1, 2) if GROUPED_PAIR else (0, 0)
    # few pairs, many experts: the grouped launches cover the list of experts that have rows instead of all of them
    slots = T * k if (EXPERT_LIST and T * k < E_local and _seg_has_list(seg, E_local)) else 0
    active = min(E_local, T * k)
    if ACTIVE_HINT_EXPECTED and n_expert:        # split-K sized for the experts a batch is expected to hit, not for all
        active = min(active, expected_active_experts(T, k, E_local, n_expert))
    if TILE_LIST and T * k >= TILE_LIST_MIN_PAIRS:
        # prompt chunks: an expert holds ~T*k/E rows, far fewer than the T the grid would have to be sized for; both grouped
        # launches walk a device-built list of the (expert, 128-token tile) pairs that exist
        tl = moe_tile_list(seg, E_local, 128, T * k)
        h = gemm_grouped(gather_rows(x, src), seg, wg, wu, T, active, pdl_flags=pair[0], bn=128, tile_list=tl)
        return gemm_grouped(h, seg, wd, None, T, active, pdl_flags=pair[1], bn=128, tile_list=tl), dest
    if GROUPED_SRC and T <= GROUPED_SRC_MAX_T and x.is_contiguous():
        # decode batches: every expert that has rows multiplies the whole (tiny) token tile and picks its tokens' columns in the
        # epilogue, so the token rows are never gathered into expert order
        h = gemm_grouped_raw(x.data_ptr(), T * k, x.shape[1], seg, wg, wu, T, active, device=x.device, src_token=src, src_rows=T,
                             pdl_flags=pair[0], n_slots=slots)
    else:
        h = gemm_grouped(gather_rows(x, src), seg, wg, wu, T, active, pdl_flags=pair[0], n_slots=slots)
    y = gemm_grouped(h, seg, wd, None, T, active, pdl_flags=pair[1], n_slots=slots)
    return y, dest


def moe_experts(x, ids, wts, wg, wu, wd, expert_base=0):
    """fp32 [T, d] sum over the local experts (API parity with the reference implementation)."""
    y, dest = moe_routed(x, ids, wts, wg, wu, wd, expert_base)
    return moe_combine(y, dest, wts, None, None).float()


def moe_ffn(x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base=0, n_expert=None, norm=None):
    """residual + shared_experts(x) + sum_k w_k expert_k(x), bf16; residual/shared may be None.
    ``norm=(weight, eps)``: returns (out, rmsnorm(out) * weight), the norm computed by the combine launch."""
    y, dest = moe_routed(x, ids, wts, wg, wu, wd, expert_base, n_expert)
    shared = None
    if wgs is not None:
        shared = gemm(gemm(x, wgs, wus), wds)
    return moe_combine(y, dest, wts, shared, residual, norm)


# ---- sampling / cache ----------------------------------------------------------------------------
def argmax(logits):
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    _ck(load().jib_argmax(logits.data_ptr(), out.data_ptr(), n, V, _stream()), "argmax")
    return out


def topk_logits(logits, k):
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    vals = torch.empty(n, k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(n, k, dtype=torch.int32, device=logits.device)
    _ck(load().jib_topk(logits.data_ptr(), vals.data_ptr(), ids.data_ptr(), n, V, k, _stream()), "topk")
    return vals, ids


def sample_topk(vals, ids, params):
    n, k = vals.shape
    assert vals.dtype == torch.float32 and ids.dtype == torch.int32 and params.dtype == torch.float32
    assert vals.is_contiguous() and ids.is_contiguous() and params.is_contiguous() and params.shape == (n, 5)
    out = torch.empty(n, dtype=torch.int32, device=vals.device)
    _ck(load().jib_sample_topk(vals.data_ptr(), ids.data_ptr(), params.data_ptr(), out.data_ptr(), n, k, _stream()), "sample_topk")
    return out


def dequantize_bf16(raw, ggml_type: int, n_elements: int):
    """``raw``: uint8 CUDA tensor holding ``n_elements`` elements of a block-quantised ggml type -> bf16 [n_elements]."""
    L = load()
    fn = L.jib_dequantize_bf16                   # bound on first use: libraries built before this entry point still load
    fn.restype, fn.argtypes = C.c_int, [C.c_uint, C.c_void_p, C.c_ulonglong, C.c_void_p, C.c_void_p]
    assert raw.dtype == torch.uint8 and raw.is_cuda and raw.is_contiguous()
    out = torch.empty(n_elements, dtype=torch.bfloat16, device=raw.device)
    with torch.cuda.device(raw.device):
        _ck(fn(int(ggml_type), raw.data_ptr(), int(n_elements), out.data_ptr(), _stream()), "dequantize_bf16")
    return out


def kv_block_copy(cache, src_blocks, dst_blocks, block_size):
    L, n_slots, row = cache.shape
    _ck(load().jib_kv_block_copy(cache.data_ptr(), n_slots * row, L, src_blocks.data_ptr(), dst_blocks.data_ptr(),
                                 src_blocks.shape[0], block_size * row, _stream()), "kv_block_copy")
