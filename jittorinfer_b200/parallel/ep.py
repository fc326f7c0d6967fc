"""Expert parallelism with data-parallel attention: all-to-all dispatch / combine of token rows.

In this mode every rank decodes its *own* batch: attention, the dense layer, the shared experts and
the lm_head are replicated, and only the routed experts are sharded (rank r owns experts
``[r*E/N, (r+1)*E/N)``).  A MoE layer therefore has to move each token's hidden row to the ranks that
own its top-k experts and bring the expert outputs back.  The reference has no such path (its expert
parallelism replicates all tokens and sums partial outputs with the post-MLP all-reduce,
src/llama-graph-deepseek2.cpp:365-368; its data-parallel mode gathers tokens with a zero-fill +
all-reduce, 317-334); this is the all-to-all that replaces both.

Two implementations of ``moe_ffn``:

* :class:`EpDispatcher` — baseline over ``torch.distributed`` (NCCL / gloo): all-gather of the
  per-expert counts (a host synchronisation), ``all_to_all_single`` of the rows, grouped experts,
  ``all_to_all_single`` back, weighted sum.
* :class:`FusedEpDispatcher` — the product path (``csrc/kernels/ep_alltoall.cu``): counts, rows and
  results move through peer-mapped buffers from inside kernels; the down-projection GEMM's epilogue
  stores each result row directly into the source rank's memory; no host synchronisation, so the
  whole layer can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops


def _grouped_experts(xs: torch.Tensor, counts: torch.Tensor, wg, wu, wd) -> torch.Tensor:
    """Rows of ``xs`` are sorted by local expert; ``counts[e]`` rows belong to expert e."""
    if xs.is_cuda and ops.use_native(xs) and xs.dtype == torch.bfloat16:
        nat = ops.nat()
        seg = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=xs.device)
        seg[1:] = torch.cumsum(counts.to(xs.device), 0).int()
        if xs.shape[0] == 0:
            return torch.empty(0, wd.shape[1], dtype=xs.dtype, device=xs.device)
        max_rows = int(counts.max())
        active = int((counts > 0).sum())
        h = nat.gemm_grouped(xs, seg, wg, wu, max_rows, active)
        return nat.gemm_grouped(h, seg, wd, None, max_rows, active)
    out = torch.empty(xs.shape[0], wd.shape[1], dtype=xs.dtype, device=xs.device)
    o = 0
    for e, n in enumerate(counts.tolist()):
        if n:
            h = ops.ref.gateup_silu(xs[o:o + n], wg[e], wu[e])
            out[o:o + n] = ops.ref.linear(h, wd[e])
        o += n
    return out


class EpDispatcher:
    """Baseline: library all-to-all."""

    fused = False

    def __init__(self, world: int, rank: int, n_expert: int, group=None):
        self.world, self.rank, self.n_expert, self.group = world, rank, n_expert, group
        self.e_local = n_expert // world
        self.n_collectives = 0

    def begin_step(self) -> None:
        pass

    def close(self) -> None:
        pass

    def moe_ffn(self, x: torch.Tensor, residual: Optional[torch.Tensor], ids: torch.Tensor, wts: torch.Tensor, wg, wu, wd,
                shared: Optional[torch.Tensor]) -> torch.Tensor:
        """x [T, d] this rank's tokens (T may be 0), ids/wts [T, k] global expert ids and weights.
        Returns residual + shared + sum_j wts[t, j] * expert_{ids[t, j]}(x[t])."""
        T, d = x.shape
        k = ids.shape[1]
        W, El = self.world, self.e_local
        dev = x.device
        flat = ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                 # expert-major = owner-major
        counts = torch.bincount(flat, minlength=self.n_expert)
        table = torch.empty(W * self.n_expert, dtype=counts.dtype, device=dev)
        dist.all_gather_into_tensor(table, counts, group=self.group)
        table_h = table.view(W, self.n_expert).cpu()             # host synchronisation: split sizes
        send_splits = table_h[self.rank].view(W, El).sum(1).tolist()
        mine = table_h[:, self.rank * El:(self.rank + 1) * El]   # [source, local expert]
        recv_splits = mine.sum(1).tolist()
        send = x[order // k].contiguous()
        recv = torch.empty(sum(recv_splits), d, dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        self.n_collectives += 3
        # received rows are source-major; the grouped GEMM wants them expert-major (stable within an expert)
        src_of = torch.repeat_interleave(torch.arange(W), torch.tensor(recv_splits))
        exp_of = torch.cat([torch.repeat_interleave(torch.arange(El), mine[s]) for s in range(W)]) if W else src_of
        perm = torch.argsort(exp_of * W + src_of, stable=True).to(dev)
        ys = _grouped_experts(recv[perm].contiguous(), mine.sum(0), wg, wu, wd)
        back = torch.empty_like(ys)
        back[perm] = ys
        ret = torch.empty(T * k, d, dtype=x.dtype, device=dev)
        dist.all_to_all_single(ret, back, send_splits, recv_splits, group=self.group)
        pairs = torch.empty_like(ret)
        pairs[order] = ret
        out = (pairs.view(T, k, d).float() * wts.view(T, k, 1).float()).sum(1)
        if shared is not None:
            out = out + shared.float()
        if residual is not None:
            out = out + residual.float()
        return out.to(x.dtype)


class EpCtx(C.Structure):
    _fields_ = [("xrecv", C.c_void_p * 8), ("meta", C.c_void_p * 8), ("counts", C.c_void_p * 8), ("yret", C.c_void_p * 8),
                ("flags", C.c_void_p * 8), ("epoch", C.c_void_p), ("status", C.c_void_p),
                ("world", C.c_int), ("rank", C.c_int), ("n_sites", C.c_int), ("E_local", C.c_int), ("d", C.c_int),
                ("max_recv_rows", C.c_int), ("max_pairs", C.c_int), ("spin_limit", C.c_uint)]


class FusedEpDispatcher(EpDispatcher):
    """All-to-all through peer memory, issued from inside kernels (plan / push / expert GEMMs / combine)."""

    fused = True

    def __init__(self, device: torch.device, world: int, rank: int, n_expert: int, d: int, k: int, n_sites: int,
                 max_tokens: int = 64, max_recv_rows: Optional[int] = None, group=None):
        super().__init__(world, rank, n_expert, group)
        from ..ops import native
        self.native = native
        self.L = native.load()
        self.device, self.d, self.k = device, d, k
        self.n_sites = n_sites + (n_sites & 1)          # even: the buffer half of a call site is then the same in every step
        self.max_tokens = max_tokens
        self.max_pairs = max_tokens * k
        # worst case: every pair of every rank lands on one rank
        self.max_recv_rows = max_recv_rows or world * self.max_pairs
        vp, i = C.c_void_p, C.c_int
        for name, args in (("jib_symm_alloc", [C.c_size_t, C.POINTER(vp), vp]), ("jib_symm_open", [vp, C.POINTER(vp)]),
                           ("jib_symm_close", [vp]), ("jib_symm_free", [vp]), ("jib_ar_epoch_bump", [vp, vp]),
                           ("jib_ep_plan", [vp, i, i, C.POINTER(EpCtx), i, vp, vp, vp]),
                           ("jib_ep_push", [vp, vp, i, i, C.POINTER(EpCtx), i, vp, vp, vp, vp]),
                           ("jib_ep_combine", [vp, vp, vp, vp, vp, i, i, C.POINTER(EpCtx), i, vp])):
            fn = getattr(self.L, name)
            fn.restype, fn.argtypes = C.c_int, args
        self._own, self._peers = [], []
        R, P, E = self.max_recv_rows, self.max_pairs, n_expert
        bufs = {"xrecv": 2 * R * d * 2, "meta": 2 * R * 4, "counts": 2 * world * E * 4, "yret": 2 * P * d * 2,
                "flags": self.n_sites * 3 * world * 4}
        self.ctx = EpCtx()
        for name, nbytes in bufs.items():
            ptrs = self._exchange(nbytes)
            arr = getattr(self.ctx, name)
            for r in range(world):
                arr[r] = ptrs[r]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        ws = native.workspace(device)
        self.ctx.epoch, self.ctx.status = self.epoch.data_ptr(), ws.status.data_ptr()
        self.ctx.world, self.ctx.rank, self.ctx.n_sites, self.ctx.E_local = world, rank, self.n_sites, self.e_local
        self.ctx.d, self.ctx.max_recv_rows, self.ctx.max_pairs = d, R, P
        self.ctx.spin_limit = int(os.environ.get("JITTORINFER_PEER_WAIT_POLLS", "0"))      # 0 = the built-in limit
        self.seg = torch.zeros(self.e_local + 1, dtype=torch.int32, device=device)
        self.pair_dst = torch.full((max(P, 1),), -1, dtype=torch.int32, device=device)
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.row_ptr = torch.zeros(R, dtype=torch.int64, device=device)
        self.site = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    _exchange = None     # bound below (shared with the all-reduce communicator)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._peers:
            self.L.jib_symm_close(p)
        self._peers = []
        dist.barrier(group=self.group)
        for p in self._own:
            self.L.jib_symm_free(p)
        self._own = []

    def begin_step(self) -> None:
        self.native._ck(self.L.jib_ar_epoch_bump(self.epoch.data_ptr(), torch.cuda.current_stream().cuda_stream), "epoch_bump")
        self.site = 0

    def moe_ffn(self, x, residual, ids, wts, wg, wu, wd, shared):
        T, d = x.shape
        k = ids.shape[1] if ids.dim() == 2 else self.k
        if T > self.max_tokens:
            raise RuntimeError(f"{T} tokens exceed the dispatcher's max_tokens={self.max_tokens}")
        site = self.site
        self.site += 1
        if site >= self.n_sites:
            raise RuntimeError("more MoE layers in one forward pass than the dispatcher was sized for")
        st = torch.cuda.current_stream().cuda_stream
        ck = self.native._ck
        ctx = C.byref(self.ctx)
        ck(self.L.jib_ep_plan(ids.data_ptr() if T else None, T, k, ctx, site, self.seg.data_ptr(), self.pair_dst.data_ptr(), st),
           "ep_plan")
        ck(self.L.jib_ep_push(x.data_ptr() if T else None, self.pair_dst.data_ptr(), T, k, ctx, site, self.seg.data_ptr(),
                              self.done.data_ptr(), self.row_ptr.data_ptr(), st), "ep_push")
        half = site & 1                                   # n_sites is even: equals the kernels' parity in every step
        x_ptr = self.ctx.xrecv[self.rank] + half * self.max_recv_rows * d * 2
        bound = min(self.max_recv_rows, self.world * self.max_tokens)        # rows one expert can receive
        expect = max(1, self.world * self.max_tokens * k // max(self.n_expert, 1))
        bn = 32 if expect <= 32 else 64 if expect <= 64 else 128
        nat = self.native
        h = nat.gemm_grouped_raw(x_ptr, self.max_recv_rows, d, self.seg, wg, wu, bound, self.e_local, bn=bn, device=self.device)
        nat.gemm_grouped_raw(h.data_ptr(), self.max_recv_rows, h.shape[1], self.seg, wd, None, bound, self.e_local, bn=bn,
                             device=self.device, out_row_ptr=self.row_ptr.data_ptr())
        out = torch.empty(T, d, dtype=torch.bfloat16, device=self.device)
        ck(self.L.jib_ep_combine(wts.data_ptr() if T else None, self.pair_dst.data_ptr(), None if shared is None else shared.data_ptr(),
                                 None if residual is None else residual.data_ptr(), out.data_ptr() if T else None, T, k, ctx, site, st),
           "ep_combine")
        self.n_collectives += 1
        return out


def _bind_exchange():
    from .comm import FusedCommunicator
    FusedEpDispatcher._exchange = FusedCommunicator._exchange


_bind_exchange()


def make_ep_dispatcher(device: torch.device, world: int, rank: int, n_expert: int, d: int, k: int, n_moe_layers: int,
                       max_tokens: int = 64, group=None):
    impl = os.environ.get("JITTORINFER_COMM", "fused").lower()
    if device.type != "cuda" or impl == "nccl":
        return EpDispatcher(world, rank, n_expert, group)
    return FusedEpDispatcher(device, world, rank, n_expert, d, k, n_moe_layers, max_tokens=max_tokens, group=group)
