"""Tensor/expert-parallel communicators.

The reference's data plane is one blocking ``HcclAllReduce`` (fp32) after ``o_proj`` and one after
the FFN/MoE block of every layer (src/llama-graph-deepseek2.cpp:294-297, 365-368;
ggml/src/ggml-cann/aclnn_ops.cpp:522-536), bootstrapped over MPI
(src/llama-context-load-utils.cpp:346-434).  Two implementations of the same interface:

* :class:`Communicator` — ``torch.distributed`` all-reduce (NCCL on GPUs, gloo on CPU).  This is
  the *baseline*, and the path for CPU tests and for batches too large for the one-shot buffers.
* :class:`FusedCommunicator` — the product path: every rank maps every peer's receive buffer and
  flag array through CUDA IPC; the row-parallel GEMMs push their tiles to the peers from the tcgen05
  epilogue and reduce in the same kernel (``jib_gemm_bf16`` with ``ar``), and the MoE partial sum
  uses the stand-alone one-shot kernel.  ``torch.distributed`` is used once, to exchange the IPC
  handles.

Both return bitwise identical results on every rank (slots are summed in rank order), which is what
lets every rank run the same scheduler and sample the same tokens without a control broadcast.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist


class Communicator:
    """Baseline: library all-reduce."""

    fused = False

    def __init__(self, world: int, rank: int, group=None):
        self.world, self.rank, self.group = world, rank, group
        self.n_collectives = 0

    def begin_step(self) -> None:
        """Called once at the start of every forward pass."""

    def all_reduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sum over ranks of ``x`` (+ residual); the reduction itself runs in fp32 as in the reference."""
        self.n_collectives += 1
        y = x.float()
        dist.all_reduce(y, group=self.group)
        if residual is not None:
            y = y + residual.float()
        return y.to(residual.dtype if residual is not None else x.dtype)

    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """all_reduce(x_shard @ w_shard^T) + residual."""
        from .. import ops
        part = ops.linear(x, w, out_dtype=torch.float32)
        out = Communicator.all_reduce(self, part, residual)      # the library path, also when a subclass calls in
        return out if residual is not None else out.to(x.dtype)

    # ---- sequence-parallel prefill: the residual stream is sharded by token rows ---------------------------------
    # With T tokens and N ranks, rank r keeps rows [r*R, (r+1)*R), R = ceil(T/N).  A row-parallel GEMM ends in a
    # reduce-scatter instead of an all-reduce (same bytes on the wire, 1/N of the norm / residual work afterwards) and
    # the next column-parallel GEMM starts from an all-gather.  These four methods are the library form (NCCL / gloo);
    # a communicator with in-kernel collectives overrides them.
    sp_min_tokens = int(os.environ.get("JITTORINFER_SP_MIN_TOKENS", "0"))      # 0 = sequence parallelism off

    def all_gather_rows(self, x_loc: torch.Tensor, final: bool = False) -> torch.Tensor:
        """``final``: the gather after the last layer (matters to communicators that reuse buffers between passes)."""
        self.n_collectives += 1
        out = torch.empty(self.world * x_loc.shape[0], x_loc.shape[1], dtype=x_loc.dtype, device=x_loc.device)
        dist.all_gather_into_tensor(out, x_loc.contiguous(), group=self.group)
        return out

    def allgather_linear(self, x_loc: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None) -> torch.Tensor:
        """(all_gather(x_loc) @ w^T), or silu(.. @ w^T) * (.. @ w2^T) with a second weight."""
        from .. import ops
        x = self.all_gather_rows(x_loc)
        return ops.gateup_silu(x, w, w2) if w2 is not None else ops.linear(x, w)

    def reduce_scatter_rows(self, part: torch.Tensor, residual_loc: Optional[torch.Tensor]) -> torch.Tensor:
        """This rank's rows of sum-over-ranks(part) (+ residual_loc); part has world * R rows."""
        self.n_collectives += 1
        R = part.shape[0] // self.world
        y = part.float().contiguous()
        out = torch.empty(R, part.shape[1], dtype=torch.float32, device=part.device)
        try:
            dist.reduce_scatter_tensor(out, y, group=self.group)
        except (RuntimeError, NotImplementedError):       # back ends without reduce-scatter (gloo): reduce, then slice
            dist.all_reduce(y, group=self.group)
            out = y[self.rank * R:(self.rank + 1) * R]
        if residual_loc is not None:
            out = out + residual_loc.float()
        return out.to(residual_loc.dtype if residual_loc is not None else part.dtype)

    def linear_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, residual_loc: Optional[torch.Tensor]) -> torch.Tensor:
        from .. import ops
        out = self.reduce_scatter_rows(ops.linear(x, w, out_dtype=torch.float32), residual_loc)
        return out if residual_loc is not None else out.to(x.dtype)

    def host_barrier(self) -> None:
        """Align the ranks on the host (used after one-off slow host work such as CUDA-graph capture)."""
        if dist.is_initialized() and self.world > 1:
            if torch.cuda.is_available() and dist.get_backend(self.group) == "nccl":
                torch.cuda.synchronize()
            dist.barrier(group=self.group)

    def close(self) -> None:
        pass


class ArCtx(C.Structure):
    _fields_ = [("recv", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("epoch", C.c_void_p), ("status", C.c_void_p),
                ("world", C.c_int), ("rank", C.c_int), ("n_sites", C.c_int), ("max_rows", C.c_int), ("d_max", C.c_int),
                ("max_tiles", C.c_int), ("recv2", C.c_void_p * 8), ("out2", C.c_void_p * 8), ("flags2", C.c_void_p * 8),
                ("max_rows2", C.c_int), ("xg", C.c_void_p * 8), ("flags3", C.c_void_p * 8), ("ag_counter", C.c_void_p),
                ("spin_limit", C.c_uint)]


class FusedCommunicator(Communicator):
    """One-shot all-reduce over peer memory, fused into the GEMM epilogue where a GEMM produces the partial."""

    fused = True
    MAX_TILES = 2048

    def __init__(self, device: torch.device, world: int, rank: int, d_max: int, n_sites: int, max_rows: int = 0,
                 group=None, max_rows_large: int = 0):
        """``max_rows``: largest batch of the one-shot path (decode; every rank receives every partial).  0 = by world size:
        the one-shot traffic grows with the number of peers -- measured on 8 GPUs it beats the library up to 64 rows and takes
        twice the library's time at 256, on 2 GPUs it still wins at 256 -- so the limit is max(64, 512 / world).
        ``max_rows_large`` > 0 also allocates the two-shot path for batches up to that size (prefill): a tile's partials
        go to one owner rank, which reduces and delivers the result to every rank."""
        super().__init__(world, rank, group)
        if max_rows <= 0:
            max_rows = max(64, 512 // max(world, 1))
        n_sites += n_sites & 1            # even: the buffer half of a call site is the same in every step
        from ..ops import native
        self.native = native
        self.L = native.load()
        self.device = device
        self.d_max, self.n_sites, self.max_rows = d_max, n_sites, max_rows
        vp = C.c_void_p
        for name, args in (("jib_symm_alloc", [C.c_size_t, C.POINTER(vp), vp]), ("jib_symm_open", [vp, C.POINTER(vp)]),
                           ("jib_symm_close", [vp]), ("jib_symm_free", [vp]), ("jib_ar_epoch_bump", [vp, vp]),
                           ("jib_allreduce_oneshot", [vp, C.c_int, vp, vp, C.c_int, C.c_int, C.POINTER(ArCtx), C.c_int, vp]),
                           ("jib_allreduce_twoshot", [vp, C.c_int, vp, C.c_int, C.c_int, C.POINTER(ArCtx), C.c_int, C.c_int, vp]),
                           ("jib_allgather_rows", [vp, C.c_int, C.c_int, C.POINTER(ArCtx), C.c_int, C.c_int, vp])):
            fn = getattr(self.L, name)
            fn.restype, fn.argtypes = C.c_int, args
        self._own, self._peers = [], []
        recv_ptrs = self._exchange(2 * world * max_rows * d_max * 4)
        flag_ptrs = self._exchange(n_sites * world * self.MAX_TILES * 4)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        ws = native.workspace(device)
        self.ctx = ArCtx()
        for i in range(world):
            self.ctx.recv[i] = recv_ptrs[i]
            self.ctx.flags[i] = flag_ptrs[i]
        self.ctx.epoch, self.ctx.status = self.epoch.data_ptr(), ws.status.data_ptr()
        self.ctx.world, self.ctx.rank, self.ctx.n_sites = world, rank, n_sites
        self.ctx.max_rows, self.ctx.d_max, self.ctx.max_tiles = max_rows, d_max, self.MAX_TILES
        self.max_rows_large = max_rows_large
        self.ctx.max_rows2 = max_rows_large
        # polls a wait on a peer's flag may take before the kernel reports the peer silent (0 = the built-in 2^20, about a second)
        self.ctx.spin_limit = int(os.environ.get("JITTORINFER_PEER_WAIT_POLLS", "0"))
        if max_rows_large > 0:
            recv2 = self._exchange(2 * world * max_rows_large * d_max * 4)
            out2 = self._exchange(2 * max_rows_large * d_max * 2)
            flags2 = self._exchange(n_sites * self.MAX_TILES * 4)
            xg = self._exchange(2 * max_rows_large * d_max * 2)
            flags3 = self._exchange(n_sites * world * 4)
            for i in range(world):
                self.ctx.recv2[i], self.ctx.out2[i], self.ctx.flags2[i] = recv2[i], out2[i], flags2[i]
                self.ctx.xg[i], self.ctx.flags3[i] = xg[i], flags3[i]
            self._ag_counter = torch.zeros(1, dtype=torch.int32, device=device)
            self.ctx.ag_counter = self._ag_counter.data_ptr()
        self.site = 0
        env = os.environ.get("JIB_FUSED_COMBINE_AR", "")
        self.fused_combine = env != "0"
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _exchange(self, nbytes: int):
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        rc = self.L.jib_symm_alloc(nbytes, C.byref(ptr), handle)
        if rc:
            raise RuntimeError(f"symmetric buffer allocation failed ({rc})")
        self._own.append(ptr.value)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(ptr.value)
                continue
            p = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            rc = self.L.jib_symm_open(buf, C.byref(p))
            if rc:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
            self._peers.append(p.value)
            ptrs.append(p.value)
        return ptrs

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

    # ---------------------------------------------------------------------------------------------
    def begin_step(self) -> None:
        rc = self.L.jib_ar_epoch_bump(self.epoch.data_ptr(), torch.cuda.current_stream().cuda_stream)
        self.native._ck(rc, "epoch_bump")
        self.site = 0

    def _next_site(self) -> int:
        s = self.site
        self.site += 1
        if s >= self.n_sites:
            raise RuntimeError("more collectives in one forward pass than the communicator was sized for")
        return s

    def all_reduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, d = x.shape
        site = self._next_site()
        if T > self.max_rows:
            if T > self.max_rows_large or d != self.d_max:
                return Communicator.all_reduce(self, x, residual)
            self.n_collectives += 1
            self.n_two_shot += 1
            rc = self.L.jib_allreduce_twoshot(x.data_ptr(), int(x.dtype == torch.float32),
                                              None if residual is None else residual.data_ptr(), T, d, C.byref(self.ctx), site, 0,
                                              torch.cuda.current_stream().cuda_stream)
            self.native._ck(rc, "allreduce_twoshot")
            return self._result_view(site, T)
        self.n_collectives += 1
        out = torch.empty(T, d, dtype=torch.bfloat16, device=x.device)
        rc = self.L.jib_allreduce_oneshot(x.data_ptr(), int(x.dtype == torch.float32),
                                          None if residual is None else residual.data_ptr(), out.data_ptr(), T, d,
                                          C.byref(self.ctx), site, torch.cuda.current_stream().cuda_stream)
        self.native._ck(rc, "allreduce_oneshot")
        return out

    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        site = self._next_site()
        T = x.shape[0]
        if T > self.max_rows:
            if T > self.max_rows_large or w.shape[0] != self.d_max:
                return Communicator.linear_all_reduce(self, x, w, residual)
            # two-shot: the GEMM's epilogue sends each tile's partial to its owner; the owner reduces and delivers
            self.n_collectives += 1
            self.n_two_shot += 1
            out = self._result_view(site, T)
            self.native.gemm(x, w, out=out, residual=residual, ar=self.ctx, ar_site=site)
            return out
        self.n_collectives += 1
        return self.native.gemm(x, w, residual=residual, ar=self.ctx, ar_site=site)

    n_two_shot = 0

    # ---- MoE block tail in one launch: expert combine + all-reduce + residual (+ the next block's norm) -----------
    # On by default (JIB_FUSED_COMBINE_AR=0 keeps the separate launches): measured per decode step of 8 sequences
    # 4.90 -> 4.80 ms on 2 GPUs, 7.25 -> 6.99 ms on 4, 12.34 -> 11.50 ms on 8.
    fused_combine = os.environ.get("JIB_FUSED_COMBINE_AR", "0") == "1"

    def moe_ffn_all_reduce(self, x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base, n_expert=None, norm=None):
        """residual + all-reduce(local experts' weighted sum + this rank's shard of the shared experts) for a decode
        batch; ``norm=(weight, eps)`` adds rmsnorm(result) * weight -> (out, normed).  One launch after the expert GEMMs
        instead of combine, all-reduce and norm."""
        T, d = x.shape
        site = self._next_site()
        nat = self.native
        y, dest = nat.moe_routed(x, ids, wts, wg, wu, wd, expert_base, n_expert)
        shared = nat.gemm(nat.gemm(x, wgs, wus), wds) if wgs is not None else None
        out = torch.empty(T, d, dtype=torch.bfloat16, device=x.device)
        normed = torch.empty(T, d, dtype=torch.bfloat16, device=x.device) if norm is not None else None
        fn = self.L.jib_moe_combine_allreduce
        if not getattr(fn, "_typed", False):
            vp = C.c_void_p
            fn.restype, fn.argtypes = C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float,
                                               C.POINTER(ArCtx), C.c_int, vp]
            fn._typed = True
        self.n_collectives += 1
        rc = fn(y.data_ptr(), dest.data_ptr(), wts.data_ptr(), None if shared is None else shared.data_ptr(),
                None if residual is None else residual.data_ptr(), None if norm is None else norm[0].data_ptr(), out.data_ptr(),
                None if normed is None else normed.data_ptr(), T, dest.shape[1], d, float(norm[1]) if norm is not None else 0.0,
                C.byref(self.ctx), site, torch.cuda.current_stream().cuda_stream)
        nat._ck(rc, "moe_combine_allreduce")
        return (out, normed) if norm is not None else out

    # ---- sequence-parallel prefill with in-kernel collectives (see Communicator for the contract) -----------------
    def _sp_fits(self, rows_total: int, d: int) -> bool:
        return 0 < rows_total <= self.max_rows_large and d == self.d_max and rows_total % self.world == 0

    def _gather_view(self, site: int, rows: int, d: int) -> torch.Tensor:
        base = self.ctx.xg[self.rank] + ((site >> 1) & 1) * self.max_rows_large * self.d_max * 2
        return self.native.tensor_from_ptr(base, (rows, self.d_max), torch.bfloat16, self.device)[:, :d]

    def _push_rows(self, x_loc: torch.Tensor, site: int, wait: bool) -> None:
        R, d = x_loc.shape
        rc = self.L.jib_allgather_rows(x_loc.contiguous().data_ptr(), R, d, C.byref(self.ctx), site, int(wait),
                                       torch.cuda.current_stream().cuda_stream)
        self.native._ck(rc, "allgather_rows")

    def all_gather_rows(self, x_loc: torch.Tensor, final: bool = False) -> torch.Tensor:
        R, d = x_loc.shape
        site = self._next_site()
        if final:
            # The gather buffer has two halves, chosen by bit 1 of the call site.  The next forward pass starts with a
            # gather at site 0 (half 0) and nothing orders it after the other ranks' reads of this result, so the last
            # gather of a pass goes to the one call site reserved for it, whose half is 1.
            site = next(t for t in range(self.n_sites - 1, -1, -1) if (t >> 1) & 1)      # the last site with bit 1 set
        if not self._sp_fits(R * self.world, d) or x_loc.dtype != torch.bfloat16:
            return Communicator.all_gather_rows(self, x_loc)
        self.n_collectives += 1
        self._push_rows(x_loc, site, wait=True)          # complete when the kernel ends: any consumer may follow
        return self._gather_view(site, R * self.world, d)

    def allgather_linear(self, x_loc: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None) -> torch.Tensor:
        R, d = x_loc.shape
        site = self._next_site()
        if not self._sp_fits(R * self.world, d) or x_loc.dtype != torch.bfloat16:
            return Communicator.allgather_linear(self, x_loc, w, w2)
        self.n_collectives += 1
        # rows are pushed without waiting; the GEMM's TMA warp waits, per token tile, for the source ranks that cover it
        self._push_rows(x_loc, site, wait=False)
        x = self._gather_view(site, R * self.world, d)
        flags = self.ctx.flags3[self.rank] + site * self.world * 4
        return self.native.gemm(x, w, w2, ag=(flags, self.epoch.data_ptr(), R, self.world))

    def reduce_scatter_rows(self, part: torch.Tensor, residual_loc: Optional[torch.Tensor]) -> torch.Tensor:
        T, d = part.shape
        site = self._next_site()
        if not self._sp_fits(T, d):
            return Communicator.reduce_scatter_rows(self, part, residual_loc)
        self.n_collectives += 1
        R = T // self.world
        rc = self.L.jib_allreduce_twoshot(part.data_ptr(), int(part.dtype == torch.float32), None, T, d, C.byref(self.ctx), site, R,
                                          torch.cuda.current_stream().cuda_stream)
        self.native._ck(rc, "reduce_scatter_rows")
        mine = self._result_view(site, T)[self.rank * R:(self.rank + 1) * R]
        return mine + residual_loc if residual_loc is not None else mine.clone()

    def linear_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, residual_loc: Optional[torch.Tensor]) -> torch.Tensor:
        T = x.shape[0]
        site = self._next_site()
        if not self._sp_fits(T, w.shape[0]):
            return Communicator.linear_reduce_scatter(self, x, w, residual_loc)
        self.n_collectives += 1
        R = T // self.world
        out = self._result_view(site, T)
        self.native.gemm(x, w, out=out, ar=self.ctx, ar_site=site, ar_rs_rows=R)     # epilogue: partials to tile owners,
        mine = out[self.rank * R:(self.rank + 1) * R]                                # reduced rows to their row owners
        return mine + residual_loc if residual_loc is not None else mine.clone()

    def _result_view(self, site: int, T: int) -> torch.Tensor:
        """This rank's copy of the two-shot result of call site ``site``: rows [0, T) of that site's half of the result
        buffer.  Valid until the call site after the next one writes the same half."""
        base = self.ctx.out2[self.rank] + (site & 1) * self.max_rows_large * self.d_max * 2
        return self.native.tensor_from_ptr(base, (T, self.d_max), torch.bfloat16, self.device)


def make_communicator(device: torch.device, world: int, rank: int, d_model: int, n_layer: int, group=None):
    impl = os.environ.get("JITTORINFER_COMM", "fused").lower()
    if device.type != "cuda" or impl == "nccl":
        return Communicator(world, rank, group)
    large = int(os.environ.get("JITTORINFER_AR_LARGE_ROWS", "2048"))
    # call sites per forward pass: 2 per layer (all-reduce form) or 4 per layer (sequence-parallel form) plus the final
    # gather, which takes a site of the spare group of four whose gather-buffer half is 1
    return FusedCommunicator(device, world, rank, d_model, 4 * n_layer + 4, group=group, max_rows_large=large)
