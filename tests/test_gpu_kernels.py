"""sm_100a kernels vs the plain-PyTorch fp32 reference of the same op (tile-edge shapes included)."""
import os

import pytest
import torch

from jittorinfer_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def nat():
    from jittorinfer_b200.ops import native
    native.load()
    yield native
    torch.cuda.synchronize()
    native.check_status()


def rnd(*shape, scale=1.0, dtype=torch.bfloat16, seed=None):
    g = torch.Generator(device="cpu")
    g.manual_seed(hash(shape) % (2 ** 31) if seed is None else seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref_mag = b.abs().max().item() + 1e-6
    assert err <= tol * ref_mag, f"max err {err} vs magnitude {ref_mag}"


@pytest.mark.parametrize("T", [1, 2, 7, 8, 16, 17, 63, 64, 65, 128, 129, 300])
@pytest.mark.parametrize("N,K", [(256, 512), (200, 192), (3648, 2048)])
def test_gemm_shapes(nat, T, N, K):
    x, w = rnd(T, K), rnd(N, K, scale=0.05)
    y = nat.gemm(x, w)
    close(y, x.float() @ w.float().T)
    nat.check_status()


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
@pytest.mark.parametrize("T", [1, 8, 40])
def test_gemm_split_k(nat, splits, T):
    x, w = rnd(T, 2048), rnd(384, 2048, scale=0.05)
    for _ in range(2):     # second launch checks that the tile counters were left at zero
        y = nat.gemm(x, w, splits=splits)
        close(y, x.float() @ w.float().T)
    nat.check_status()


def test_gemm_residual_f32_out(nat):
    x, w, r = rnd(5, 1024), rnd(640, 1024, scale=0.05), rnd(5, 640)
    close(nat.gemm(x, w, residual=r), x.float() @ w.float().T + r.float())
    rf = r.float()
    y = nat.gemm(x, w, residual=rf, out_dtype=torch.float32)
    assert y.dtype == torch.float32
    close(y, x.float() @ w.float().T + rf, tol=1e-3)


@pytest.mark.parametrize("T,splits", [(1, 0), (8, 0), (8, 4), (33, 1), (200, 0)])
def test_gemm_gateup_silu(nat, T, splits):
    x, wg, wu = rnd(T, 1024), rnd(1408, 1024, scale=0.05), rnd(1408, 1024, scale=0.05, seed=3)
    y = nat.gemm(x, wg, wu, splits=splits)
    g, u = x.float() @ wg.float().T, x.float() @ wu.float().T
    close(y, torch.nn.functional.silu(g) * u)
    nat.check_status()


def test_gemm_several_waves_takes_the_persistent_kernel(nat, monkeypatch):
    """Launches of several waves of wide tiles run as one CTA per SM walking the tile list with two accumulator sets in
    tensor memory: dense with a residual and a ragged last token tile, gate|up, and the grouped pair of a prompt chunk
    (tile list).  Each against fp32 and against the one-tile-per-CTA kernel (bitwise: same tiles, same order of sums)."""
    import os
    x, w, res = rnd(2000, 1088), rnd(5120, 1088, scale=0.05), rnd(2000, 5120, seed=7)
    y = nat.gemm(x, w, residual=res)
    close(y, x.float() @ w.float().T + res.float(), tol=1e-2)
    x2, wg, wu = rnd(1500, 512), rnd(4096, 512, scale=0.05), rnd(4096, 512, scale=0.05, seed=3)
    y2 = nat.gemm(x2, wg, wu)
    close(y2, torch.nn.functional.silu(x2.float() @ wg.float().T) * (x2.float() @ wu.float().T))
    w4 = rnd(2048, 1088, scale=0.05, seed=11)          # between one and two waves of 256-token tiles: 128-token tiles instead
    y4 = nat.gemm(x, w4)
    close(y4, x.float() @ w4.float().T, tol=1e-2)
    T, E, k, d, F = 2048, 64, 6, 1024, 768
    xm = rnd(T, d)
    eg, eu, ed = rnd(E, F, d, scale=0.05), rnd(E, F, d, scale=0.05, seed=5), rnd(E, d, F, scale=0.05)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(DEV)
    wts = torch.rand(T, k, generator=g).to(DEV)
    y3 = nat.moe_experts(xm, ids, wts, eg, eu, ed, 0)
    close(y3, ref.moe_experts(xm, ids, wts, eg, eu, ed, 0), tol=3e-2)
    nat.check_status()
    # a rank's share of every DeepSeek-V2 expert at TP 8 (192 of 1536 FFN columns: a ragged second feature tile for gate|up,
    # three k-blocks for down) at prompt-chunk size
    T, E, k, d, F = 1024, 160, 6, 5120, 192
    xm = rnd(T, d, scale=0.3)
    eg, eu, ed = rnd(E, F, d, scale=0.02), rnd(E, F, d, scale=0.02, seed=5), rnd(E, d, F, scale=0.05)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(DEV)
    wts = torch.rand(T, k, generator=g).to(DEV)
    y5 = nat.moe_experts(xm, ids, wts, eg, eu, ed, 0)
    close(y5, ref.moe_experts(xm, ids, wts, eg, eu, ed, 0), tol=3e-2)
    nat.check_status()
    # the same three through the other kernel (the switch is read once per process by the library: a child process)
    import subprocess, sys
    code = ("import torch, sys; sys.path.insert(0, %r); from tests.test_gpu_kernels import rnd, DEV; from jittorinfer_b200.ops import native as nat; nat.load();"
            "x, w, res = rnd(2000, 1088), rnd(5120, 1088, scale=0.05), rnd(2000, 5120, seed=7);"
            "x2, wg, wu = rnd(1500, 512), rnd(4096, 512, scale=0.05), rnd(4096, 512, scale=0.05, seed=3);"
            "w4 = rnd(2048, 1088, scale=0.05, seed=11);"
            "torch.save([nat.gemm(x, w, residual=res).cpu(), nat.gemm(x2, wg, wu).cpu(), nat.gemm(x, w4).cpu()], sys.argv[1]); nat.check_status()") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import tempfile
    with tempfile.TemporaryDirectory() as td:
        out = os.path.join(td, "o.pt")
        subprocess.run([sys.executable, "-c", code, out], check=True, env=dict(os.environ, JIB_GEMM_PERSIST="0"), timeout=300)
        a, b, c4 = torch.load(out)
    assert torch.equal(a, y.cpu()) and torch.equal(b, y2.cpu()) and torch.equal(c4, y4.cpu())


def test_gemm_strided_rows(nat):
    big = rnd(9, 1000)
    x = big[:, 104:104 + 512]            # row stride 1000, 16-byte aligned start
    w = rnd(256, 512, scale=0.05)
    close(nat.gemm(x, w), x.float() @ w.float().T)


@pytest.mark.parametrize("T", [1, 8, 70])
def test_q_absorb_v_up(nat, T):
    H, dn, dr, r, dv = 16, 128, 64, 512, 128
    q = rnd(T, H * (dn + dr))
    w_uk = rnd(H, r, dn, scale=0.05)
    q_out = torch.zeros(T, H, r + dr, dtype=torch.bfloat16, device=DEV)
    q_nope = q.view(T, H, dn + dr)[..., :dn]
    nat.q_absorb(q_nope, w_uk, q_out, r)
    exp = torch.zeros_like(q_out)
    ref.q_absorb(q_nope, w_uk, exp, r)
    close(q_out[..., :r], exp[..., :r])
    assert q_out[..., r:].abs().max().item() == 0
    o_lat, w_uv = rnd(T, H, r), rnd(H, dv, r, scale=0.05)
    close(nat.v_up(o_lat, w_uv), ref.v_up(o_lat, w_uv))
    nat.check_status()


@pytest.mark.parametrize("T,E,k,d,F", [(1, 8, 2, 512, 384), (8, 64, 6, 512, 384), (50, 64, 6, 512, 384), (300, 16, 4, 512, 384),
                                       (8, 160, 6, 5120, 192), (1, 160, 6, 5120, 192)])     # last two: a rank's share of every
def test_moe_routed(nat, T, E, k, d, F):                                                     # DeepSeek-V2 expert at TP 8
    x = rnd(T, d)
    wg, wu, wd = rnd(E, F, d, scale=0.05), rnd(E, F, d, scale=0.05, seed=5), rnd(E, d, F, scale=0.05)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(DEV)
    wts = torch.rand(T, k, generator=g).to(DEV)
    for base, El in ((0, E), (E // 2, E // 2)):       # all experts local / second half local (expert parallel)
        out = nat.moe_experts(x, ids, wts, wg[base:base + El].contiguous(), wu[base:base + El].contiguous(),
                              wd[base:base + El].contiguous(), base)
        exp = ref.moe_experts(x, ids, wts, wg[base:base + El], wu[base:base + El], wd[base:base + El], base)
        close(out, exp, tol=3e-2)
    nat.check_status()


def test_moe_permute_is_stable_sort(nat):
    T, k, E = 37, 6, 64
    g = torch.Generator().manual_seed(1)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(DEV)
    seg, src, dest = nat.moe_permute(ids, 0, E)
    flat = ids.flatten().cpu()
    order = torch.sort(flat, stable=True).indices
    assert torch.equal(src.cpu(), (order // k).int())
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(seg.cpu()[1:] - seg.cpu()[:-1], counts.int())
    inv = torch.empty_like(order)
    inv[order] = torch.arange(T * k)
    assert torch.equal(dest.flatten().cpu(), inv.int())


@pytest.mark.parametrize("E,k,ng,tg,sig", [(64, 6, 1, 1, False), (160, 6, 8, 3, False), (8, 2, 1, 1, False), (16, 4, 4, 2, True)])
def test_moe_gate(nat, E, k, ng, tg, sig):
    T, d = 9, 2048
    g = rnd(T, d)
    wr = rnd(E, d, dtype=torch.float32, scale=0.05)
    ids, w = nat.moe_gate(g, wr, None, k, ng, tg, 16.0, False, sig)
    ids2, w2 = ref.moe_gate(g, wr, None, k, ng, tg, 16.0, False, sig)
    assert torch.equal(ids.cpu(), ids2.cpu())
    close(w, w2, tol=1e-4)
    ids, w = nat.moe_gate(g, wr, None, k, ng, tg, 1.0, True, sig)
    ids2, w2 = ref.moe_gate(g, wr, None, k, ng, tg, 1.0, True, sig)
    close(w, w2, tol=1e-4)
    # shared experts appended as always-selected experts E, E+1 with weight 1
    ids, w = nat.moe_gate(g, wr, None, k, ng, tg, 16.0, False, sig, 2)
    ids2, w2 = ref.moe_gate(g, wr, None, k, ng, tg, 16.0, False, sig, 2)
    assert ids.shape == (T, k + 2) and torch.equal(ids.cpu(), ids2.cpu())
    assert torch.equal(ids[:, k:].cpu(), torch.tensor([[E, E + 1]], dtype=torch.int32).expand(T, 2))
    close(w, w2, tol=1e-4)


@pytest.mark.parametrize("d", [512, 1536, 2048, 5120])
def test_rmsnorm(nat, d):
    x, r, w = rnd(11, d), rnd(11, d), rnd(d, dtype=torch.float32) + 1
    n, s = nat.rmsnorm(x, w, 1e-6, r)
    n2, s2 = ref.rmsnorm(x, w, 1e-6, r)
    assert torch.equal(s, s2)
    close(n, n2, tol=1e-2)
    n, _ = nat.rmsnorm(x, w, 1e-6)
    close(n, ref.rmsnorm(x, w, 1e-6)[0], tol=1e-2)


def test_mla_qkv_post_and_embed(nat):
    T, H, dn, dr, r = 10, 16, 128, 64, 512
    q, ckv, w = rnd(T, H * (dn + dr)), rnd(T, r + dr), rnd(r, dtype=torch.float32) + 1
    table = ref.yarn_table(256, dr, 10000.0, 0.025, 1.0, 0.73, 10, 23, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV) * 7
    slots = torch.tensor([5, 3, -1, 9, 64, 65, 66, 0, 1, 127], dtype=torch.int32, device=DEV)
    c1 = torch.zeros(128, r + dr, dtype=torch.bfloat16, device=DEV)
    c2 = c1.clone()
    q1 = torch.zeros(T, H, r + dr, dtype=torch.bfloat16, device=DEV)
    q2 = q1.clone()
    nat.mla_qkv_post(q, ckv, w, 1e-6, table, pos, slots, c1, q1, H, dn, dr, r)
    ref.mla_qkv_post(q, ckv, w, 1e-6, table, pos, slots, c2, q2, H, dn, dr, r)
    close(c1, c2, tol=1e-2)
    close(q1, q2, tol=1e-2)
    emb = rnd(1000, 256)
    ids = torch.randint(0, 1000, (33,), dtype=torch.int32, device=DEV)
    assert torch.equal(nat.embed_gather(emb, ids), emb[ids.long()])


@pytest.mark.parametrize("r,dr,H", [(512, 64, 16), (64, 16, 16), (512, 64, 32), (64, 16, 4)])
@pytest.mark.parametrize("lens,qlens", [([1], [1]), ([70, 300, 5, 129], [1, 1, 1, 1]), ([40, 200], [40, 73]), ([0, 33], [1, 1]),
                                        ([41, 200, 7], [41, 73, 1]), ([1000, 1500, 129, 64, 1], [1, 1, 1, 1, 1]), ([700], [300])])
def test_mla_attention(nat, r, dr, H, lens, qlens):
    bs = 64
    nb_per = 24
    B = len(lens)
    cache = rnd(B * nb_per * bs, r + dr)
    g = torch.Generator().manual_seed(7)
    perm = torch.randperm(B * nb_per, generator=g).view(B, nb_per).int().to(DEV)
    T = sum(qlens)
    q = rnd(T, H, r + dr, scale=0.3)
    qs = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    o = nat.mla_attention(q, cache, perm, sl, qs, 0.11, r, bs, max(qlens))
    o2 = ref.mla_attention(q, cache, perm, sl, qs, 0.11, r, bs)
    close(o, o2)


def test_argmax_topk(nat):
    x = rnd(6, 102400, dtype=torch.float32)
    x[2, 77] = 50.0
    x[3, 5] = x[3, 9] = 60.0       # tie -> lower index
    am = nat.argmax(x)
    assert am.tolist() == torch.argmax(x, -1).tolist() or am[3].item() == 5
    assert am[2].item() == 77 and am[3].item() == 5
    for k in (1, 40, 64):
        v, i = nat.topk_logits(x, k)
        v2, i2 = torch.topk(x, k, dim=-1)
        assert torch.equal(v, v2)
        assert torch.equal(torch.gather(x, 1, i.long()), v)


def test_kv_block_copy(nat):
    L, nb, bs, row = 3, 10, 64, 576
    cache = rnd(L, nb * bs, row)
    exp = cache.clone()
    src = torch.tensor([7, 9], dtype=torch.int32, device=DEV)
    dst = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    nat.kv_block_copy(cache, src, dst, bs)
    ref.kv_block_copy(exp, src, dst, bs)
    assert torch.equal(cache, exp)


@pytest.mark.parametrize("T,k,E", [(1024, 6, 64), (2048, 8, 66), (700, 6, 160)])
def test_moe_permute_multi_cta(nat, T, k, E):
    """Batches of 4096 pairs and more take the histogram / scan / scatter kernels: same stable sort by expert as the
    single-CTA kernel."""
    ids = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
    assert nat.PERMUTE_MULTI and T * k >= nat.PERMUTE_MULTI_MIN
    seg, src, dest = nat.moe_permute(ids, 0, E)
    flat = ids.flatten().long().cpu()
    order = torch.sort(flat, stable=True).indices
    inv = torch.empty_like(order)
    inv[order] = torch.arange(T * k)
    assert torch.equal(dest.flatten().cpu().long(), inv)
    assert torch.equal(src.cpu().long(), order // k)
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(seg.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))


@pytest.mark.parametrize("T,d,E,k,n_group,topk_group,n_shared,base,E_local",
                         [(1, 2048, 64, 6, 1, 1, 2, 0, 66), (8, 2048, 64, 6, 1, 1, 2, 0, 66), (64, 2048, 64, 6, 1, 1, 0, 0, 64),
                          (8, 5120, 160, 6, 8, 3, 0, 40, 20), (33, 5120, 160, 6, 8, 3, 0, 0, 160)])
def test_fused_route_matches_the_separate_kernels(nat, T, d, E, k, n_group, topk_group, n_shared, base, E_local):
    """[RMSNorm +] router logits + gating + expert sort in one launch (decode batches): bitwise the ids, weights, sort
    (and normalised rows) of the separate launches; a second call checks that the last-CTA counter was left at zero."""
    y = rnd(T, d)
    w_router = torch.randn(E, d, device=DEV, dtype=torch.float32) * 0.05
    w_norm = torch.rand(d, device=DEV, dtype=torch.float32) + 0.5
    saved = nat.FUSED_ROUTE
    try:
        for pre in (None, (w_norm, 1e-6), None):
            nat.FUSED_ROUTE = False
            g = y if pre is None else nat.rmsnorm(y, pre[0], pre[1])[0]
            ids0, wts0 = nat.moe_gate(g, w_router, None, k, n_group, topk_group, 1.0, False, False, n_shared)
            seg0, src0, dest0 = nat.moe_permute(ids0, base, E_local)
            nat.FUSED_ROUTE = True
            res = nat.moe_gate(y, w_router, None, k, n_group, topk_group, 1.0, False, False, n_shared, False, (base, E_local), pre)
            ids1, wts1 = res[0], res[1]
            seg1, src1, dest1 = nat.moe_permute(ids1, base, E_local)
            torch.cuda.synchronize()
            assert not nat._route_stash                       # the sort came from the fused launch
            if pre is not None:
                assert torch.equal(res[2], g)                 # the rows the router normalised = the norm kernel's rows
            assert torch.equal(ids0, ids1) and torch.equal(wts0, wts1)
            assert torch.equal(seg0, seg1) and torch.equal(dest0, dest1)
            n_local = int(seg0[-1])
            assert torch.equal(src0[:n_local], src1[:n_local]) and bool((src1[n_local:] == -1).all())
            assert int(nat.workspace(y.device).route_counter.item()) == 0
    finally:
        nat.FUSED_ROUTE = saved


def test_gate_matches_the_fp32_reference(nat):
    """ids of the gate kernel against the PyTorch restatement (softmax top-k, group-limited variant)."""
    for T, d, E, k, ng, tg in ((8, 2048, 64, 6, 1, 1), (33, 5120, 160, 6, 8, 3)):
        g = rnd(T, d)
        w_router = torch.randn(E, d, device=DEV, dtype=torch.float32) * 0.05
        ids, wts = nat.moe_gate(g, w_router, None, k, ng, tg, 1.0, False, False, 0)
        ids_r, wts_r = ref.moe_gate(g, w_router, None, k, ng, tg, 1.0, False, False, 0)
        assert torch.equal(ids.sort(-1).values, ids_r.sort(-1).values)
        close(wts.sort(-1).values, wts_r.sort(-1).values, tol=1e-4)


@pytest.mark.parametrize("T,E,k,F,d", [(1, 66, 8, 1408, 2048), (8, 66, 8, 1408, 2048), (33, 66, 8, 1408, 2048), (64, 20, 6, 1536, 5120),
                                       (5, 8, 2, 128, 256)])
def test_grouped_gateup_reads_tokens_in_place(nat, T, E, k, F, d):
    """Decode batches: the grouped gate|up GEMM given the unsorted token rows and the sort's source index equals, bit for
    bit, the same GEMM over rows gathered into expert order (same split of K); both track the fp32 reference."""
    x = rnd(T, d)
    wg, wu = rnd(E, F, d, scale=0.03), rnd(E, F, d, scale=0.03, seed=9)
    gen = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(T)]).int().to(DEV)
    seg, src, dest = nat.moe_permute(ids, 0, E)
    active = min(E, T * k)
    for _ in range(2):
        h0 = nat.gemm_grouped(nat.gather_rows(x, src), seg, wg, wu, T, active)
        h1 = nat.gemm_grouped_raw(x.data_ptr(), T * k, d, seg, wg, wu, T, active, device=x.device, src_token=src, src_rows=T)
        torch.cuda.synchronize()
        assert torch.equal(h0, h1)
        if T * k < E:
            # few pairs: the launch covers the sort's list of experts that have rows instead of all E experts
            assert nat._seg_has_list(seg, E)
            h2 = nat.gemm_grouped_raw(x.data_ptr(), T * k, d, seg, wg, wu, T, active, device=x.device, src_token=src, src_rows=T,
                                      n_slots=T * k)
            h3 = nat.gemm_grouped(nat.gather_rows(x, src), seg, wg, wu, T, active, n_slots=T * k)
            torch.cuda.synchronize()
            assert torch.equal(h0, h2) and torch.equal(h0, h3)
    flat = ids.flatten().long()
    order = torch.sort(flat, stable=True).indices
    xs = x.float()[order // k]
    e_of = flat[order]
    want = torch.nn.functional.silu(torch.einsum("rd,rfd->rf", xs, wg.float()[e_of])) * torch.einsum("rd,rfd->rf", xs, wu.float()[e_of])
    close(h1, want, tol=3e-2)
    nat.check_status()


@pytest.mark.parametrize("T,k,d,with_shared", [(1, 8, 2048, False), (8, 8, 2048, False), (64, 6, 2048, True), (8, 6, 5120, True),
                                               (300, 6, 5120, False), (5, 6, 512, False)])
def test_combine_fused_with_the_next_norm(nat, T, k, d, with_shared):
    """Expert combine + the RMSNorm that follows it in one launch: the same two tensors as the two launches (the kernel
    keeps the reduction order of the norm kernel; a last-bit difference from instruction selection is tolerated)."""
    n_rows = T * k
    y = rnd(n_rows, d)
    dest = torch.randperm(n_rows, device=DEV).int().view(T, k)
    dest[0, 0] = -1                                       # a pair whose expert lives elsewhere
    wts = torch.rand(T, k, device=DEV, dtype=torch.float32)
    shared = rnd(T, d) if with_shared else None
    residual = rnd(T, d)
    w = torch.rand(d, device=DEV, dtype=torch.float32) + 0.5
    out0 = nat.moe_combine(y, dest, wts, shared, residual)
    norm0, _ = nat.rmsnorm(out0, w, 1e-6)
    out1, norm1 = nat.moe_combine(y, dest, wts, shared, residual, norm=(w, 1e-6))
    torch.cuda.synchronize()
    assert torch.equal(out0, out1)
    assert (norm0.float() - norm1.float()).abs().max().item() <= 2 ** -7 * norm0.float().abs().max().item()
    assert (norm0 != norm1).float().mean().item() < 0.01


@pytest.mark.parametrize("k", [8, 64, 128])
def test_device_sampler_matches_the_reference(nat, k):
    """top-k / top-p / min-p / temperature + one draw per row: the ids of the PyTorch fp32 restatement, except for draws
    that land within rounding distance of a boundary."""
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    vals = torch.sort(torch.randn(n, k, device=DEV, generator=g) * 2.5, dim=-1, descending=True).values.contiguous()
    ids = torch.stack([torch.randperm(50000, device=DEV, generator=g)[:k] for _ in range(8)]).repeat(n // 8, 1).int().contiguous()
    params = torch.zeros(n, 5, device=DEV)
    params[:, 0] = torch.tensor([0.0, 0.6, 1.0, 1.7], device=DEV).repeat(n // 4)
    params[:, 1] = torch.tensor([0.0, 5.0, 40.0, 500.0], device=DEV).repeat_interleave(n // 4)
    params[:, 2] = torch.rand(n, device=DEV, generator=g).clamp(0.2, 1.0)
    params[:, 3] = torch.rand(n, device=DEV, generator=g) * 0.1 * (torch.rand(n, device=DEV, generator=g) < 0.5)
    params[:, 4] = torch.rand(n, device=DEV, generator=g)
    got = nat.sample_topk(vals, ids, params)
    want = ref.sample_topk(vals, ids, params)
    torch.cuda.synchronize()
    agree = (got == want).float().mean().item()
    assert agree > 0.995, agree
    greedy = params[:, 0] <= 0
    assert torch.equal(got[greedy], ids[greedy, 0])


def test_device_dequantize_matches_the_host_expander():
    import numpy as np
    from jittorinfer_b200.gguf import quants as Q
    from jittorinfer_b200.ops import native
    rng = np.random.default_rng(0)
    for t, (blk, bsz) in Q.TRAITS.items():
        x = rng.standard_normal(blk * 4099).astype(np.float32)          # an odd number of blocks: the last thread block is partial
        raw = Q.quantize(t, x)
        want = Q.dequantize_torch(t, raw.reshape(-1, bsz), torch.bfloat16)
        got = native.dequantize_bf16(torch.from_numpy(raw).cuda(), t, x.size).cpu()
        diff = (got.float() - want.float()).abs()
        assert float((diff / want.float().abs().clamp_min(1e-3)).max()) < 1e-2, Q.NAMES[t]      # fused multiply-add may move one bf16 ulp
        assert float((got != want).float().mean()) < 1e-3, Q.NAMES[t]


@pytest.mark.parametrize("lens", [[(130, 130)], [(300, 300), (64, 64)], [(128, 400), (200, 200), (70, 1000)]])
def test_prefill_attention_per_head_form(nat, lens):
    """Prompt-chunk attention over K / V expanded from the cached latent rows (tcgen05, queries on the M axis) against an
    fp32 restatement: several sequences per batch, chunks that continue a cached prefix (query rows are the LAST rows of a
    sequence), partial tiles, block tables in scrambled order."""
    H, dn, dr, dv, r, bs = 16, 128, 64, 128, 512, 64
    g = torch.Generator().manual_seed(len(lens))
    n_seqs = len(lens)
    S_all = [s for _, s in lens]
    n_blocks = sum((s + bs - 1) // bs for s in S_all) + 3
    cache = (torch.randn(n_blocks * bs, r + dr, generator=g) * 0.5).bfloat16().to(DEV)
    perm = torch.randperm(n_blocks - 1, generator=g) + 1
    max_blocks = max((s + bs - 1) // bs for s in S_all)
    bt = torch.zeros(n_seqs, max_blocks, dtype=torch.int32)
    used = 0
    for b, s in enumerate(S_all):
        nb = (s + bs - 1) // bs
        bt[b, :nb] = perm[used:used + nb].int()
        used += nb
    T = sum(q for q, _ in lens)
    q = (torch.randn(T, H * (dn + dr), generator=g) * 0.5).bfloat16().to(DEV)
    w_kv_b = (torch.randn(H * (dn + dv), r, generator=g) * 0.05).bfloat16().to(DEV)
    q_start = torch.tensor([0] + list(torch.tensor([ql for ql, _ in lens]).cumsum(0)), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(S_all, dtype=torch.int32, device=DEV)
    scale = 0.07
    meta = {"total_kv": sum(S_all), "n_q_tiles": sum((ql + 127) // 128 for ql, _ in lens)}
    out = nat.mha_prefill(q, cache, w_kv_b, bt.to(DEV), seq_lens, q_start, scale, H, bs, meta)
    torch.cuda.synchronize()
    nat.check_status()
    # reference
    row0 = 0
    for b, (ql, S) in enumerate(lens):
        slots = torch.cat([bt[b, i].long() * bs + torch.arange(bs) for i in range((S + bs - 1) // bs)])[:S].to(DEV)
        lat = cache[slots].float()
        kv = (lat[:, :r] @ w_kv_b.float().T).bfloat16().float().view(S, H, dn + dv)      # the kernel reads the bf16 expansion
        k = torch.cat([kv[..., :dn], lat[:, None, r:].expand(S, H, dr)], dim=-1)
        v = kv[..., dn:]
        qq = q[row0:row0 + ql].float().view(ql, H, dn + dr)
        s = torch.einsum("thd,shd->hts", qq, k) * scale
        pos = torch.arange(S - ql, S, device=DEV)
        mask = torch.arange(S, device=DEV)[None, :] > pos[:, None]
        s = s.masked_fill(mask[None], float("-inf"))
        want = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), v).reshape(ql, H * dv)
        got = out[row0:row0 + ql].float()
        err = (got - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 1e-3, (b, err, want.abs().max().item())
        row0 += ql
