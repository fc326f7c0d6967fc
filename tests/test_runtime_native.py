"""Native host runtime: paged KV allocator and scheduler (no GPU)."""
import numpy as np
import torch

from jittorinfer_b200.runtime.engine import _StepIO
from jittorinfer_b200.runtime.native_rt import PagedKV, Scheduler


def test_kv_append_rm_cp_cow():
    kv = PagedKV(8, 4, 4)
    s = kv.append(0, 6)
    assert list(s) == [0, 1, 2, 3, 4, 5] and kv.used_blocks == 2
    assert kv.seq_cp(0, 1)                           # share prefix: refcounts bump, no new blocks
    assert kv.used_blocks == 2 and kv.refcount(0) == 2 and kv.seq_len(1) == 6
    s1 = kv.append(1, 1)                             # partially filled shared tail block -> copy-on-write
    src, dst = kv.take_copies()
    assert list(src) == [1] and list(dst) == [2] and s1[0] == 2 * 4 + 2
    assert kv.refcount(1) == 1 and kv.check()
    assert not kv.seq_rm(0, 1, 3)                    # hole in the middle is not representable
    assert kv.seq_rm(0, 4, -1) and kv.seq_len(0) == 4 and kv.check()
    assert kv.seq_rm(1, 0, -1) and kv.check()
    assert kv.append(2, 4 * 7) is not None and kv.append(3, 1) is None   # out of blocks: refused, unchanged
    assert kv.check()


def test_kv_defrag_compacts_and_keeps_tables_valid():
    kv = PagedKV(16, 4, 4)
    for s in range(4):
        kv.append(s, 12)
    kv.seq_rm(0, 0, -1)
    kv.seq_rm(2, 0, -1)
    frag = kv.fragmentation()
    assert frag > 0.4
    before = {s: kv.seq_len(s) for s in range(4)}
    src, dst = kv.defrag(64)
    assert len(src) > 0 and set(dst.tolist()).isdisjoint(src.tolist())
    assert kv.fragmentation() == 0.0 and kv.check()
    assert {s: kv.seq_len(s) for s in range(4)} == before
    assert max(max(kv.seq_blocks(1)), max(kv.seq_blocks(3))) < 6


def _run(sched, io, sample, max_steps=10000):
    out = {}
    for _ in range(max_steps):
        info = sched.step(io.arrays)
        n_tok, n_seq, n_out = int(info[0]), int(info[1]), int(info[2])
        if n_tok == 0:
            if sched.idle():
                break
            continue
        assert io.h["q_start"][n_seq] == n_tok
        toks = np.array([sample(r) for r in sched.out_reqs(n_out)], dtype=np.int32)
        sched.commit(toks, n_out)
        for rid, slot, tok, fin, npmt, ndec in sched.take_events():
            out.setdefault(rid, []).append((tok, fin))
    return out


def test_scheduler_chunked_prefill_budget_and_stop_rules():
    kv = PagedKV(64, 16, 4)
    sched = Scheduler(kv, 4, 32, 256, eos_id=7)
    io = _StepIO(32, 4, 16, torch.device("cpu"))
    sched.add(1, list(range(100, 170)), max_new=5)            # 70-token prompt: 32+32+6 chunks
    sched.add(2, [1, 2, 3], max_new=50)                       # stops on EOS
    sched.add(3, [4, 5], max_new=3, ignore_eos=True)
    out = _run(sched, io, lambda rid: 7 if rid in (2, 3) else 9)
    assert [t for t, _ in out[1]] == [9] * 5 and out[1][-1][1] == "length"
    assert out[2] == [(7, "stop")]
    assert [f for _, f in out[3]] == [None, None, "length"]
    st = sched.stats()
    assert st["finished"] == 3 and st["prompt_tokens"] == 75 and kv.check()


def test_scheduler_prefix_reuse_and_preemption():
    kv = PagedKV(12, 16, 2)
    sched = Scheduler(kv, 2, 64, 512, eos_id=-1)
    io = _StepIO(64, 2, 32, torch.device("cpu"))
    p = list(range(40))
    sched.add(1, p, max_new=2)
    _run(sched, io, lambda rid: 3)
    sched.add(2, p + [99, 98], max_new=2)                      # shares 40 cached tokens with the idle slot
    _run(sched, io, lambda rid: 3)
    assert sched.stats()["prefix_hits"] == 1
    # two long generations in a 12-block cache: the younger one is preempted, both still finish
    sched.add(3, list(range(60)), max_new=60)
    sched.add(4, list(range(60, 120)), max_new=60)
    out = _run(sched, io, lambda rid: 5)
    assert len(out[3]) == 60 and len(out[4]) == 60 and sched.stats()["preemptions"] >= 1 and kv.check()


def test_multi_cta_expert_sort_algorithm_matches_a_stable_sort():
    """Host restatement of the three-kernel expert sort used for large batches (per-chunk histogram, scan over chunks and
    experts, scatter with the rank inside the warp and the prefix over the warps of the chunk): the result must be the
    stable sort by expert that the single-CTA kernel produces, including pairs of experts this rank does not own."""
    import numpy as np
    rng = np.random.default_rng(0)
    for n, k, E_total, base, E_local in ((5000, 6, 64, 0, 64), (16384, 8, 66, 0, 66), (3000, 6, 160, 40, 20), (1024, 2, 8, 0, 8)):
        ids = rng.integers(0, E_total, size=n).astype(np.int64)
        le = ids - base
        le[(le < 0) | (le >= E_local)] = -1
        chunk = 1024
        n_chunks = (n + chunk - 1) // chunk
        tmp = np.zeros((n_chunks, E_local), dtype=np.int64)
        for c in range(n_chunks):                                         # permute_count_kernel
            part = le[c * chunk:(c + 1) * chunk]
            for e in part[part >= 0]:
                tmp[c, e] += 1
        total = tmp.sum(0)                                                # permute_scan_kernel
        tmp = np.cumsum(tmp, axis=0) - tmp
        seg = np.concatenate([[0], np.cumsum(total)])
        tmp += seg[:-1][None, :]
        dest = np.full(n, -1, dtype=np.int64)
        src = np.full(n, -1, dtype=np.int64)
        for c in range(n_chunks):                                         # permute_scatter_kernel
            warp_cnt = np.zeros((32, E_local), dtype=np.int64)
            ranks = {}
            for t in range(chunk):
                i = c * chunk + t
                if i >= n or le[i] < 0:
                    continue
                w, lane = divmod(t, 32)
                lanes = [l for l in range(32) if c * chunk + w * 32 + l < n and le[c * chunk + w * 32 + l] == le[i]]
                ranks[i] = (w, lanes.index(lane))
                warp_cnt[w, le[i]] = len(lanes)
            warp_off = np.cumsum(warp_cnt, axis=0) - warp_cnt
            for i, (w, r) in ranks.items():
                row = tmp[c, le[i]] + warp_off[w, le[i]] + r
                dest[i] = row
                src[row] = i // k
        owned = np.nonzero(le >= 0)[0]
        order = owned[np.argsort(le[owned], kind="stable")]
        want = np.full(n, -1, dtype=np.int64)
        want[order] = np.arange(len(order))
        assert np.array_equal(dest, want)
        assert np.array_equal(src[:len(order)], order // k) and np.all(src[len(order):] == -1)
        assert seg[-1] == len(order)


def test_scheduler_deferred_commit_gives_the_synchronous_events():
    """commit_deferred / resolve (the engine runs one step ahead of the sampled ids): the same requests, with a
    deterministic "sampler" that depends on the request and its step, end with the same tokens and reasons as with
    commit(); the unknown-token marker never survives in a slot's history; an end-of-sequence token costs exactly one
    extra fed token, whose output is dropped."""
    EOS = 7

    def sample(rid, n):                                  # request 2 produces the end-of-sequence token as its 4th token
        return EOS if (rid == 2 and n == 3) else 100 + 10 * rid + n

    def run(deferred):
        kv = PagedKV(64, 16, 4)
        sched = Scheduler(kv, 4, 64, 256, EOS)
        io = _StepIO(64, 4, 16, torch.device("cpu"))
        sched.add(1, list(range(20, 40)), max_new=9)
        sched.add(2, list(range(40, 45)), max_new=30)
        sched.add(3, list(range(50, 83)), max_new=3, ignore_eos=True)
        count, out, fed, pending = {}, {}, 0, None
        for _ in range(200):
            if pending is not None and deferred and sched.can_run_ahead():
                sched.commit_deferred(len(pending))
                info = sched.step(io.arrays)
                fed += int(info[0])
                nxt = None
                if int(info[0]):
                    assert (io.h["tokens"][:int(info[0])] == -2).all()          # only ids still on the device are fed
                    nxt = [int(r) for r in sched.out_reqs(int(info[2]))]
                toks = np.array([sample(r, count.setdefault(r, 0)) for r in pending], dtype=np.int32)
                for r in pending:
                    count[r] += 1
                sched.resolve(toks, len(pending))
                pending = nxt
            else:
                if pending is not None:
                    toks = np.array([sample(r, count.setdefault(r, 0)) for r in pending], dtype=np.int32)
                    for r in pending:
                        count[r] += 1
                    sched.commit(toks, len(pending))
                    pending = None
                else:
                    info = sched.step(io.arrays)
                    fed += int(info[0])
                    if int(info[0]) == 0 and sched.idle():
                        break
                    if int(info[2]):
                        pending = [int(r) for r in sched.out_reqs(int(info[2]))]
                    else:
                        sched.commit(np.empty(0, dtype=np.int32), 0)
            for rid, slot, tok, fin, npmt, ndec in sched.take_events():
                out.setdefault(rid, []).append((tok, fin))
        assert kv.check() and sched.idle()
        return out, fed

    sync, fed_sync = run(False)
    ahead, fed_ahead = run(True)
    assert sync == ahead
    assert [t for t, _ in sync[2]] == [120, 121, 122, EOS] and sync[2][-1][1] == "stop"
    assert len(sync[1]) == 9 and sync[1][-1][1] == "length" and len(sync[3]) == 3
    assert fed_ahead == fed_sync + 1                     # the token fed to request 2 after its end-of-sequence token


def test_scheduler_random_workloads_sync_and_deferred_agree():
    """Seeded random workloads (prompt lengths, token limits, end-of-sequence hits, cancellations, arrivals over time, a
    cache small enough to force eviction and preemption): the scheduler driven with commit() and the one driven with
    commit_deferred() / resolve() whenever can_run_ahead() allows give every request the same tokens and finish reason;
    the allocator stays consistent; no unknown-token marker is ever fed except as a step's device-fed input."""
    import random
    EOS = 3

    def sample(rid, n, eos_at):
        return EOS if eos_at.get(rid) == n else 10 + (rid * 7919 + n * 104729) % 900

    def run(seed, deferred):
        rng = random.Random(seed)
        n_slots = rng.choice([2, 3, 4])
        bs = rng.choice([4, 8, 16])
        kv = PagedKV(rng.choice([12, 24, 64]), bs, n_slots)
        n_ctx_slot = bs * rng.choice([4, 6])
        sched = Scheduler(kv, n_slots, rng.choice([8, 32]), n_ctx_slot, EOS)
        io = _StepIO(64, n_slots, n_ctx_slot // bs + 1, torch.device("cpu"))
        n_req = rng.randint(3, 9)
        arrivals, eos_at, cancels = {}, {}, {}
        common = [rng.randint(10, 900) for _ in range(2 * n_ctx_slot)]          # some prompts share a prefix, some exceed the slot
        for rid in range(1, n_req + 1):
            n_tok = rng.randint(1, n_ctx_slot - 2) if rng.random() < 0.8 else rng.randint(n_ctx_slot, 2 * n_ctx_slot)
            prompt = [rng.randint(10, 900) for _ in range(n_tok)]
            if rng.random() < 0.5:
                cut = rng.randint(1, n_tok)
                prompt[:cut] = common[:cut]
            arrivals.setdefault(rng.randint(0, 12), []).append((rid, prompt, rng.choice([-1, 1, 3, 9, 30]), rng.random() < 0.2))
            if rng.random() < 0.4:
                eos_at[rid] = rng.randint(0, 12)
            if rng.random() < 0.2:
                cancels[rid] = rng.randint(1, 25)
        count, out, pending, n_deferred = {}, {}, None, 0
        for it in range(600):
            done = False
            for rid, prompt, max_new, ign in arrivals.get(it, []):
                sched.add(rid, prompt, max_new=max_new, ignore_eos=ign)
            for rid, when in cancels.items():
                if when == it:
                    sched.cancel(rid)

            def ids_of(p):
                toks = np.array([sample(r, count.setdefault(r, 0), eos_at) for r in p], dtype=np.int32)
                for r in p:
                    count[r] += 1
                return toks
            if pending is not None and deferred and sched.can_run_ahead():
                sched.commit_deferred(len(pending))
                n_deferred += 1
                info = sched.step(io.arrays)
                nxt = [int(r) for r in sched.out_reqs(int(info[2]))] if int(info[0]) else None
                sched.resolve(ids_of(pending), len(pending))
                pending = nxt
            elif pending is not None:
                sched.commit(ids_of(pending), len(pending))
                pending = None
            else:
                info = sched.step(io.arrays)
                if int(info[0]) == 0:
                    done = sched.idle() and it > 14
                elif int(info[2]):
                    pending = [int(r) for r in sched.out_reqs(int(info[2]))]
                else:
                    sched.commit(np.empty(0, dtype=np.int32), 0)
            for rid, slot, tok, fin, npmt, ndec in sched.take_events():
                out.setdefault(rid, []).append((tok, fin))
            assert kv.check()
            if done:
                break
        assert sched.idle(), seed
        return out, n_deferred

    total_deferred = 0
    for seed in range(60):
        a, _ = run(seed, False)
        b, nd = run(seed, True)
        total_deferred += nd
        # a cancelled request may have produced one token more or less by the time the cancel lands (ids arrive a step
        # later when running ahead); everything else must be identical
        for rid in set(a) | set(b):
            ta, tb = a.get(rid, []), b.get(rid, [])
            if any(f == "cancelled" for _, f in ta + tb):
                n = min(len(ta), len(tb)) - 1
                assert [t for t, _ in ta[:n]] == [t for t, _ in tb[:n]], (seed, rid)
            else:
                assert ta == tb, (seed, rid, ta, tb)
    assert total_deferred > 100


def test_mixed_prompt_budget_bounds_prefill_next_to_decoding_sequences():
    """With a budget for prompt tokens in steps that also decode, a long prompt arriving while another request generates is
    fed in small chunks (the running request gets a token every step), and in full-size chunks once nothing decodes."""
    kv = PagedKV(64, 16, 4)
    sched = Scheduler(kv, 4, 64, 512, 2)
    sched.set_mixed_prompt_budget(8)
    io = _StepIO(64, 4, 33, torch.device("cpu"))
    sched.add(1, list(range(10, 20)), max_new=12, ignore_eos=True)
    info = sched.step(io.arrays)
    assert int(info[0]) == 10                               # nothing decodes yet: the whole prompt in one step
    sched.commit(np.array([50], dtype=np.int32), 1)
    sched.add(2, list(range(100, 200)), max_new=2, ignore_eos=True)
    sizes = []
    for _ in range(40):
        info = sched.step(io.arrays)
        n_tok, n_out = int(info[0]), int(info[2])
        if n_tok == 0:
            break
        sizes.append((n_tok, int(info[3])))                 # tokens in the step, decoding sequences in it
        sched.commit(np.full(n_out, 60, dtype=np.int32), n_out)
        sched.take_events()
    mixed = [n for n, dec in sizes if dec >= 1 and n > dec]
    assert mixed and max(mixed) <= 1 + 8                    # one decode token + at most 8 prompt tokens
    assert any(n > 9 and dec == 0 for n, dec in sizes)      # after request 1 ended, the rest of the prompt goes at full width
    assert kv.check()


def test_per_request_n_keep_decides_which_head_survives_a_cut():
    """A prompt longer than a slot loses whole chunks from its middle; the head that stays is the request's ``n_keep``
    (examples/server/server.cpp:90, 1390-1415 reads it per request), the scheduler's default when the request names none,
    and "as much of the prompt as fits" when it is negative -- also after a preemption re-queues the request."""
    def first_step_tokens(n_keep, default_keep=0):
        kv = PagedKV(64, 16, 2)
        sched = Scheduler(kv, 2, 512, 64, eos_id=7, n_keep=default_keep)
        io = _StepIO(512, 2, 8, torch.device("cpu"))
        sched.add(1, list(range(1000, 1200)), max_new=2, n_keep=n_keep)        # 200 tokens into a slot of 64
        info = sched.step(io.arrays)
        return io.h["tokens"][: int(info[0])].tolist()

    t0 = first_step_tokens(None)
    assert t0[0] != 1000 and t0[-1] == 1199 and len(t0) < 64               # default 0: nothing of the head is kept
    t5 = first_step_tokens(5)
    assert t5[:5] == [1000, 1001, 1002, 1003, 1004] and t5[5] > 1004 and t5[-1] == 1199 and len(t5) < 64
    assert first_step_tokens(None, default_keep=5) == t5                    # the engine-wide default does the same
    assert first_step_tokens(0, default_keep=5) == t0                       # and a request may ask for less
    tall = first_step_tokens(-1)
    assert tall[:60] == list(range(1000, 1060)) and tall[-1] == 1199 and len(tall) < 64
