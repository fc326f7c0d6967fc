"""Interleaving model of the peer-memory protocols (no GPU, no processes).

The fused collectives never reset a flag and reuse two buffer halves, so their safety rests on an ordering argument: a
rank can run ahead of the slowest rank only until its next wait, and that is never far enough to overwrite data somebody
has yet to read.  Here every rank is a little program of single memory operations (store a tagged value into a peer's
buffer, store a flag, wait for flags, load and check a tag) and a scheduler runs the ranks in random orders -- thousands
of interleavings per protocol, including "one rank races ahead as far as it can".  A load that sees a value written for
another call site or another step is a protocol bug.  The programs mirror the kernels:

* one-shot all-reduce (comm_fused.cu / the GEMM epilogue, ``args.ar``): push to every peer, signal, wait, reduce;
* two-shot all-reduce and its reduce-scatter form (partials to a tile owner, delivery to all ranks / to the row owner);
* expert-parallel all-to-all (ep_alltoall.cu): counts, rows, returned outputs, three flag phases per call site;
* the sequence-parallel layer (all-gather, GEMM+reduce-scatter, all-gather, reduce-scatter) with the gather buffer
  indexed by ``(site >> 1) & 1`` and the reduce buffers by ``site & 1``.

What the model cannot show is memory ordering inside one GPU (release/acquire, proxy fences): that is by construction
in the kernels (``st.release.sys`` after ``__threadfence_system``, ``ld.acquire.sys`` before the loads).
"""
import random

import pytest


class Sim:
    """Shared memory = dict; ranks = generators yielding ("store", key, value) | ("wait", fn) | ("check", key, value)."""

    def __init__(self, programs, seed, bias=None):
        self.mem = {}
        self.programs = programs
        self.pending = [None] * len(programs)
        self.done = [False] * len(programs)
        self.rng = random.Random(seed)
        self.bias = bias                    # rank that is scheduled whenever it can run (races ahead)
        self.steps = 0

    def _next(self, r):
        if self.pending[r] is None and not self.done[r]:
            try:
                self.pending[r] = next(self.programs[r])
            except StopIteration:
                self.done[r] = True
        return self.pending[r]

    def _runnable(self, r):
        op = self._next(r)
        if op is None:
            return False
        return op[0] != "wait" or op[1](self.mem)

    def run(self, max_steps=2_000_000):
        n = len(self.programs)
        while not all(self.done):
            ready = [r for r in range(n) if self._runnable(r)]
            if not ready and all(self.done):
                break
            assert ready, "deadlock: every rank waits"
            if self.bias is not None and self.bias in ready and self.rng.random() < 0.9:
                r = self.bias
            else:
                r = self.rng.choice(ready)
            op = self.pending[r]
            self.pending[r] = None
            if op[0] == "store":
                self.mem[op[1]] = op[2]
            elif op[0] == "check":
                got = self.mem.get(op[1])
                assert got == op[2], f"rank {r}: {op[1]} holds {got}, expected {op[2]}"
            self.steps += 1
            assert self.steps < max_steps


def parity(site, n_sites, epoch):
    return (site + (epoch % 2) * (n_sites & 1)) & 1


# ---- programs ---------------------------------------------------------------------------------------------------------
def one_shot(rank, world, n_sites, n_epochs):
    for epoch in range(1, n_epochs + 1):
        for site in range(n_sites):
            par = parity(site, n_sites, epoch)
            for p in range(world):
                yield ("store", ("recv", p, par, rank), (epoch, site))
            for p in range(world):
                yield ("store", ("flag", p, site, rank), epoch)
            yield ("wait", lambda m, s=site, e=epoch: all(m.get(("flag", rank, s, src)) == e for src in range(world)))
            for src in range(world):
                yield ("check", ("recv", rank, par, src), (epoch, site))


def two_shot(rank, world, n_sites, n_epochs, n_tiles=3, rows_per_rank=0):
    """rows_per_rank > 0: reduce-scatter form -- tile t's result is delivered to rank (t % world) only ("row owner"),
    which is the only one that reads it; every rank still waits for the owner's delivery flag."""
    for epoch in range(1, n_epochs + 1):
        for site in range(n_sites):
            par = site & 1
            for tile in range(n_tiles):
                owner = (tile + site) % world
                yield ("store", ("recv2", owner, par, tile, rank), (epoch, site))
                yield ("store", ("flag", owner, site, tile, rank), epoch)
                if rank == owner:
                    yield ("wait", lambda m, s=site, t=tile, e=epoch: all(m.get(("flag", rank, s, t, src)) == e for src in range(world)))
                    for src in range(world):
                        yield ("check", ("recv2", rank, par, tile, src), (epoch, site))
                    targets = [tile % world] if rows_per_rank else range(world)
                    for p in targets:
                        yield ("store", ("out2", p, par, tile), (epoch, site))
                    for p in range(world):
                        yield ("store", ("flag2", p, site, tile), epoch)
                yield ("wait", lambda m, s=site, t=tile, e=epoch: m.get(("flag2", rank, s, t)) == e)
            # the consumer (next kernel on the stream) reads the result after the whole kernel
            for tile in range(n_tiles):
                if not rows_per_rank or tile % world == rank:
                    yield ("check", ("out2", rank, par, tile), (epoch, site))


def ep_layer(rank, world, n_sites, n_epochs):
    for epoch in range(1, n_epochs + 1):
        for site in range(n_sites):
            par = parity(site, n_sites, epoch)
            tag = (epoch, site)
            for p in range(world):                                   # plan: counts to everybody
                yield ("store", ("counts", p, par, rank), tag)
            for p in range(world):
                yield ("store", ("f0", p, site, rank), epoch)
            yield ("wait", lambda m, s=site, e=epoch: all(m.get(("f0", rank, s, src)) == e for src in range(world)))
            for src in range(world):
                yield ("check", ("counts", rank, par, src), tag)
            for p in range(world):                                   # push: my rows into the owners' buffers
                yield ("store", ("xrecv", p, par, rank), tag)
            for p in range(world):
                yield ("store", ("f1", p, site, rank), epoch)
            yield ("wait", lambda m, s=site, e=epoch: all(m.get(("f1", rank, s, src)) == e for src in range(world)))
            for src in range(world):                                 # expert GEMMs read what arrived ...
                yield ("check", ("xrecv", rank, par, src), tag)
            for src in range(world):                                 # ... and store the results into the sources
                yield ("store", ("yret", src, par, rank), tag)
            for p in range(world):                                   # combine: signal, wait, read
                yield ("store", ("f2", p, site, rank), epoch)
            yield ("wait", lambda m, s=site, e=epoch: all(m.get(("f2", rank, s, src)) == e for src in range(world)))
            for owner in range(world):
                yield ("check", ("yret", rank, par, owner), tag)


def sp_layers(rank, world, n_layers, n_epochs, final_site=None):
    """Per layer: all-gather (site 4l), GEMM+reduce-scatter (4l+1), all-gather (4l+2), reduce-scatter (4l+3); after the
    last layer one more all-gather (the rows for the output head) at ``final_site`` (default 4 * n_layers + 2, whose
    gather-buffer half differs from the half the next pass's first gather uses)."""
    if final_site is None:
        final_site = 4 * n_layers + 2
    def gather(site, epoch):
        par = (site >> 1) & 1
        for p in range(world):
            yield ("store", ("xg", p, par, rank), (epoch, site))
        for p in range(world):
            yield ("store", ("f3", p, site, rank), epoch)
        yield ("wait", lambda m: all(m.get(("f3", rank, site, src)) == epoch for src in range(world)))
        for src in range(world):
            yield ("check", ("xg", rank, par, src), (epoch, site))

    for epoch in range(1, n_epochs + 1):
        for layer in range(n_layers):
            for which, site in enumerate(range(4 * layer, 4 * layer + 4)):
                if which % 2 == 0:
                    yield from gather(site, epoch)
                else:
                    par = site & 1
                    owner = site % world                         # one tile per call site, its owner rotates
                    yield ("store", ("recv2", owner, par, rank), (epoch, site))
                    yield ("store", ("flag", owner, site, rank), epoch)
                    if rank == owner:
                        yield ("wait", lambda m, s=site, e=epoch: all(m.get(("flag", rank, s, src)) == e for src in range(world)))
                        for src in range(world):
                            yield ("check", ("recv2", rank, par, src), (epoch, site))
                        for p in range(world):                   # each rank's rows of the tile
                            yield ("store", ("out2", p, par), (epoch, site))
                        for p in range(world):
                            yield ("store", ("flag2", p, site), epoch)
                    yield ("wait", lambda m, s=site, e=epoch: m.get(("flag2", rank, s)) == e)
                    yield ("check", ("out2", rank, par), (epoch, site))
        yield from gather(final_site, epoch)


PROTOCOLS = {
    "one_shot_even_sites": lambda r, w: one_shot(r, w, 4, 3),
    "one_shot_odd_sites": lambda r, w: one_shot(r, w, 3, 4),
    "two_shot": lambda r, w: two_shot(r, w, 4, 3),
    "two_shot_reduce_scatter": lambda r, w: two_shot(r, w, 4, 3, rows_per_rank=1),
    "ep_all_to_all_even_sites": lambda r, w: ep_layer(r, w, 2, 3),
    "ep_all_to_all_odd_sites": lambda r, w: ep_layer(r, w, 3, 4),
    "sequence_parallel_layers": lambda r, w: sp_layers(r, w, 2, 3),
}


@pytest.mark.parametrize("name", sorted(PROTOCOLS))
@pytest.mark.parametrize("world", [2, 4])
def test_no_interleaving_reads_stale_or_overwritten_data(name, world):
    for seed in range(60):
        Sim([PROTOCOLS[name](r, world) for r in range(world)], seed).run()
    for fast in range(world):                                   # one rank always runs when it can
        for seed in range(10):
            Sim([PROTOCOLS[name](r, world) for r in range(world)], 1000 + seed, bias=fast).run()


def test_the_model_catches_a_final_gather_that_shares_its_half_with_the_next_pass():
    """The gather after the last layer must not use the buffer half that the next forward pass's first gather uses: a
    rank that runs ahead would overwrite rows a slower rank has not read yet.  Site 4 * n_layers has that flaw (half 0,
    like site 0); the model finds it."""
    tripped = 0
    for seed in range(200):
        try:
            Sim([sp_layers(r, 2, 2, 3, final_site=8) for r in range(2)], seed, bias=seed % 2).run()
        except AssertionError:
            tripped += 1
    assert tripped > 0


def test_the_model_catches_a_protocol_without_double_buffering():
    """Sanity of the tool itself: with one buffer half instead of two, a rank that races ahead overwrites a slot that a
    slower rank has not reduced yet -- some interleaving must trip the check."""
    def single_buffer(rank, world, n_sites, n_epochs):
        for op in one_shot(rank, world, n_sites, n_epochs):
            if op[0] in ("store", "check") and op[1][0] == "recv":
                key = list(op[1])
                key[2] = 0                                       # every call site uses half 0
                op = (op[0], tuple(key), op[2])
            yield op

    tripped = 0
    for seed in range(200):
        try:
            Sim([single_buffer(r, 2, 4, 3) for r in range(2)], seed, bias=seed % 2).run()
        except AssertionError:
            tripped += 1
    assert tripped > 0


# ---- CTA residency: the two-shot epilogue when a launch has more tiles than the GPU holds CTAs ----------------------------
# A resident CTA of tile t sends its partial to the tile's owner; on the owner it then waits for every rank's partial of
# tile t, and everywhere it waits for the owner's delivery before it leaves and frees its slot.  With more tiles than
# slots, progress therefore needs the CTA of tile t to become resident on EVERY rank: guaranteed when all ranks dispatch
# their tiles in the same order (the hardware dispatches blockIdx in order, and every rank launches the same grid), not
# guaranteed for an arbitrary order.  The model: every rank has `slots` CTA slots and a dispatch order; a slot takes the
# next tile when its CTA has finished.
def _two_shot_resident(world, n_tiles, slots, orders, seed):
    rng = random.Random(seed)
    sent = set()            # (tile, src): partial stored at the owner
    delivered = set()       # tile: owner has reduced and delivered
    nxt = [0] * world       # next position in the rank's dispatch order
    res = [[] for _ in range(world)]      # resident CTAs: [tile, stage]  stage 0 = to send, 1 = sent (owner: to reduce), 2 = wait delivery
    done = [0] * world
    for _ in range(100000):
        moves = []
        for r in range(world):
            if len(res[r]) < slots and nxt[r] < n_tiles:
                moves.append(("dispatch", r, None))
            for cta in res[r]:
                t, st = cta
                owner = t % world
                if st == 0:
                    moves.append(("send", r, cta))
                elif st == 1 and r == owner and all((t, s) in sent for s in range(world)):
                    moves.append(("reduce", r, cta))
                elif (st == 2 or (st == 1 and r != owner)) and t in delivered:
                    moves.append(("leave", r, cta))
        if not moves:
            return all(d == n_tiles for d in done)
        kind, r, cta = rng.choice(moves)
        if kind == "dispatch":
            res[r].append([orders[r][nxt[r]], 0])
            nxt[r] += 1
        elif kind == "send":
            sent.add((cta[0], r))
            cta[1] = 1
        elif kind == "reduce":
            delivered.add(cta[0])
            cta[1] = 2
        else:
            res[r].remove(cta)
            done[r] += 1
    raise AssertionError("model did not terminate")


def test_two_shot_with_more_tiles_than_resident_ctas_needs_one_dispatch_order():
    world, n_tiles, slots = 4, 40, 3
    same = [list(range(n_tiles))] * world
    assert all(_two_shot_resident(world, n_tiles, slots, same, seed) for seed in range(200))
    # the assumption is load-bearing: one rank walking its tiles backwards fills its slots with tiles whose CTAs are not
    # resident elsewhere, and every rank ends up waiting (in the kernels such a wait is bounded and reports a timeout)
    mixed = [list(range(n_tiles))] * (world - 1) + [list(reversed(range(n_tiles)))]
    assert not any(_two_shot_resident(world, n_tiles, slots, mixed, seed) for seed in range(50))


# ---- the persistent GEMM's roles inside one CTA (gemm_persistent_kernel): TMA producer, MMA issuer, four epilogue warps ------------
# mbarriers are modelled as phase counters; a wait on parity P passes when the phase of parity P has completed, i.e. when the
# barrier's current phase has the other parity -- exactly what mbarrier.test_wait.parity answers.  Ring slots and accumulator
# sets carry tags, so a slot overwritten before the MMA read it, or an accumulator set reused before all four epilogue warps
# read it, shows as a wrong tag.
def _phase_wait(key, parity):
    return lambda mem: (mem.get(key, 0) & 1) != parity


def _persistent_roles(stages, num_kb, n_items, n_epi=4):
    def producer():
        it = 0
        for j in range(n_items):
            for kb in range(num_kb):
                s, ph = it % stages, (it // stages) & 1
                yield ("wait", _phase_wait(("empty", s), ph ^ 1))
                yield ("store", ("ring", s), (j, kb))
                yield ("add", ("full", s))                     # the TMA transaction completes the slot's phase
                it += 1

    def mma():
        it = 0
        for j in range(n_items):
            b = j & 1
            yield ("wait", _phase_wait(("acc_empty", b), ((j >> 1) & 1) ^ 1))
            for kb in range(num_kb):
                s, ph = it % stages, (it // stages) & 1
                yield ("wait", _phase_wait(("full", s), ph))
                yield ("check", ("ring", s), (j, kb))
                yield ("store", ("acc", b), (j, kb))
                yield ("add", ("empty", s))                    # tcgen05.commit: the slot may be refilled
                it += 1
            yield ("add", ("acc_ready", b))

    def epilogue(w):
        for j in range(n_items):
            b = j & 1
            yield ("wait", _phase_wait(("acc_ready", b), (j >> 1) & 1))
            yield ("check", ("acc", b), (j, num_kb - 1))
            yield ("arrive", ("acc_empty", b), n_epi)          # the phase completes with the fourth warp's arrival
    return [producer(), mma()] + [epilogue(w) for w in range(n_epi)]


class _PhaseSim(Sim):
    """Sim plus two barrier operations: "add" completes a phase, "arrive" completes one after `count` arrivals."""

    def run(self, max_steps=2_000_000):
        n = len(self.programs)
        while not all(self.done):
            ready = [r for r in range(n) if self._runnable(r)]
            if not ready and all(self.done):
                break
            assert ready, "deadlock: every role waits"
            r = self.bias if self.bias is not None and self.bias in ready and self.rng.random() < 0.9 else self.rng.choice(ready)
            op = self.pending[r]
            self.pending[r] = None
            if op[0] == "store":
                self.mem[op[1]] = op[2]
            elif op[0] == "check":
                assert self.mem.get(op[1]) == op[2], f"role {r} read {self.mem.get(op[1])} at {op[1]}, expected {op[2]}"
            elif op[0] == "add":
                self.mem[op[1]] = self.mem.get(op[1], 0) + 1
            elif op[0] == "arrive":
                k = ("pending",) + op[1]
                self.mem[k] = self.mem.get(k, 0) + 1
                if self.mem[k] == op[2]:
                    self.mem[k] = 0
                    self.mem[op[1]] = self.mem.get(op[1], 0) + 1
            self.steps += 1
            assert self.steps < max_steps


@pytest.mark.parametrize("stages,num_kb", [(3, 1), (4, 2), (4, 5), (6, 22), (4, 32)])
def test_persistent_gemm_pipeline_never_reads_a_slot_or_an_accumulator_out_of_turn(stages, num_kb):
    for seed in range(60):
        for bias in (None, 0, 1, 2):                           # also: the producer, the MMA issuer or one epilogue warp races ahead
            _PhaseSim(_persistent_roles(stages, num_kb, n_items=7), seed, bias).run()


def test_the_pipeline_model_catches_a_single_accumulator_set():
    """Without the second accumulator set (b = 0 for every tile, the wait parities unchanged) the MMA issuer overwrites what
    the epilogue has yet to read, or the roles block each other: the model has to notice."""
    def broken(stages, num_kb, n_items):
        roles = _persistent_roles(stages, num_kb, n_items)

        def one_set(gen):
            for op in gen:
                if len(op) > 1 and isinstance(op[1], tuple) and op[1][0] in ("acc", "acc_ready", "acc_empty"):
                    op = (op[0], (op[1][0], 0)) + tuple(op[2:])
                elif op[0] == "wait":
                    pass
                yield op
        return [one_set(g) for g in roles]
    with pytest.raises(AssertionError):
        for seed in range(40):
            _PhaseSim(broken(4, 2, 7), seed, 1).run()


# ---- the prompt-attention kernel's roles (mha_prefill_kernel): TMA producer, MMA issuer, four softmax warps ---------------------------
# K tiles are double-buffered, the V and P tiles single, S double-buffered in tensor memory; Q.K^T of tile t + 1 is issued before
# P.V of tile t.  Tags: ("K", t) in a K slot, ("V", t), ("S", t) in an S buffer, ("P", t).
def _mha_roles(n_tiles, n_smx=4, rescale_at=()):
    def producer():
        for t in range(n_tiles):
            s = t & 1
            yield ("wait", _phase_wait(("k_empty", s), ((t >> 1) & 1) ^ 1))
            yield ("store", ("K", s), t)
            yield ("add", ("k_full", s))
            yield ("wait", _phase_wait(("v_empty",), (t & 1) ^ 1))
            yield ("store", ("V",), t)
            yield ("add", ("v_full",))

    def mma():
        def pv(t):
            yield ("wait", _phase_wait(("p_full",), t & 1))
            yield ("wait", _phase_wait(("v_full",), t & 1))
            yield ("check", ("P",), t)
            yield ("check", ("V",), t)
            yield ("store", ("O",), t)
            yield ("add", ("o_done",))          # committed first: see the kernel
            yield ("add", ("v_empty",))
            yield ("add", ("p_empty",))
        for t in range(n_tiles):
            s, ph = t & 1, (t >> 1) & 1
            yield ("wait", _phase_wait(("k_full", s), ph))
            yield ("wait", _phase_wait(("s_empty", s), ph ^ 1))
            yield ("check", ("K", s), t)
            yield ("store", ("S", s), t)
            yield ("add", ("k_empty", s))
            yield ("add", ("s_full", s))
            if t >= 1:
                yield from pv(t - 1)
        yield from pv(n_tiles - 1)

    def softmax(w):
        for t in range(n_tiles):
            s = t & 1
            yield ("wait", _phase_wait(("s_full", s), (t >> 1) & 1))
            yield ("check", ("S", s), t)
            yield ("arrive", ("s_empty", s), n_smx)           # scores are in registers: the S buffer goes back at once
            if t in rescale_at and t > 0:                       # the exponent base moved: O is rescaled after the products in flight
                yield ("wait", _phase_wait(("o_done",), (t - 1) & 1))
                yield ("check", ("O",), t - 1)
            if t > 0:
                yield ("wait", _phase_wait(("p_empty",), (t - 1) & 1))
            if w == 0:
                yield ("store", ("P",), t)
            yield ("arrive", ("p_full",), n_smx)
        yield ("wait", _phase_wait(("o_done",), (n_tiles - 1) & 1))
        yield ("check", ("O",), n_tiles - 1)
    return [producer(), mma()] + [softmax(w) for w in range(n_smx)]


@pytest.mark.parametrize("n_tiles", [1, 2, 3, 8, 17])
def test_prompt_attention_pipeline_never_reads_a_tile_out_of_turn(n_tiles):
    """(This model found that the three barriers a P.V product completes must be completed with o_done first: with o_done last a
    softmax warp could see p_empty of product t, finish tile t + 1 and ask for o_done while that barrier was still a whole
    phase behind -- and a parity wait cannot tell "the phase before" from "this phase".)"""
    for seed in range(40):
        for bias in (None, 0, 1, 2):
            _PhaseSim(_mha_roles(n_tiles, rescale_at=(1, 2, 5, 16)), seed, bias).run()


# ---- the decode attention kernel's roles (mla_flash_kernel): TMA producer, MMA issuer, four softmax warps -------------------------------
# A ring of latent "pair" slots (4 pairs per KV tile, NPAIR slots) that BOTH products of a tile read, two slots for the rope
# chunk, one S buffer, one P buffer, O accumulated in place.
def _flash_roles(n_tiles, npair, n_smx=4):
    def producer():
        for it in range(n_tiles):
            s = it & 1
            yield ("wait", _phase_wait(("rope_free", s), ((it >> 1) & 1) ^ 1))
            yield ("store", ("rope", s), it)
            yield ("add", ("rope_full", s))
            for m in range(4):
                u = it * 4 + m
                s = u % npair
                yield ("wait", _phase_wait(("lat_free", s), ((u // npair) & 1) ^ 1))
                yield ("store", ("lat", s), (it, m))
                yield ("add", ("lat_full", s))

    def mma():
        for it in range(n_tiles):
            for m in range(4):
                u = it * 4 + m
                s = u % npair
                yield ("wait", _phase_wait(("lat_full", s), (u // npair) & 1))
                yield ("check", ("lat", s), (it, m))
            s = it & 1
            yield ("wait", _phase_wait(("rope_full", s), (it >> 1) & 1))
            yield ("check", ("rope", s), it)
            yield ("add", ("rope_free", s))
            yield ("store", ("S",), it)
            yield ("add", ("s_ready",))
            yield ("wait", _phase_wait(("p_ready",), it & 1))
            yield ("check", ("P",), it)
            for m in range(4):
                s = (it * 4 + m) % npair
                yield ("check", ("lat", s), (it, m))          # the second product reads the same copy of the tile
                yield ("add", ("lat_free", s))
            yield ("store", ("O",), it)
            yield ("add", ("o_ready",))

    def softmax(w):
        for it in range(n_tiles):
            yield ("wait", _phase_wait(("s_ready",), it & 1))
            yield ("check", ("S",), it)
            if it > 0:
                yield ("wait", _phase_wait(("o_ready",), (it - 1) & 1))
                yield ("check", ("O",), it - 1)                 # running-max correction of what the products so far left
            if w == 0:
                yield ("store", ("P",), it)
            yield ("arrive", ("p_ready",), n_smx)
        yield ("wait", _phase_wait(("o_ready",), (n_tiles - 1) & 1))
        yield ("check", ("O",), n_tiles - 1)
    return [producer(), mma()] + [softmax(w) for w in range(n_smx)]


@pytest.mark.parametrize("n_tiles,npair", [(1, 5), (2, 4), (3, 5), (9, 4), (10, 5)])
def test_decode_attention_pipeline_never_reads_a_tile_out_of_turn(n_tiles, npair):
    for seed in range(40):
        for bias in (None, 0, 1, 2):
            _PhaseSim(_flash_roles(n_tiles, npair), seed, bias).run()
