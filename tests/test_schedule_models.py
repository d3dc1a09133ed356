"""CPU models of three pieces of device-side bookkeeping, checked against what the planner emits.

1. The mbarrier ring protocol of the inline fused kernel (TMA producer of x tiles -> transform warp
   groups taking k-blocks round-robin -> UMMA issuer, over a shared-memory ring and a tensor-memory
   slot ring).  A parity wait only tells "the phase with this parity has completed": a waiter that
   is two phases away from its barrier gets the wrong answer (it passes early, or blocks for ever).
   The model runs the agents under many interleavings and checks at every wait that the parity test
   agrees with what the waiter means.  It must pass for every ring the planner can emit and fail
   for ring depths that are not a multiple of the group count (the one GPU fault on record came
   from exactly that).

1b. The hand-over of a single-buffered accumulator in halves between the UMMA issuer and the
   epilogue warps of the plain GEMM (commits that arrive late and in order, 8 or 16 warps).

2. The tile split of the weight-streaming kernel (whole tiles, owners, donors): every
   (tile, k-block) is streamed exactly once, donors' slots are unique, and the contributor range
   an owner computes matches who really contributes.
"""

import itertools
import random

import pytest


# ------------------------------------------------------------------------------------------------
# 1. ring / phase model
# ------------------------------------------------------------------------------------------------
class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.completed = count, 0, 0

    def arrive(self):
        self.pending += 1
        if self.pending == self.count:
            self.pending, self.completed = 0, self.completed + 1

    def parity_test(self, parity):  # what mbarrier.try_wait.parity answers
        return (self.completed & 1) != parity


class Ring:
    def __init__(self, depth):
        self.depth, self.s, self.ph, self.passes = depth, 0, 0, 0

    def advance(self):
        self.s += 1
        if self.s == self.depth:
            self.s, self.ph, self.passes = 0, self.ph ^ 1, self.passes + 1


class Violation(AssertionError):
    pass


def x_producer(bars, a_stages, units):
    ring = Ring(a_stages)
    for _ in range(units):
        yield ("wait", bars["empty_a"][ring.s], ring.ph ^ 1, ring.passes)        # released `passes` times so far
        yield ("arrive", bars["full_a"][ring.s])
        ring.advance()


def transform_group(bars, g, groups, a_stages, a_slots, units):
    ring, slot = Ring(a_stages), Ring(a_slots)
    for it in range(units):
        if it % groups == g:
            yield ("wait", bars["full_a"][ring.s], ring.ph, ring.passes + 1)       # filled passes+1 times
            yield ("wait", bars["a_free"][slot.s], slot.ph ^ 1, slot.passes)
            yield ("arrive", bars["empty_a"][ring.s])
            yield ("arrive", bars["a_ready"][slot.s])
        ring.advance()
        slot.advance()


def issuer(bars, a_slots, units):
    slot = Ring(a_slots)
    for _ in range(units):
        yield ("wait", bars["a_ready"][slot.s], slot.ph, slot.passes + 1)
        yield ("arrive", bars["a_free"][slot.s])                                  # the UMMA's commit
        slot.advance()


def run_ring_model(a_stages, a_slots, groups, units, seed, bias=None):
    """Runs the agents under one interleaving; raises Violation on a wrong parity answer or a deadlock."""
    rng = random.Random(seed)
    bars = {name: [Barrier(1) for _ in range(n)] for name, n in
            (("full_a", a_stages), ("empty_a", a_stages), ("a_ready", a_slots), ("a_free", a_slots))}
    agents = [x_producer(bars, a_stages, units), issuer(bars, a_slots, units)]
    agents += [transform_group(bars, g, groups, a_stages, a_slots, units) for g in range(groups)]
    pending = [next(a, None) for a in agents]
    while any(op is not None for op in pending):
        live = [i for i, op in enumerate(pending) if op is not None]
        order = sorted(live, key=lambda i: (bias(i) if bias else 0, rng.random()))
        progressed = False
        for i in order:
            op = pending[i]
            if op[0] == "arrive":
                op[1].arrive()
            else:
                _, bar, parity, need = op
                says, means = bar.parity_test(parity), bar.completed >= need
                if says != means:
                    raise Violation(f"agent {i}: parity test says {says} but {bar.completed} phases are complete and {need} are needed")
                if not says:
                    continue
            pending[i] = next(agents[i], None)
            progressed = True
            break
        if not progressed:
            raise Violation("deadlock: every agent is blocked")


BIASES = [None, lambda i: -i, lambda i: i, lambda i: 0 if i >= 2 else 1, lambda i: 1 if i >= 2 else 0]


def check_ring(a_stages, a_slots, groups, units=37, seeds=6):
    for bias in BIASES:
        for seed in range(seeds):
            run_ring_model(a_stages, a_slots, groups, units, seed, bias)


def test_rings_the_planner_emits_keep_every_waiter_within_one_phase(native_lib):
    from autotune import native
    from autotune.runner.candidate import enumerate_grid

    seen = set()
    for c in enumerate_grid("rmsnorm_matmul", tile_k=(64, 128), stages=(1, 2, 3, 4, 5, 6)):
        cfg = dict(c.config, norm_mode=1)
        if native.cfg_check("rmsnorm_matmul", cfg, 4096, 11008, 4096)[0] != native.OK:
            continue
        ring = native.describe_launch("rmsnorm_matmul", cfg, 4096, 11008, 4096)["x_ring"]
        seen.add((ring["a_stages"], ring["a_slots"], ring["groups"]))
    assert seen, "no inline candidate fits: the test would check nothing"
    for a_stages, a_slots, groups in sorted(seen):
        assert a_stages % groups == 0 and a_slots % groups == 0, (a_stages, a_slots, groups)
        check_ring(a_stages, a_slots, groups)


@pytest.mark.parametrize("a_stages,a_slots,groups", [(2, 4, 4), (3, 4, 4), (3, 8, 4), (2, 6, 4), (1, 4, 4)])
def test_ring_depths_that_are_not_multiples_of_the_group_count_are_caught(a_stages, a_slots, groups):
    """The fault on record: four transform groups over a shared-memory ring of 2 or 3 stages.  A group
    can then reach a stage two phases before its turn and the parity test lets it through.  (Not
    every depth that is not a multiple of the group count fails -- 6 stages with 4 groups is safe,
    because the group's previous k-block already proves enough loads -- but the planner only emits
    multiples, which always are.)"""
    with pytest.raises(Violation):
        check_ring(a_stages, a_slots, groups)


def test_plain_single_consumer_rings_pass():
    for depth in (1, 2, 3, 4, 6, 12):
        check_ring(depth, depth, 1)


# ------------------------------------------------------------------------------------------------
# 1b. accumulator handed over in halves (plain GEMM, single accumulator of two UMMA blocks)
# ------------------------------------------------------------------------------------------------
# acc_full[h] / acc_empty[h] stand for half h and flip once per tile.  The issuer issues half 0 and
# half 1 one after the other in every k-block; the last k-block commits half 0 between them, the
# first one waits for half 1 to be drained between them.  A commit arrives when the UMMAs before it
# have completed: later than it is issued, in issue order.  Every epilogue warp drains half 0,
# hands it back, then drains half 1.
def halves_issuer(bars, tiles, nkb):
    ph = 0
    for t in range(tiles):
        yield ("wait", bars["acc_empty"][0], ph ^ 1, t)
        for kb in range(nkb):
            if kb == nkb - 1:
                yield ("commit", bars["acc_full"][0])          # after half 0's UMMAs of the last k-block
            if kb == 0:
                yield ("wait", bars["acc_empty"][1], ph ^ 1, t)
        yield ("commit", bars["acc_full"][1])
        ph ^= 1


def halves_epilogue_warp(bars, tiles):
    ph = 0
    for t in range(tiles):
        for h in (0, 1):
            yield ("wait", bars["acc_full"][h], ph, t + 1)
            yield ("arrive", bars["acc_empty"][h])
        ph ^= 1


def run_halves_model(tiles, nkb, warps, seed, bias=None):
    rng = random.Random(seed)
    bars = {"acc_full": [Barrier(1), Barrier(1)], "acc_empty": [Barrier(warps), Barrier(warps)]}
    agents = [halves_issuer(bars, tiles, nkb)] + [halves_epilogue_warp(bars, tiles) for _ in range(warps)]
    pending = [next(a, None) for a in agents]
    commits = []   # issued, not yet arrived; they arrive in issue order
    while any(op is not None for op in pending) or commits:
        if commits and (rng.random() < 0.3 or all(op is None for op in pending)):
            commits.pop(0).arrive()
            continue
        live = [i for i, op in enumerate(pending) if op is not None]
        progressed = False
        for i in sorted(live, key=lambda i: (bias(i) if bias else 0, rng.random())):
            op = pending[i]
            if op[0] == "arrive":
                op[1].arrive()
            elif op[0] == "commit":
                commits.append(op[1])
            else:
                _, bar, parity, need = op
                says, means = bar.parity_test(parity), bar.completed >= need
                if says != means:
                    raise Violation(f"agent {i}: parity test says {says}, {bar.completed} phases complete, {need} needed")
                if not says:
                    continue
            pending[i] = next(agents[i], None)
            progressed = True
            break
        if not progressed:
            if not commits:
                raise Violation("deadlock: every agent is blocked")
            commits.pop(0).arrive()
    assert all(b.completed == tiles for pair in bars.values() for b in pair)


def test_accumulator_halves_protocol():
    """One to several tiles, tiles of one, two and many k-blocks, 8 warps (one CTA) and 16 (a pair)."""
    for tiles, nkb, warps in itertools.product((1, 2, 5), (1, 2, 7), (8, 16)):
        for bias in BIASES:
            for seed in range(3):
                run_halves_model(tiles, nkb, warps, seed, bias)


def test_halves_model_notices_a_missing_hand_back():
    """An issuer that does not wait for half 1 to be drained before the next tile's first k-block
    would be caught as a barrier that ends with the wrong number of completed phases -- here: the
    model's own bookkeeping of an epilogue that forgets to hand half 1 back deadlocks."""
    def forgetful(bars, tiles):
        ph = 0
        for t in range(tiles):
            yield ("wait", bars["acc_full"][0], ph, t + 1)
            yield ("arrive", bars["acc_empty"][0])
            yield ("wait", bars["acc_full"][1], ph, t + 1)      # drains half 1 but never releases it
            ph ^= 1

    bars = {"acc_full": [Barrier(1), Barrier(1)], "acc_empty": [Barrier(1), Barrier(1)]}
    agents = [halves_issuer(bars, 2, 3), forgetful(bars, 2)]
    pending = [next(a, None) for a in agents]
    commits, steps = [], 0
    with pytest.raises(Violation):
        while any(op is not None for op in pending) or commits:
            steps += 1
            progressed = False
            if commits:
                commits.pop(0).arrive()
                progressed = True
            for i, op in enumerate(pending):
                if op is None:
                    continue
                if op[0] == "arrive":
                    op[1].arrive()
                elif op[0] == "commit":
                    commits.append(op[1])
                else:
                    if not op[1].parity_test(op[2]):
                        continue
                pending[i] = next(agents[i], None)
                progressed = True
            if not progressed:
                raise Violation("deadlock: every agent is blocked")


# ------------------------------------------------------------------------------------------------
# 2. tile split of the weight-streaming kernel (mirrors prepare_skinny / SkinnyWork)
# ------------------------------------------------------------------------------------------------
def skinny_layout(N, K, tile_k, sms=148):
    T, nkb, grid = (N + 255) // 256, (K + tile_k - 1) // tile_k, min(sms, 160)
    if T < grid and T * nkb < grid:
        grid = T * nkb
    base, R = divmod(T, grid)
    D = grid - R if R else 0
    don = 0
    if R and D:
        lead = 0 if base else (192 * 1024) // (256 * tile_k * 2)
        lead = min(lead, R * nkb // grid // 8)
        own = max(1, min(nkb, (R * nkb + D * lead + grid - 1) // grid))
        don = nkb - own
    return dict(grid=grid, T=T, nkb=nkb, base=base, R=R, D=D, don=don, rot=5)


def skinny_segments(L, b):
    nkb, base, R, D, don, rot = (L[k] for k in ("nkb", "base", "R", "D", "don", "rot"))
    whole = lambda bt: ("whole", R + b * base + bt, 0, nkb, (b * rot + 7 * bt) % nkb)  # noqa: E731
    out = []
    if b < D:
        if don:
            V = R * don
            u, end = V * b // D, V * (b + 1) // D
            while u < end:
                t = u // don
                lo, stop = u - t * don, min(end, (t + 1) * don)
                out.append(("donate", t, lo, lo + stop - u, lo))
                u = stop
        out += [whole(bt) for bt in range(base)]
    else:
        out += [whole(bt) for bt in range(base)]
        if b - D < R:
            out.append(("own" if don else "whole", b - D, don, nkb, don + (b * rot) % (nkb - don)))
    return out


@pytest.mark.parametrize("N,K,tile_k", list(itertools.product(
    [8, 72, 256, 1000, 4096, 9472, 18944, 28672, 32768, 37888, 40000, 65536], [64, 192, 4096, 8192], [64, 128])))
def test_skinny_split_streams_every_unit_once(N, K, tile_k):
    L = skinny_layout(N, K, tile_k)
    cover = {}
    for b in range(L["grid"]):
        for kind, t, lo, hi, start in skinny_segments(L, b):
            assert 0 <= t < L["T"] and lo < hi and lo <= start < hi
            walk = [start + i if start + i < hi else start + i - (hi - lo) for i in range(hi - lo)]
            assert sorted(walk) == list(range(lo, hi))                 # the wrapped K loop visits its range once
            for kb in walk:
                assert (t, kb) not in cover
                cover[(t, kb)] = (b, kind)
            if kind == "donate":
                assert b + t < L["T"] + 160                            # the slot index stays inside the scratch
    assert len(cover) == L["T"] * L["nkb"]
    R, D, don = L["R"], L["D"], L["don"]
    if don:
        V = R * don
        slots = set()
        for t in range(R):
            lo, hi = ((t * don + 1) * D - 1) // V, ((t + 1) * don * D - 1) // V     # what the owner computes
            donors = sorted({cover[(t, kb)][0] for kb in range(don)})
            assert donors[0] == lo and donors[-1] == hi
            assert all(cover[(t, kb)][1] == "donate" for kb in range(don))
            assert all(cover[(t, kb)] == (D + t, "own") for kb in range(don, L["nkb"]))
            for d in donors:
                assert (d + t) not in slots                             # one slot per (donor, tile)
                slots.add(d + t)


def test_skinny_model_agrees_with_the_library(native_lib):
    from autotune import native

    for N, K in [(28672, 8192), (37888, 8192), (65536, 4096), (4096, 4096), (256, 512)]:
        L = skinny_layout(N, K, 128)
        d = native.describe_launch("rmsnorm_matmul", None, 16, N, K)
        if d["sm_count_from_device"] and d["sm_count"] != 148:
            continue
        assert (d["grid"], d["whole_tiles_per_cta"], d["shared_tiles"], d["k_blocks"]) == (L["grid"], L["base"], L["R"], L["nkb"])
