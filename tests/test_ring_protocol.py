"""The fused depthwise -> pointwise kernel's barrier protocol, simulated on the CPU.

`sepconv_tcgen05_kernel` synchronises its TMA producer, its depthwise thread groups and its MMA
issuer through mbarriers that are waited on by phase PARITY.  A parity wait is only correct for a
waiter that observes every phase of its barrier; when the depthwise warps were first split into
two groups working on alternate k-blocks over SHARED rings, a group could see the parity of a
phase it had skipped and run ahead (over-arrivals, then deadlock).  The kernel therefore gives
every A slot, raw stage and barrier to exactly one group (`ring_pos` in
tfjs-core_b200/csrc/sepconv_tcgen05.cu).  This test restates that mapping and drives the four
roles with random interleavings for every ring geometry the kernel instantiates: no wait may pass
before the completion it stands for, no barrier may be over-arrived, and every role must finish.
It also shows that the shared-ring mapping fails the same check.
"""
import random

import pytest


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.completions = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "over-arrival"
        if self.pending == 0:
            self.pending = self.count
            self.completions += 1

    def test(self, parity):  # mbarrier.test_wait.parity: true once the phase of that parity is over
        return (self.completions & 1) != parity


def ring_pos_owned(seq, size, groups):
    """(index, phase parity, completions that must precede a consumer's pass): group seq % groups owns
    size / groups consecutive entries and cycles through them."""
    per = size // groups
    group, turn = seq % groups, seq // groups
    return group * per + turn % per, (turn // per) & 1, turn // per


def ring_pos_shared(seq, size, groups):
    return seq % size, (seq // size) & 1, seq // size


def simulate(ring_pos, groups, raw_stages, a_slots, parts, w_stages, k_blocks, tiles, seed):
    rnd = random.Random(seed)
    warps = 8 // groups
    raw_full = [Barrier(1) for _ in range(raw_stages)]
    raw_empty = [Barrier(warps) for _ in range(raw_stages)]
    a_full = [Barrier(warps) for _ in range(a_slots)]
    a_empty = [Barrier(1) for _ in range(a_slots)]
    w_full = [Barrier(1) for _ in range(w_stages)]
    w_empty = [Barrier(1) for _ in range(w_stages)]

    def wait(bar, parity, completions_needed):
        while not bar.test(parity):
            yield
        assert bar.completions >= completions_needed, "a wait passed on the parity of an earlier phase"

    def producer():  # weights and windows in program order; the kernel's polling variant only relaxes this
        rn = ws = wturn = 0
        for _ in range(tiles * k_blocks):
            yield from wait(w_empty[ws], (wturn & 1) ^ 1, wturn)
            yield
            w_full[ws].arrive()
            ws += 1
            if ws == w_stages:
                ws, wturn = 0, wturn + 1
            for _ in range(parts):
                rs, phase, need = ring_pos(rn, raw_stages, groups)
                yield from wait(raw_empty[rs], phase ^ 1, need)
                yield
                raw_full[rs].arrive()
                rn += 1

    def mma():
        ws = wturn = 0
        for n in range(tiles * k_blocks):
            slot, phase, need = ring_pos(n, a_slots, groups)
            yield from wait(w_full[ws], wturn & 1, wturn + 1)
            yield from wait(a_full[slot], phase, need + 1)
            yield
            w_empty[ws].arrive()
            a_empty[slot].arrive()
            ws += 1
            if ws == w_stages:
                ws, wturn = 0, wturn + 1

    def depthwise_warp(group):
        for n in range(tiles * k_blocks):
            if n % groups != group:
                continue
            slot, phase, need = ring_pos(n, a_slots, groups)
            yield from wait(a_empty[slot], phase ^ 1, need)
            for part in range(parts):
                rs, rphase, rneed = ring_pos(n * parts + part, raw_stages, groups)
                yield from wait(raw_full[rs], rphase, rneed + 1)
                yield
                raw_empty[rs].arrive()
            yield
            a_full[slot].arrive()

    alive = [producer(), mma()] + [depthwise_warp(g) for g in range(groups) for _ in range(warps)]
    steps = 0
    while alive:
        role = rnd.choice(alive)
        try:
            next(role)
        except StopIteration:
            alive.remove(role)
        steps += 1
        assert steps < 2_000_000, "deadlock"


def simulate_in_place(ring_pos, groups, raw_stages, w_stages, k_blocks, tiles, seed):
    """The 256-column stride-1 variant: a group writes the A tile over its own window, so a raw
    stage goes TMA -> depthwise group -> MMA and is freed by the MMAs' commit."""
    rnd = random.Random(seed)
    warps = 8 // groups
    raw_full = [Barrier(1) for _ in range(raw_stages)]
    raw_empty = [Barrier(1) for _ in range(raw_stages)]
    a_full = [Barrier(warps) for _ in range(raw_stages)]
    w_full = [Barrier(1) for _ in range(w_stages)]
    w_empty = [Barrier(1) for _ in range(w_stages)]

    def wait(bar, parity, completions_needed):
        while not bar.test(parity):
            yield
        assert bar.completions >= completions_needed, "a wait passed on the parity of an earlier phase"

    def producer():  # polls both rings; a step advances whichever is free
        rn = wn = 0
        total = tiles * k_blocks
        while rn < total or wn < total:
            moved = False
            if rn < total:
                rs, phase, need = ring_pos(rn, raw_stages, groups)
                if raw_empty[rs].test(phase ^ 1):
                    assert raw_empty[rs].completions >= need
                    raw_full[rs].arrive()
                    rn += 1
                    moved = True
            if wn < total:
                ws, wturn = wn % w_stages, wn // w_stages
                if w_empty[ws].test((wturn & 1) ^ 1):
                    assert w_empty[ws].completions >= wturn
                    w_full[ws].arrive()
                    wn += 1
                    moved = True
            yield moved

    def mma():
        for n in range(tiles * k_blocks):
            rs, phase, need = ring_pos(n, raw_stages, groups)
            ws, wturn = n % w_stages, n // w_stages
            yield from wait(a_full[rs], phase, need + 1)
            yield from wait(w_full[ws], wturn & 1, wturn + 1)
            yield
            w_empty[ws].arrive()
            raw_empty[rs].arrive()

    def depthwise_warp(group):
        for n in range(tiles * k_blocks):
            if n % groups != group:
                continue
            rs, phase, need = ring_pos(n, raw_stages, groups)
            yield from wait(raw_full[rs], phase, need + 1)
            yield
            a_full[rs].arrive()

    alive = [producer(), mma()] + [depthwise_warp(g) for g in range(groups) for _ in range(warps)]
    steps = 0
    while alive:
        role = rnd.choice(alive)
        try:
            next(role)
        except StopIteration:
            alive.remove(role)
        steps += 1
        assert steps < 2_000_000, "deadlock"


def test_in_place_tiles_are_safe():
    for seed in range(8):
        simulate_in_place(ring_pos_owned, 2, 4, 2, 8, 5, seed)


# (groups, raw stages, A slots, raw stages per k-block, weight stages, k-blocks per tile, tiles per CTA)
GEOMETRIES = [
    (2, 4, 2, 1, 4, 1, 25),   # block 1: 32 channels, N = 64
    (2, 4, 2, 1, 3, 4, 9),    # block 3: 128 channels, N = 128
    (2, 8, 2, 1, 4, 1, 25),   # the stem (im2col threads instead of depthwise threads)
    (1, 3, 2, 2, 2, 2, 9),    # block 2: stride 2, one group, two half-windows per k-block, three window stages
    (1, 2, 2, 2, 2, 4, 7),    # block 4
]


@pytest.mark.parametrize("geometry", GEOMETRIES)
def test_group_owned_rings_are_safe(geometry):
    for seed in range(8):
        simulate(ring_pos_owned, *geometry, seed)


def test_shared_rings_between_two_groups_are_not():
    failures = 0
    for seed in range(12):
        try:
            simulate(ring_pos_shared, 2, 2, 2, 2, 3, 4, 7, seed)  # stride-2 geometry split over two groups
        except AssertionError:
            failures += 1
    assert failures > 0
