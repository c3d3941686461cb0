"""A model of the expert-parallel exchange protocol of the layer kernel (csrc/s14_moe_umma.cu, final
stage; include/polaris_s14_cuda.h, s14_cmd_routed_moe_layer_ep), run as interleaved Python
coroutines on the CPU.  Rules modelled, per rank and step s (the rank's own count):

* publish: for every slot the rank owns, store (value, s + 1) into buffer s % 2 of EVERY rank;
* wait: poll the own buffer s % 2, slot by slot, until the number is >= s + 1; after `limit` polls
  the rank gives the step up and reports it; a number > s + 1 anywhere means that a peer gave up on
  this rank earlier and ran ahead: the rank reports it and waits for nothing more in this step (the
  words it still misses belong to steps its peers have left behind and would never come), so it
  runs at full speed until it is level again; in every case the step count advances.

Properties checked: with every rank scheduled fairly nothing is reported and every rank mixes
exactly its step's values (two buffers are enough); after one rank stalls for a long time the
others report time-outs, the late rank reports overwritten values, and all ranks fall into step
again, after which nothing more is reported."""
import random

import pytest

N_SLOTS = 7


class Rank:
    def __init__(self, rank, world, limit):
        self.rank, self.world, self.limit = rank, world, limit
        self.buf = [[(None, 0)] * N_SLOTS for _ in range(2)]  # (value, number), zeroed like the real buffer
        self.step = 0
        self.log = []  # (step, kind) with kind in {"ok", "timeout", "ahead"}


def owner(slot, step, world):
    return (slot * 5 + step * 3) % world  # any rule all ranks agree on


def run_step(me, ranks):
    """Generator: yields between memory operations so that a scheduler can interleave the ranks."""
    s = me.step
    for slot in range(N_SLOTS):
        if owner(slot, s, me.world) == me.rank:
            for peer in ranks:
                peer.buf[s & 1][slot] = ((me.rank, s, slot), s + 1)
                yield
    kind, got = "ok", []
    behind = lambda: any(me.buf[s & 1][j][1] > s + 1 for j in range(N_SLOTS))  # the kernel's threads poll side by side
    for slot in range(N_SLOTS):
        polls = 0
        while kind == "ok" and me.buf[s & 1][slot][1] < s + 1:  # a rank that gave up or is behind waits for nothing more
            if behind():
                kind = "ahead"
                break
            polls += 1
            if polls > me.limit:
                kind = "timeout"
                break
            yield
        value, number = me.buf[s & 1][slot]
        if number > s + 1 and kind == "ok":
            kind = "ahead"
        got.append(value)
    if kind == "ok":  # nothing reported: every value is this step's
        assert got == [(owner(slot, s, me.world), s, slot) for slot in range(N_SLOTS)], (me.rank, s, got)
    me.log.append((s, kind))
    me.step = s + 1


def simulate(world, n_steps, limit, seed, stall=None):
    """stall = (rank, at_step, ticks): the rank is not scheduled for `ticks` scheduler turns when it
    reaches that step."""
    rng = random.Random(seed)
    ranks = [Rank(r, world, limit) for r in range(world)]
    gens = [None] * world
    sleeping = {}
    while any(r.step < n_steps for r in ranks):
        # fair random scheduler: ranks in random order, one operation each per turn
        for i in rng.sample(range(world), world):
            r = ranks[i]
            if r.step >= n_steps:
                continue
            if stall and i == stall[0] and r.step == stall[1] and gens[i] is None and i not in sleeping:
                sleeping[i] = stall[2]
            if sleeping.get(i, 0) > 0:
                sleeping[i] -= 1
                continue
            if gens[i] is None:
                gens[i] = run_step(r, ranks)
            try:
                next(gens[i])
            except StopIteration:
                gens[i] = None
    return ranks


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fairly_scheduled_ranks_report_nothing_and_mix_their_own_step(world):
    for seed in range(5):
        ranks = simulate(world, n_steps=40, limit=10_000, seed=seed)
        for r in ranks:
            assert [k for _, k in r.log] == ["ok"] * 40


@pytest.mark.parametrize("world", [2, 4, 8])
def test_a_long_stall_is_reported_and_the_ranks_fall_into_step_again(world):
    limit = 50
    ranks = simulate(world, n_steps=60, limit=limit, seed=3, stall=(1, 10, 12 * limit))
    late, others = ranks[1], [r for r in ranks if r.rank != 1]
    for r in others:
        kinds = [k for _, k in r.log]
        assert "timeout" in kinds[10:]           # they gave steps up while rank 1 was away
        assert kinds[-15:] == ["ok"] * 15        # and run clean again afterwards
    kinds = [k for _, k in late.log]
    assert "ahead" in kinds[10:] or "timeout" in kinds[10:]  # its values had been overwritten
    assert kinds[-15:] == ["ok"] * 15
    assert len({r.step for r in ranks}) == 1
