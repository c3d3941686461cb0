"""A model of the expert-parallel exchange protocol of the layer kernel (csrc/s14_moe_umma.cu, final
stage; include/polaris_s14_cuda.h, s14_cmd_routed_moe_layer_ep), run as interleaved Python
coroutines on the CPU.  Rules modelled, per rank and step s (the rank's own count):

* credits: every rank's buffer holds, per peer, the number of steps that peer has finished; a rank
  starts step s only when every peer's credit in its own buffer is >= s - 1 (so nobody still reads
  buffer s % 2 for step s - 2); after `limit` polls it reports that and goes on with the step all the
  same -- the peer it overwrites is hopelessly late, finds later steps' numbers in its buffer and
  catches up at full speed, as below; a rank that wrote nothing after such a wait would leave the
  late rank waiting for words that never come, and the two would stay apart for good; at the end of
  a step the rank stores its new step count into every peer's buffer;
* publish: for every slot the rank owns, store (value, s + 1) into buffer s % 2 of EVERY rank;
* wait: poll the own buffer s % 2, slot by slot, until the number is >= s + 1; after `limit` polls
  the rank gives the step up and reports it; a number > s + 1 anywhere means that a peer gave up on
  this rank earlier and ran ahead: the rank reports it and waits for nothing more in this step (the
  words it still misses belong to steps its peers have left behind and would never come), so it
  runs at full speed until it is level again; in every case the step count advances.

Properties checked: with every rank scheduled fairly nothing is reported and every rank mixes
exactly its step's values (two buffers are enough); after one rank stalls for a long time the
others report time-outs, the late rank reports overwritten values, and all ranks fall into step
again, after which nothing more is reported; and a slow rank that owns no slot at all -- for which
nobody waits in the exchange itself -- still reads every step's values intact, because the credits
hold the others back (without them its buffer would be overwritten two steps later)."""
import random

import pytest

N_SLOTS = 7


class Rank:
    def __init__(self, rank, world, limit):
        self.rank, self.world, self.limit = rank, world, limit
        self.buf = [[(None, 0)] * N_SLOTS for _ in range(2)]  # (value, number), zeroed like the real buffer
        self.credit = [0] * world  # steps every peer has finished, as far as this rank has been told
        self.step = 0
        self.log = []  # (step, kind) with kind in {"ok", "timeout", "ahead", "credit"}


def owner(slot, step, world):
    return (slot * 5 + step * 3) % world  # any rule all ranks agree on


def finish_step(me, ranks, s, kind):
    me.log.append((s, kind))
    me.step = s + 1
    for peer in ranks:
        peer.credit[me.rank] = s + 1


def run_step(me, ranks, owner=owner, use_credits=True):
    """Generator: yields between memory operations so that a scheduler can interleave the ranks."""
    s = me.step
    kind = "ok"
    if use_credits:
        polls = 0
        while any(me.credit[p] < s - 1 for p in range(me.world) if p != me.rank):
            polls += 1
            if polls > me.limit:  # reported; the step goes on
                kind = "credit"
                break
            yield
    for slot in range(N_SLOTS):
        if owner(slot, s, me.world) == me.rank:
            for peer in ranks:
                peer.buf[s & 1][slot] = ((me.rank, s, slot), s + 1)
                yield
    got, waited_out = [], kind == "credit"
    behind = lambda: any(me.buf[s & 1][j][1] > s + 1 for j in range(N_SLOTS))  # the kernel's threads poll side by side
    for slot in range(N_SLOTS):
        polls = 0
        while kind in ("ok", "credit") and me.buf[s & 1][slot][1] < s + 1:  # a rank that gave up or is behind waits for nothing more
            if behind():
                kind = "ahead"
                break
            polls += 1
            if polls > me.limit:
                kind = "timeout"
                break
            yield
        value, number = me.buf[s & 1][slot]
        if number > s + 1 and kind in ("ok", "credit"):
            kind = "ahead"
        got.append(value)
    if kind == "ok" and not waited_out:  # nothing reported: every value is this step's
        assert got == [(owner(slot, s, me.world), s, slot) for slot in range(N_SLOTS)], (me.rank, s, got)
    finish_step(me, ranks, s, kind)


def simulate(world, n_steps, limit, seed, stall=None, owner=owner, use_credits=True, slow=None):
    """stall = (rank, at_step, ticks): the rank is not scheduled for `ticks` scheduler turns when it
    reaches that step.  slow = (rank, k): the rank is scheduled only every k-th turn."""
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
            if slow and i == slow[0] and rng.randrange(slow[1]):
                continue
            if gens[i] is None:
                gens[i] = run_step(r, ranks, owner, use_credits)
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


def test_a_slow_rank_that_owns_nothing_is_protected_by_the_credits():
    """Rank 1 owns no slot, so no rank ever waits for it in the exchange, and it is scheduled ten times
    less often than rank 0.  With the credits it still mixes exactly its own step's values in every
    step (run_step asserts that) and nothing is reported.  Without them rank 0 runs ahead and
    overwrites the buffers rank 1 has not read yet, which rank 1 sees as later steps' numbers."""
    rank0_owns_all = lambda slot, step, world: 0
    ranks = simulate(2, n_steps=40, limit=100_000, seed=11, owner=rank0_owns_all, slow=(1, 10))
    for r in ranks:
        assert [k for _, k in r.log] == ["ok"] * 40
    ranks = simulate(2, n_steps=40, limit=100_000, seed=11, owner=rank0_owns_all, slow=(1, 10), use_credits=False)
    assert "ahead" in [k for _, k in ranks[1].log]


def test_a_credit_wait_that_runs_out_is_reported_and_the_ranks_fall_into_step_again():
    """A peer that is away for longer than the wait limit: the others report the credit wait (the
    kernel's status 0x5505) or the word wait, go on, and run clean again once it is back."""
    limit = 50
    ranks = simulate(2, n_steps=60, limit=limit, seed=5, stall=(1, 10, 12 * limit))
    kinds = [k for _, k in ranks[0].log]
    assert "credit" in kinds[10:] or "timeout" in kinds[10:]
    assert kinds[-15:] == ["ok"] * 15
    assert len({r.step for r in ranks}) == 1
