"""CPU: a host model of the (value, epoch) pair exchange that the fused GEMV + all-reduce and the one-shot all-reduce
use on peer memory, run under randomised interleavings of the ranks' steps.

The protocol (``csrc/kernels/gemv_ar.cu``, ``collective.cu``): every value travels as one 8-byte (value, epoch) pair
into slot `rank` of every peer's staging buffer, staging is double-buffered by the parity of the launch's epoch, a
rank polls only its OWN staging until every pair it needs carries the launch's epoch, reduces in rank order, and only
then (stream order) starts its next launch.  The model checks the two claims the kernels rely on:

* a rank never reduces a value of another launch (no stale pair of epoch e - 2 in the same parity is accepted, no pair
  of epoch e + 2 can land before the pairs of e were read), whatever the interleaving and whatever the sizes of
  consecutive launches;
* a rank is at most one launch ahead of any peer, which is why two parities suffice.

It also shows what the epoch in the pair buys: with pairs replaced by bare values plus ONE flag per (rank, launch)
written after the values WITHOUT a fence, an interleaving exists in which a reader sees the flag before the values.
"""
import random

import pytest


class Rank:
    def __init__(self, rank, world, cap):
        self.rank, self.world = rank, world
        # staging[parity][src][i] = (value, epoch)
        self.staging = [[[(0.0, 0)] * cap for _ in range(world)] for _ in range(2)]
        self.epoch = 1                 # epoch of the launch this rank runs next
        self.phase = "idle"
        self.out = []


def run(world, sizes, seed, cap=16):
    """Every rank runs len(sizes) launches; launch k reduces sizes[k] values.  A step of the scheduler is ONE pair store
    or ONE poll attempt of one rank, picked at random.  Returns the largest lead (in launches) one rank had over another."""
    rng = random.Random(seed)
    ranks = [Rank(r, world, cap) for r in range(world)]
    val = lambda r, k, i: float((r + 1) * 1000 + k * 37 + i)           # rank r's local partial of launch k, element i
    todo = {r: None for r in range(world)}                             # pending pair stores of the rank's current launch
    done = [0] * world
    lead = 0
    while min(done) < len(sizes):
        r = rng.randrange(world)
        me = ranks[r]
        k = done[r]
        if k == len(sizes):
            continue
        n, e = sizes[k], me.epoch
        if todo[r] is None:                                            # launch starts: pairs to every peer, any order
            todo[r] = [(p, i) for p in range(world) if p != r for i in range(n)]
            rng.shuffle(todo[r])
        if todo[r]:
            p, i = todo[r].pop()
            ranks[p].staging[e & 1][r][i] = (val(r, k, i), e)          # one 8-byte store: value and epoch together
            continue
        # all pairs are on their way: poll the local staging (one attempt = look at every awaited pair once)
        mine = me.staging[e & 1]
        if all(mine[src][i][1] == e for src in range(world) if src != r for i in range(n)):
            got = [sum(val(r, k, i) if src == r else mine[src][i][0] for src in range(world)) for i in range(n)]
            want = [sum(val(src, k, i) for src in range(world)) for i in range(n)]
            assert got == want, (r, k, got, want)
            me.epoch += 1
            done[r] += 1
            todo[r] = None
            lead = max(lead, max(done) - min(done))
    return lead


@pytest.mark.parametrize("world", [2, 4, 8])
def test_pairs_never_mix_launches_and_two_parities_suffice(world):
    leads = []
    for seed in range(40):
        rng = random.Random(1000 + seed)
        sizes = [rng.choice([1, 3, 8, 16]) for _ in range(12)]         # consecutive launches of different widths
        leads.append(run(world, sizes, seed))
    assert max(leads) <= 1                                             # nobody gets two launches ahead of a peer
    assert max(leads) == 1                                             # and the interleavings did exercise the overlap


def test_flag_after_unfenced_values_can_be_seen_first():
    """The alternative without epochs in the data: values, then a flag, no fence in between.  Stores to a peer may
    become visible in any order, so a schedule that delivers the flag first makes the reader reduce a stale value:
    the reason the first form of the kernel needed a system-scope fence per launch, and the pair form does not."""
    staging, flag = [0.0], [0]
    pending = [("value", 42.0), ("flag", 1)]                           # issued in this order by the writer
    pending.reverse()                                                  # ... and delivered in the other
    seen = None
    for kind, v in pending:
        if kind == "value":
            staging[0] = v
        else:
            flag[0] = v
        if flag[0] == 1 and seen is None:
            seen = staging[0]                                          # the reader acts as soon as the flag is up
    assert seen == 0.0                                                 # stale: the value had not landed yet
