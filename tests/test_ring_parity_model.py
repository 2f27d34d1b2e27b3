"""CPU: host model of an mbarrier-guarded shared-memory ring with several consumer threads, the hazard behind the ring
depths of ``csrc/kernels/fp8w_gemm.cu`` (several MMA issuer threads take the stages of one ring in turn).

An mbarrier wait only sees the PARITY of the barrier's phase: ``try_wait.parity(u & 1)`` for the u-th use of a slot
passes when the parity of the completed fills differs from u's.  That is right while the waiter is in step with the
barrier and wrong when it is a whole use ahead of the slot's previous fill (same parity as "already filled").  A
consumer gets there only if the slot's previous use belongs to ANOTHER consumer and has not even been produced when
this one arrives: with C consumers taking items in turn and a ring of depth D that needs D < C (the first form of the
kernel: four issuers on a three-deep ring, wrong results and timeouts).  From D >= C on, a consumer's own previous
item is at least as new as the slot's previous use, so the in-order producer has filled that use before the consumer
can come back.  The kernel uses depths that are multiples of its issuer count, which is inside the safe region and
also makes the slot -> issuer assignment static.  The model runs both regions under randomised schedules.
"""
import random

import pytest


def run(depth, consumers, items, seed):
    """Producer fills item i into slot i % depth after the slot's previous use was released; consumer i % consumers
    takes item i after a parity wait on the slot's full barrier.  Returns the items that were read wrongly."""
    rng = random.Random(seed)
    slot_item = [None] * depth
    fills = [0] * depth              # completed fills of a slot (the full barrier's phase count)
    frees = [0] * depth              # completed releases (the empty barrier's phase count)
    next_fill = 0
    cursor = list(range(consumers))  # the next item of every consumer
    wrong = []
    steps = 0
    while any(c < items for c in cursor) or next_fill < items:
        steps += 1
        if steps > 100000:   # a consumer that took a slot too early can leave the ring stuck: that is a failure too
            wrong.append(("stuck", next_fill))
            break
        actor = rng.randrange(consumers + 1)
        if actor == consumers:                                   # the producer
            if next_fill < items:
                s, u = next_fill % depth, next_fill // depth
                if frees[s] >= u:                                # exact: one producer thread, in program order
                    slot_item[s] = next_fill
                    fills[s] += 1
                    next_fill += 1
            continue
        i = cursor[actor]
        if i >= items:
            continue
        s, u = i % depth, i // depth
        if (fills[s] & 1) != (u & 1):                            # try_wait.parity(u & 1)
            if slot_item[s] != i:
                wrong.append((i, slot_item[s]))
            frees[s] = max(frees[s], u + 1)                      # release the slot for its next fill
            cursor[actor] = i + consumers
    return wrong


@pytest.mark.parametrize("depth,consumers", [(4, 4), (8, 4), (4, 2), (6, 2), (8, 2), (5, 4), (6, 4), (3, 2)])
def test_depth_of_at_least_the_consumer_count_never_reads_a_foreign_fill(depth, consumers):
    for seed in range(60):
        assert run(depth, consumers, 64, seed) == []


@pytest.mark.parametrize("depth,consumers", [(3, 4), (2, 4), (1, 2), (2, 3)])
def test_shallower_rings_admit_a_schedule_that_reads_a_slot_too_early(depth, consumers):
    assert any(run(depth, consumers, 64, seed) for seed in range(200))
