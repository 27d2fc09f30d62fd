"""Discrete-event simulation of the mbarrier protocol of the tcgen05 dsd kernel
(``sparta_b200/csrc/bsmm_dsd_tc.cu``): four producer warps, two converter sets, twelve issuers, rings
of 6 load slots / 4 or 6 activation slots / 40 W blocks, waits that name a phase by its parity only.

The simulation runs the roles' wait / arrive sequences under random timing with the mbarrier rules
(a wait for parity P succeeds when the barrier's current phase has the other parity; an arrival beyond
the expected count is an error) and checks that nothing deadlocks, that no barrier receives too many
arrivals, and that no operand is overwritten while a later stage still needs it.  It is how a waiter
falling two phases behind a barrier (which then blocks for ever) was found in a design that was never
shipped; the kernel's scheme passes.  Keep it in step with the kernel when the protocol changes."""
import heapq
import random

import numpy as np
import pytest

NP, KX, KW, NPROD = 12, 6, 40, 4


class Barrier:
    def __init__(self, count, name):
        self.count, self.pending, self.phase, self.name = count, count, 0, name

    def arrive(self, n=1):
        self.pending -= n
        assert self.pending >= 0, f'arrival overflow on {self.name}'
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, parity):  # mbarrier.try_wait.parity
        return (self.phase & 1) != parity


def wait_for_table(need):
    """Latest earlier step whose W blocks still occupy the ring positions step s needs (-1: none)."""
    cum = np.concatenate([[0], np.cumsum(need)])
    table = []
    for s in range(len(need)):
        target = cum[s + 1] - KW
        f = -1
        if target > 0:
            f = int(np.searchsorted(cum[:s + 1], target, side='left')) - 1
        table.append(f)
    return cum, table


def simulate(need, seed, KA=4, NISS=12):
    """KA activation slots in tensor memory, NISS issuer warps (4 / 12 for panels of 12 block columns,
    6 / 10 for panels of 10, 6 / 8 for panels of 8)."""
    rnd = random.Random(seed)
    n = len(need)
    cum, wait_for = wait_for_table(need)
    full = [Barrier(1, f'full{i}') for i in range(KX)]
    empty = [Barrier(NISS, f'empty{i}') for i in range(KX)]
    afull = [Barrier(4, f'afull{i}') for i in range(KA)]
    accum = Barrier(NISS, 'accum')
    x_owner = [None] * KX   # step whose X tile sits in the shared-memory slot
    a_owner = [None] * KA   # step whose activations sit in the tensor-memory slot
    w_owner = {}            # W ring position -> step that still needs it
    mma_left = [NISS] * n
    jitter = rnd.uniform

    def producer(j):
        for s in range(j, n, NPROD):
            slot = s % KX
            if s >= KX:  # own slot's previous use: the barrier's next use is s itself
                yield ('wait', empty[slot], ((s - KX) // KX) & 1)
            wf = wait_for[s]
            if wf >= 0 and wf > s - KX:  # previous use of that barrier is known released, next use > s
                yield ('wait', empty[wf % KX], (wf // KX) & 1)
            yield ('delay', jitter(100, 600))
            assert x_owner[slot] is None, f'X slot {slot} overwritten: holds {x_owner[slot]}, new {s}'
            x_owner[slot] = s
            for q in range(cum[s], cum[s + 1]):
                assert q % KW not in w_owner, f'W slot {q % KW} of step {w_owner.get(q % KW)} overwritten by {s}'
                w_owner[q % KW] = s
            yield ('delay', jitter(200, 1200))  # the loads land
            yield ('arrive', full[slot], 1)

    def converter(c):
        for s in range(c, n, 2):
            slot, aslot = s % KX, s % KA
            if s >= KA:
                yield ('wait', empty[(s - KA) % KX], ((s - KA) // KX) & 1)
            yield ('wait', full[slot], (s // KX) & 1)
            assert x_owner[slot] == s, f'converter of step {s} reads X slot holding {x_owner[slot]}'
            yield ('delay', jitter(100, 400))
            assert a_owner[aslot] is None, f'A slot {aslot} of step {a_owner[aslot]} overwritten by {s}'
            a_owner[aslot] = s
            yield ('arrive', afull[aslot], 4)  # the set's four warps

    def issuer(i):
        for s in range(n):
            slot, aslot = s % KX, s % KA
            yield ('wait', afull[aslot], (s // KA) & 1)
            assert a_owner[aslot] == s, f'issuer {i} at step {s} reads A slot holding {a_owner[aslot]}'
            yield ('delay', jitter(50, 700) if rnd.random() < 0.5 else jitter(20, 100))
            mma_left[s] -= 1
            if mma_left[s] == 0:  # the step's operands are dead
                a_owner[aslot] = None
                x_owner[slot] = None
                for q in range(cum[s], cum[s + 1]):
                    del w_owner[q % KW]
            yield ('arrive', empty[slot], 1)
        yield ('arrive', accum, 1)

    roles = [producer(j) for j in range(NPROD)] + [converter(0), converter(1)] + [issuer(i) for i in range(NISS)]
    now = 0.0
    ready = [(0.0, k) for k in range(len(roles))]
    heapq.heapify(ready)
    waiting = {}
    while ready or waiting:
        assert ready, 'deadlock: ' + ', '.join(f'role {k} on {b.name} parity {p} (phase {b.phase})'
                                               for k, (b, p) in waiting.items())
        now, k = heapq.heappop(ready)
        while True:
            try:
                op = next(roles[k])
            except StopIteration:
                break
            if op[0] == 'delay':
                heapq.heappush(ready, (now + op[1], k))
                break
            if op[0] == 'arrive':
                op[1].arrive(op[2])
                for kk, (b, par) in list(waiting.items()):
                    if b.done(par):
                        del waiting[kk]
                        heapq.heappush(ready, (now + jitter(20, 150), kk))
                continue
            if op[1].done(op[2]):
                continue
            waiting[k] = (op[1], op[2])
            break
    assert accum.phase == 1
    assert not w_owner and all(o is None for o in x_owner) and all(o is None for o in a_owner)


@pytest.mark.parametrize('ka,niss', [(4, 12), (6, 10), (6, 8)])
@pytest.mark.parametrize('density', [0.02, 0.1, 0.25, 0.5, 1.0])
def test_protocol_under_random_timing(density, ka, niss):
    rs = np.random.RandomState(int(density * 1000) + ka)
    for trial in range(8):
        need = np.maximum(1, rs.binomial(2 * niss, density, size=rs.randint(1, 100)))
        simulate(need, seed=trial, KA=ka, NISS=niss)


def test_wait_for_table_small_case():
    # ring of 40: step 3 needs positions 36..47, i.e. the space of steps 0 (12 blocks); step 4 wraps further
    cum, table = wait_for_table(np.array([12, 12, 12, 12, 12]))
    assert list(cum) == [0, 12, 24, 36, 48, 60]
    assert table == [-1, -1, -1, 0, 1]
