"""Discrete-event simulation of the mbarrier protocol of the tcgen05 dsd kernel
(``sparta_b200/csrc/bsmm_dsd_tc.cu``): one X producer warp, three W producer warps, two converter sets,
one issuer warp per block column; a ring of 12 steps for the "full" barriers, X slots in shared memory
that the converters free, activation slots in tensor memory and a ring of 40 or 48 W blocks that the
issuers free (per step or per pair of steps); waits that name a phase by its parity only.

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

KS, NWPROD = 12, 3


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


def wait_for_table(need, KW=48):
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


def simulate(need, seed, KA=3, NISS=10, KX=4, PAIR=1, KW=40):
    """KA activation slots in tensor memory, NISS issuer warps (one per block column of the panel), KX
    X slots in shared memory, PAIR steps released together by the issuers, KW W ring slots.  The kernel as
    built (four K-blocks per step): PAIR 1 and KA / NISS / KX / KW of 2 / 12 / 3 / 48, 3 / 10 / 4 / 40 or
    4 / 8 / 4 / 40; its variant with two K-blocks per step: KX 5, PAIR 2 and 4 / 12, 6 / 10 or 6 / 8."""
    KP = KS // PAIR
    rnd = random.Random(seed)
    n = len(need)
    cum, wait_for = wait_for_table(need, KW)
    full = [Barrier(2, f'full{i}') for i in range(KS)]      # X producer + W producer
    empty = [Barrier(NISS, f'empty{i}') for i in range(KP)]
    pair_wait = lambda t: ('wait', empty[(t // PAIR) % KP], ((t // PAIR) // KP) & 1)  # release of step t
    afull = [Barrier(4, f'afull{i}') for i in range(KA)]
    xfree = [Barrier(4, f'xfree{i}') for i in range(KX)]
    accum = Barrier(NISS, 'accum')
    x_owner = [None] * KX   # step whose X tile sits in the shared-memory slot
    a_owner = [None] * KA   # step whose activations sit in the tensor-memory slot
    w_owner = {}            # W ring position -> step that still needs it
    mma_left = [NISS] * n
    jitter = rnd.uniform

    def x_producer():
        for s in range(n):
            xslot = s % KX
            if s >= KX:  # the converters have read the slot's previous tile (one warp, in order: no aliasing)
                yield ('wait', xfree[xslot], ((s - KX) // KX) & 1)
            yield ('delay', jitter(50, 300))
            assert x_owner[xslot] is None, f'X slot {xslot} overwritten: holds {x_owner[xslot]}, new {s}'
            x_owner[xslot] = s
            yield ('delay', jitter(200, 1200))  # the load lands
            yield ('arrive', full[s % KS], 1)

    def w_producer(j):
        for s in range(j, n, NWPROD):
            if s >= KS:  # own barrier slot's previous use: the barrier's next use is s itself
                yield pair_wait(s - KS)
            wf = wait_for[s]
            if wf >= 0 and wf > s - KS:  # previous use of that barrier is known released, next use > s
                yield pair_wait(wf)
            yield ('delay', jitter(100, 600))
            for q in range(cum[s], cum[s + 1]):
                assert q % KW not in w_owner, f'W slot {q % KW} of step {w_owner.get(q % KW)} overwritten by {s}'
                w_owner[q % KW] = s
            yield ('delay', jitter(200, 1200))  # the loads land
            yield ('arrive', full[s % KS], 1)

    def converter(c):
        for s in range(c, n, 2):
            xslot, aslot = s % KX, s % KA
            yield ('wait', full[s % KS], (s // KS) & 1)   # the tile has landed: half of it goes to registers at once
            assert x_owner[xslot] == s, f'converter of step {s} reads X slot holding {x_owner[xslot]}'
            yield ('delay', jitter(50, 150))
            if s >= KA:
                yield pair_wait(s - KA)
            yield ('delay', jitter(100, 400))
            assert a_owner[aslot] is None, f'A slot {aslot} of step {a_owner[aslot]} overwritten by {s}'
            a_owner[aslot] = s
            x_owner[xslot] = None
            yield ('arrive', afull[aslot], 4)  # the set's four warps
            yield ('arrive', xfree[xslot], 4)

    def issuer(i):
        for s in range(n):
            slot, aslot = s % KS, s % KA
            yield ('wait', afull[aslot], (s // KA) & 1)
            assert a_owner[aslot] == s, f'issuer {i} at step {s} reads A slot holding {a_owner[aslot]}'
            yield ('delay', jitter(50, 700) if rnd.random() < 0.5 else jitter(20, 100))
            mma_left[s] -= 1
            if mma_left[s] == 0:  # the step's operands are dead
                a_owner[aslot] = None
                for q in range(cum[s], cum[s + 1]):
                    del w_owner[q % KW]
            if s % PAIR == PAIR - 1 or s == n - 1:
                yield ('arrive', empty[(s // PAIR) % KP], 1)
        yield ('arrive', accum, 1)

    roles = [x_producer()] + [w_producer(j) for j in range(NWPROD)] + [converter(0), converter(1)] + [issuer(i) for i in range(NISS)]
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


# (activation slots, issuers, X slots, steps released together, K-blocks per step, W ring slots)
CONFIGS = [(2, 12, 3, 1, 4, 48), (3, 10, 4, 1, 4, 40), (4, 8, 4, 1, 4, 40),     # the kernel as built
           (4, 12, 5, 2, 2, 48), (6, 10, 5, 2, 2, 48), (6, 8, 5, 2, 2, 48)]     # its variant with two K-blocks per step


@pytest.mark.parametrize('ka,niss,kx,pair,kg,kw', CONFIGS)
@pytest.mark.parametrize('density', [0.02, 0.1, 0.25, 0.5, 1.0])
def test_protocol_under_random_timing(density, ka, niss, kx, pair, kg, kw):
    rs = np.random.RandomState(int(density * 1000) + ka)
    for trial in range(6):
        need = np.maximum(1, rs.binomial(kg * niss, density, size=rs.randint(1, 100)))
        simulate(need, seed=trial, KA=ka, NISS=niss, KX=kx, PAIR=pair, KW=kw)


def test_wait_for_table_small_case():
    # ring of 48: step 2 needs positions 40..59, i.e. the space of step 0 (20 blocks); step 3 wraps further
    cum, table = wait_for_table(np.array([20, 20, 20, 20, 20]))
    assert list(cum) == [0, 20, 40, 60, 80, 100]
    assert table == [-1, -1, 0, 1, 2]
