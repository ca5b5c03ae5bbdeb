"""Model check of the barrier protocol of the exact-similarity tcgen05 kernel
(zipage_b200/csrc/zp_redundancy_exact_tc.cu) on the CPU.

The kernel's four roles (TMA producer, MMA issuer, epilogue, row-sum warps) are replayed as
coroutines over Python models of the mbarriers (phase counter + parity wait, which cannot tell a
phase from the one two later) and of the three rotating page slots (`SlotFifo`), under random
schedules and random job lengths.  Checked: no deadlock; the MMA issuer always finds the page it
expects in the slot it computes; the row page a row-sum warp reads is never overwritten while it
reads.  The same file shows why the row-sum role may not wait on a slot's `full` barrier: that
variant aliases phases and loses a page within a few jobs.
"""
import random
from collections import deque

import pytest


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, parity):          # mbarrier.try_wait.parity
        return (self.phase & 1) != parity


class Fifo:                           # the slots in the order in which they become free
    def __init__(self):
        self.q, self.u = deque([0, 1, 2]), [0, 0, 0]

    def pop(self):
        return self.q.popleft()

    def push(self, v):
        self.q.append(v)

    def use(self, v):                 # parity of the number of earlier loads into slot v
        r = self.u[v] & 1
        self.u[v] += 1
        return r


class Violation(Exception):
    pass


def run(seed, njobs=40, rowsum_waits_on_full=False):
    rnd = random.Random(seed)
    jobs = [rnd.randint(1, 9) for _ in range(njobs)]
    full, empty = [Bar(1) for _ in range(3)], [Bar(1) for _ in range(3)]
    tfull, tempty = [Bar(1), Bar(1)], [Bar(1), Bar(1)]
    adone, aready = [Bar(1), Bar(1)], [Bar(1), Bar(1)]
    content, reading = [None] * 3, {}

    def wait(bar, parity):
        while not bar.done(parity):
            yield

    def producer():
        f, pend, done_jobs = Fifo(), [0, 0, 0], 0

        def load(slot, what):
            yield from wait(empty[slot], (f.use(slot) & 1) ^ 1)
            if pend[slot]:            # the row-sum warps still read the row page this slot held
                k = pend[slot] - 1
                yield from wait(adone[k & 1], (k >> 1) & 1)
                pend[slot] = 0
            if slot in reading:
                raise Violation("page overwritten while the row-sum warps read it")
            content[slot] = what
            for _ in range(rnd.randint(0, 5)):
                yield
            full[slot].arrive()

        for j, nb in enumerate(jobs):
            sa = f.pop()
            yield from load(sa, ("A", j))
            for i in range(nb):
                sb = f.pop()
                f.push(sb)
                yield from load(sb, ("B", j, i))
            f.push(sa)
            done_jobs += 1
            pend[sa] = done_jobs

    def mma():
        f, use = Fifo(), 0
        for j, nb in enumerate(jobs):
            sa = f.pop()
            yield from wait(full[sa], f.use(sa))
            if content[sa] != ("A", j):
                raise Violation("wrong row page")
            aready[j & 1].arrive()
            for i in range(nb):
                sb = f.pop()
                f.push(sb)
                yield from wait(full[sb], f.use(sb))
                if content[sb] != ("B", j, i):
                    raise Violation("wrong column page")
                for g in range(2):
                    yield from wait(tempty[g], (use & 1) ^ 1)
                    for _ in range(rnd.randint(1, 4)):
                        yield
                    if content[sa] != ("A", j):
                        raise Violation("row page lost under the products")
                    tfull[g].arrive()
                use += 1
                empty[sb].arrive()
            empty[sa].arrive()
            f.push(sa)

    def epilogue():
        use = 0
        for nb in jobs:
            for _ in range(nb):
                for g in range(2):
                    yield from wait(tfull[g], use & 1)
                    for _ in range(rnd.randint(0, 3)):
                        yield
                    tempty[g].arrive()
                    for _ in range(rnd.randint(0, 6)):
                        yield
                use += 1

    def rowsum():
        f, nj = Fifo(), 0
        for j, nb in enumerate(jobs):
            sa = f.pop()
            if rowsum_waits_on_full:
                yield from wait(full[sa], f.use(sa))
            else:
                yield from wait(aready[nj & 1], (nj >> 1) & 1)
            reading[sa] = j
            for _ in range(rnd.randint(0, 40)):
                if content[sa] != ("A", j):
                    raise Violation("the row-sum warps read a page that is not theirs")
                yield
            del reading[sa]
            adone[nj & 1].arrive()
            nj += 1
            for _ in range(nb):
                sb = f.pop()
                f.push(sb)
                if rowsum_waits_on_full:
                    f.use(sb)
            f.push(sa)

    procs = [producer(), mma(), epilogue(), rowsum()]
    alive, steps = [True] * 4, 0
    while any(alive):
        i = rnd.randrange(4)
        if alive[i]:
            try:
                next(procs[i])
            except StopIteration:
                alive[i] = False
        steps += 1
        if steps > 400000:
            raise Violation("deadlock")


@pytest.mark.parametrize("seed", range(25))
def test_protocol_has_no_deadlock_and_loses_no_page(seed):
    run(seed)


def test_waiting_on_the_slot_barrier_from_the_row_sum_role_is_unsafe():
    """The variant that was on the GPU first (and timed out there): it fails in the model too."""
    failures = 0
    for seed in range(10):
        try:
            run(seed, rowsum_waits_on_full=True)
        except Violation:
            failures += 1
    assert failures > 0
