"""Model check of the synchronisation protocol of the prefill attention kernel (csrc/kernels/attn_prefill.cu).

The kernel has eleven roles per CTA (a TMA producer, one MMA issuer per query tile, four softmax warps per query
tile) that meet on mbarriers whose phases are told apart by one parity bit.  This test restates the protocol as
small Python coroutines over a model of those barriers and of the asynchronous agents (TMA loads complete later,
`tcgen05.commit` arrives when the issuer's earlier MMAs have finished) and runs it under random interleavings for
many shapes.  It checks what a wrong parity, a missing release or a wrong ring order would break:

* no role waits forever (every run ends with all roles finished),
* every consumer sees the data it expects: the ring stage holds the K / V tile the MMA is issued for until that MMA
  has finished, S_t holds the scores of the tile the softmax is about to read, P_t the probabilities of the tile
  whose P V is issued, and O_t has received every earlier P V when it is rescaled or written out,
* nothing is overwritten while a consumer still needs it.

It is a model of the code, kept next to it on purpose: a change of the ring order, of a barrier count or of a
parity expression has to be made in both places, and the model says at once whether the new protocol can hang.
"""
import random

import pytest

KV_STAGES = 3


class Barrier:
    """mbarrier: `count` arrivals complete a phase; a parity test passes when the phase of that parity is over."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
        if self.pending == 0:
            self.pending = self.count
            self.phase += 1

    def test(self, parity):
        return (self.phase & 1) != parity


class Sim:
    def __init__(self, n0, n1, lo0, lo1, seed, lockstep=True):
        """Query tile t attends to KV tiles [lo_t, lo_t + n_t) of the CTA's union range (n1 = 0: no second tile).
        lockstep=False lets an issuer release the stage of a KV tile its query tile skips without waiting for the
        load, which is how the kernel first was written."""
        self.rng = random.Random(seed)
        self.lockstep = lockstep
        self.two = n1 > 0
        self.a_lo = [lo0, lo1 if self.two else 0]
        self.a_hi = [lo0 + n0, lo1 + n1 if self.two else 0]
        self.n_union = max(self.a_hi[0], self.a_hi[1]) if self.two else self.a_hi[0]
        assert min(self.a_lo[0], self.a_lo[1] if self.two else self.a_lo[0]) == 0
        self.kv_full = [Barrier(1) for _ in range(KV_STAGES)]
        self.kv_empty = [Barrier(2 if self.two else 1) for _ in range(KV_STAGES)]
        self.s_full = [Barrier(1), Barrier(1)]
        self.s_empty = [Barrier(4), Barrier(4)]
        self.p_full = [Barrier(4), Barrier(4)]
        self.o_full = [Barrier(1), Barrier(1)]
        self.turn = [[Barrier(1) for _ in range(4)] for _ in range(2)]
        # data tags
        self.stage_tag = [None] * KV_STAGES          # ("K" | "V", x) once the load has landed
        self.stage_readers = [0] * KV_STAGES         # MMAs in flight that read the stage
        self.s_tag = [None, None]                    # local iteration whose scores S_t holds
        self.s_unread = [0, 0]                       # softmax warps that have not read S_t yet
        self.p_tag = [[None] * 4, [None] * 4]        # per softmax warp: iteration whose probabilities it wrote
        self.p_readers = [0, 0]
        self.o_count = [0, 0]                        # P V products accumulated into O_t
        self.events = []                             # (time, fn): asynchronous completions
        self.time = 0
        self.mma_done_at = [0, 0]                    # per issuer: completion time of its latest MMA

    # ---- asynchronous agents
    def later(self, delay, fn):
        self.events.append((self.time + delay, self.rng.random(), fn))

    def run_events(self):
        due = sorted(e for e in self.events if e[0] <= self.time)
        self.events = [e for e in self.events if e[0] > self.time]
        for _, _, fn in due:
            fn()

    def commit(self, t, fn):
        """tcgen05.commit by issuer t: `fn` runs once all MMAs the issuer has issued so far are complete."""
        self.later(max(0, self.mma_done_at[t] - self.time), fn)

    def mma(self, t, start_fn, done_fn):
        """An MMA group by issuer t: executes after the issuer's earlier groups (in order), takes a while."""
        begin = max(self.time, self.mma_done_at[t]) + self.rng.randint(0, 3)
        end = begin + self.rng.randint(1, 6)
        self.mma_done_at[t] = end
        self.later(begin - self.time, start_fn)
        self.later(end - self.time, done_fn)

    # ---- roles (generators yield a predicate to wait for, or None to be rescheduled)
    def producer(self):
        seq = 0
        order = [("K", 0)]
        for u in range(self.n_union):
            if u + 1 < self.n_union:
                order.append(("K", u + 1))
            order.append(("V", u))
        for kind, x in order:
            st, ph = seq % KV_STAGES, (seq // KV_STAGES) & 1
            seq += 1
            yield lambda st=st, ph=ph: self.kv_empty[st].test(ph ^ 1)
            assert self.stage_readers[st] == 0, "ring stage overwritten while an MMA still reads it"

            def landed(st=st, kind=kind, x=x):
                assert self.stage_readers[st] == 0
                self.stage_tag[st] = (kind, x)
                self.kv_full[st].arrive()

            self.stage_tag[st] = None
            self.later(self.rng.randint(1, 12), landed)

    def issuer(self, t):
        if t == 1 and not self.two:
            return
        seq = 0
        a_lo, a_hi = self.a_lo[t], self.a_hi[t]

        def read_stage(st, want):
            def start():
                assert self.stage_tag[st] == want, (self.stage_tag[st], want)
                self.stage_readers[st] += 1
            return start

        def do_k(x):
            nonlocal seq
            if x >= self.n_union:
                return
            item = seq
            seq += 1
            st, par = item % KV_STAGES, (item // KV_STAGES) & 1
            if self.lockstep or a_lo <= x < a_hi:
                yield lambda: self.kv_full[st].test(par)
            if a_lo <= x < a_hi:
                lit = x - a_lo
                yield lambda: self.s_empty[t].test((lit & 1) ^ 1)
                assert self.s_unread[t] == 0, "S_t overwritten before every softmax warp has read it"

                def done(st=st, lit=lit):
                    self.stage_readers[st] -= 1
                    assert self.s_unread[t] == 0
                    self.s_tag[t] = lit
                    self.s_unread[t] = 4

                self.mma(t, read_stage(st, ("K", x)), done)
                self.commit(t, self.s_full[t].arrive)
            self.commit(t, self.kv_empty[st].arrive)

        def do_v(x):
            nonlocal seq
            item = seq
            seq += 1
            st, par = item % KV_STAGES, (item // KV_STAGES) & 1
            if self.lockstep or a_lo <= x < a_hi:
                yield lambda: self.kv_full[st].test(par)
            if a_lo <= x < a_hi:
                lit = x - a_lo
                yield lambda: self.p_full[t].test(lit & 1)

                def start(st=st, lit=lit):
                    read_stage(st, ("V", x))()
                    assert self.p_tag[t] == [lit] * 4, (self.p_tag[t], lit)
                    self.p_readers[t] += 1

                def done(st=st, lit=lit):
                    self.stage_readers[st] -= 1
                    self.p_readers[t] -= 1
                    assert self.o_count[t] == lit, "P V products reach O_t out of order"
                    self.o_count[t] += 1

                self.mma(t, start, done)
                self.commit(t, self.o_full[t].arrive)
            self.commit(t, self.kv_empty[st].arrive)

        yield from do_k(0)
        for u in range(self.n_union):
            yield from do_k(u + 1)
            yield from do_v(u)

    def softmax(self, t, quad):
        n = self.a_hi[t] - self.a_lo[t]
        n_other = self.a_hi[1 - t] - self.a_lo[1 - t]
        for it in range(n):
            yield lambda it=it: self.s_full[t].test(it & 1)
            assert self.s_tag[t] == it, (self.s_tag[t], it)
            self.s_unread[t] -= 1                        # scores are in registers
            self.s_empty[t].arrive()
            yield None
            rescale = it > 0 and self.rng.random() < 0.3
            p_free = it == 0
            if rescale:
                yield lambda it=it: self.o_full[t].test((it - 1) & 1)
                assert self.o_count[t] == it, "O_t rescaled before the previous P V has finished"
                p_free = True
            if not p_free:
                yield lambda it=it: self.o_full[t].test((it - 1) & 1)
            assert self.p_readers[t] == 0, "P_t overwritten while P V still reads it"
            if (it >= 1 and it - 1 < n_other) if t == 0 else (it < n_other):
                yield lambda it=it: self.turn[t][quad].test(((it - 1) if t == 0 else it) & 1)
            yield None
            self.p_tag[t][quad] = it
            self.turn[1 - t][quad].arrive()
            self.p_full[t].arrive()
        if n > 0:
            yield lambda: self.o_full[t].test((n - 1) & 1)
            assert self.o_count[t] == n, "O_t written out before its last P V has finished"

    # ---- scheduler
    def run(self, max_steps=200000):
        roles = {"producer": self.producer(), "issuer0": self.issuer(0), "issuer1": self.issuer(1)}
        for t in range(2):
            for q in range(4):
                roles[f"softmax{t}{q}"] = self.softmax(t, q)
        waiting = {}
        for name, gen in list(roles.items()):
            try:
                waiting[name] = next(gen)
            except StopIteration:
                del roles[name]
        steps = 0
        while roles:
            steps += 1
            assert steps < max_steps, "too many steps"
            self.run_events()
            ready = [nm for nm in roles if waiting[nm] is None or waiting[nm]()]
            if not ready:
                assert self.events, f"deadlock: {sorted(roles)} wait and nothing is in flight"
                self.time = min(e[0] for e in self.events)
                continue
            nm = self.rng.choice(ready)
            try:
                waiting[nm] = next(roles[nm])
            except StopIteration:
                del roles[nm]
            if self.rng.random() < 0.5:
                self.time += 1
        self.time = max([self.time] + [e[0] for e in self.events])
        self.run_events()
        return steps


SHAPES = [
    # n0, n1, lo0, lo1: query tile t attends to union KV tiles [lo_t, lo_t + n_t)
    (1, 0, 0, 0),      # one short query tile, second tile absent
    (5, 0, 0, 0),
    (1, 1, 0, 0),
    (1, 2, 0, 0),      # causal: the second tile has one more (diagonal) KV tile
    (4, 5, 0, 0),
    (7, 7, 0, 0),      # non-causal
    (9, 10, 0, 0),
    (3, 3, 0, 1),      # sliding window: the second tile starts one KV tile later
    (2, 3, 0, 1),
    (6, 2, 0, 0),      # end of context cuts the second tile short
]


@pytest.mark.parametrize("n0,n1,lo0,lo1", SHAPES)
def test_protocol_finishes_and_keeps_its_data_under_random_interleavings(n0, n1, lo0, lo1):
    for seed in range(60):
        Sim(n0, n1, lo0, lo1, seed).run()


def test_the_model_notices_a_broken_protocol():
    """The checks have teeth: a ring whose items come in an order the issuers do not consume hangs or hands the MMA
    the wrong tile."""
    class WrongOrder(Sim):
        def producer(self):
            seq = 0
            order = []
            for u in range(self.n_union):                 # K(u), V(u) instead of K(u+1), V(u)
                order += [("K", u), ("V", u)]
            for kind, x in order:
                st, ph = seq % KV_STAGES, (seq // KV_STAGES) & 1
                seq += 1
                yield lambda st=st, ph=ph: self.kv_empty[st].test(ph ^ 1)

                def landed(st=st, kind=kind, x=x):
                    self.stage_tag[st] = (kind, x)
                    self.kv_full[st].arrive()

                self.later(self.rng.randint(1, 12), landed)

    with pytest.raises(AssertionError):
        for seed in range(20):
            WrongOrder(4, 5, 0, 0, seed).run()


def test_the_model_notices_an_issuer_that_releases_stages_it_has_not_seen_loaded():
    """The defect the first two-issuer version had on the GPU (wrong results for a sequence whose second query tile
    ends early): an issuer that runs ahead through KV tiles it skips arrives twice on one phase of a ring barrier
    and frees a stage the other issuer still reads."""
    caught = 0
    for seed in range(40):
        try:
            Sim(6, 2, 0, 0, seed, lockstep=False).run()
        except AssertionError:
            caught += 1
    assert caught > 0
