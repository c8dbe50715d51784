"""Discrete-event model of the attention kernel's barrier protocol (fa_fwd_sm100.cu),
run on CPU under random interleavings.

Each role of the kernel is an agent (a generator): the TMA loader, the MMA-issue thread,
the two softmax warpgroups, the correction warpgroup (a warpgroup's 128 threads act
alike, so each is one agent and a 128- or 256-arrival barrier counts 1 or 2 here), plus
two asynchronous engines the hardware provides: the TMA unit, which completes loads
some time after they are issued, and the tensor pipe, which executes the issued MMAs and
commits in order. A scheduler picks any agent that can move, at random.

Checked on every run: no deadlock; no barrier is ever two phases ahead of one of its
waiters (a parity wait could not tell); and no buffer is overwritten before its last
reader is done -- the K/V ring slots, the Q tiles, the per-tile basis, the per-item row
sums, and the O accumulators. The model also shows why the l_free hand-over exists:
without it the row sums of a short item are overwritten before the epilogue reads them.
"""
import random

import pytest

from test_attention_schedule import tile_counts


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.done = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.done = self.count, self.done + 1


class Kernel:
    def __init__(self, items, slots, stream, causal, rng, use_l_free=True):
        self.items, self.slots, self.stream, self.causal = items, slots, stream, causal
        self.rng, self.use_l_free = rng, use_l_free
        B = lambda c: [Bar(c), Bar(c)]
        self.q_full, self.q_free, self.s_full = B(1), B(1), B(1)
        self.basis, self.l_ready, self.l_free, self.o_done = B(1), B(1), B(1), B(1)
        self.p_full = [[Bar(2), Bar(2)], [Bar(2), Bar(2)]]
        self.kv_full = [Bar(1) for _ in range(slots)]
        self.kv_free = [Bar(1) for _ in range(slots)]
        self.tma, self.pipe = [], []                  # issued, not yet completed
        self.slot_reads = [0] * slots                 # MMAs issued on a slot, not yet executed
        self.q_item, self.q_reads = [-1, -1], [0, 0]  # item whose Q is loaded; reads outstanding
        self.neg_read, self.l_read = [True, True], [True, True]
        self.o_free = [True, True]

    def wait(self, bar, n):
        """Block until phase n of `bar` has completed (the kernel waits on parity n & 1)."""
        while bar.done <= n:
            yield
        assert bar.done == n + 1, "a barrier ran two phases ahead of a waiter"

    # ---- engines --------------------------------------------------------------------
    def tma_engine(self):
        while True:
            if self.tma and self.rng.random() < 0.7:
                kind, idx, item, bar = self.tma.pop(0)
                if kind == "kv":
                    assert self.slot_reads[idx] == 0, "ring slot overwritten under an MMA"
                else:
                    assert self.q_reads[idx] == 0, "Q tile overwritten under an MMA"
                    self.q_item[idx] = item
                bar.arrive()
            yield

    def pipe_engine(self):
        while True:
            if self.pipe and self.rng.random() < 0.7:
                op = self.pipe.pop(0)
                if op[0] == "qk":
                    _, s, slot, item = op
                    assert self.q_item[s] == item, "scores computed on another item's Q"
                    self.slot_reads[slot] -= 1
                    self.q_reads[s] -= 1
                elif op[0] == "pv":
                    _, s, slot, first = op
                    if first:
                        assert self.o_free[s], "O overwritten before the epilogue read it"
                        self.o_free[s] = False
                    self.slot_reads[slot] -= 1
                else:
                    op[1].arrive()
            yield

    # ---- roles ----------------------------------------------------------------------
    def loader(self):
        it = 0

        def kv_load():
            nonlocal it
            s, n = it % self.slots, it // self.slots
            if n > 0:
                yield from self.wait(self.kv_free[s], n - 1)
            self.tma.append(("kv", s, None, self.kv_full[s]))
            it += 1

        for i, (nt0, nt1) in enumerate(self.items):
            if i > 0:
                yield from self.wait(self.q_free[0], i - 1)
            self.tma.append(("q", 0, i, self.q_full[0]))
            yield from kv_load()
            if i > 0:
                yield from self.wait(self.q_free[1], i - 1)
            self.tma.append(("q", 1, i, self.q_full[1]))
            for j in range(nt1):
                yield from kv_load()
                if j + 1 < nt1:
                    yield from kv_load()
            yield

    def mma(self):
        slots = self.slots
        pos = 0                      # ring position: slot = pos % slots, fill index = pos // slots
        cnt_pv = [0, 0]
        commit = lambda bar: self.pipe.append(("commit", bar))

        def wait_tile(p):
            yield from self.wait(self.kv_full[p % slots], p // slots)

        def qk(s, p, item):
            self.slot_reads[p % slots] += 1
            self.q_reads[s] += 1
            self.pipe.append(("qk", s, p % slots, item))
            commit(self.s_full[s])

        def first_qk(s, p, item, nt_s):
            yield from self.wait(self.q_full[s], item)
            qk(s, p, item)
            if nt_s == 1:
                commit(self.q_free[s])

        def start_item(i):
            nonlocal pos
            yield from wait_tile(pos)
            yield from first_qk(0, pos, i, self.items[i][0])
            yield from first_qk(1, pos, i, self.items[i][1])
            commit(self.kv_free[pos % slots])
            pos += 1

        n = len(self.items)
        if n:
            yield from start_item(0)
        for i, nt in enumerate(self.items):
            chain = self.stream and i + 1 < n
            for j in range(nt[1]):
                vs, ks = pos, pos + 1
                last = j + 1 == nt[1]
                need_k = (not last) or chain
                yield from wait_tile(vs)
                if need_k:
                    yield from wait_tile(ks)
                for s in range(2):
                    if not self.causal or j < nt[s]:
                        for h in range(2):
                            yield from self.wait(self.p_full[s][h], cnt_pv[s])
                        self.slot_reads[vs % slots] += 1
                        self.pipe.append(("pv", s, vs % slots, j == 0))
                        cnt_pv[s] += 1
                        if j + 1 < nt[s]:
                            qk(s, ks, i)
                            if j + 2 == nt[s]:
                                commit(self.q_free[s])
                        else:
                            commit(self.o_done[s])
                    if last and chain:
                        yield from first_qk(s, ks, i + 1, self.items[i + 1][s])
                commit(self.kv_free[vs % slots])
                if need_k:
                    commit(self.kv_free[ks % slots])
                pos += 2 if need_k else 1
                yield
            if i + 1 < n and not self.stream:
                yield from start_item(i + 1)

    def softmax(self, s):
        cnt_s = 0
        for i, nt in enumerate(self.items):
            for j in range(nt[s]):
                yield from self.wait(self.s_full[s], cnt_s)
                cnt_s += 1
                yield                                   # row maximum
                assert self.neg_read[s], "basis overwritten before the correction warps read it"
                self.neg_read[s] = False
                self.basis[s].arrive()
                yield                                   # exponentials, first half of P
                self.p_full[s][0].arrive()
                yield
                self.p_full[s][1].arrive()
            if i > 0 and self.use_l_free:
                yield from self.wait(self.l_free[s], i - 1)
            assert self.l_read[s], "row sums overwritten before the epilogue read them"
            self.l_read[s] = False
            self.l_ready[s].arrive()

    def correction(self):
        self.p_full[0][0].arrive()
        self.p_full[1][0].arrive()
        cnt = [0, 0]
        for i, nt in enumerate(self.items):
            for j in range(nt[1]):
                for s in range(2):
                    if j < nt[s]:
                        yield from self.wait(self.s_full[s], cnt[s])
                        yield from self.wait(self.basis[s], cnt[s])
                        cnt[s] += 1
                        self.neg_read[s] = True
                        if j > 0:
                            yield                       # O rescale, if any
                            self.p_full[s][0].arrive()
                        yield                           # its share of the exponentials
                        self.p_full[s][1].arrive()
            for s in range(2):
                yield from self.wait(self.o_done[s], i)
                yield from self.wait(self.l_ready[s], i)
                self.l_read[s] = True
                self.l_free[s].arrive()
                yield                                   # O -> registers
                self.o_free[s] = True
                self.p_full[s][0].arrive()
                yield                                   # stores

    def run(self, max_steps=4_000_000, skew=False):
        """skew: every role and engine gets a speed of its own for the run (some a
        hundred times slower than others), which reaches interleavings that a uniform
        choice practically never does."""
        roles = {"loader": self.loader(), "mma": self.mma(), "softmax0": self.softmax(0),
                 "softmax1": self.softmax(1), "correction": self.correction()}
        engines = [self.tma_engine(), self.pipe_engine()]
        w = {k: self.rng.choice([0.03, 0.3, 1.0, 4.0]) if skew else 1.0 for k in roles}
        ew = [self.rng.choice([0.1, 1.0, 5.0]) if skew else 1.0 for _ in engines]
        idle = 0
        for _ in range(max_steps):
            if not roles:
                break
            before = self._state()
            names = list(roles)
            name = self.rng.choices(names, [w[n] for n in names])[0]
            try:
                next(roles[name])
            except StopIteration:
                del roles[name]
            next(self.rng.choices(engines, ew)[0])
            idle = idle + 1 if self._state() == before and name in roles else 0
            assert idle < 200000, f"deadlock; still running: {sorted(roles)}"
        assert not roles, "step limit"
        while self.pipe or self.tma:                    # drain the engines
            next(engines[0]), next(engines[1])

    def _state(self):
        bars = self.q_full + self.q_free + self.s_full + self.basis + self.l_ready + self.l_free + self.o_done
        bars += self.p_full[0] + self.p_full[1] + self.kv_full + self.kv_free
        return tuple((b.done, b.pending) for b in bars) + (len(self.tma), len(self.pipe))


def _item_lists(causal):
    out = []
    for nmb, nt_all in [(1, 1), (1, 2), (2, 3), (2, 4), (4, 8)]:
        order = list(range(nmb - 1, -1, -1)) if causal else list(range(nmb))
        out.append([tile_counts(mb, nt_all, causal) for mb in order] * 4)
    if causal:
        out.append([tile_counts(mb, 16, True) for mb in (7, 0, 6, 1, 5, 2)])   # pair mode
    return out


@pytest.mark.parametrize("slots,stream", [(5, True), (8, False)])
@pytest.mark.parametrize("causal", [False, True])
def test_protocol_holds_under_random_interleavings(slots, stream, causal):
    for items in _item_lists(causal):
        for seed in range(12):
            Kernel(items, slots, stream, causal, random.Random(seed)).run()
            if seed < 4:
                Kernel(items, slots, stream, causal, random.Random(1000 + seed)).run(skew=True)


def test_model_sees_the_hazard_l_free_closes():
    """One-tile items as one stream, no l_free: some interleaving lets a stage's softmax
    publish the next item's row sums before the epilogue has read this item's."""
    items = [tile_counts(0, 1, True)] * 8
    hits = 0
    for seed in range(40):
        try:
            Kernel(items, 5, True, True, random.Random(seed), use_l_free=False).run()
        except AssertionError as e:
            assert "row sums" in str(e) or "two phases" in str(e), e
            hits += 1
    assert hits > 0
