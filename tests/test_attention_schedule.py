"""Host model of the attention kernel's work distribution and of the MMA role's ring and
barrier bookkeeping (fa_fwd_sm100.cu: ItemIter, tile_counts, causal_pair_mode,
fa_mma_role and the loader in fa_fwd_kernel), checked on CPU:

  * every (block, batch*head) item is taken by exactly one CTA, whatever the mode;
  * the paired causal schedule gives every pair the same number of key tiles;
  * the chooser between the two static causal schedules never picks the one whose
    longest CTA is more than a tenth longer;
  * the MMA role waits for the K/V ring slots in exactly the order, and with exactly the
    phase parities, in which the loader fills them, releases every slot once, and
    commits q_free / o_done once and s_full nt times per stage and item -- with the
    items chained into one stream (head dim 128) and without (head dim 64).
"""
import itertools

import pytest

SM = 148


def tile_counts(mb, nt_all, causal):
    if causal:
        return min(2 * mb + 1, nt_all), min(2 * mb + 2, nt_all)
    return nt_all, nt_all


def items_of(cta, grid, bh, nmb, causal, pair_mode):
    """The (mb, bh) items CTA `cta` takes, in order (ItemIter::next)."""
    out, v = [], 0
    if not causal or not pair_mode:
        while cta + v * grid < bh * nmb:
            w = cta + v * grid
            v += 1
            out.append((nmb - 1 - w % nmb if causal else w % nmb, w // nmb))
        return out
    pph = (nmb + 1) // 2
    while True:
        q = cta + (v >> 1) * grid
        if q >= bh * pph:
            return out
        b, t = divmod(q, pph)
        far = nmb - 1 - t
        second = v & 1
        v += 1
        if not second:
            out.append((far, b))
        elif t != far:
            out.append((t, b))


def causal_pair_mode(bh, nmb, nt_all, sm=SM):
    items, pph = bh * nmb, (nmb + 1) // 2
    pairs = bh * pph
    ln = lambda mb: sum(tile_counts(mb, nt_all, True))
    gi, gp = min(items, sm), min(pairs, sm)
    worst_i = max(sum(ln(nmb - 1 - w % nmb) for w in range(c, items, gi)) for c in range(gi))
    worst_p = 0
    for c in range(gp):
        s = 0
        for q in range(c, pairs, gp):
            t = q % pph
            far = nmb - 1 - t
            s += ln(far) + (ln(t) if t != far else 0)
        worst_p = max(worst_p, s)
    return (1 if worst_p * 10 <= worst_i * 11 else 0), worst_i, worst_p


@pytest.mark.parametrize("causal,pair_mode", [(False, 0), (True, 0), (True, 1)])
def test_every_item_exactly_once(causal, pair_mode):
    for bh, nmb in itertools.product([1, 2, 3, 7, 64, 150, 333], [1, 2, 3, 4, 5, 16, 33]):
        units = bh * ((nmb + 1) // 2) if (causal and pair_mode) else bh * nmb
        grid = min(units, SM)
        seen = []
        for cta in range(grid):
            seen += items_of(cta, grid, bh, nmb, causal, pair_mode)
        assert sorted(seen) == sorted(itertools.product(range(nmb), range(bh))), (bh, nmb)


def test_pairs_are_equally_long():
    for nmb in [2, 4, 16, 32]:           # S a multiple of 512
        nt_all = 2 * nmb
        for cta in range(min(SM, 5 * (nmb // 2))):
            its = items_of(cta, min(SM, 5 * (nmb // 2)), 5, nmb, True, 1)
            for a, b in zip(its[0::2], its[1::2]):
                assert a[1] == b[1]
                assert sum(tile_counts(a[0], nt_all, True)) + sum(tile_counts(b[0], nt_all, True)) == 4 * nmb + 2


def test_chooser_keeps_within_a_tenth():
    for bh, nmb in itertools.product([1, 4, 16, 37, 64, 256], [1, 2, 5, 9, 16, 32]):
        for nt_all in (2 * nmb - 1, 2 * nmb):
            mode, worst_i, worst_p = causal_pair_mode(bh, nmb, nt_all)
            assert (worst_p * 10 <= worst_i * 11) == bool(mode), (bh, nmb, nt_all)
            if nmb == 1:
                assert mode == 1 and worst_p == worst_i      # a lone block is its own pair
    assert causal_pair_mode(256, 32, 64)[0] == 1          # the large causal configuration uses pairs


def loader_fills(item_tiles, slots):
    """(slot, parity) of every K/V tile in the order the loader issues them: per item
    K_0, then V_j and K_{j+1} alternately (nt1 of each)."""
    fills, it = [], 0
    for nt0, nt1 in item_tiles:
        for _ in range(2 * nt1):
            fills.append((it % slots, (it // slots) & 1))
            it += 1
    return fills


def mma_role(item_tiles, slots, stream, causal):
    """The MMA role's slot waits / releases and per-item commits, as fa_mma_role issues them."""
    waits, frees, log = [], [], []
    slot, ph = 0, 0

    def advance(n):
        nonlocal slot, ph
        slot += n
        if slot >= slots:
            slot -= slots
            ph ^= 1

    def first_qk(i, s, nt_s):
        log.append(("s_full", i, s))
        if nt_s == 1:
            log.append(("q_free", i, s))

    def start_item(i, nts):
        waits.append((slot, ph))
        first_qk(i, 0, nts[0])
        first_qk(i, 1, nts[1])
        frees.append(slot)
        advance(1)

    n = len(item_tiles)
    if n:
        start_item(0, item_tiles[0])
    for i, nt in enumerate(item_tiles):
        have2 = i + 1 < n
        chain = stream and have2
        for j in range(nt[1]):
            VS, KS = slot, (slot + 1) % slots
            last = j + 1 == nt[1]
            need_k = (not last) or chain
            waits.append((VS, ph))
            if need_k:
                waits.append((KS, ph ^ 1 if KS == 0 else ph))
            for s in range(2):
                if not causal or j < nt[s]:
                    log.append(("pv", i, s))
                    if j + 1 < nt[s]:
                        log.append(("s_full", i, s))
                        if j + 2 == nt[s]:
                            log.append(("q_free", i, s))
                    else:
                        log.append(("o_done", i, s))
                if last and chain:
                    first_qk(i + 1, s, item_tiles[i + 1][s])
            frees.append(VS)
            if need_k:
                frees.append(KS)
            advance(2 if need_k else 1)
        if have2 and not stream:
            start_item(i + 1, item_tiles[i + 1])
    return waits, frees, log


@pytest.mark.parametrize("slots,stream", [(5, True), (8, False), (5, False), (8, True)])
@pytest.mark.parametrize("causal", [False, True])
def test_mma_role_follows_the_loader(slots, stream, causal):
    cases = []
    for nmb, nt_all in [(1, 1), (1, 2), (2, 3), (2, 4), (3, 5), (8, 16), (5, 9)]:
        order = list(range(nmb - 1, -1, -1)) if causal else list(range(nmb))
        cases.append([tile_counts(mb, nt_all, causal) for mb in order] * 3)
    if causal:   # a pair-mode CTA: far block, near block, far block, ...
        cases.append([tile_counts(mb, 32, True) for mb in (15, 0, 14, 1, 13, 2)])
    for item_tiles in cases:
        waits, frees, log = mma_role(item_tiles, slots, stream, causal)
        fills = loader_fills(item_tiles, slots)
        assert waits == fills, (item_tiles, slots, stream)
        assert frees == [s for s, _ in fills]
        for i, nt in enumerate(item_tiles):
            for s in range(2):
                assert log.count(("q_free", i, s)) == 1
                assert log.count(("o_done", i, s)) == 1
                assert log.count(("s_full", i, s)) == nt[s] == log.count(("pv", i, s))
                # a stage's scores of tile t are issued before its P V of tile t
                ev = [e[0] for e in log if e[1:] == (i, s) and e[0] in ("s_full", "pv")]
                depth = 0
                for e in ev:
                    depth += 1 if e == "s_full" else -1
                    assert 0 <= depth <= 1
