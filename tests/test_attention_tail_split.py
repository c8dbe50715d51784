"""The attention kernel's work distribution with the last round cut along the key axis
(ptx.jl_b200/csrc/attn_sched.cuh, plan_schedule in fa_fwd_sm100.cu), checked on CPU through
ptxb200_fa_plan, which runs the very code the launcher and the kernel run.

The reference deals whole (m_block, batch*head) items round robin
(test/gpu/blackwell/flash_attention_defs.jl:269-272); these tests pin what the cut adds:
every key tile of every item is still computed exactly once, the pieces of an item sit in
consecutive CTAs with exactly one combiner, every piece that is parked is the first thing
its CTA runs in the tail (one scratch slot per CTA), no piece is shorter than two tiles,
and the busiest CTA is never busier than under the plain round robin.
"""
import ctypes
import itertools

import pytest

SM = 148
FA_SINGLE_BLOCKS, FA_NO_TAIL_SPLIT, FA_ALWAYS = 0x2, 0x4, 0x8
MAX_SEGS, MAX_PARTS = 8, 8


def plan(pkg, BH, S, causal, flags=0, sm=SM):
    cap = 16 + sm * (1 + 6 * MAX_SEGS)
    buf = (ctypes.c_int * cap)()
    n = pkg.native.lib().ptxb200_fa_plan(1, BH, S, int(causal), flags, sm, buf, cap)
    assert n >= 10, n
    v = list(buf)[:n]
    keys = ["nmb", "bh", "nt_all", "causal", "pair", "grid", "full", "tail_units", "tail_steps", "tail_ctas"]
    sc = dict(zip(keys, v[:10]))
    ctas, i = [], 10
    if sc["tail_units"] > 0:
        for _ in range(sc["tail_ctas"]):
            k = v[i]
            i += 1
            segs = [tuple(v[i + 6 * j: i + 6 * j + 6]) for j in range(k)]
            i += 6 * k
            ctas.append(segs)
    assert i == n
    return sc, ctas


def item_steps(mb, nt_all, causal):
    return min(2 * mb + 2, nt_all) if causal else nt_all


def unit_items(sc, q):
    n = sc["nmb"]
    if not sc["causal"] or not sc["pair"]:
        bh, r = divmod(q, n)
        return [(n - 1 - r if sc["causal"] else r, bh)]
    pph = (n + 1) // 2
    bh, t = divmod(q, pph)
    far = n - 1 - t
    return [(far, bh)] + ([(t, bh)] if t != far else [])


def units_total(sc):
    return sc["bh"] * ((sc["nmb"] + 1) // 2 if (sc["causal"] and sc["pair"]) else sc["nmb"])


def check_plan(sc, ctas):
    """All invariants of one plan; returns (busiest CTA's steps, steps of the round robin part)."""
    nt_all, causal = sc["nt_all"], sc["causal"]
    covered = {}
    # round robin part
    per_cta = [0] * sc["grid"]
    for q in range(sc["full"]):
        for mb, bh in unit_items(sc, q):
            ln = item_steps(mb, nt_all, causal)
            for j in range(ln):
                assert (mb, bh, j) not in covered
                covered[(mb, bh, j)] = "rr"
            per_cta[q % sc["grid"]] += ln
    assert sc["full"] % sc["grid"] == 0 or sc["tail_units"] == 0
    rr_worst = max(per_cta)
    if sc["tail_units"] == 0:
        assert sc["full"] == units_total(sc)
        assert len(covered) == sum(item_steps(mb, nt_all, causal) for mb in range(sc["nmb"])) * sc["bh"]
        return rr_worst, rr_worst
    assert sc["full"] + sc["tail_units"] == units_total(sc)
    assert 2 <= sc["tail_ctas"] <= sc["grid"] and sc["tail_units"] < sc["grid"]
    line = 0
    for c, segs in enumerate(ctas):
        assert 1 <= len(segs) <= MAX_SEGS, (c, segs)
        for i, (mb, bh, j0, j1, ln, n_other) in enumerate(segs):
            assert ln == item_steps(mb, nt_all, causal)
            assert 0 <= j0 < j1 <= ln
            whole = j0 == 0 and j1 == ln
            assert whole or j1 - j0 >= (2 if causal else 1), (c, segs)
            if causal:
                # the item's first stage (one tile fewer unless the sequence ends first) is never empty
                full0 = min(2 * mb + 1, nt_all)
                assert min(j1, full0) - j0 >= 1
            if j0 > 0:
                assert i == 0, "a parked piece must be its CTA's first tail segment"
                assert n_other == 0
            if j0 == 0 and j1 < ln:
                assert i == len(segs) - 1, "a combiner's piece ends its CTA's span"
                assert 1 <= n_other <= MAX_PARTS - 1
                # the following CTAs continue the item, in order, up to its end
                at = j1
                for k in range(1, n_other + 1):
                    m2, b2, a0, a1, l2, no2 = ctas[c + k][0]
                    assert (m2, b2, a0, l2) == (mb, bh, at, ln) and no2 == 0
                    at = a1
                assert at == ln
            else:
                assert n_other == 0 or j0 > 0
            for j in range(j0, j1):
                assert (mb, bh, j) not in covered, (mb, bh, j)
                covered[(mb, bh, j)] = c
            per_cta[c] += j1 - j0
            line += j1 - j0
    assert line == sc["tail_steps"]
    want = sum(item_steps(mb, nt_all, causal) for mb in range(sc["nmb"])) * sc["bh"]
    assert len(covered) == want
    return max(per_cta), rr_worst


def legacy_worst(pkg, BH, S, causal, flags):
    sc, _ = plan(pkg, BH, S, causal, flags | FA_NO_TAIL_SPLIT)
    assert sc["tail_units"] == 0
    per = [0] * sc["grid"]
    for q in range(sc["full"]):
        per[q % sc["grid"]] += sum(item_steps(mb, sc["nt_all"], causal) for mb, _ in unit_items(sc, q))
    return max(per)


@pytest.mark.parametrize("causal", [False, True])
def test_every_tile_once_and_never_busier_than_round_robin(pkg, causal):
    n_split = n_forced = 0
    for BH, S in itertools.product([1, 2, 3, 5, 8, 13, 32, 37, 64, 100, 149, 256, 300],
                                   [128, 200, 256, 300, 512, 640, 1000, 1024, 2048, 4096, 5000, 8192]):
        if BH * S > 1_000_000:
            continue
        for flags in ([0, FA_SINGLE_BLOCKS] if causal else [0]):
            # the default policy cuts only where it expects a gain of a twelfth or more ...
            sc, ctas = plan(pkg, BH, S, causal, flags)
            worst, _ = check_plan(sc, ctas)
            if sc["tail_units"] > 0:
                n_split += 1
                assert (worst + 3) * 100 <= legacy_worst(pkg, BH, S, causal, flags) * 92, (BH, S, flags)
            # ... and a forced cut is valid wherever one is possible
            sc, ctas = plan(pkg, BH, S, causal, flags | FA_ALWAYS)
            check_plan(sc, ctas)
            n_forced += sc["tail_units"] > 0
    assert n_split > 10 and n_forced > 40      # the sweep does exercise the cut


def test_flag_keeps_the_round_robin(pkg):
    for BH, S, causal in [(8, 4096, False), (32, 8192, True), (3, 1000, True)]:
        sc, ctas = plan(pkg, BH, S, causal, FA_NO_TAIL_SPLIT)
        assert sc["tail_units"] == 0 and not ctas
        check_plan(sc, ctas)


def test_an_eighth_of_the_headline_problem_fills_every_sm(pkg):
    """B*H = 8 heads of S = 4096 (one GPU's share of the headline problem split eight
    ways): 128 items of 32 steps on 148 SMs. The round robin leaves 20 SMs idle for the whole
    launch; cut, every SM runs 27-28 steps. The default policy leaves this launch whole --
    a second segment with its parking and merging costs about three steps, measured, and
    four are saved -- so the cut is forced here."""
    assert plan(pkg, 8, 4096, False)[0]["tail_units"] == 0
    sc, ctas = plan(pkg, 8, 4096, False, FA_ALWAYS)
    assert (sc["grid"], sc["full"], sc["tail_units"], sc["tail_steps"], sc["tail_ctas"]) == (148, 0, 128, 4096, 148)
    worst, _ = check_plan(sc, ctas)
    per = [sum(j1 - j0 for _, _, j0, j1, _, _ in segs) for segs in ctas]
    assert worst == 28 and min(per) >= 27
    assert max(len(s) for s in ctas) <= 2


def test_causal_long_context_share(pkg):
    """32 heads of S = 8192 causal (an eighth of the long-context configuration): 512 pairs
    of 66 steps; three full rounds and 68 pairs cut over 148 SMs."""
    sc, ctas = plan(pkg, 32, 8192, True)       # cut by default: 4 rounds of 66 steps become 3 and 30 steps
    assert sc["pair"] == 1 and sc["full"] == 444 and sc["tail_units"] == 68
    worst, rr = check_plan(sc, ctas)
    assert rr == 3 * 66 and worst <= rr + 33
    assert legacy_worst(pkg, 32, 8192, True, 0) == 4 * 66


def test_other_sm_counts(pkg):
    for sm in (16, 132, 148, 160, 240):
        for BH, S, causal in [(8, 4096, False), (5, 3000, True), (40, 768, False)]:
            sc, ctas = plan(pkg, BH, S, causal, FA_ALWAYS, sm)
            check_plan(sc, ctas)
