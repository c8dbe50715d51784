"""Host model of the GEMM's stream-K tail schedule (gemm_sm100.cu: Sched / UnitIter /
sk_owner and the policy in launch_gemm), checked exhaustively on CPU: every
k-iteration of every tile is covered exactly once, a CTA parks at most one partial
tile per slab, and the reducer's arithmetic (which CTAs hold parts of a tile, in
which slab) agrees with what the CTAs do."""
import itertools

SM = 148
MIN_ITERS = 8


def policy(tiles, kiters, sm=SM):
    """-> (grid, dp_tiles, sk_tiles, sk_ctas), as launch_gemm decides."""
    if tiles * 2 <= sm:
        ctas = min(tiles * kiters // MIN_ITERS, sm)
        if ctas >= 2 * tiles:
            return ctas, 0, tiles, ctas
    return min(tiles, sm), tiles, 0, 0


def general(tiles, kiters, sk_tiles, ctas, sm=SM):
    """A schedule the kernel supports though the policy does not pick it: whole tiles
    first, the last sk_tiles cut along K over `ctas` CTAs."""
    return (sm if tiles - sk_tiles > 0 else ctas), tiles - sk_tiles, sk_tiles, ctas


def units_of(cta, grid, dp_tiles, sk_tiles, sk_ctas, kiters):
    out, i = [], 0
    while cta + i * grid < dp_tiles:
        out.append((cta + i * grid, 0, kiters, 0))
        i += 1
    if cta < sk_ctas:
        total = sk_tiles * kiters
        begin = it = total * cta // sk_ctas
        end = total * (cta + 1) // sk_ctas
        while it < end:
            t = it // kiters
            k0 = it - t * kiters
            ln = min(end - it, kiters - k0)
            out.append((dp_tiles + t, k0, k0 + ln, 0 if it == begin else 1))
            it += ln
    return out


def sk_owner(x, total, ctas):
    return ((x + 1) * ctas - 1) // total


def check(tiles, kiters, sched=None):
    grid, dp, sk, ctas = sched or policy(tiles, kiters)
    assert dp + sk == tiles and grid <= SM
    cover = {}
    parts = {}
    for c in range(grid):
        slabs_used = set()
        for tile, k0, k1, slab in units_of(c, grid, dp, sk, ctas, kiters):
            assert 0 <= k0 < k1 <= kiters
            for k in range(k0, k1):
                assert (tile, k) not in cover
                cover[(tile, k)] = c
            if not (k0 == 0 and k1 == kiters):
                assert tile >= dp and slab not in slabs_used
                slabs_used.add(slab)
                parts.setdefault(tile, []).append((c, slab))
    assert len(cover) == tiles * kiters
    total = sk * kiters
    for tile, got in parts.items():
        x0 = (tile - dp) * kiters
        c_first = sk_owner(x0, total, ctas)
        nseg = sk_owner(x0 + kiters - 1, total, ctas) - c_first + 1
        want = [(c, 0 if total * c // ctas >= x0 else 1) for c in range(c_first, c_first + nseg)]
        assert sorted(got) == want, (tiles, kiters, tile)
        assert nseg >= 2
    return sk


def test_schedule_covers_every_iteration_once():
    split = 0
    for tiles, kiters in itertools.product(list(range(1, 80)) + [100, 147, 148, 149, 296, 2048],
                                           [1, 2, 4, 8, 16, 31, 64, 128, 256]):
        split += 1 if check(tiles, kiters) else 0
    assert split > 100          # the policy does take the split path on many of these
    # mixed schedules (whole tiles, then a tail cut along K)
    for tiles, sk, ctas, kiters in [(256, 108, 148, 128), (300, 4, 37, 64), (149, 1, 148, 256), (200, 52, 100, 31)]:
        assert check(tiles, kiters, general(tiles, kiters, sk, ctas)) == sk


def test_policy_examples():
    assert policy(2048, 128)[2] == 0            # 8192^3: left alone
    assert policy(1, 128) == (16, 0, 1, 16)     # one tile, K = 8192: sixteen CTAs share it
    assert policy(4, 128) == (64, 0, 4, 64)
    assert policy(32, 128) == (148, 0, 32, 148)
    assert policy(74, 8)[2] == 0                # K too short to give every CTA 8 iterations twice over
    assert policy(75, 128)[2] == 0              # more than half the SMs busy anyway
