"""Work partition of the 9..32-token W4A16 GEMM (csrc/gemv_w4a16_strip.cuh), restated in
Python and checked exhaustively on small cases: units (strip set, quantisation group) are cut
into one contiguous range per CTA, the groups of a set inside a range are shared out among the
K slices of the CTA, a set cut between CTAs is finished by its last contributor from one
partial slot per contributor.  The properties the kernel relies on:
every unit is taken by exactly one (CTA, slice); the contributor interval computed from a set's
first and last unit is exactly the set of CTAs whose ranges meet the set; a CTA never uses one of
its two partial slots for two different cut sets; the per-slice walk (cursor) visits the units in
the order the consumer loop does."""
import itertools

import pytest


def cta_range(total, ncta, cta):
    base, rem = divmod(total, ncta)
    u0 = cta * base + min(cta, rem)
    return u0, u0 + base + (1 if cta < rem else 0)


def share(s, u0, u1, G, wk, WK):
    ga, gb = max(u0 - s * G, 0), min(u1 - s * G, G)
    n = gb - ga
    base, rem = divmod(n, WK) if n > 0 else (0, 0)
    a = ga + wk * base + min(wk, rem)
    return a, a + base + (1 if wk < rem else 0)


def owner_of_unit(u, total, ncta):
    base, rem = divmod(total, ncta)
    cut = rem * (base + 1)
    return u // (base + 1) if u < cut else rem + (u - cut) // base


def cursor_walk(u0, u1, G, wk, WK):
    """seek / next of W4sCursor: first unit at or after a strip set, then group by group."""
    out = []
    s = u0 // G
    while s * G < u1:
        a, b = share(s, u0, u1, G, wk, WK)
        out.extend((s, g) for g in range(a, b))
        s += 1
    return out


@pytest.mark.parametrize("sets,G,ncta,WK", [
    (1, 4, 3, 2), (2, 4, 148, 2), (16, 16, 148, 2), (16, 32, 148, 2), (56, 32, 148, 2), (112, 32, 148, 2),
    (7, 5, 4, 3), (9, 112, 148, 4), (3, 1, 2, 2), (1002, 32, 148, 2), (33, 7, 148, 4),
])
def test_every_unit_is_taken_once_and_contributors_match(sets, G, ncta, WK):
    total = sets * G
    ncta = min(ncta, total)          # the launcher never starts more CTAs than units
    taken = {}
    slots_used = {}
    for cta in range(ncta):
        u0, u1 = cta_range(total, ncta, cta)
        assert u1 > u0
        s_first, s_last = u0 // G, (u1 - 1) // G
        for wk in range(WK):
            consumer = []
            for s in range(s_first, s_last + 1):
                a, b = share(s, u0, u1, G, wk, WK)
                consumer.extend((s, g) for g in range(a, b))
            assert consumer == cursor_walk(u0, u1, G, wk, WK)
            for unit in consumer:
                assert unit not in taken
                taken[unit] = (cta, wk)
        for s in range(s_first, s_last + 1):
            whole = u0 <= s * G and (s + 1) * G <= u1
            c_first = owner_of_unit(s * G, total, ncta)
            c_last = owner_of_unit(s * G + G - 1, total, ncta)
            meets = [c for c in range(ncta) if cta_range(total, ncta, c)[0] < (s + 1) * G
                     and cta_range(total, ncta, c)[1] > s * G]
            assert meets == list(range(c_first, c_last + 1))
            assert whole == (c_first == c_last)
            if not whole:
                slot = 1 if cta == c_first else 0
                assert (cta, slot) not in slots_used, "a partial slot serves one cut set per launch"
                slots_used[(cta, slot)] = s
    assert set(taken) == set(itertools.product(range(sets), range(G)))


@pytest.mark.parametrize("M,expected", [(9, [9]), (16, [16]), (17, [17]), (24, [24]), (32, [32]), (33, [24, 9]),
                                        (40, [24, 16]), (48, [24, 24]), (63, [32, 31]), (64, [32, 32])])
def test_token_chunks_are_equal_in_whole_token_tiles(M, expected):
    """qlinear.cu: up to 64 tokens go in ceil(M / 32) chunks of equal size rounded up to 8 tokens."""
    nchunks = (M + 31) // 32
    chunk = ((M + nchunks - 1) // nchunks + 7) // 8 * 8
    got = [min(chunk, M - m0) for m0 in range(0, M, chunk)]
    assert got == expected
    assert sum(got) == M and max(got) <= 32
