"""GPU parity of the two table steps Einsum::prove runs ahead of its sumcheck: permute_evals_by_ranges
(src/basicblock/einsum.rs:142-198) and fix_variables_zkgpt (src/util/poly.rs:1378-1473)."""
import random

import pytest

import pyoracle as o
from zkes_b200 import fix_variables_zkgpt, permute_evals_by_ranges
from zkes_b200._lib import ZkError

pytestmark = pytest.mark.gpu


def random_ranges(rnd, n):
    """A random partition of 0..n into contiguous ranges, in random order."""
    cuts = sorted(rnd.sample(range(1, n), rnd.randrange(0, min(n - 1, 4) + 1))) if n > 1 else []
    edges = [0] + cuts + [n]
    ranges = [(edges[i], edges[i + 1]) for i in range(len(edges) - 1)]
    rnd.shuffle(ranges)
    return ranges


@pytest.mark.parametrize("n", [1, 2, 5, 9, 12])
@pytest.mark.parametrize("integers", [False, True])
def test_permute_matches_oracle(ctx, n, integers):
    rnd = random.Random(100 * n + integers)
    for _ in range(3):
        ranges = random_ranges(rnd, n)
        if integers:
            evals = [rnd.randrange(-(1 << 127), 1 << 127) for _ in range(1 << n)]
        else:
            evals = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
        assert permute_evals_by_ranges(ctx, evals, n, ranges, integers=integers) == o.permute_evals_by_ranges(evals, n, ranges)


def test_permute_identity_and_swap(ctx):
    evals = list(range(16))
    assert permute_evals_by_ranges(ctx, evals, 4, [(0, 4)]) == evals
    # halves swapped: new index = (old >> 2) | ((old & 3) << 2)
    out = permute_evals_by_ranges(ctx, evals, 4, [(2, 4), (0, 2)])
    assert out == [((i & 3) << 2) | (i >> 2) for i in range(16)]
    # empty ranges are allowed inside the list
    assert permute_evals_by_ranges(ctx, evals, 4, [(0, 0), (0, 4), (4, 4)]) == evals


@pytest.mark.parametrize("ranges", [[(0, 2)], [(0, 3), (2, 4)], [(0, 5)], [(3, 2), (0, 4)]])
def test_permute_rejects_bad_ranges(ctx, ranges):
    with pytest.raises(ZkError):
        permute_evals_by_ranges(ctx, list(range(16)), 4, ranges)


@pytest.mark.parametrize("num_vars,k", [(4, 0), (4, 1), (6, 3), (8, 4), (10, 5), (11, 6), (12, 9), (13, 13), (14, 7)])
def test_fix_variables_zkgpt_matches_oracle(ctx, num_vars, k):
    """Small quantised values (the Einsum witnesses), with a q_bits below their range so the reference's
    quotient / remainder branch is taken in the restatement too."""
    rnd = random.Random(17 * num_vars + k)
    t = [rnd.randrange(-(1 << 12), 1 << 12) if rnd.random() < 0.9 else 0 for _ in range(1 << num_vars)]
    r = [rnd.randrange(o.R_MOD) for _ in range(k)]
    got = fix_variables_zkgpt(ctx, num_vars, t, r, 10).evaluations
    assert got == o.fix_variables_zkgpt(num_vars, t, r, 10)
    assert got == o.fix_variables([v % o.R_MOD for v in t], r)


@pytest.mark.parametrize("num_vars,k", [(6, 2), (9, 5), (12, 8)])
def test_fix_variables_zkgpt_wide_integers(ctx, num_vars, k):
    """Magnitudes up to 2^127 (every i128), extremes included: the four-limb path."""
    rnd = random.Random(91 * num_vars + k)
    edge = [-(1 << 127), (1 << 127) - 1, -1, 1, 1 << 32, -(1 << 32), (1 << 64) + 5, 0]
    t = [rnd.choice(edge) if rnd.random() < 0.2 else rnd.randrange(-(1 << 127), 1 << 127) for _ in range(1 << num_vars)]
    r = [rnd.randrange(o.R_MOD) for _ in range(k)]
    assert fix_variables_zkgpt(ctx, num_vars, t, r).evaluations == o.fix_variables([v % o.R_MOD for v in t], r)


def test_fix_variables_zkgpt_einsum_size(ctx):
    """num_vars = 18 (the size from which Einsum::prove takes this path), checked through linearity:
    folding t = a + 3 b equals fold(a) + 3 fold(b), and one column against the direct sum."""
    rnd = random.Random(18)
    num_vars, k = 18, 7
    a = [rnd.randrange(-(1 << 10), 1 << 10) for _ in range(1 << num_vars)]
    b = [rnd.randrange(-(1 << 10), 1 << 10) for _ in range(1 << num_vars)]
    r = [rnd.randrange(o.R_MOD) for _ in range(k)]
    fa = fix_variables_zkgpt(ctx, num_vars, a, r).evaluations
    fb = fix_variables_zkgpt(ctx, num_vars, b, r).evaluations
    fc = fix_variables_zkgpt(ctx, num_vars, [x + 3 * y for x, y in zip(a, b)], r).evaluations
    assert fc == [(x + 3 * y) % o.R_MOD for x, y in zip(fa, fb)]
    eq = o.precompute_eq(r)
    for c in (0, 1, 777, (1 << (num_vars - k)) - 1):
        assert fa[c] == sum(e * a[c * (1 << k) + i] for i, e in enumerate(eq)) % o.R_MOD
