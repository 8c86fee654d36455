"""eq tables and fix_variables_from_right on the GPU against the oracle, with the closed forms of
tests/test_lagrange_basis.rs and tests/test_fix_variables.rs:278-307."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, evaluate_lagrange_basis, fix_variables_from_right

pytestmark = pytest.mark.gpu
M = o.R_MOD


def test_lagrange_basis_closed_forms(ctx):
    assert evaluate_lagrange_basis(ctx, []) == [1]  # test_lagrange_basis.rs:121-127
    r0, r1 = 3, 10
    assert evaluate_lagrange_basis(ctx, [r0]) == [(1 - r0) % M, r0]
    assert evaluate_lagrange_basis(ctx, [r0, r1]) == [(1 - r0) * (1 - r1) % M, r0 * (1 - r1) % M, (1 - r0) * r1 % M, r0 * r1 % M]
    assert evaluate_lagrange_basis(ctx, [1, 0, 1]) == [1 if i == 5 else 0 for i in range(8)]  # vertices :97-118


@pytest.mark.parametrize("k", [1, 4, 9, 10, 11, 14])
def test_lagrange_basis_random(ctx, k):
    rnd = random.Random(k)
    pt = [rnd.randrange(M) for _ in range(k)]
    got = evaluate_lagrange_basis(ctx, pt)
    assert got == o.evaluate_lagrange_basis(pt)
    assert sum(got) % M == 1  # partition of unity :66-73


def test_from_right_closed_form(ctx):
    f = DenseMLPoly.from_evaluations([1, 2, 3, 4])
    assert fix_variables_from_right(ctx, f, [0]).evaluations == [1, 2]
    assert fix_variables_from_right(ctx, f, [1]).evaluations == [3, 4]
    assert fix_variables_from_right(ctx, f, [7]).evaluations == [15, 16]
    assert fix_variables_from_right(ctx, f, []).evaluations == [1, 2, 3, 4]


@pytest.mark.parametrize("n,k", [(1, 1), (4, 2), (6, 6), (10, 3), (12, 6), (13, 12), (14, 2), (15, 8)])
def test_from_right_random(ctx, n, k):
    rnd = random.Random(100 * n + k)
    f = [rnd.randrange(M) for _ in range(1 << n)]
    pt = [rnd.randrange(M) for _ in range(k)]
    got = fix_variables_from_right(ctx, DenseMLPoly.from_evaluations(f), pt).evaluations
    assert got == o.fix_variables_from_right(f, pt)
    # the same polynomial: binding the low variables afterwards gives the full evaluation
    if n <= 12:
        lowpt = [rnd.randrange(M) for _ in range(n - k)]
        assert o.evaluate_multilinear_extension(got, lowpt) == o.evaluate_multilinear_extension(f, lowpt + pt)


@pytest.mark.parametrize("n", [0, 1, 3, 8, 11, 15])
def test_evaluate_at_point(ctx, n):
    """DenseMLPoly::evaluate_at_point (poly.rs:788-791); test_kzh2.rs:149-175 relies on it."""
    rnd = random.Random(900 + n)
    f = [rnd.randrange(M) for _ in range(1 << n)]
    pt = [rnd.randrange(M) for _ in range(n)]
    assert DenseMLPoly.from_evaluations(f).evaluate_at_point(ctx, pt) == o.evaluate_multilinear_extension(f, pt)
    if n == 3:  # a vertex picks one table entry
        assert DenseMLPoly.from_evaluations(f).evaluate_at_point(ctx, [1, 0, 1]) == f[5]
