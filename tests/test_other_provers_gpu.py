"""SparseBoolSumcheckProver and GeneralLinearSumcheckProver on the GPU against the oracle
(src/crypto/sumcheck/linear_prover.rs:193-656), including the committed golden vectors."""
import json
import os
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, GeneralLinearSumcheckProver, SparseBoolSumcheckProver, Transcript
from zkes_b200._lib import ZkError

pytestmark = pytest.mark.gpu
M = o.R_MOD
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "sumcheck.json")))


def ints(xs):
    return [int(x, 16) for x in xs]


def test_sparse_bool_golden(ctx):
    for case in GOLD["sparse_bool"]:
        t = Transcript(b"range")
        p = SparseBoolSumcheckProver(case["n"], t)
        pr = p.prove(ctx, ints(case["weights"]), case["positions"], ints(case["eq_point"]), t)
        assert pr.round_messages == [ints(m) for m in case["round_messages"]]
        assert pr.final_eval == int(case["final_eval"], 16)
        assert t.challenge_scalar(b"after") == int(case["tail"], 16)


@pytest.mark.parametrize("n,terms,k", [(0, 1, 1), (1, 1, 1), (1, 2, 2), (3, 1, 8), (6, 3, 10), (9, 5, 100), (12, 4, 2000),
                                       (13, 5, 512), (10, 0, 0), (8, 2, 0),
                                       (14, 64, 8192), (15, 40, 3000)])  # pairs by the hundred per warp; and mostly lone entries
def test_sparse_bool_random(ctx, n, terms, k):
    rnd = random.Random(n * 31 + terms * 7 + k)
    w = [rnd.randrange(M) for _ in range(terms)]
    pos = [rnd.sample(range(1 << n), min(k, 1 << n)) for _ in range(terms)]  # unsorted, as hash-map keys arrive
    pt = [rnd.randrange(M) for _ in range(n)]
    t = Transcript(b"range")
    p = SparseBoolSumcheckProver(n, t)
    pr = p.prove(ctx, w, pos, pt, t)
    ot = o.Transcript(b"range")
    op = o.SparseBoolSumcheckProver(n, ot)
    opr = op.prove(w, pos, pt, ot)
    assert pr.round_messages == opr.round_messages and p.challenges == op.challenges
    assert pr.final_eval == opr.final_eval
    assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
    # selection tables are 0/1, so the claimed sum is 0 (dag/mod.rs:1343-1351) and the verifier accepts
    vt = o.Transcript(b"range")
    res, _ = o.SumcheckVerifier(n, 3, vt).verify(vt, pr.round_messages, 0)
    assert res == pr.final_eval


def test_sparse_bool_lookup_scale_verifies(ctx):
    """At the size of one of the trace's boolean checks (48 selection terms of 2^17 ones over 2^21 positions, 6.3
    million entries: every warp's span is thousands of entries long and crosses terms, the pair queue fills many
    times) the oracle's prover would take minutes; instead the proof must pass the verifier with claimed sum 0
    (dag/mod.rs:1343-1351) and its final value must be eq(point, r) sum_j w_j s_j(r) (s_j(r) - 1) with the s_j(r)
    summed independently from the eq table of the challenges."""
    import numpy as np
    n_low, digit_log, terms = 17, 4, 48
    n = n_low + digit_log
    rnd = random.Random(2024)
    rng = np.random.default_rng(11)
    w = [rnd.randrange(M) for _ in range(terms)]
    pt = [rnd.randrange(M) for _ in range(n)]
    base = np.arange(1 << n_low, dtype=np.uint64)
    pos = [((rng.integers(0, 1 << digit_log, size=1 << n_low, dtype=np.uint64) << np.uint64(n_low)) | base).tolist()
           for _ in range(terms)]
    t = Transcript(b"range")
    p = SparseBoolSumcheckProver(n, t)
    pr = p.prove(ctx, w, pos, pt, t)
    vt = o.Transcript(b"range")
    res, chals = o.SumcheckVerifier(n, 3, vt).verify(vt, pr.round_messages, 0)
    assert res is not None and res == pr.final_eval and chals == p.challenges
    eq_r = o.evaluate_lagrange_basis(chals)
    inner = 0
    for wj, pj in zip(w, pos):
        v = sum(eq_r[x] for x in pj) % M
        inner += wj * v * (v - 1)
    eq_val = 1
    for a, b in zip(pt, chals):
        eq_val = eq_val * ((a * b + (1 - a) * (1 - b)) % M) % M
    assert pr.final_eval == eq_val * inner % M


def test_sparse_bool_rejects_duplicates(ctx):
    t = Transcript(b"range")
    p = SparseBoolSumcheckProver(3, t)
    with pytest.raises(ZkError):
        p.prove(ctx, [1], [[2, 2]], [1, 2, 3], t)
    with pytest.raises(ZkError):
        p.prove(ctx, [1], [[8]], [1, 2, 3], t)


@pytest.mark.parametrize("n,num_poly,terms", [(0, 2, 1), (1, 2, 1), (3, 3, 2), (5, 2, 3), (6, 4, 2), (9, 3, 4), (11, 5, 2)])
def test_general_linear(ctx, n, num_poly, terms):
    rnd = random.Random(n * 100 + num_poly * 10 + terms)
    scalars = [rnd.randrange(M) for _ in range(terms)]
    arrays = [[[rnd.randrange(M) for _ in range(1 << n)] for _ in range(num_poly - 1)] for _ in range(terms)]
    eq = o.evaluate_lagrange_basis([rnd.randrange(M) for _ in range(n)])
    t = Transcript(b"general")
    p = GeneralLinearSumcheckProver(n, num_poly, t)
    pr = p.prove(ctx, (scalars, [[DenseMLPoly.from_evaluations(x) for x in term] for term in arrays],
                       DenseMLPoly.from_evaluations(eq)), t)
    ot = o.Transcript(b"general")
    op = o.GeneralLinearSumcheckProver(n, num_poly, ot)
    opr = op.prove((scalars, arrays, eq), ot)
    assert pr.round_messages == opr.round_messages and p.challenges == op.challenges
    assert pr.final_eval == opr.final_eval
    assert [[v[0] for v in term] for term in p.a_arrays] == [[tb[0] for tb in term] for term in op.final_tables]
    claimed = 0
    for x in range(1 << n):
        inner = 0
        for a, term in zip(scalars, arrays):
            g = a
            for tb in term:
                g = g * tb[x] % M
            inner += g
        claimed += eq[x] * inner
    vt = o.Transcript(b"general")
    res, _ = o.SumcheckVerifier(n, num_poly, vt).verify(vt, pr.round_messages, claimed % M)
    assert res == pr.final_eval
