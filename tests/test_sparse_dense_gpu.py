"""GPU parity of the sparse x dense product sumcheck against the oracle's dense prover on
[a.to_dense(), b] (the definition of this prover's output)."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, SparseDenseSumcheckProver, Transcript
from zkes_b200._lib import ZkError

pytestmark = pytest.mark.gpu


def run_case(ctx, n, nnz, seed, small_values=True):
    rnd = random.Random(seed)
    idx = sorted(rnd.sample(range(1 << n), nnz))
    if small_values:
        vals = [o.fr_from_int(rnd.randrange(-128, 128)) for _ in idx]  # int8 lifted, zeros allowed
    else:
        vals = [rnd.randrange(o.R_MOD) for _ in idx]
    dense = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    t = Transcript(b"sd_sumcheck")
    prover = SparseDenseSumcheckProver(n, t)
    proof = prover.prove(ctx, idx, vals, DenseMLPoly.from_evaluations(dense), t)
    ot = o.Transcript(b"sd_sumcheck")
    oprover, oproof = o.sparse_dense_prove(n, idx, vals, dense, ot)
    assert proof.round_messages == oproof.round_messages
    assert prover.challenges == oprover.challenges
    assert proof.final_eval == oproof.final_eval
    assert [a[0] for a in prover.a_arrays] == [a[0] for a in oprover.a_arrays]
    assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
    # the restated verifier accepts with the true claimed sum
    claimed = sum(v * dense[i] for i, v in zip(idx, vals)) % o.R_MOD
    vt = o.Transcript(b"sd_sumcheck")
    ver = o.SumcheckVerifier(n, 2, vt)
    res, _ = ver.verify(vt, proof.round_messages, claimed)
    assert res == proof.final_eval


@pytest.mark.parametrize("n,nnz", [(0, 0), (0, 1), (1, 0), (1, 1), (1, 2), (3, 1), (4, 16), (6, 5), (8, 3), (10, 64),
                                   (12, 40), (12, 4096), (13, 700), (14, 1000), (16, 300)])
def test_sparse_dense_matches_dense_prover(ctx, n, nnz):
    run_case(ctx, n, nnz, seed=100 * n + nnz)


def test_full_width_values(ctx):
    run_case(ctx, 11, 200, seed=7, small_values=False)


def test_adjacent_runs(ctx):
    """Entries in consecutive runs exercise the even/odd pairing and the compaction."""
    n = 10
    idx = list(range(5, 40)) + list(range(511, 530)) + [1022, 1023]
    rnd = random.Random(3)
    vals = [rnd.randrange(1, o.R_MOD) for _ in idx]
    dense = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    t = Transcript(b"sd")
    p = SparseDenseSumcheckProver(n, t)
    proof = p.prove(ctx, idx, vals, DenseMLPoly.from_evaluations(dense), t)
    ot = o.Transcript(b"sd")
    _, oproof = o.sparse_dense_prove(n, idx, vals, dense, ot)
    assert proof.round_messages == oproof.round_messages and proof.final_eval == oproof.final_eval


def test_rejects_unsorted_or_out_of_range(ctx):
    dense = DenseMLPoly.from_evaluations([1] * 16)
    for bad in ([3, 2], [1, 1], [5, 16]):
        t = Transcript(b"sd")
        p = SparseDenseSumcheckProver(4, t)
        with pytest.raises(ZkError):
            p.prove(ctx, bad, [1, 1], dense, t)
