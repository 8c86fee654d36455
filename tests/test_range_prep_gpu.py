"""GPU parity of the range-proof preprocessing of Dag::prove_range (src/dag/mod.rs:1314-1340): the
scatter-add of Lagrange weights into the table, the middle claim, the beta*gamma-weighted sum of the
auxiliary polynomials, and the table polynomial range_dense(n) + alpha."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, range_aux_accumulate, range_table
from zkes_b200._lib import ZkError

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k,table_log,n_sel", [(0, 0, 1), (1, 1, 2), (3, 2, 8), (6, 4, 64), (10, 8, 1024), (12, 8, 3000),
                                               (9, 11, 512), (8, 3, 0)])
def test_aux_accumulate_matches_oracle(ctx, k, table_log, n_sel):
    rnd = random.Random(1000 * k + table_log)
    acc = DenseMLPoly.from_evaluations([0] * (1 << table_log))
    want_acc = [0] * (1 << table_log)
    for call in range(3):  # three auxiliary polynomials into one running sum
        point = [rnd.randrange(o.R_MOD) for _ in range(k)]
        # every input index selects one table entry (a lookup), in no particular order
        inputs = list(range(1 << k))
        rnd.shuffle(inputs)
        selection = [(inputs[e % (1 << k)], rnd.randrange(1 << table_log)) for e in range(n_sel)]
        beta_gamma = rnd.randrange(o.R_MOD)
        got_mid = range_aux_accumulate(ctx, point, selection, beta_gamma, table_log, acc)
        want_mid, want_acc = o.range_aux_accumulate(point, selection, beta_gamma, table_log, want_acc)
        assert got_mid == want_mid
        assert acc.evaluations == want_acc


def test_aux_accumulate_one_hot_table(ctx):
    """All pairs on one table entry: the limb counters of that entry take every addend."""
    rnd = random.Random(5)
    k, table_log = 11, 4
    point = [rnd.randrange(o.R_MOD) for _ in range(k)]
    selection = [(i, 9) for i in range(1 << k)]
    acc = DenseMLPoly.from_evaluations([7] * (1 << table_log))
    mid = range_aux_accumulate(ctx, point, selection, 3, table_log, acc)
    # the Lagrange weights sum to one
    assert mid == 9
    assert acc.evaluations == [7 + (3 if t == 9 else 0) for t in range(1 << table_log)]


def test_aux_accumulate_rejects_bad_index(ctx):
    acc = DenseMLPoly.from_evaluations([0] * 4)
    with pytest.raises(ZkError):
        range_aux_accumulate(ctx, [5, 6], [(4, 0)], 1, 2, acc)
    with pytest.raises(ZkError):
        range_aux_accumulate(ctx, [5, 6], [(0, 4)], 1, 2, acc)


@pytest.mark.parametrize("n", [0, 1, 4, 8, 13])
def test_range_table(ctx, n):
    alpha = random.Random(n).randrange(o.R_MOD)
    assert range_table(ctx, n, alpha).evaluations == o.range_table(n, alpha)
