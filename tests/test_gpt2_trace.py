"""The GPT-2-small trace replay: its call list has the reference DAG's shapes (CPU), and a reduced model runs
every kind of call through the C ABI on the GPU."""
from collections import Counter

import pytest

from zkes_b200 import gpt2_trace


def test_call_list_shapes():
    prove, dense, lookups = gpt2_trace.model_calls()  # sequence length 128
    # per layer: four 2^20 and two 2^22 weight matrices, the 2^19 GELU constant (src/dag/gpt2.rs, src/bin/gpt2.rs:102-125)
    c = Counter(dense)
    assert c[20] == 48 and c[22] == 24 and c[19] == 12 and c[17] == 1 and c[14] == 1
    sumchecks = [x for x in prove if x[0] == "sumcheck"]
    # the six weight einsums of a layer bsi,ij->bsj: three tables (x, w, eq), 10 or 12 summed variables (einsum.rs:541-553)
    assert sum(1 for x in sumchecks if x[1:] == (3, 10)) >= 12 * 5 and sum(1 for x in sumchecks if x[1:] == (3, 12)) == 12
    # the two element-wise products of the GELU run over all 19 variables of the MLP activation
    assert sum(1 for x in sumchecks if x[1:] == (3, 19)) == 24
    # integer-table folds only from 2^18 entries on (einsum.rs:504-519)
    assert all(x[1] >= 18 for x in prove if x[0] == "intfold") and all(x[1] < 18 for x in prove if x[0] == "fold")
    # lookups over activations of 2^17, 2^18 and 2^19 elements; terms of the boolean sumchecks fit the 32-bit key space
    assert set(lookups) == {17, 18, 19}
    for n, nodes in Counter(lookups).items():
        assert (nodes * gpt2_trace.TABLE_BLOCKS) << (n + gpt2_trace.TABLE_BLOCK_LOG) <= 1 << 32


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [2, 3])
def test_reduced_trace_runs(ctx, dims):
    rep = gpt2_trace.run(ctx, seq_len=8, layers=1, dims=dims)
    assert rep["value"] > 0 and rep["commit_s"] > 0
    assert rep["calls"]["sparse_bool_proves"] == 3 and rep["calls"]["dense_commits"] == 20
