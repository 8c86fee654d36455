"""The bounded wait of the peer exchange (sharded proves) on one GPU: a rank whose partner never
writes must give up after its poll limit, report ZK_ERR_TIMEOUT and leave the context usable.
The partner is missing by construction (both exchange boxes are one scratch box); nothing faults."""
import ctypes
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, LinearSumcheckProver, Transcript
from zkes_b200._lib import ZK_ERR_ARG, ZK_ERR_COMM, ZK_ERR_TIMEOUT, ZK_MEM_HOST, ZkError, lib

pytestmark = pytest.mark.gpu


def test_wait_for_a_missing_rank_runs_out(ctx):
    assert lib.zk_comm_wait_selftest(ctx.handle, 20000) == ZK_ERR_TIMEOUT
    assert b"ran out" in lib.zk_last_error()
    assert lib.zk_comm_wait_selftest(ctx.handle, 0) == ZK_ERR_ARG
    # the context still proves, and a second time-out does not disturb it either
    for _ in range(2):
        rnd = random.Random(11)
        n = 6
        f = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
        g = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
        t = Transcript(b"after_timeout")
        proof = LinearSumcheckProver(n, 2, t).prove(ctx, [DenseMLPoly.from_evaluations(f), DenseMLPoly.from_evaluations(g)], t)
        ot = o.Transcript(b"after_timeout")
        oproof = o.LinearSumcheckProver(n, 2, ot).prove([f, g], ot)
        assert proof.round_messages == oproof.round_messages and proof.final_eval == oproof.final_eval
        assert lib.zk_comm_wait_selftest(ctx.handle, 5000) == ZK_ERR_TIMEOUT


def test_failed_sharded_call_retires_the_communicator(ctx):
    """A sharded call that fails leaves the ranks' exchange counters in doubt, so the communicator refuses
    every later sharded call with ZK_ERR_COMM until it is freed and made anew (one rank is enough to see
    the rule; the two-GPU form is in test_sharded_gpu.py)."""
    from zkes_b200 import dist as zd
    rnd = random.Random(12)
    n = 7
    f = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    g = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    ot = o.Transcript(b"retire")
    want = o.LinearSumcheckProver(n, 2, ot).prove([f, g], ot)

    def prove(comm):
        t = Transcript(b"retire")
        t.append_u64(b"num_var", n)
        t.append_u64(b"num_poly", 2)
        return zd.sharded_linear_prove(ctx, comm, n, [DenseMLPoly.from_evaluations(f), DenseMLPoly.from_evaluations(g)], t)

    comm = zd.Comm(ctx, rank=0, world=1)
    msgs, _, _, fin = prove(comm)
    assert msgs == want.round_messages and fin == want.final_eval
    rc = lib.zk_sumcheck_linear_prove_sharded(ctx.handle, comm.handle, n, 0, None, ZK_MEM_HOST, None, None, None, None, None,
                                              None, None)
    assert rc == ZK_ERR_ARG
    with pytest.raises(ZkError) as e:
        prove(comm)
    assert e.value.code == ZK_ERR_COMM and "zk_comm_init again" in str(e.value)
    out = (ctypes.c_uint64 * 12)()
    assert lib.zk_msm_g1_sharded(ctx.handle, comm.handle, None, ZK_MEM_HOST, None, ZK_MEM_HOST, 0, out) == ZK_ERR_COMM
    comm.close()
    comm = zd.Comm(ctx, rank=0, world=1)
    msgs, _, _, fin = prove(comm)
    assert msgs == want.round_messages and fin == want.final_eval
    comm.close()
