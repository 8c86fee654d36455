"""The bounded wait of the peer exchange (sharded proves) on one GPU: a rank whose partner never
writes must give up after its poll limit, report ZK_ERR_TIMEOUT and leave the context usable.
The partner is missing by construction (both exchange boxes are one scratch box); nothing faults."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, LinearSumcheckProver, Transcript
from zkes_b200._lib import ZK_ERR_ARG, ZK_ERR_TIMEOUT, lib

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
