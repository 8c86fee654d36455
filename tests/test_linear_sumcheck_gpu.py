"""GPU parity of LinearSumcheckProver and the LSB fold against the big-integer oracle.

Mirrors tests/test_linear_sumcheck.rs and tests/test_fix_variables.rs of the reference: small
hand-checkable tables first, then seeded random tables; every proof must be accepted by the
restated SumcheckVerifier and match the oracle prover bit for bit."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, LinearSumcheckProver, Transcript

pytestmark = pytest.mark.gpu


def run_both(ctx, tables, label=b"sumcheck"):
    n = len(tables[0]).bit_length() - 1
    ell = len(tables)
    t = Transcript(label)
    prover = LinearSumcheckProver(n, ell, t)
    proof = prover.prove(ctx, [DenseMLPoly.from_evaluations(p) for p in tables], t)
    ot = o.Transcript(label)
    oprover = o.LinearSumcheckProver(n, ell, ot)
    oproof = oprover.prove(tables, ot)
    assert proof.round_messages == oproof.round_messages
    assert prover.challenges == oprover.challenges
    assert proof.final_eval == oproof.final_eval
    assert [a[0] for a in prover.a_arrays] == [a[0] for a in oprover.a_arrays]
    # transcripts end in the same state
    assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
    return prover, proof


def verify(proof, n, ell, claimed, label=b"sumcheck"):
    vt = o.Transcript(label)
    v = o.SumcheckVerifier(n, ell, vt)
    res, ch = v.verify(vt, proof.round_messages, claimed)
    assert res is not None, "verifier rejected an honest proof"
    assert res == proof.final_eval
    return ch


def eval_prod(tables, i):
    v = 1
    for t in tables:
        v = v * t[i] % o.R_MOD
    return v


def test_constant_polynomials(ctx):  # test_linear_sumcheck.rs:19-62, claimed sum 4
    _, proof = run_both(ctx, [[1, 1, 1, 1], [1, 1, 1, 1]])
    assert len(proof.round_messages) == 2 and all(len(m) == 3 for m in proof.round_messages)
    verify(proof, 2, 2, 4)


def test_identity_polynomials(ctx):  # :65-110, claimed sum 1
    _, proof = run_both(ctx, [[0, 1, 0, 1], [0, 0, 1, 1]])
    verify(proof, 2, 2, 1)


def test_single_variable(ctx):  # :113-134, one table, claimed sum 1
    _, proof = run_both(ctx, [[0, 1]])
    assert len(proof.round_messages) == 1 and len(proof.round_messages[0]) == 2
    verify(proof, 1, 1, 1)


def test_all_zero(ctx):  # :237-275, all-zero tables give all-zero messages
    _, proof = run_both(ctx, [[0] * 8, [0] * 8])
    assert all(v == 0 for m in proof.round_messages for v in m)
    assert proof.final_eval == 0


def test_deterministic(ctx):  # :428-473
    rnd = random.Random(9)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(16)] for _ in range(2)]
    _, p1 = run_both(ctx, tables)
    _, p2 = run_both(ctx, tables)
    assert p1.round_messages == p2.round_messages and p1.final_eval == p2.final_eval


@pytest.mark.parametrize("ell", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [1, 2, 3, 5, 6, 7, 10])
def test_random_tables(ctx, n, ell):
    rnd = random.Random(1000 * ell + n)
    edge = [0, 1, o.R_MOD - 1, o.R_MOD - 2]
    tables = [[rnd.choice(edge) if rnd.random() < 0.1 else rnd.randrange(o.R_MOD) for _ in range(1 << n)]
              for _ in range(ell)]
    prover, proof = run_both(ctx, tables)
    claimed = 0
    for x in range(1 << n):
        g = 1
        for t in tables:
            g = g * t[x] % o.R_MOD
        claimed += g
    ch = verify(proof, n, ell, claimed % o.R_MOD)
    prod = 1
    for t in tables:
        prod = prod * o.evaluate_multilinear_extension(t, ch) % o.R_MOD
    assert prod == proof.final_eval


def test_bench_style_tables(ctx):  # benches/sumcheck_prover.rs:20-34: entry i*2^n + j + 1
    n = 8
    tables = [[i * (1 << n) + j + 1 for j in range(1 << n)] for i in range(2)]
    run_both(ctx, tables, label=b"sumcheck_bench")


def test_medium_size_many_blocks(ctx):
    n = 14  # several tiles per warp and a multi-block grid reduction
    rnd = random.Random(77)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(2)]
    run_both(ctx, tables)


def test_callback_transcript(ctx):
    """The per-round callback form drives an external transcript (here the oracle's)."""
    import ctypes
    from zkes_b200.field import from_mont_array, to_mont_array

    rnd = random.Random(5)
    n = 6
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(2)]
    ext = o.Transcript(b"sumcheck")
    ext.append_u64(b"num_var", n)
    ext.append_u64(b"num_poly", 2)

    def cb(user, msgs, n_msgs, out):
        import numpy as np
        vals = from_mont_array(np.ctypeslib.as_array(msgs, shape=(n_msgs, 4)))
        for v in vals:
            ext.append_scalar(b"round_message", v)
        ch = to_mont_array([ext.challenge_scalar(b"challenge")])[0]
        for k in range(4):
            out[k] = int(ch[k])
        return 0

    dummy = Transcript(b"unused")
    prover = LinearSumcheckProver(n, 2, dummy)
    proof = prover.prove(ctx, [DenseMLPoly.from_evaluations(p) for p in tables], dummy, fs_callback=cb)
    ot = o.Transcript(b"sumcheck")
    op = o.LinearSumcheckProver(n, 2, ot)
    oproof = op.prove(tables, ot)
    assert proof.round_messages == oproof.round_messages and proof.final_eval == oproof.final_eval


def test_shape_errors(ctx):  # linear_prover.rs:44-52 panics become ZK_ERR_ARG / assertions
    t = Transcript(b"sumcheck")
    prover = LinearSumcheckProver(3, 2, t)
    with pytest.raises(AssertionError):
        prover.prove(ctx, [DenseMLPoly.from_evaluations([1, 2, 3, 4])] * 2, t)
    with pytest.raises(AssertionError):
        prover.prove(ctx, [], t)


# ---- fold: tests/test_fix_variables.rs dense cases
def test_fix_variables_known_answers(ctx):
    f = DenseMLPoly.from_evaluations([1, 2, 3, 4])
    assert f.fix_variables(ctx, [0]).evaluations == [1, 3]  # :19-48
    assert f.fix_variables(ctx, [1]).evaluations == [2, 4]
    assert f.fix_variables(ctx, []).evaluations == [1, 2, 3, 4]
    g = DenseMLPoly.from_evaluations(list(range(1, 9)))  # 3 variables, :89-122
    assert g.fix_variables(ctx, [1, 0]).evaluations == [2, 6]
    assert g.fix_variables(ctx, [0, 1, 1]).evaluations == [7]


@pytest.mark.parametrize("n,k", [(1, 1), (5, 2), (6, 6), (9, 3), (13, 13), (15, 4)])
def test_fix_variables_random(ctx, n, k):
    rnd = random.Random(31 * n + k)
    f = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    pt = [rnd.randrange(o.R_MOD) for _ in range(k)]
    assert DenseMLPoly.from_evaluations(f).fix_variables(ctx, pt).evaluations == o.fix_variables(f, pt)


@pytest.mark.parametrize("ell", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [0, 1, 4, 9, 10, 11, 13])
def test_device_tail_option(ctx, n, ell):
    """ZK_OPT_DEVICE_TAIL (on by default) keeps the rounds on the device with the transcript in a warp; switched
    off, every round goes through the per-round kernels with the transcript on the host.  Every output and the
    transcript state must be the same."""
    from zkes_b200._lib import ZK_OPT_DEVICE_TAIL
    rnd = random.Random(5000 + 10 * n + ell)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(ell)]
    run_both(ctx, tables)  # default: device-resident rounds
    ctx.set_option(ZK_OPT_DEVICE_TAIL, 0)
    try:
        run_both(ctx, tables)
    finally:
        ctx.set_option(ZK_OPT_DEVICE_TAIL, 1)


@pytest.mark.parametrize("n,ell", [(12, 1), (14, 3), (15, 2), (16, 2), (12, 4)])
def test_resident_rounds(ctx, n, ell):
    """Tables above 1024 entries: the cooperative multi-block kernel runs all rounds with the transcript on the
    device, the later ones prepared ahead of their challenges."""
    rnd = random.Random(9100 + 10 * n + ell)
    edge = [0, 1, o.R_MOD - 1]
    tables = [[rnd.choice(edge) if rnd.random() < 0.05 else rnd.randrange(o.R_MOD) for _ in range(1 << n)]
              for _ in range(ell)]
    _, proof = run_both(ctx, tables, label=b"resident-%d" % n)
    claimed = sum(eval_prod(tables, i) for i in range(1 << n)) % o.R_MOD if n <= 12 else None
    if claimed is not None:
        verify(proof, n, ell, claimed, label=b"resident-%d" % n)


@pytest.mark.parametrize("ell", [1, 2, 3, 4])
@pytest.mark.parametrize("label_len", list(range(1, 40, 3)) + [150, 165, 166, 167, 200])
def test_device_transcript_block_boundaries(ctx, label_len, ell):
    """The device transcript meets the sponge's 166-byte block boundary at a position set by what was absorbed
    before the prover ran: sweep that position so framing bytes, labels and data each straddle a boundary."""
    rnd = random.Random(7000 + 10 * label_len + ell)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << 4)] for _ in range(ell)]
    run_both(ctx, tables, label=bytes(rnd.randrange(256) for _ in range(label_len)))


@pytest.mark.parametrize("ell", [1, 2, 3])
@pytest.mark.parametrize("n", [2, 3, 4, 6, 9, 12, 14])
def test_run_ahead_thresholds(ctx, n, ell):
    """ZK_OPT_AHEAD_LOG moves the round from which the multi-round kernel prepares messages ahead of their
    challenges (0: never, and the single-block kernel finishes; 2: only the very last rounds; large: from the
    second round on).  Messages, challenges, final values and the transcript state must not depend on it."""
    from zkes_b200._lib import ZK_OPT_AHEAD_LOG
    rnd = random.Random(7300 + 10 * n + ell)
    edge = [0, 1, o.R_MOD - 1]
    tables = [[rnd.choice(edge) if rnd.random() < 0.1 else rnd.randrange(o.R_MOD) for _ in range(1 << n)]
              for _ in range(ell)]
    try:
        for log in (0, 2, 5, 10, 24):
            ctx.set_option(ZK_OPT_AHEAD_LOG, log)
            run_both(ctx, tables, label=b"ahead-%d" % log)
    finally:
        ctx.set_option(ZK_OPT_AHEAD_LOG, 15)


def test_run_ahead_large_tables(ctx):
    """Two tables of 2^16 entries with the run-ahead threshold above the table size: every round but the first is
    prepared ahead, with many units per warp and every worker block busy."""
    from zkes_b200._lib import ZK_OPT_AHEAD_LOG
    n = 16
    rnd = random.Random(99)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(2)]
    try:
        ctx.set_option(ZK_OPT_AHEAD_LOG, 20)
        run_both(ctx, tables, label=b"ahead-large")
    finally:
        ctx.set_option(ZK_OPT_AHEAD_LOG, 15)


def test_run_ahead_option_range(ctx):
    from zkes_b200._lib import ZK_OPT_AHEAD_LOG
    for bad in (-1, 25):
        with pytest.raises(Exception):
            ctx.set_option(ZK_OPT_AHEAD_LOG, bad)
    ctx.set_option(ZK_OPT_AHEAD_LOG, 15)
