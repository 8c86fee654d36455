"""The library's host-side SumcheckVerifier (verifier.rs:7-70 behind zk_sumcheck_verify) against the
oracle's restatement: same accept / reject decisions, running sums and challenges.  No device is used."""
import random

import pyoracle as o
from zkes_b200 import SumcheckVerifier, Transcript


def honest_proof(n, ell, seed, label=b"verify"):
    rnd = random.Random(seed)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(ell)]
    t = o.Transcript(label)
    proof = o.LinearSumcheckProver(n, ell, t).prove(tables, t)
    claimed = 0
    for i in range(1 << n):
        p = 1
        for tb in tables:
            p = p * tb[i] % o.R_MOD
        claimed = (claimed + p) % o.R_MOD
    return tables, proof, claimed


def both(n, ell, msgs, claimed, label=b"verify"):
    t, ot = Transcript(label), o.Transcript(label)
    got = SumcheckVerifier(n, ell, t).verify(t, msgs, claimed)
    want = o.SumcheckVerifier(n, ell, ot).verify(ot, msgs, claimed)
    assert got == (want[0], list(want[1]))
    if want[0] is not None:  # the transcripts moved alike
        assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
    return got


def test_accepts_honest_proofs():
    for n, ell in [(0, 1), (1, 1), (3, 2), (5, 3), (4, 4), (6, 2)]:
        tables, proof, claimed = honest_proof(n, ell, 10 * n + ell)
        res, chal = both(n, ell, proof.round_messages, claimed)
        assert res == proof.final_eval
        assert len(chal) == n
        vals = [o.evaluate_multilinear_extension(tb, chal) for tb in tables]
        prod = 1
        for v in vals:
            prod = prod * v % o.R_MOD
        assert res == prod


def test_rejects_like_the_reference():
    n, ell = 4, 2
    _, proof, claimed = honest_proof(n, ell, 77)
    msgs = [list(m) for m in proof.round_messages]
    assert both(n, ell, msgs, (claimed + 1) % o.R_MOD) == (None, [])        # wrong claimed sum
    assert both(n, ell, msgs[:-1], claimed) == (None, [])                    # a round is missing
    bad = [list(m) for m in msgs]
    bad[2][1] = (bad[2][1] + 5) % o.R_MOD
    assert both(n, ell, bad, claimed) == (None, [])                          # round 2 does not continue round 1
    short = [m[:-1] for m in msgs]
    assert both(n, ell, short, claimed) == (None, [])                        # degree bound
