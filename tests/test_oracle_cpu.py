"""CPU checks of the oracle itself: known answers the reference's tests make derivable by hand,
Keccak against hashlib, the committed golden vectors, and agreement of the two restatements."""
import hashlib
import json
import os
import random

import pytest

import coracle as c
import pyoracle as o

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "sumcheck.json")))


def ints(xs):
    return [int(x, 16) for x in xs]


def test_keccak_against_hashlib():
    for msg in (b"", b"abc", b"q" * 135, b"q" * 136, b"z" * 777):
        assert o.sponge(msg, 136, 0x06, 32) == hashlib.sha3_256(msg).digest()
        assert o.sponge(msg, 168, 0x1F, 300) == hashlib.shake_128(msg).digest(300)


def test_merlin_known_answer():
    t = o.Transcript(b"test protocol")
    t.append_message(b"some label", b"some data")
    got = t.challenge_bytes(b"challenge", 32).hex()
    assert got == GOLD["merlin"]["simple"]
    # The vector the merlin crate pins for this exchange in its own unit test `equivalence_simple`
    # (merlin 3.0.0, src/transcript.rs: protocol label "test protocol", append_message("some label",
    # "some data"), 32 challenge bytes under "challenge").
    assert got == "d5a21972d0d5fe320c0d263fac7fffb8145aa640af6e9bca177c03c7efcf0615"


def test_fix_variables_hand_cases():  # tests/test_fix_variables.rs:19-140
    assert o.fix_variables([1, 2, 3, 4], [0]) == [1, 3]
    assert o.fix_variables([1, 2, 3, 4], [1]) == [2, 4]
    assert c.fix_variables([1, 2, 3, 4], [0]) == [1, 3]
    r = 5  # f(x0, x1) = 1 + x0 + 2 x1 on [1,2,3,4]: binding x0 = 5 gives [6, 8]
    assert o.fix_variables([1, 2, 3, 4], [r]) == [6, 8]
    g = list(range(1, 9))
    assert o.fix_variables(g, [1, 0]) == [2, 6]
    assert c.fix_variables(g, [0, 1, 1]) == [7]
    # fix_variables_from_right against the closed form (:278-307): binding x1 of [1,2,3,4]
    assert o.fix_variables_from_right([1, 2, 3, 4], [0]) == [1, 2]
    assert o.fix_variables_from_right([1, 2, 3, 4], [1]) == [3, 4]
    assert c.fix_from_right([1, 2, 3, 4], [7]) == [(1 + 7 * 2) % o.R_MOD, (2 + 7 * 2) % o.R_MOD]


def test_lagrange_basis_hand_cases():  # tests/test_lagrange_basis.rs:16-127
    assert o.evaluate_lagrange_basis([]) == [1]
    r0, r1 = 3, 10
    m = o.R_MOD
    assert o.evaluate_lagrange_basis([r0]) == [(1 - r0) % m, r0]
    assert o.evaluate_lagrange_basis([r0, r1]) == [(1 - r0) * (1 - r1) % m, r0 * (1 - r1) % m, (1 - r0) * r1 % m, r0 * r1 % m]
    rnd = random.Random(1)
    pt = [rnd.randrange(m) for _ in range(5)]
    assert sum(o.evaluate_lagrange_basis(pt)) % m == 1  # partition of unity
    assert o.evaluate_lagrange_basis([1, 0, 1]) == [1 if i == 5 else 0 for i in range(8)]  # vertices
    assert c.eq_table(pt) == o.evaluate_lagrange_basis(pt)


def test_claimed_sums_verify():  # tests/test_linear_sumcheck.rs: sums 4, 1, 1
    for tables, claimed in (([[1, 1, 1, 1], [1, 1, 1, 1]], 4), ([[0, 1, 0, 1], [0, 0, 1, 1]], 1), ([[0, 1]], 1)):
        n = len(tables[0]).bit_length() - 1
        t = o.Transcript(b"sumcheck")
        p = o.LinearSumcheckProver(n, len(tables), t)
        pr = p.prove(tables, t)
        vt = o.Transcript(b"sumcheck")
        res, ch = o.SumcheckVerifier(n, len(tables), vt).verify(vt, pr.round_messages, claimed)
        assert res == pr.final_eval and ch == p.challenges
        vt = o.Transcript(b"sumcheck")
        bad, _ = o.SumcheckVerifier(n, len(tables), vt).verify(vt, pr.round_messages, claimed + 1)
        assert bad is None


def test_golden_linear_both_oracles():
    for case in GOLD["linear"]:
        tables = [ints(t) for t in case["tables"]]
        label = case["label"].encode()
        n = len(tables[0]).bit_length() - 1
        t = o.Transcript(label)
        p = o.LinearSumcheckProver(n, len(tables), t)
        pr = p.prove(tables, t)
        want = [ints(m) for m in case["round_messages"]]
        assert pr.round_messages == want and pr.final_eval == int(case["final_eval"], 16)
        cp = c.linear_prove(label, tables)
        assert cp.round_messages == want and cp.challenges == ints(case["challenges"])
        assert cp.final_eval == int(case["final_eval"], 16) and cp.tail == int(case["tail"], 16)


def test_golden_sparse_dense_and_bool():
    import numpy as np
    for case in GOLD["sparse_dense"]:
        cp = c.sparse_dense_prove_mont(b"sd_sumcheck", case["n"], np.array(case["idx"], dtype=np.uint64),
                                       c.mont(ints(case["vals"])), c.mont(ints(case["dense"])))
        assert cp.round_messages == [ints(m) for m in case["round_messages"]]
        assert cp.final_eval == int(case["final_eval"], 16) and cp.tail == int(case["tail"], 16)
    for case in GOLD["sparse_bool"]:
        cp = c.sparse_bool_prove(b"range", case["n"], ints(case["weights"]), case["positions"], ints(case["eq_point"]))
        assert cp.round_messages == [ints(m) for m in case["round_messages"]]
        assert cp.final_eval == int(case["final_eval"], 16) and cp.tail == int(case["tail"], 16)
        vt = o.Transcript(b"range")  # the range-proof claim is 0 (dag/mod.rs:1343-1351)
        res, _ = o.SumcheckVerifier(case["n"], 3, vt).verify(vt, [ints(m) for m in case["round_messages"]], 0)
        assert res == int(case["final_eval"], 16)


def test_golden_poly_helpers():
    g = GOLD["poly"]
    f, pt = ints(g["f"]), ints(g["point"])
    assert c.eq_table(pt[:4]) == ints(g["eq"]) == o.evaluate_lagrange_basis(pt[:4])
    assert c.fix_variables(f, pt[:3]) == ints(g["fix_lsb_3"])
    assert c.fix_from_right(f, pt[:2]) == ints(g["fix_right_2"])
    assert c.mle_eval(f, pt) == int(g["mle"], 16)
    assert o.gen_uniform_fr(7, 3, 5, 4) == ints(g["uniform_seed7"])
    assert o.gen_small_fr(7, 3, 5, 8, 8) == ints(g["small_seed7_bits8"])


def test_chacha_against_cryptography():
    """The input generator's keystream is RFC 8439 ChaCha20 (checked against `cryptography`)."""
    import struct
    from cryptography.hazmat.primitives.ciphers import Cipher, algorithms
    key = struct.pack("<QQ16x", 9, 4)
    for counter in (0, 1, 77):
        nonce = struct.pack("<I12x", counter)  # library layout: 32-bit counter then 96-bit nonce
        ks = Cipher(algorithms.ChaCha20(key, nonce), mode=None).encryptor().update(b"\x00" * 64)
        assert ks == o.gen_bytes(9, 4, counter, 1)


def test_multithreaded_oracle_matches_single():
    rnd = random.Random(8)
    tables = [[rnd.randrange(o.R_MOD) for _ in range(1 << 13)] for _ in range(2)]
    c.set_threads(1)
    a = c.linear_prove(b"x", tables)
    c.set_threads(4)
    b = c.linear_prove(b"x", tables)
    c.set_threads(1)
    assert a.round_messages == b.round_messages and a.final_eval == b.final_eval


def test_permute_evals_by_ranges_hand_cases():
    """src/basicblock/einsum.rs:142-198: identity, swapped halves, and the inverse of a permutation."""
    evals = list(range(16))
    assert o.permute_evals_by_ranges(evals, 4, [(0, 4)]) == evals
    out = o.permute_evals_by_ranges(evals, 4, [(2, 4), (0, 2)])
    assert out == [((i & 3) << 2) | (i >> 2) for i in range(16)]
    assert o.permute_evals_by_ranges(out, 4, [(2, 4), (0, 2)]) == evals
    with pytest.raises(AssertionError):
        o.permute_evals_by_ranges(evals, 4, [(0, 3)])
    with pytest.raises(AssertionError):
        o.permute_evals_by_ranges(evals, 4, [(0, 3), (2, 4)])


@pytest.mark.parametrize("num_vars,k,q_bits", [(4, 0, 3), (5, 2, 2), (7, 3, 4), (8, 5, 12), (9, 9, 3)])
def test_fix_variables_zkgpt_is_the_lsb_fold_of_the_lifted_integers(num_vars, k, q_bits):
    """The table-of-multiples algorithm of src/util/poly.rs:1378-1473 (both its lookup and its quotient branch)
    computes sum_b eq(r)[b] t[c n + b], i.e. DenseMLPoly::fix_variables on the integers lifted to the field."""
    rnd = random.Random(num_vars * 100 + k)
    t = [rnd.randrange(-(1 << 9), 1 << 9) for _ in range(1 << num_vars)]
    r = [rnd.randrange(o.R_MOD) for _ in range(k)]
    assert o.fix_variables_zkgpt(num_vars, t, r, q_bits) == o.fix_variables([v % o.R_MOD for v in t], r)


def test_g1_compressed_encoding_round_trip():
    """The flag convention of the compressed form: generator (1, 2) has the smaller y, its negative the larger."""
    g = (1, 2)
    assert o.g1_serialize_compressed(g) == bytes([1]) + bytes(31)
    assert o.g1_serialize_compressed((1, o.Q_MOD - 2)) == bytes([1]) + bytes(30) + bytes([0x80])
    assert o.g1_serialize_compressed(None) == bytes(31) + bytes([0x40])
    rnd = random.Random(3)
    for _ in range(20):
        p = o.g1_mul(g, rnd.randrange(1, o.R_MOD))
        assert o.g1_deserialize_compressed(o.g1_serialize_compressed(p)) == p
    assert o.g1_deserialize_compressed(o.g1_serialize_compressed(None)) is None


def test_cpp_g1_against_bigint_oracle():
    """oracle/g1.h (Jacobian formulas, bucket-method MSM on threads) against the big-integer restatement."""
    rnd = random.Random(5)
    pts = [o.g1_mul(o.G1_GEN, rnd.randrange(1, o.R_MOD)) for _ in range(70)]
    pts[7] = None
    sc = [rnd.randrange(o.R_MOD) if i % 3 else o.fr_from_int(rnd.randrange(-128, 128)) for i in range(70)]
    sc[11] = 0
    assert c.g1_mul(o.G1_GEN, 12345) == o.g1_mul(o.G1_GEN, 12345)
    for n in (0, 1, 2, 31, 32, 70):
        assert c.g1_msm(pts[:n], sc[:n]) == o.g1_msm(pts[:n], sc[:n]), n
    c.set_threads(4)
    big = [pts[i % 70] for i in range(4500)]  # above the threshold at which the points are split over threads
    bs = [rnd.randrange(o.R_MOD) for _ in range(4500)]
    folded = [sum(bs[i] for i in range(j, 4500, 70)) % o.R_MOD for j in range(70)]
    assert c.g1_msm(big, bs) == o.g1_msm(pts, folded)
    rows = c.g1_msm_rows_mont(c.affine_array(pts[:16]), c.mont(sc[:64]), 4)
    assert rows == [o.g1_msm(pts[:16], sc[16 * r:16 * r + 16]) for r in range(4)]
    p = pts[0]
    assert c.g1_msm([p, p], [1, 1]) == o.g1_mul(p, 2)  # the doubling branch of the mixed addition
    assert c.g1_msm([p, o.g1_neg(p)], [5, 5]) is None
    c.set_threads(1)


def test_boolean_check_entrywise_identity():
    """The algebra the CUDA message kernel of the boolean-check prover relies on (zkes_b200/csrc/general.cu), checked
    in big integers against the pairwise form of linear_prover.rs:529-591: a pair (v0, v1) contributes, at c = 0..3,
    aux (aux - 1) eq with aux = v0 + c (v1 - v0); taken entry by entry that is, per entry of value v on side b with
    q = v^2 and the per-position record {eq(b), eq(2) * (1 + b), eq(3) * (2 + b)}:
      T(b) += (q - v) rec0;  T(2) += (b ? 2q - v : q + v) rec1;  T(3) += (b ? 3q - v : 2q + v) rec2,
    plus, where both sides are present, T(2) -= 4 v0 v1 eq(2) and T(3) -= 6 v0 v1 (2 eq(3)).  With every value one
    (the first round) a lone entry gives 2 eq(2), 6 eq(3) and a pair nothing."""
    M = o.R_MOD
    rnd = random.Random(5)
    for case in range(200):
        v0 = rnd.randrange(M) if case % 3 != 1 else 0
        v1 = rnd.randrange(M) if case % 3 != 2 else 0
        if case >= 150:  # first-round shape: present entries are one
            v0, v1 = (1 if v0 else 0), (1 if v1 else 0)
        e0, e1 = rnd.randrange(M), rnd.randrange(M)
        e = [e0, e1, (2 * e1 - e0) % M, (3 * e1 - 2 * e0) % M]
        pair = []
        for cc in range(4):
            aux = (v0 + cc * (v1 - v0)) % M
            pair.append(aux * (aux - 1) * e[cc] % M)
        t = [0, 0, 0, 0]
        for b, v in ((0, v0), (1, v1)):
            if v == 0:
                continue
            q = v * v % M
            rec = [e[b], e[2] * (1 + b) % M, e[3] * (2 + b) % M]
            t[b] += (q - v) * rec[0]
            t[2] += ((2 * q - v) if b else (q + v)) * rec[1]
            t[3] += ((3 * q - v) if b else (2 * q + v)) * rec[2]
        if v0 and v1:
            t[2] -= 4 * v0 * v1 * e[2]
            t[3] -= 6 * v0 * v1 * (2 * e[3])
        assert [x % M for x in t] == pair
        if case >= 150:
            lone = (v0 == 1) != (v1 == 1)
            assert pair == ([0, 0, 2 * e[2] % M, 6 * e[3] % M] if lone else [0, 0, 0, 0])
