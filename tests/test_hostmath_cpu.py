"""The device field arithmetic (zkes_b200/csrc/ff.cuh) compiled for the host, where its carry
chains take their portable C form, against Python integers."""
import ctypes
import os
import random
import subprocess

import pytest

import pyoracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
R = 1 << 256


@pytest.fixture(scope="module")
def hm():
    so = os.path.join(HERE, "hostmath", "libffhost.so")
    src = os.path.join(HERE, "hostmath", "ff_host.cpp")
    subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-x", "c++", src, "-o", so], check=True)
    return ctypes.CDLL(so)


def buf(x, n=8):
    return (ctypes.c_uint32 * n)(*[(x >> (32 * i)) & 0xFFFFFFFF for i in range(n)])


def val(b):
    return sum(int(v) << (32 * i) for i, v in enumerate(b))


@pytest.mark.parametrize("name,p", [("fr", o.R_MOD), ("fq", o.Q_MOD)])
def test_field_ops(hm, name, p):
    rnd = random.Random(5)
    edge = [0, 1, 2, p - 1, p - 2, R % p, (p - 1) // 2, 0xFFFFFFFF, (1 << 224) - 1]
    rv = lambda: rnd.choice(edge) if rnd.random() < 0.2 else rnd.randrange(p)  # noqa: E731
    out = (ctypes.c_uint32 * 8)()
    rinv = pow(R, -1, p)
    for it in range(3000):
        a, b = rv(), rv()
        getattr(hm, f"zkh_{name}_mul")(buf(a), buf(b), out)
        assert val(out) == a * b * rinv % p
        bb = rnd.randrange(R) if it % 3 else R - 1  # second operand may be any 256-bit value
        getattr(hm, f"zkh_{name}_mul")(buf(a), buf(bb), out)
        assert val(out) == a * bb * rinv % p
        getattr(hm, f"zkh_{name}_mul_fixed")(buf(a), buf(b), out)
        assert val(out) == a * b * rinv % p
        getattr(hm, f"zkh_{name}_add")(buf(a), buf(b), out)
        assert val(out) == (a + b) % p
        getattr(hm, f"zkh_{name}_sub")(buf(a), buf(b), out)
        assert val(out) == (a - b) % p
    for _ in range(5):
        a = rv()
        getattr(hm, f"zkh_{name}_inv")(buf(a), out)
        am = a * rinv % p
        assert val(out) == ((pow(am, -1, p) * R % p) if am else 0)
        getattr(hm, f"zkh_{name}_to_mont")(buf(a), out)
        assert val(out) == a * R % p


@pytest.mark.parametrize("name,p", [("fr", o.R_MOD), ("fq", o.Q_MOD)])
def test_double_fold_formula(hm, name, p):
    """t0 + r0 d01 + r1 (t2 - t0) + r0 r1 (d23 - d01) equals two successive folds."""
    rnd = random.Random(12)
    out = (ctypes.c_uint32 * 8)()
    edge = [0, 1, p - 1, p - 2]
    for it in range(500):
        r0, r1 = rnd.randrange(p), rnd.randrange(p)
        t = [rnd.choice(edge) if rnd.random() < 0.3 else rnd.randrange(p) for _ in range(4)]
        xs = (ctypes.c_uint32 * 16)(*[((v * R % p) >> (32 * i)) & 0xFFFFFFFF for v in (r0, r1) for i in range(8)])
        ts = (ctypes.c_uint32 * 32)(*[((v * R % p) >> (32 * i)) & 0xFFFFFFFF for v in t for i in range(8)])
        getattr(hm, f"zkh_{name}_fold2")(xs, ts, out)
        a = (t[0] + r0 * (t[1] - t[0])) % p
        b = (t[2] + r0 * (t[3] - t[2])) % p
        assert val(out) == ((a + r1 * (b - a)) % p) * R % p


@pytest.mark.parametrize("name,p", [("fr", o.R_MOD), ("fq", o.Q_MOD)])
def test_lazy_dot_product(hm, name, p):
    rnd = random.Random(6)
    out = (ctypes.c_uint32 * 8)()
    rinv = pow(R, -1, p)
    for n in (1, 4, 5, 6, 37, 300):
        for worst in (True, False):
            a = [p - 1 if worst else rnd.randrange(p) for _ in range(n)]
            b = [p - 1 if worst else rnd.randrange(p) for _ in range(n)]
            ab = (ctypes.c_uint32 * (8 * n))(*[(x >> (32 * i)) & 0xFFFFFFFF for x in a for i in range(8)])
            bb = (ctypes.c_uint32 * (8 * n))(*[(x >> (32 * i)) & 0xFFFFFFFF for x in b for i in range(8)])
            getattr(hm, f"zkh_{name}_dot")(ab, bb, n, out)
            assert val(out) == sum(x * y for x, y in zip(a, b)) * rinv % p


def test_wide_product(hm):
    rnd = random.Random(7)
    w = (ctypes.c_uint32 * 16)()
    for it in range(3000):
        a = rnd.randrange(R) if it % 5 else R - 1
        b = rnd.randrange(R) if it % 7 else R - 1
        hm.zkh_mul_wide(buf(a), buf(b), w)
        assert val(w) == a * b


def aff_buf(pt):
    q = o.Q_MOD
    if pt is None:
        return (ctypes.c_uint32 * 16)()
    x, y = pt[0] * R % q, pt[1] * R % q
    return (ctypes.c_uint32 * 16)(*[(v >> (32 * i)) & 0xFFFFFFFF for v in (x, y) for i in range(8)])


def aff_val(b):
    q = o.Q_MOD
    rinv = pow(R, -1, q)
    x = sum(int(v) << (32 * i) for i, v in enumerate(b[:8])) * rinv % q
    y = sum(int(v) << (32 * i) for i, v in enumerate(b[8:16])) * rinv % q
    return None if x == 0 and y == 0 else (x, y)


def test_g1_group_law(hm):
    rnd = random.Random(11)
    g = o.G1_GEN
    out = (ctypes.c_uint32 * 16)()
    pts = [o.g1_mul(g, rnd.randrange(1, o.R_MOD)) for _ in range(4)]
    cases = []
    for _ in range(30):
        cases.append((rnd.choice(pts), rnd.randrange(0, 50), rnd.choice(pts + [None]), rnd.choice(pts + [None]),
                      rnd.randrange(0, 50), rnd.randrange(0, 3)))
    p = pts[0]
    # exceptional cases: P + P, P + (-P), infinity operands, doubling of the result
    cases += [(p, 1, p, p, 0, 0), (p, 1, o.g1_neg(p), p, 0, 1), (p, 0, None, p, 0, 0), (p, 2, o.g1_neg(p), o.g1_neg(p), 1, 0),
              (p, 3, p, p, 4, 2), (p, 1, None, p, 1, 0), (p, 5, o.g1_neg(p), o.g1_mul(p, 4), 1, 0)]
    for a, k1, b, c, k2, dbls in cases:
        hm.zkh_g1_combo(aff_buf(a), k1, aff_buf(b), aff_buf(c), k2, dbls, out)
        want = o.g1_add(o.g1_add(o.g1_mul(a, k1), b), o.g1_mul(c, k2) if c else None)
        for _ in range(dbls):
            want = o.g1_add(want, want)
        assert aff_val(out) == want
        assert o.g1_is_on_curve(aff_val(out))
    jac = (ctypes.c_uint32 * 24)()
    hm.zkh_g1_jacobian(aff_buf(p), 7, jac)
    q = o.Q_MOD
    rinv = pow(R, -1, q)
    X, Y, Z = [sum(int(v) << (32 * i) for i, v in enumerate(jac[8 * k:8 * k + 8])) * rinv % q for k in range(3)]
    zi = pow(Z, -1, q)
    assert (X * zi * zi % q, Y * zi * zi * zi % q) == o.g1_mul(p, 7)


def test_device_form_transcript_matches_oracle(hm):
    """strobe_dev.cuh (the single-thread GPU transcript) against the oracle's Merlin, continuing
    from an arbitrary mid-stream state over many rounds."""
    rnd = random.Random(21)
    t = o.Transcript(b"sumcheck")
    t.append_u64(b"num_var", 20)
    t.append_u64(b"num_poly", 2)
    t.append_message(b"x", bytes(rnd.randrange(256) for _ in range(77)))
    state = (ctypes.c_uint8 * 200)(*t.strobe.state)
    pos3 = (ctypes.c_uint32 * 3)(t.strobe.pos, t.strobe.pos_begin, t.strobe.cur_flags)
    ch = (ctypes.c_uint32 * 8)()
    for rounds in range(40):
        n = rnd.choice([2, 3, 4, 5])
        scalars = [rnd.randrange(o.R_MOD) for _ in range(n)]
        buf = (ctypes.c_uint32 * (8 * n))(*[((v * R % o.R_MOD) >> (32 * i)) & 0xFFFFFFFF for v in scalars for i in range(8)])
        hm.zkh_strobe_round(state, pos3, buf, n, ch)
        for s_ in scalars:
            t.append_scalar(b"round_message", s_)
        want = t.challenge_scalar(b"challenge")
        assert val(ch) == want * R % o.R_MOD
        assert bytes(state) == bytes(t.strobe.state)
        assert (pos3[0], pos3[1]) == (t.strobe.pos, t.strobe.pos_begin)
