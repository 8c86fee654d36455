"""GPU MSM against the big-integer oracle: P::G1::msm semantics (kzh2.rs:640,658), the shared-base
batched form, sparse_msm (polycommit/mod.rs:10-31), small (quantised) and full-width scalars,
points at infinity, repeated and opposite points, empty input."""
import random

import numpy as np
import pytest

import pyoracle as o
from zkes_b200 import curve

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def points():
    rnd = random.Random(42)
    pts = [o.g1_mul(o.G1_GEN, rnd.randrange(1, o.R_MOD)) for _ in range(96)]
    return pts


def small(rnd, bits):
    return o.fr_from_int(rnd.randrange(-(1 << (bits - 1)), 1 << (bits - 1)))


@pytest.mark.parametrize("n,kind", [(0, "full"), (1, "full"), (2, "full"), (7, "full"), (33, "full"), (96, "full"),
                                    (1, "int8"), (50, "int8"), (96, "int16"), (96, "mixed"), (40, "zero")])
def test_msm_matches_oracle(ctx, points, n, kind):
    rnd = random.Random(n * 7 + len(kind))
    bases = points[:n]
    if kind == "full":
        sc = [rnd.choice([0, 1, o.R_MOD - 1, (o.R_MOD - 1) // 2, (o.R_MOD + 1) // 2]) if rnd.random() < 0.2 else rnd.randrange(o.R_MOD)
              for _ in range(n)]
    elif kind == "int8":
        sc = [small(rnd, 8) for _ in range(n)]
        if n:
            sc[0] = o.fr_from_int(-128)
    elif kind == "int16":
        sc = [small(rnd, 16) for _ in range(n)]
    elif kind == "mixed":
        sc = [small(rnd, 16) if i % 2 else rnd.randrange(o.R_MOD) for i in range(n)]
    else:
        sc = [0] * n
    got = curve.msm(ctx, curve.affine_to_array(bases), sc)
    assert got == o.g1_msm(bases, sc)


def test_msm_special_points(ctx, points):
    p = points[0]
    bases = [p, p, o.g1_neg(p), None, points[1], None, p]
    sc = [3, 5, 8, 12345, 7, 0, o.R_MOD - 1]
    assert curve.msm(ctx, curve.affine_to_array(bases), sc) == o.g1_msm(bases, sc)
    # everything cancels
    assert curve.msm(ctx, curve.affine_to_array([p, o.g1_neg(p)]), [77, 77]) is None
    # the same point many times in one bucket (doubling inside the mixed addition)
    assert curve.msm(ctx, curve.affine_to_array([p] * 40), [9] * 40) == o.g1_mul(p, 360)


def test_msm_length_mismatch(ctx, points):
    with pytest.raises(ValueError):
        curve.msm(ctx, curve.affine_to_array(points[:3]), [1, 2])


@pytest.mark.parametrize("rows,n,kind", [(1, 16, "int8"), (5, 16, "int8"), (8, 32, "full"), (3, 7, "mixed"), (64, 4, "int8")])
def test_batched_msm(ctx, points, rows, n, kind):
    rnd = random.Random(rows * 100 + n)
    bases = points[:n]
    mk = {"int8": lambda i: small(rnd, 8), "full": lambda i: rnd.randrange(o.R_MOD),
          "mixed": lambda i: small(rnd, 16) if i % 2 else rnd.randrange(o.R_MOD)}[kind]
    mat = [[mk(i) for i in range(n)] for _ in range(rows)]
    if rows > 2:
        mat[1] = [0] * n  # an all-zero row gives the identity
    got = curve.msm_batched(ctx, curve.affine_to_array(bases), mat)
    assert got == [o.g1_msm(bases, r) for r in mat]


@pytest.mark.parametrize("bits", [8, 16])
def test_batched_msm_many_rows(ctx, points, bits):
    """Thousands of short rows over shared bases (the shape of a commitment's d_x rows): the bucket
    sums of a row are then reduced by eight lanes, four rows to a warp.  Sampled rows against the oracle."""
    rnd = random.Random(bits)
    n = 256
    bases = [points[i % len(points)] if i < len(points) else o.g1_mul(o.G1_GEN, 1000 + i) for i in range(n)]
    rows = 1100
    mat = [[small(rnd, bits) for _ in range(n)] for _ in range(rows)]
    mat[7] = [0] * n
    mat[8] = [o.fr_from_int(-(1 << (bits - 1)))] * n  # the largest magnitude everywhere
    got = curve.msm_batched(ctx, curve.affine_to_array(bases), mat)
    for r in (0, 7, 8, 9, 511, 1024, rows - 1):
        assert got[r] == o.g1_msm(bases, mat[r]), r


def test_sparse_msm(ctx, points):
    rnd = random.Random(5)
    idx = [rnd.randrange(len(points)) for _ in range(50)]  # repeats allowed
    sc = [1] * 50  # selection polynomials: all-ones scalars (sparse_kzh2.rs)
    want = o.g1_msm([points[i] for i in idx], sc)
    assert curve.sparse_msm(ctx, curve.affine_to_array(points), idx, sc) == want
    sc = [rnd.randrange(o.R_MOD) for _ in idx]
    assert curve.sparse_msm(ctx, curve.affine_to_array(points), idx, sc) == o.g1_msm([points[i] for i in idx], sc)
    assert curve.sparse_msm(ctx, curve.affine_to_array(points), [], []) is None
    from zkes_b200._lib import ZkError
    with pytest.raises(ZkError):
        curve.sparse_msm(ctx, curve.affine_to_array(points), [len(points)], [1])
    with pytest.raises(ValueError):
        curve.sparse_msm(ctx, curve.affine_to_array(points), [1, 2], [1])


def test_msm_medium_int8_linearity(ctx, points):
    """2^13 points (repeating the 96 bases) with int8 scalars: compare with the per-base totals."""
    rnd = random.Random(8)
    n = 1 << 13
    idx = [i % len(points) for i in range(n)]
    sc = [rnd.randrange(-128, 128) for _ in range(n)]
    tot = [0] * len(points)
    for i, s in zip(idx, sc):
        tot[i] += s
    want = o.g1_msm(points, [t % o.R_MOD for t in tot])
    bases = curve.affine_to_array(points)[np.array(idx)]
    got = curve.msm(ctx, np.ascontiguousarray(bases), [o.fr_from_int(s) for s in sc])
    assert got == want
    st = curve.last_stats(ctx)
    assert st["windows"] == 1 and st["max_bits"] <= 8


def test_normalize(ctx, points):
    from zkes_b200.field import Q_MOD, to_mont_array
    rnd = random.Random(2)
    rows = []
    for p in points[:10] + [None]:
        if p is None:
            rows += [1, 1, 0]
        else:
            z = rnd.randrange(1, Q_MOD)
            rows += [p[0] * z * z % Q_MOD, p[1] * z * z * z % Q_MOD, z]
    jac = to_mont_array(rows, Q_MOD).reshape(-1, 12)
    assert curve.normalize(ctx, jac) == points[:10] + [None]


@pytest.mark.parametrize("n,kind", [(1 << 14, "full"), (1 << 15, "mixed"), (3000, "int8"), (1 << 13, "int16")])
def test_msm_against_cpp_oracle_thousands_of_points(ctx, n, kind):
    """Sizes the big-integer oracle cannot reach: the bases are an SRS vector generated on the device
    (distinct multiples of g, read back), the expected point comes from the C++ bucket-method MSM."""
    import ctypes

    import coracle
    from zkes_b200 import kzh
    from zkes_b200._lib import ZK_MEM_HOST, check, lib
    from zkes_b200.field import to_mont_array

    coracle.set_threads(8)
    rnd = random.Random(n + len(kind))
    log = (n - 1).bit_length()
    xl = log // 2
    tx = [rnd.randrange(1, o.R_MOD) for _ in range(1 << xl)]
    ty = [rnd.randrange(1, o.R_MOD) for _ in range(1 << (log - xl))]
    srs = kzh.KZHSRS.setup(ctx, 2, log, o.g1_mul(o.G1_GEN, 31337), tx, ty, alpha=5)
    bases = np.zeros((n, 8), dtype=np.uint64)
    check(lib.zk_kzh_srs_read(ctx.handle, srs.handle, 0, 0, n, ctypes.c_void_p(bases.ctypes.data)), "zk_kzh_srs_read")
    srs.close()
    if kind == "full":
        sc = [rnd.randrange(o.R_MOD) for _ in range(n)]
    elif kind == "mixed":
        sc = [small(rnd, 16) if (i >> 6) % 2 else rnd.randrange(o.R_MOD) for i in range(n)]
    else:
        sc = [small(rnd, 8 if kind == "int8" else 16) for _ in range(n)]
    sm = to_mont_array(sc)
    out = np.zeros((1, 12), dtype=np.uint64)
    vp = ctypes.c_void_p
    check(lib.zk_msm_g1(ctx.handle, vp(bases.ctypes.data), ZK_MEM_HOST, vp(sm.ctypes.data), ZK_MEM_HOST, n,
                        vp(out.ctypes.data), ZK_MEM_HOST), "zk_msm_g1")
    assert curve.jacobian_to_affine_py(out)[0] == coracle.g1_msm_mont(bases, sm)
