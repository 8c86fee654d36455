"""KZH2 / KZH3 setup, commit and open on the GPU against the oracle (which restates kzh2.rs and
kzh3.rs), plus the identities the reference's verifiers check (kzh2.rs:763-789, kzh3.rs:836-886)
and the trapdoor identity C = (sum_i f_i t_i) g.  Mirrors tests/test_kzh2.rs:42-175 (n in 2, 4, 6)
and tests/test_kzh3.rs:31-85 (n in 3, 4)."""
import random

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, kzh

pytestmark = pytest.mark.gpu
M = o.R_MOD


def trapdoors(seed, n_x, n_y, n_z=0):
    d = o.gen_uniform_fr(seed, 0, 0, 1 + n_x + n_y + max(n_z, 1))
    return d[0], d[1:1 + n_x], d[1 + n_x:1 + n_x + n_y], d[1 + n_x + n_y:]


@pytest.mark.parametrize("n,kind", [(2, "full"), (3, "int8"), (4, "full"), (5, "mixed"), (6, "int8")])
def test_kzh2_commit_open(ctx, n, kind):
    rnd = random.Random(n)
    xl, yl = o.kzh2_degrees(n)
    gk, tx, ty, rest = trapdoors(2, 1 << xl, 1 << yl)
    alpha = rest[0]
    osrs = o.KZH2SRS(n, gk, tx, ty, alpha)
    srs = kzh.KZHSRS.setup(ctx, 2, n, osrs.g, tx, ty, alpha=alpha)
    assert (srs.x_log, srs.y_log) == (xl, yl)
    assert srs.read(0, 0, 1 << n) == osrs.h_xy and srs.read(1, 0, 1 << yl) == osrs.h_y
    mk = {"full": lambda i: rnd.randrange(M), "int8": lambda i: o.fr_from_int(rnd.randrange(-128, 128)),
          "mixed": lambda i: o.fr_from_int(rnd.randrange(-2 ** 15, 2 ** 15)) if i % 2 else rnd.randrange(M)}[kind]
    f = [mk(i) for i in range(1 << n)]
    poly = DenseMLPoly.from_evaluations(f)
    com = kzh.commit(ctx, srs, poly)
    oc, odx = o.kzh2_commit(osrs, f)
    assert com.c == oc and com.d_x == odx
    assert com.c == o.g1_mul(osrs.g, sum(a * b for a, b in zip(f, osrs.t_xy)) % M)  # trapdoor identity
    pt = [rnd.randrange(M) for _ in range(n)]
    d_x, f_star = kzh.kzh2_open(ctx, srs, pt, com, poly)
    _, ofs = o.kzh2_open(osrs, pt, odx, f)
    assert f_star == ofs and d_x == odx
    r_y, r_x = o.split_input([yl, xl], pt)
    assert o.g1_msm(d_x, o.evaluate_lagrange_basis(r_x)) == o.g1_msm(osrs.h_y, f_star)  # kzh2.rs:763-789
    assert o.evaluate_multilinear_extension(f_star, r_y) == o.evaluate_multilinear_extension(f, pt)  # test_kzh2.rs:149-175


def test_kzh2_small_poly_and_short_point(ctx):
    """A polynomial with fewer variables than the SRS is zero-extended; a short point is left-padded."""
    rnd = random.Random(9)
    n = 6
    gk, tx, ty, rest = trapdoors(3, 8, 8)
    osrs = o.KZH2SRS(n, gk, tx, ty, rest[0])
    srs = kzh.KZHSRS.upload(ctx, 2, n, osrs.h_xy, osrs.h_y)
    f = [rnd.randrange(M) for _ in range(16)]
    poly = DenseMLPoly.from_evaluations(f)
    com = kzh.commit(ctx, srs, poly)
    oc, odx = o.kzh2_commit(osrs, f)
    assert com.c == oc and com.d_x == odx
    pt = [rnd.randrange(M) for _ in range(4)]
    _, f_star = kzh.kzh2_open(ctx, srs, pt, com, poly)
    assert f_star == o.kzh2_open(osrs, pt, odx, f)[1]


@pytest.mark.parametrize("n,kind", [(3, "full"), (4, "int8"), (5, "full"), (7, "mixed")])
def test_kzh3_commit_open(ctx, n, kind):
    rnd = random.Random(30 + n)
    xl, yl, zl = o.kzh3_degrees(n)
    gk, tx, ty, tz = trapdoors(3, 1 << xl, 1 << yl, 1 << zl)
    tz = tz[:1 << zl]
    osrs = o.KZH3SRS(n, gk, tx, ty, tz)
    srs = kzh.KZHSRS.setup(ctx, 3, n, osrs.g, tx, ty, tau_z=tz)
    assert (srs.x_log, srs.y_log, srs.z_log) == (xl, yl, zl)
    assert srs.read(0, 0, 1 << n) == osrs.h_xyz and srs.read(1, 0, 1 << (yl + zl)) == osrs.h_yz
    assert srs.read(2, 0, 1 << zl) == osrs.h_z
    mk = {"full": lambda i: rnd.randrange(M), "int8": lambda i: o.fr_from_int(rnd.randrange(-128, 128)),
          "mixed": lambda i: o.fr_from_int(rnd.randrange(-2 ** 15, 2 ** 15)) if (i >> 2) % 2 else rnd.randrange(M)}[kind]
    f = [mk(i) for i in range(1 << n)]
    poly = DenseMLPoly.from_evaluations(f)
    com = kzh.commit(ctx, srs, poly)
    oc, odx = o.kzh3_commit(osrs, f)
    assert com.c == oc and com.d_x == odx
    assert com.c == o.g1_mul(osrs.g, sum(a * b for a, b in zip(f, osrs.t_xyz)) % M)
    pt = [rnd.randrange(M) for _ in range(n)]
    d_x, d_y, c_y, f_star = kzh.kzh3_open(ctx, srs, pt, com, poly)
    _, ody, ocy, ofs = o.kzh3_open(osrs, pt, odx, f)
    assert d_y == ody and c_y == ocy and f_star == ofs
    r_z, r_y, r_x = o.split_input([zl, yl, xl], pt)
    assert c_y == o.g1_msm(d_x, o.evaluate_lagrange_basis(r_x))  # kzh3.rs:836-852
    assert o.g1_msm(osrs.h_z, f_star) == o.g1_msm(d_y, o.evaluate_lagrange_basis(r_y))
    assert o.evaluate_multilinear_extension(f_star, r_z) == o.evaluate_multilinear_extension(f, pt)


def test_kzh_argument_errors(ctx):
    from zkes_b200._lib import ZkError
    gk, tx, ty, rest = trapdoors(2, 2, 2)
    osrs = o.KZH2SRS(2, gk, tx, ty, rest[0])
    srs = kzh.KZHSRS.upload(ctx, 2, 2, osrs.h_xy, osrs.h_y)
    big = DenseMLPoly.from_evaluations([1] * 8)
    with pytest.raises(ZkError):
        kzh.commit(ctx, srs, big)  # more variables than the SRS supports
    with pytest.raises(ZkError):
        kzh.kzh3_open(ctx, srs, [1, 2], kzh.commit(ctx, srs, DenseMLPoly.from_evaluations([1, 2, 3, 4])),
                      DenseMLPoly.from_evaluations([1, 2, 3, 4]))


@pytest.mark.parametrize("dims,n,nnz,ones", [(2, 4, 5, False), (2, 6, 20, True), (3, 5, 9, False), (3, 7, 40, True), (2, 6, 0, False)])
def test_sparse_kzh_commit_open(ctx, dims, n, nnz, ones):
    """sparse_kzh2 / sparse_kzh3 commit and open (sparse_kzh2.rs:14-127, sparse_kzh3.rs:32-232); `ones`
    mirrors the selection polynomials of the range proofs (all-one values)."""
    rnd = random.Random(1000 * dims + n)
    if dims == 2:
        xl, yl = o.kzh2_degrees(n)
        gk, tx, ty, rest = trapdoors(7, 1 << xl, 1 << yl)
        osrs = o.KZH2SRS(n, gk, tx, ty, rest[0])
        srs = kzh.KZHSRS.upload(ctx, 2, n, osrs.h_xy, osrs.h_y)
    else:
        xl, yl, zl = o.kzh3_degrees(n)
        gk, tx, ty, tz = trapdoors(8, 1 << xl, 1 << yl, 1 << zl)
        osrs = o.KZH3SRS(n, gk, tx, ty, tz[:1 << zl])
        srs = kzh.KZHSRS.upload(ctx, 3, n, osrs.h_xyz, osrs.h_yz, osrs.h_z)
    ev = {i: (1 if ones else rnd.randrange(M)) for i in rnd.sample(range(1 << n), nnz)}
    com = kzh.sparse_commit(ctx, srs, ev)
    oc, odx = (o.sparse_kzh2_commit if dims == 2 else o.sparse_kzh3_commit)(osrs, ev)
    assert com.c == oc and com.d_x == odx
    dense = [ev.get(i, 0) for i in range(1 << n)]
    assert (oc, odx) == (o.kzh2_commit if dims == 2 else o.kzh3_commit)(osrs, dense)  # same commitment as the dense form
    for plen in (n, n - 2):
        pt = [rnd.randrange(M) for _ in range(plen)]
        if dims == 2:
            _, fs = kzh.sparse_kzh2_open(ctx, srs, pt, com, ev)
            assert fs == o.sparse_kzh2_open(osrs, pt, odx, ev)[1]
        else:
            _, dy, cy, fs = kzh.sparse_kzh3_open(ctx, srs, pt, com, ev)
            _, ody, ocy, ofs = o.sparse_kzh3_open(osrs, pt, odx, ev)
            assert (dy, cy, fs) == (ody, ocy, ofs)


@pytest.mark.parametrize("dims,n,nnz", [(2, 6, 20), (2, 8, 200), (3, 7, 40), (3, 9, 300), (2, 6, 1), (2, 6, 64)])
def test_selection_polynomial_commit(ctx, dims, n, nnz):
    """A selection polynomial passes no values (every listed entry is one): its commitment is computed as plain
    sums of SRS points over runs of the ordered index list, whatever order the caller lists them in; with explicit
    ones, or with an index listed twice, it goes through the general MSM.  All must give the oracle's commitment."""
    import ctypes
    import numpy as np
    from zkes_b200 import curve
    from zkes_b200._lib import check, lib
    from zkes_b200.field import to_mont_array
    rnd = random.Random(77 * dims + n)
    if dims == 2:
        xl, yl = o.kzh2_degrees(n)
        gk, tx, ty, rest = trapdoors(7, 1 << xl, 1 << yl)
        osrs = o.KZH2SRS(n, gk, tx, ty, rest[0])
        srs = kzh.KZHSRS.upload(ctx, 2, n, osrs.h_xy, osrs.h_y)
    else:
        xl, yl, zl = o.kzh3_degrees(n)
        gk, tx, ty, tz = trapdoors(8, 1 << xl, 1 << yl, 1 << zl)
        osrs = o.KZH3SRS(n, gk, tx, ty, tz[:1 << zl])
        srs = kzh.KZHSRS.upload(ctx, 3, n, osrs.h_xyz, osrs.h_yz, osrs.h_z)
    positions = sorted(rnd.sample(range(1 << n), nnz))
    ev = {i: 1 for i in positions}
    oc, odx = (o.sparse_kzh2_commit if dims == 2 else o.sparse_kzh3_commit)(osrs, ev)

    def commit(order, with_values):
        idx = np.array(order, dtype=np.uint64)
        vals = to_mont_array([1] * len(order)) if with_values else None
        c = np.zeros((1, 8), dtype=np.uint64)
        dx = np.zeros((1 << srs.x_log, 12), dtype=np.uint64)
        vp = ctypes.c_void_p
        check(lib.zk_sparse_kzh_commit(ctx.handle, srs.handle, len(order), vp(idx.ctypes.data),
                                       vp(vals.ctypes.data) if vals is not None else None, vp(c.ctypes.data), vp(dx.ctypes.data)),
              "zk_sparse_kzh_commit")
        return kzh.KZHCommitment(srs, curve.affine_from_array(c)[0], dx)

    shuffled = positions[:]
    rnd.shuffle(shuffled)
    for order, with_values in ((positions, False), (shuffled, False), (positions, True)):
        com = commit(order, with_values)
        assert com.c == oc and com.d_x == odx
    if nnz > 1:  # an index listed twice counts twice, as in the reference's loop over the entries
        twice = shuffled + [shuffled[0]]
        ev2 = dict(ev)
        ev2[shuffled[0]] = 2
        oc2, odx2 = (o.sparse_kzh2_commit if dims == 2 else o.sparse_kzh3_commit)(osrs, ev2)
        com = commit(twice, False)
        assert com.c == oc2 and com.d_x == odx2


@pytest.mark.parametrize("n", [2, 4, 5])
def test_kzh2_verify_g1(ctx, n):
    """The G1 / field steps of kzh2_verify (kzh2.rs:763-789) on the device: an honest opening passes,
    and each tampered part fails at the step the reference would fail at (tests/test_kzh2.rs:42-175
    checks only that honest openings verify)."""
    rnd = random.Random(400 + n)
    xl, yl = o.kzh2_degrees(n)
    gk, tx, ty, rest = trapdoors(5, 1 << xl, 1 << yl)
    osrs = o.KZH2SRS(n, gk, tx, ty, rest[0])
    srs = kzh.KZHSRS.setup(ctx, 2, n, osrs.g, tx, ty, alpha=rest[0])
    f = [rnd.randrange(M) for _ in range(1 << n)]
    poly = DenseMLPoly.from_evaluations(f)
    com = kzh.commit(ctx, srs, poly)
    pt = [rnd.randrange(M) for _ in range(n)]
    d_x, f_star = kzh.kzh2_open(ctx, srs, pt, com, poly)
    value = o.evaluate_multilinear_extension(f, pt)
    assert kzh.verify_g1(ctx, srs, pt, value, com.d_x_jac, f_star) == (True, 0)
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, f_star) == (True, 0)  # affine d_x as the proof carries it
    assert kzh.verify_g1(ctx, srs, pt, (value + 1) % M, d_x, f_star) == (False, 3)
    bad_f = list(f_star)
    bad_f[0] = (bad_f[0] + 1) % M
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, bad_f) == (False, 2)
    bad_dx = list(d_x)
    bad_dx[-1] = o.g1_add(bad_dx[-1], osrs.g) if bad_dx[-1] is not None else osrs.g
    assert kzh.verify_g1(ctx, srs, pt, value, bad_dx, f_star) == (False, 2)


@pytest.mark.parametrize("n", [3, 4, 7])
def test_kzh3_verify_g1(ctx, n):
    """Checks 2, 4 and 5 of kzh3_verify (kzh3.rs:836-886)."""
    rnd = random.Random(500 + n)
    xl, yl, zl = o.kzh3_degrees(n)
    gk, tx, ty, tz = trapdoors(6, 1 << xl, 1 << yl, 1 << zl)
    tz = tz[:1 << zl]
    osrs = o.KZH3SRS(n, gk, tx, ty, tz)
    srs = kzh.KZHSRS.setup(ctx, 3, n, osrs.g, tx, ty, tau_z=tz)
    f = [o.fr_from_int(rnd.randrange(-2 ** 15, 2 ** 15)) if i % 3 else rnd.randrange(M) for i in range(1 << n)]
    poly = DenseMLPoly.from_evaluations(f)
    com = kzh.commit(ctx, srs, poly)
    pt = [rnd.randrange(M) for _ in range(n)]
    d_x, d_y, c_y, f_star = kzh.kzh3_open(ctx, srs, pt, com, poly)
    value = o.evaluate_multilinear_extension(f, pt)
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, f_star, d_y=d_y, c_y=c_y) == (True, 0)
    assert kzh.verify_g1(ctx, srs, pt, (value + 5) % M, d_x, f_star, d_y=d_y, c_y=c_y) == (False, 5)
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, f_star, d_y=d_y, c_y=o.g1_add(c_y, osrs.g) if c_y else osrs.g) == (False, 2)
    bad_dy = list(d_y)
    bad_dy[0] = o.g1_add(bad_dy[0], osrs.g) if bad_dy[0] is not None else osrs.g
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, f_star, d_y=bad_dy, c_y=c_y) == (False, 4)
    bad_f = list(f_star)
    bad_f[-1] = (bad_f[-1] + 1) % M
    assert kzh.verify_g1(ctx, srs, pt, value, d_x, bad_f, d_y=d_y, c_y=c_y) == (False, 4)
