"""KZH at benchmark sizes, checked through size-independent properties (no CPU MSM is feasible):
the trapdoor identity C = (sum_i f_i t_i) g computed by contracting f with the trapdoor vectors,
single rows of d_x the same way, and the opening identities of kzh2.rs:763-789 / kzh3.rs:836-886
with f(point) obtained by an independent kernel path (the LSB fold)."""
import ctypes
import random

import numpy as np
import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, kzh
from zkes_b200._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
from zkes_b200.field import from_mont_array, to_mont_array

pytestmark = pytest.mark.gpu
M = o.R_MOD
G = o.g1_mul(o.G1_GEN, 987654321)


def dev_uniform(ctx, seed, stream, count):
    import torch
    t = torch.empty((count, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_uniform_fr(ctx.handle, seed, stream, 0, count, t.data_ptr()), "gen")
    return t


def host_ints(t):
    return from_mont_array(t.cpu().numpy().view(np.uint64))


def contract_high(ctx, n, f_ptr, k, weights):
    """out[lo] = sum_hi weights[hi] f[hi * 2^(n-k) + lo] on the device."""
    w = to_mont_array(weights)
    out = np.zeros((1 << (n - k), 4), dtype=np.uint64)
    check(lib.zk_weighted_fold_from_right(ctx.handle, n, ctypes.c_void_p(f_ptr), ZK_MEM_DEVICE, k, ctypes.c_void_p(w.ctypes.data),
                                          ZK_MEM_HOST, ctypes.c_void_p(out.ctypes.data), ZK_MEM_HOST), "weighted_fold")
    return from_mont_array(out)


def mle_at(ctx, n, f_ptr, point):
    pt = to_mont_array(point)
    out = np.zeros((1, 4), dtype=np.uint64)
    check(lib.zk_fold_lsb(ctx.handle, n, ctypes.c_void_p(f_ptr), ZK_MEM_DEVICE, n, ctypes.c_void_p(pt.ctypes.data),
                          ctypes.c_void_p(out.ctypes.data), ZK_MEM_HOST), "fold_lsb")
    return from_mont_array(out)[0]


def test_kzh2_int8_2p24(ctx):
    """2^24 int8 evaluations (quantised weights) on a 2^12 x 2^12 split, seed 2."""
    import torch
    n, xl, yl = 24, 12, 12
    tx, ty = host_ints(dev_uniform(ctx, 2, 1, 1 << xl)), host_ints(dev_uniform(ctx, 2, 2, 1 << yl))
    alpha = 1234567890123456789
    srs = kzh.KZHSRS.setup(ctx, 2, n, G, tx, ty, alpha=alpha)
    f = torch.empty((1 << n, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_small_fr(ctx.handle, 2, 7, 0, 1 << n, 8, f.data_ptr()), "gen")
    poly = DenseMLPoly(n, device_ptr=f.data_ptr())
    com = kzh.commit(ctx, srs, poly)
    # C = (sum_x tau_x[x] sum_y tau_y[y] f[x, y]) g
    gy = contract_high(ctx, n, f.data_ptr(), xl, tx)
    s = sum(a * b for a, b in zip(gy, ty)) % M
    assert com.c == o.g1_mul(G, s)
    # rows of d_x: d_x[i] = (alpha sum_y tau_y[y] f[i, y]) g
    d_x = com.d_x
    for i in (0, 1, 2047, 4095):
        row = host_ints(f[i << yl:(i + 1) << yl])
        assert d_x[i] == o.g1_mul(G, alpha * sum(a * b for a, b in zip(row, ty)) % M)
    # open: f_star(r_y) = f(point), and sum_i eq(r_x)[i] d_x[i] = MSM(h_y, f_star) in the exponent
    rnd = random.Random(3)
    pt = [rnd.randrange(M) for _ in range(n)]
    _, f_star = kzh.kzh2_open(ctx, srs, pt, com, poly)
    r_y, r_x = pt[:yl], pt[yl:]
    assert o.evaluate_multilinear_extension(f_star, r_y) == mle_at(ctx, n, f.data_ptr(), pt)
    eqx = o.evaluate_lagrange_basis(r_x)
    # sum_x eq(r_x)[x] f[x, .] by the weighted contraction (a different launch shape of the column-sum kernel)
    assert contract_high(ctx, n, f.data_ptr(), xl, eqx) == f_star
    # verifier identity in the exponent: sum_i eq[i] d_x[i] = MSM(h_y, f_star) = (alpha sum_y tau_y[y] f_star[y]) g
    sample = random.Random(5).sample(range(1 << xl), 3)
    for i in sample:
        row = host_ints(f[i << yl:(i + 1) << yl])
        assert d_x[i] == o.g1_mul(G, alpha * sum(a * b for a, b in zip(row, ty)) % M)
    srs.close()


def run_kzh3_mix(ctx, n):
    """KZH3 commit + open of 2^n evaluations in alternating x-slabs of int16 fixed-point activations
    (N(0,1) * 2^8 rounded) and full-width values, checked by the trapdoor identities and the
    identities of kzh3_verify (kzh3.rs:836-886)."""
    import torch
    xl, yl, zl = o.kzh3_degrees(n)
    tx = host_ints(dev_uniform(ctx, 3, 1, 1 << xl))
    ty = host_ints(dev_uniform(ctx, 3, 2, 1 << yl))
    tz = host_ints(dev_uniform(ctx, 3, 3, 1 << zl))
    srs = kzh.KZHSRS.setup(ctx, 3, n, G, tx, ty, tau_z=tz)
    f = torch.empty((1 << n, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_uniform_fr(ctx.handle, 3, 7, 0, 1 << n, f.data_ptr()), "gen")
    slab = 1 << (yl + zl)
    for x in range(0, 1 << xl, 2):  # even slabs: N(0,1) * 2^8 rounded
        check(lib.zk_gen_gauss_fr(ctx.handle, 3, 8, x * slab, slab, 8, f[x * slab:(x + 1) * slab].data_ptr()), "gen")
    torch.cuda.synchronize()
    small = host_ints(f[:64])
    assert all(v < (1 << 15) or M - v < (1 << 15) for v in small) and len(set(small)) > 8
    poly = DenseMLPoly(n, device_ptr=f.data_ptr())
    com = kzh.commit(ctx, srs, poly)
    gyz = contract_high(ctx, n, f.data_ptr(), xl, tx)  # [y, z]
    tyz = [ty[i >> zl] * tz[i & ((1 << zl) - 1)] % M for i in range(1 << (yl + zl))]
    assert com.c == o.g1_mul(G, sum(a * b for a, b in zip(gyz, tyz)) % M)
    d_x = com.d_x
    for i in (0, 1, (1 << xl) - 1):  # an activation slab, a full-width slab, the last slab
        row = host_ints(f[i * slab:(i + 1) * slab])
        assert d_x[i] == o.g1_mul(G, sum(a * b for a, b in zip(row, tyz)) % M)
    rnd = random.Random(4)
    pt = [rnd.randrange(M) for _ in range(n)]
    _, d_y, c_y, f_star = kzh.kzh3_open(ctx, srs, pt, com, poly)
    r_z, r_y, r_x = pt[:zl], pt[zl:zl + yl], pt[zl + yl:]
    assert o.evaluate_multilinear_extension(f_star, r_z) == mle_at(ctx, n, f.data_ptr(), pt)
    f_prime = contract_high(ctx, n, f.data_ptr(), xl, o.evaluate_lagrange_basis(r_x))
    assert c_y == o.g1_mul(G, sum(a * b for a, b in zip(f_prime, tyz)) % M)  # c_y = MSM(h_yz, f_prime) = sum eq d_x
    for i in (0, 77, (1 << yl) - 1):
        row = f_prime[i << zl:(i + 1) << zl]
        assert d_y[i] == o.g1_mul(G, sum(a * b for a, b in zip(row, tz)) % M)
    assert o.g1_mul(G, sum(a * b for a, b in zip(f_star, tz)) % M) == o.g1_msm(d_y, o.evaluate_lagrange_basis(r_y))
    srs.close()
    del f
    torch.cuda.empty_cache()


def test_kzh3_mix_reduced(ctx):
    """The int16 / full-width mix at n = 22 (8, 7, 7)."""
    run_kzh3_mix(ctx, 22)


def test_kzh3_mix_full_size(ctx):
    """n = 28 on the 2^10 x 2^9 x 2^9 split: 8 GiB of evaluations against a 16 GiB h_xyz; the commitment's
    MSM makes about 2.3 * 10^9 digit entries, the size at which 32-bit entry counts and offsets are closest
    to their limit."""
    run_kzh3_mix(ctx, 28)
