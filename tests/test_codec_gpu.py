"""arkworks' compressed G1 encoding on the device against the oracle (serialize_compressed as used by
src/crypto/polycommit/kzh3.rs:406-411 and src/crypto/srs_storage.rs:15-58)."""
import random

import pytest

import pyoracle as o
from zkes_b200 import curve
from zkes_b200._lib import ZkError

pytestmark = pytest.mark.gpu
G = (1, 2)


def test_known_encodings(ctx):
    assert curve.serialize_compressed(ctx, [G]) == bytes([1]) + bytes(31)
    assert curve.serialize_compressed(ctx, [(1, o.Q_MOD - 2)]) == bytes([1]) + bytes(30) + bytes([0x80])
    assert curve.serialize_compressed(ctx, [None]) == bytes(31) + bytes([0x40])
    assert curve.serialize_compressed(ctx, []) == b""
    assert curve.deserialize_compressed(ctx, bytes([1]) + bytes(31)) == [G]
    assert curve.deserialize_compressed(ctx, bytes(31) + bytes([0x40])) == [None]


@pytest.mark.parametrize("count", [1, 33, 1000])
def test_round_trip_matches_oracle(ctx, count):
    rnd = random.Random(count)
    pts = [None if rnd.random() < 0.05 else o.g1_mul(G, rnd.randrange(1, o.R_MOD)) for _ in range(count)]
    data = curve.serialize_compressed(ctx, pts)
    assert data == b"".join(o.g1_serialize_compressed(p) for p in pts)
    assert curve.deserialize_compressed(ctx, data) == pts
    assert [o.g1_deserialize_compressed(data[32 * i:32 * i + 32]) for i in range(min(count, 40))] == pts[:40]


def test_rejects_invalid_encodings(ctx):
    good = o.g1_serialize_compressed(G)
    # x with no point above it: x^3 + 3 a non-residue
    x = 2
    while pow((x ** 3 + 3) % o.Q_MOD, (o.Q_MOD - 1) // 2, o.Q_MOD) == 1:
        x += 1
    cases = [x.to_bytes(32, "little"),                                   # not on the curve
             (o.Q_MOD + 1).to_bytes(32, "little"),                       # x >= q (x = 1 mod q is otherwise fine)
             bytes(31) + bytes([0xC0]),                                   # infinity with the sign flag
             bytes([1]) + bytes(30) + bytes([0x40])]                      # infinity with a non-zero x
    for bad in cases:
        with pytest.raises(ZkError):
            curve.deserialize_compressed(ctx, good + bad)
        with pytest.raises(ValueError):
            o.g1_deserialize_compressed(bad)


def test_commitment_transcript_bytes(ctx):
    """KZH3 commitments bind to the transcript by their compressed c (kzh3.rs:406-411), KZH2 ones by nothing."""
    from zkes_b200 import DenseMLPoly, kzh
    rnd = random.Random(77)
    d = o.gen_uniform_fr(9, 0, 0, 32)
    srs3 = kzh.KZHSRS.setup(ctx, 3, 3, o.g1_mul(G, d[0]), d[1:3], d[3:5], tau_z=d[5:7])
    srs2 = kzh.KZHSRS.setup(ctx, 2, 2, o.g1_mul(G, d[0]), d[1:3], d[3:5], alpha=d[5])
    f = [rnd.randrange(o.R_MOD) for _ in range(8)]
    c3 = kzh.commit(ctx, srs3, DenseMLPoly.from_evaluations(f))
    c2 = kzh.commit(ctx, srs2, DenseMLPoly.from_evaluations(f[:4]))
    assert c3.to_transcript_bytes(ctx) == o.g1_serialize_compressed(c3.c)
    assert c2.to_transcript_bytes(ctx) == b""


def test_srs_file_and_opening_round_trip(ctx, tmp_path):
    """`{n}.srs` written from a device SRS and read back gives the same G1 vectors (and hands the G2 part through);
    a KZH3 opening survives its bincode form, and its point bytes are the compressed encoding the oracle gives."""
    import random

    import pyoracle as o
    from zkes_b200 import DenseMLPoly, curve, kzh, wire

    rnd = random.Random(8)
    n = 7
    xl, yl, zl = o.kzh3_degrees(n)
    tx, ty, tz = ([rnd.randrange(1, o.R_MOD) for _ in range(1 << lg)] for lg in (xl, yl, zl))
    srs = kzh.KZHSRS.setup(ctx, 3, n, o.g1_mul(o.G1_GEN, 5), tx, ty, tau_z=tz)
    g2 = {k: bytes(rnd.randrange(256) for _ in range(64 * c)) for k, c in (("v_x", 1 << xl), ("v_y", 1 << yl), ("v_z", 1 << zl), ("v", 1))}
    path = tmp_path / wire.srs_file_name(n)
    kzh.store_kzh3_srs(ctx, srs, path, g2["v_x"], g2["v_y"], g2["v_z"], g2["v"])
    loaded, g2_back = kzh.load_kzh3_srs(ctx, path, n)
    assert g2_back == g2
    for which, count in ((0, 1 << n), (1, 1 << (yl + zl)), (2, 1 << zl)):
        assert loaded.read(which, 0, count) == srs.read(which, 0, count)
    with open(path, "rb") as f:
        raw = wire.read_kzh3_srs(f)
    osrs = o.KZH3SRS(n, 5, tx, ty, tz)
    assert raw["h_z"] == b"".join(o.g1_serialize_compressed(p) for p in osrs.h_z)
    with pytest.raises(ValueError):
        kzh.load_kzh3_srs(ctx, path, n + 1)
    # an opening through bincode and back
    poly = DenseMLPoly.from_evaluations([rnd.randrange(o.R_MOD) for _ in range(1 << n)])
    com = kzh.commit(ctx, loaded, poly)
    pt = [rnd.randrange(o.R_MOD) for _ in range(n)]
    d_x, d_y, c_y, f_star = kzh.kzh3_open(ctx, loaded, pt, com, poly)
    dy_jac = curve.affine_to_array(d_y)
    jac = lambda pts: kzh._jac_array(pts)  # noqa: E731
    data = kzh.kzh3_opening_to_bincode(ctx, com.d_x_jac, jac(d_y), c_y, f_star)
    bx, by, bc, fn, fe = wire.kzh3_opening_from_bincode(data)
    assert curve.deserialize_compressed(ctx, bx) == d_x and curve.deserialize_compressed(ctx, by) == d_y
    assert curve.deserialize_compressed(ctx, bc) == [c_y] and (fn, fe) == (zl, f_star)
    assert bc == o.g1_serialize_compressed(c_y)
    del dy_jac
    srs.close()
    loaded.close()
