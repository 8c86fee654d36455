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
