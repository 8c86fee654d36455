"""The file formats of zkes_b200/wire.py: byte layouts against hand-assembled strings (ark-serialize's compressed
struct framing of `{n}.srs`, bincode 1.3's default encoding of the proof structs) and round trips."""
import io
import random
import struct

import pytest

from zkes_b200 import wire


def test_sumcheck_proof_layout_and_round_trip():
    msgs = [[1, 2, 3], [wire.R_MOD - 1, 0, 5]]
    data = wire.sumcheck_proof_to_bincode(7, msgs)
    # final_eval: u64 32 | 32 LE bytes; round_messages: u64 2 | (u64 3 | 3 x (u64 32 | 32 bytes)) x 2
    head = struct.pack("<Q", 32) + (7).to_bytes(32, "little") + struct.pack("<Q", 2) + struct.pack("<Q", 3)
    assert data[:len(head)] == head
    assert data[len(head):len(head) + 40] == struct.pack("<Q", 32) + (1).to_bytes(32, "little")
    assert len(data) == 40 + 8 + 2 * (8 + 3 * 40)
    assert wire.sumcheck_proof_from_bincode(data) == (7, msgs)
    with pytest.raises(ValueError):
        wire.sumcheck_proof_from_bincode(data + b"\0")
    with pytest.raises(ValueError):
        wire.sumcheck_proof_from_bincode(data[:-1])
    bad = bytearray(data)
    bad[8:40] = wire.R_MOD.to_bytes(32, "little")  # not reduced
    with pytest.raises(ValueError):
        wire.sumcheck_proof_from_bincode(bytes(bad))


def test_kzh3_opening_round_trip():
    rnd = random.Random(1)
    pts = lambda k: bytes(rnd.randrange(256) for _ in range(32 * k))  # noqa: E731
    d_x, d_y, c_y = pts(4), pts(2), pts(1)
    f_star = [rnd.randrange(wire.R_MOD) for _ in range(4)]
    data = wire.kzh3_opening_to_bincode(d_x, d_y, c_y, 2, f_star)
    assert data[:8] == struct.pack("<Q", 4) and data[8:16] == struct.pack("<Q", 32) and data[16:48] == d_x[:32]
    assert len(data) == (8 + 4 * 40) + (8 + 2 * 40) + 40 + (8 + 8 + 4 * 40)
    assert wire.kzh3_opening_from_bincode(data) == (d_x, d_y, c_y, 2, f_star)


def test_kzh3_srs_file_layout_and_round_trip():
    rnd = random.Random(2)
    blob = lambda n: bytes(rnd.randrange(256) for _ in range(n))  # noqa: E731
    h_xyz, h_yz, h_z = blob(32 * 8), blob(32 * 4), blob(32 * 2)
    v_x, v_y, v_z, v = blob(64 * 2), blob(64 * 2), blob(64 * 2), blob(64)
    f = io.BytesIO()
    wire.write_kzh3_srs(f, (2, 2, 2), h_xyz, h_yz, h_z, v_x, v_y, v_z, v)
    data = f.getvalue()
    assert data[:24] == struct.pack("<QQQ", 2, 2, 2)
    assert data[24:32] == struct.pack("<Q", 8) and data[32:32 + 256] == h_xyz
    assert len(data) == 24 + (8 + 256) + (8 + 128) + (8 + 64) + 3 * (8 + 128) + 64
    got = wire.read_kzh3_srs(io.BytesIO(data))
    assert got == {"degrees": (2, 2, 2), "h_xyz": h_xyz, "h_yz": h_yz, "h_z": h_z, "v_x": v_x, "v_y": v_y, "v_z": v_z, "v": v}
    with pytest.raises(ValueError):
        wire.read_kzh3_srs(io.BytesIO(data[:-3]))
    assert wire.srs_file_name(20) == "20.srs"
