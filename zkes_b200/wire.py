"""File formats around the hot path, on the host: the reference's `{n}.srs` files and its bincode proof files.

Both are byte layouts of third-party serialisers that are not in this tree (ark-serialize 0.5 and bincode 1.3);
they are restated from those crates' published formats and from the reference's own (de)serialisation glue:

  KZH3SRS   `store_kzh3_srs` / `load_kzh3_srs` (src/crypto/srs_storage.rs:15-58) write the derived
            `CanonicalSerialize` of the struct (src/crypto/polycommit/kzh3.rs:34-46) in compressed mode: the fields in
            declaration order; a `usize` is a little-endian u64; a `Vec<T>` is a u64 length followed by the items; a
            G1 point is 32 bytes, a G2 point 64 bytes (x little-endian, the sign / infinity flags in the top bits of
            the last byte).  G1 points are produced and consumed by the library's codec (zk_g1_compress /
            zk_g1_decompress); G2 points are outside the accelerated path and pass through here as opaque 64-byte
            strings.
  proofs    `serialize_proof` (src/util/serialization.rs:91-107) is `bincode::serialize` with the default options:
            fixed-width little-endian integers, u64 sequence lengths, struct fields in order with no framing.  Field
            elements and points go through `ark_se` / `ark_se_vec` / `se_nested_vec` (serialization.rs:14-21, 74-88;
            src/crypto/sumcheck/prover.rs:17-36), i.e. each one as a length-prefixed byte string of its compressed form.

Parity status: unpinned against arkworks / bincode (neither can be built here); the tests check the layouts against
hand-assembled byte strings and round trips.
"""
from __future__ import annotations

import io
import struct

R_MOD = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001
G1_BYTES, G2_BYTES, FR_BYTES = 32, 64, 32


def _u64(v: int) -> bytes:
    return struct.pack("<Q", v)


def _read(f, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise ValueError("unexpected end of data")
    return b


def _read_u64(f) -> int:
    return struct.unpack("<Q", _read(f, 8))[0]


def fr_to_bytes(x: int) -> bytes:
    return (x % R_MOD).to_bytes(FR_BYTES, "little")


def fr_from_bytes(b: bytes) -> int:
    v = int.from_bytes(b, "little")
    if len(b) != FR_BYTES or v >= R_MOD:
        raise ValueError("not a canonical field element")
    return v


# ----------------------------------------------------------------------------- {n}.srs
def _write_points(f, blob: bytes, item: int):
    if len(blob) % item:
        raise ValueError("point vector is not a whole number of points")
    f.write(_u64(len(blob) // item))
    f.write(blob)


def _read_points(f, item: int) -> bytes:
    return _read(f, _read_u64(f) * item)


def write_kzh3_srs(f, degrees, h_xyz: bytes, h_yz: bytes, h_z: bytes, v_x: bytes, v_y: bytes, v_z: bytes, v: bytes):
    """KZH3SRS::serialize_compressed.  degrees = (degree_x, degree_y, degree_z) as the struct holds them (element
    counts); the G1 vectors are concatenated 32-byte compressed points, the G2 vectors 64-byte ones."""
    for d in degrees:
        f.write(_u64(d))
    for blob in (h_xyz, h_yz, h_z):
        _write_points(f, blob, G1_BYTES)
    for blob in (v_x, v_y, v_z):
        _write_points(f, blob, G2_BYTES)
    if len(v) != G2_BYTES:
        raise ValueError("v is one G2 point")
    f.write(v)


def read_kzh3_srs(f) -> dict:
    out = {"degrees": tuple(_read_u64(f) for _ in range(3))}
    for name in ("h_xyz", "h_yz", "h_z"):
        out[name] = _read_points(f, G1_BYTES)
    for name in ("v_x", "v_y", "v_z"):
        out[name] = _read_points(f, G2_BYTES)
    out["v"] = _read(f, G2_BYTES)
    return out


def srs_file_name(maximum_degree: int) -> str:
    """`{maximum_degree}.srs` (srs_storage.rs:20, 45)."""
    return f"{maximum_degree}.srs"


# ----------------------------------------------------------------------------- bincode proofs
def _bytes_field(b: bytes) -> bytes:  # serialize_bytes / Vec<u8>: u64 length, raw bytes
    return _u64(len(b)) + b


def _read_bytes_field(f, expect: int) -> bytes:
    n = _read_u64(f)
    if n != expect:
        raise ValueError(f"byte string of {n} bytes where {expect} were expected")
    return _read(f, n)


def sumcheck_proof_to_bincode(final_eval: int, round_messages) -> bytes:
    """SumcheckProof { final_eval, round_messages } (prover.rs:7-14)."""
    out = [_bytes_field(fr_to_bytes(final_eval)), _u64(len(round_messages))]
    for msg in round_messages:
        out.append(_u64(len(msg)))
        out.extend(_bytes_field(fr_to_bytes(v)) for v in msg)
    return b"".join(out)


def sumcheck_proof_from_bincode(data: bytes):
    f = io.BytesIO(data)
    final_eval = fr_from_bytes(_read_bytes_field(f, FR_BYTES))
    msgs = []
    for _ in range(_read_u64(f)):
        msgs.append([fr_from_bytes(_read_bytes_field(f, FR_BYTES)) for _ in range(_read_u64(f))])
    if f.read(1):
        raise ValueError("trailing bytes")
    return final_eval, msgs


def _points_seq(blob: bytes) -> bytes:  # ark_se_vec: a sequence of length-prefixed compressed points
    if len(blob) % G1_BYTES:
        raise ValueError("point vector is not a whole number of points")
    n = len(blob) // G1_BYTES
    return _u64(n) + b"".join(_bytes_field(blob[G1_BYTES * i:G1_BYTES * (i + 1)]) for i in range(n))


def _read_points_seq(f) -> bytes:
    return b"".join(_read_bytes_field(f, G1_BYTES) for _ in range(_read_u64(f)))


def dense_poly_to_bincode(n: int, evaluations) -> bytes:
    """DenseMLPoly { n, evaluations } (util/poly.rs:762-768)."""
    return _u64(n) + _u64(len(evaluations)) + b"".join(_bytes_field(fr_to_bytes(v)) for v in evaluations)


def _read_dense_poly(f):
    n = _read_u64(f)
    return n, [fr_from_bytes(_read_bytes_field(f, FR_BYTES)) for _ in range(_read_u64(f))]


def kzh3_opening_to_bincode(d_x: bytes, d_y: bytes, c_y: bytes, f_star_n: int, f_star) -> bytes:
    """KZH3Opening { d_x, d_y, c_y, f_star } (kzh3.rs:104-117); points as compressed G1 bytes."""
    if len(c_y) != G1_BYTES:
        raise ValueError("c_y is one G1 point")
    return _points_seq(d_x) + _points_seq(d_y) + _bytes_field(c_y) + dense_poly_to_bincode(f_star_n, f_star)


def kzh3_opening_from_bincode(data: bytes):
    f = io.BytesIO(data)
    d_x, d_y = _read_points_seq(f), _read_points_seq(f)
    c_y = _read_bytes_field(f, G1_BYTES)
    n, evals = _read_dense_poly(f)
    if f.read(1):
        raise ValueError("trailing bytes")
    return d_x, d_y, c_y, n, evals
