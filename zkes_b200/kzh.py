"""Host-side mirror of the KZH2 / KZH3 commitment interface (src/crypto/polycommit/kzh2.rs,
kzh3.rs), G1 side: setup from trapdoors, commit, open.  Pairing checks stay with the caller."""
from __future__ import annotations

import ctypes
from ctypes import c_uint32, c_void_p

import numpy as np

from . import curve
from ._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
from .field import from_mont_array, to_mont_array


def _p(a):
    return c_void_p(a.ctypes.data)


class KZHSRS:
    """KZH2SRS (kzh2.rs:27-35) / KZH3SRS (kzh3.rs:33-45), resident on the device."""

    def __init__(self, ctx, dims: int, n: int, handle):
        self.ctx, self.dims, self.n, self.handle = ctx, dims, n, handle
        x, y, z = c_uint32(), c_uint32(), c_uint32()
        check(lib.zk_kzh_srs_shape(handle, ctypes.byref(x), ctypes.byref(y), ctypes.byref(z)), "zk_kzh_srs_shape")
        self.x_log, self.y_log, self.z_log = x.value, y.value, z.value

    @classmethod
    def setup(cls, ctx, dims: int, n: int, g, tau_x, tau_y, tau_z=None, alpha=None):
        """setup_kzh2_srs (kzh2.rs:502-555) / setup_kzh3_srs (kzh3.rs:463-563) from sampled trapdoors."""
        h = c_void_p()
        ga = curve.affine_to_array([g])
        tx, ty = to_mont_array(tau_x), to_mont_array(tau_y)
        tz = to_mont_array(tau_z) if tau_z is not None else None
        al = to_mont_array([alpha]) if alpha is not None else None
        check(lib.zk_kzh_srs_setup(ctx.handle, dims, n, _p(ga), _p(tx), _p(ty), _p(tz) if tz is not None else None,
                                   _p(al) if al is not None else None, ctypes.byref(h)), "zk_kzh_srs_setup")
        return cls(ctx, dims, n, h)

    @classmethod
    def upload(cls, ctx, dims: int, n: int, h_full, h_mid, h_low=None):
        h = c_void_p()
        a, b = curve.affine_to_array(h_full), curve.affine_to_array(h_mid)
        c = curve.affine_to_array(h_low) if h_low is not None else None
        check(lib.zk_kzh_srs_upload(ctx.handle, dims, n, _p(a), _p(b), _p(c) if c is not None else None, ZK_MEM_HOST,
                                    ctypes.byref(h)), "zk_kzh_srs_upload")
        return cls(ctx, dims, n, h)

    def read(self, which: int, offset: int, count: int):
        out = np.zeros((max(count, 1), 8), dtype=np.uint64)
        check(lib.zk_kzh_srs_read(self.ctx.handle, self.handle, which, offset, count, _p(out)), "zk_kzh_srs_read")
        return curve.affine_from_array(out[:count])

    def close(self):
        if self.handle:
            lib.zk_kzh_srs_free(self.ctx.handle, self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KZHCommitment:
    """KZH2Commitment / KZH3Commitment: affine c and aux.d_x (projective), kzh2.rs:103-107."""

    def __init__(self, srs, c, d_x_jac):
        self.srs, self.c, self.d_x_jac = srs, c, d_x_jac

    @property
    def d_x(self):
        return curve.jacobian_to_affine_py(self.d_x_jac)

    def to_transcript_bytes(self, ctx) -> bytes:
        """Commitment::to_transcript_bytes: the compressed c for KZH3 (kzh3.rs:406-411), nothing for KZH2
        (the trait's default, polycommit/mod.rs:408-412)."""
        return curve.serialize_compressed(ctx, [self.c]) if self.srs.dims == 3 else b""


def _evals_arg(poly):
    if poly.device_ptr is not None:
        return c_void_p(poly.device_ptr), ZK_MEM_DEVICE
    return _p(poly.mont), ZK_MEM_HOST


def commit(ctx, srs: KZHSRS, poly) -> KZHCommitment:
    """kzh2_commit (kzh2.rs:619-673) / kzh3_commit (kzh3.rs:645-700)."""
    c = np.zeros((1, 8), dtype=np.uint64)
    dx = np.zeros((1 << srs.x_log, 12), dtype=np.uint64)
    ptr, mem = _evals_arg(poly)
    check(lib.zk_kzh_commit(ctx.handle, srs.handle, poly.n, ptr, mem, _p(c), _p(dx)), "zk_kzh_commit")
    return KZHCommitment(srs, curve.affine_from_array(c)[0], dx)


def kzh2_open(ctx, srs: KZHSRS, point, com: KZHCommitment, poly):
    """kzh2_open (kzh2.rs:676-710) -> (d_x, f_star)."""
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << srs.y_log, 4), dtype=np.uint64)
    ptr, mem = _evals_arg(poly)
    check(lib.zk_kzh2_open(ctx.handle, srs.handle, poly.n, ptr, mem, _p(pt), len(point), _p(out)), "zk_kzh2_open")
    return com.d_x, from_mont_array(out)


def kzh3_open(ctx, srs: KZHSRS, point, com: KZHCommitment, poly):
    """kzh3_open (kzh3.rs:702-787) -> (d_x, d_y, c_y, f_star)."""
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    dy = np.zeros((1 << srs.y_log, 12), dtype=np.uint64)
    cy = np.zeros((1, 8), dtype=np.uint64)
    fs = np.zeros((1 << srs.z_log, 4), dtype=np.uint64)
    ptr, mem = _evals_arg(poly)
    check(lib.zk_kzh3_open(ctx.handle, srs.handle, poly.n, ptr, mem, _p(pt), len(point), _p(com.d_x_jac), _p(dy), _p(cy),
                           _p(fs)), "zk_kzh3_open")
    return com.d_x, curve.jacobian_to_affine_py(dy), curve.affine_from_array(cy)[0], from_mont_array(fs)


def _jac_array(points_or_jac):
    """(len, 12) Jacobian array from either such an array or a list of affine points (None = infinity)."""
    if isinstance(points_or_jac, np.ndarray):
        return points_or_jac
    out = np.zeros((max(len(points_or_jac), 1), 12), dtype=np.uint64)
    aff = curve.affine_to_array(points_or_jac)
    one = to_mont_array([1], curve.Q_MOD)[0]
    for i, p in enumerate(points_or_jac):
        if p is None:      # infinity: z = 0 (x = y = 1 as to_jacobian writes it)
            out[i, 0:4] = one
            out[i, 4:8] = one
            continue
        out[i, :8] = aff[i]
        out[i, 8:] = one
    return out


def verify_g1(ctx, srs: KZHSRS, point, output: int, d_x, f_star, d_y=None, c_y=None):
    """The G1 / field part of kzh2_verify (kzh2.rs:763-789) and kzh3_verify (kzh3.rs:836-886): returns
    (ok, number of the first failing check in the reference's numbering, 0 if none).  Pairing checks are the caller's."""
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    outp = to_mont_array([output])
    dx = _jac_array(d_x)
    dy = _jac_array(d_y) if d_y is not None else None
    cy = curve.affine_to_array([c_y]) if srs.dims == 3 else None
    fs = to_mont_array(f_star)
    ok, failed = ctypes.c_int(0), ctypes.c_int(0)
    check(lib.zk_kzh_verify_g1(ctx.handle, srs.handle, _p(pt), len(point), _p(outp), _p(dx), _p(dy) if dy is not None else None,
                               _p(cy) if cy is not None else None, _p(fs), ctypes.byref(ok), ctypes.byref(failed)),
          "zk_kzh_verify_g1")
    return bool(ok.value), failed.value


def sparse_commit(ctx, srs: KZHSRS, evaluations: dict) -> KZHCommitment:
    """sparse_kzh2_commit (sparse_kzh2.rs:14-82) / sparse_kzh3_commit (sparse_kzh3.rs:32-110);
    evaluations: {index: value} as SparseMLPoly.evaluations."""
    idx = np.array(list(evaluations.keys()) or [0], dtype=np.uint64)
    vals = to_mont_array(list(evaluations.values())) if evaluations else np.zeros((1, 4), dtype=np.uint64)
    c = np.zeros((1, 8), dtype=np.uint64)
    dx = np.zeros((1 << srs.x_log, 12), dtype=np.uint64)
    check(lib.zk_sparse_kzh_commit(ctx.handle, srs.handle, len(evaluations), _p(idx), _p(vals), _p(c), _p(dx)),
          "zk_sparse_kzh_commit")
    return KZHCommitment(srs, curve.affine_from_array(c)[0], dx)


def sparse_kzh2_open(ctx, srs: KZHSRS, point, com: KZHCommitment, evaluations: dict):
    idx = np.array(list(evaluations.keys()) or [0], dtype=np.uint64)
    vals = to_mont_array(list(evaluations.values())) if evaluations else np.zeros((1, 4), dtype=np.uint64)
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << srs.y_log, 4), dtype=np.uint64)
    check(lib.zk_sparse_kzh2_open(ctx.handle, srs.handle, len(evaluations), _p(idx), _p(vals), _p(pt), len(point), _p(out)),
          "zk_sparse_kzh2_open")
    return com.d_x, from_mont_array(out)


def sparse_kzh3_open(ctx, srs: KZHSRS, point, com: KZHCommitment, evaluations: dict):
    idx = np.array(list(evaluations.keys()) or [0], dtype=np.uint64)
    vals = to_mont_array(list(evaluations.values())) if evaluations else np.zeros((1, 4), dtype=np.uint64)
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    dy = np.zeros((1 << srs.y_log, 12), dtype=np.uint64)
    cy = np.zeros((1, 8), dtype=np.uint64)
    fs = np.zeros((1 << srs.z_log, 4), dtype=np.uint64)
    check(lib.zk_sparse_kzh3_open(ctx.handle, srs.handle, len(evaluations), _p(idx), _p(vals), _p(pt), len(point),
                                  _p(com.d_x_jac), _p(dy), _p(cy), _p(fs)), "zk_sparse_kzh3_open")
    return com.d_x, curve.jacobian_to_affine_py(dy), curve.affine_from_array(cy)[0], from_mont_array(fs)


# ---- file formats (zkes_b200/wire.py): `{n}.srs` and bincode openings, with the points coded on the device
def store_kzh3_srs(ctx, srs: KZHSRS, path, v_x: bytes = b"", v_y: bytes = b"", v_z: bytes = b"", v: bytes = bytes(64)):
    """store_kzh3_srs (src/crypto/srs_storage.rs:15-35): the G1 vectors of the device-resident SRS in compressed form;
    the G2 vectors (64-byte compressed points, kept by the caller: the verifier side is not on the device) pass through."""
    from . import wire
    assert srs.dims == 3
    blobs = []
    for which, count in ((0, 1 << srs.n), (1, 1 << (srs.y_log + srs.z_log)), (2, 1 << srs.z_log)):
        pts = np.zeros((count, 8), dtype=np.uint64)
        check(lib.zk_kzh_srs_read(ctx.handle, srs.handle, which, 0, count, _p(pts)), "zk_kzh_srs_read")
        out = np.zeros(count * 32, dtype=np.uint8)
        check(lib.zk_g1_compress(ctx.handle, _p(pts), ZK_MEM_HOST, count, _p(out), ZK_MEM_HOST), "zk_g1_compress")
        blobs.append(out.tobytes())
    with open(path, "wb") as f:
        wire.write_kzh3_srs(f, (1 << srs.x_log, 1 << srs.y_log, 1 << srs.z_log), blobs[0], blobs[1], blobs[2], v_x, v_y, v_z, v)


def load_kzh3_srs(ctx, path, n: int):
    """load_kzh3_srs (srs_storage.rs:39-58) -> (device SRS, {"v_x", "v_y", "v_z", "v"}: the G2 part as stored)."""
    from . import wire
    with open(path, "rb") as f:
        d = wire.read_kzh3_srs(f)
    arrays = []
    for name in ("h_xyz", "h_yz", "h_z"):
        count = len(d[name]) // 32
        src = np.frombuffer(d[name], dtype=np.uint8).copy()
        pts = np.zeros((count, 8), dtype=np.uint64)
        check(lib.zk_g1_decompress(ctx.handle, _p(src), ZK_MEM_HOST, count, _p(pts), ZK_MEM_HOST), "zk_g1_decompress")
        arrays.append(pts)
    h = c_void_p()
    check(lib.zk_kzh_srs_upload(ctx.handle, 3, n, _p(arrays[0]), _p(arrays[1]), _p(arrays[2]), ZK_MEM_HOST, ctypes.byref(h)),
          "zk_kzh_srs_upload")
    srs = KZHSRS(ctx, 3, n, h)
    if d["degrees"] != (1 << srs.x_log, 1 << srs.y_log, 1 << srs.z_log):
        srs.close()
        raise ValueError(f"the file holds degrees {d['degrees']}, not those of {n} variables")
    return srs, {k: d[k] for k in ("v_x", "v_y", "v_z", "v")}


def kzh3_opening_to_bincode(ctx, d_x_jac: np.ndarray, d_y_jac: np.ndarray, c_y, f_star) -> bytes:
    """The bincode form of KZH3Opening (kzh3.rs:104-117, util/serialization.rs:91-98): projective points are written
    in compressed affine form, as ark-serialize does for a Projective."""
    from . import wire
    blobs = []
    for jac in (d_x_jac, d_y_jac):
        n = jac.shape[0]
        aff = np.zeros((n, 8), dtype=np.uint64)
        check(lib.zk_g1_normalize(ctx.handle, _p(jac), ZK_MEM_HOST, n, _p(aff), ZK_MEM_HOST), "zk_g1_normalize")
        out = np.zeros(n * 32, dtype=np.uint8)
        check(lib.zk_g1_compress(ctx.handle, _p(aff), ZK_MEM_HOST, n, _p(out), ZK_MEM_HOST), "zk_g1_compress")
        blobs.append(out.tobytes())
    return wire.kzh3_opening_to_bincode(blobs[0], blobs[1], curve.serialize_compressed(ctx, [c_y]),
                                        len(f_star).bit_length() - 1, f_star)
