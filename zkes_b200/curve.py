"""Host-side helpers for G1 points in the library's wire form and thin wrappers over the MSM
entry points (the PairingG1 seam of src/crypto/polycommit/mod.rs:72-92)."""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import numpy as np

from ._lib import ZK_MEM_HOST, check, lib
from .field import Q_MOD, from_mont_array, to_mont_array


def affine_to_array(points) -> np.ndarray:
    """[(x, y) | None] -> (n, 8) uint64 (Montgomery mod q; infinity = zeros)."""
    flat = []
    for p in points:
        flat += [0, 0] if p is None else [p[0], p[1]]
    return to_mont_array(flat, Q_MOD).reshape(-1, 8) if flat else np.zeros((0, 8), dtype=np.uint64)


def affine_from_array(arr):
    vals = from_mont_array(np.asarray(arr).reshape(-1, 4), Q_MOD)
    out = []
    for i in range(0, len(vals), 2):
        out.append(None if vals[i] == 0 and vals[i + 1] == 0 else (vals[i], vals[i + 1]))
    return out


def jacobian_to_affine_py(arr):
    """(n, 12) uint64 Jacobian rows -> affine tuples, normalised with Python integers."""
    vals = from_mont_array(np.asarray(arr).reshape(-1, 4), Q_MOD)
    out = []
    for i in range(0, len(vals), 3):
        x, y, z = vals[i:i + 3]
        if z == 0:
            out.append(None)
            continue
        zi = pow(z, -1, Q_MOD)
        out.append((x * zi * zi % Q_MOD, y * zi * zi * zi % Q_MOD))
    return out


def _p(a):
    return c_void_p(a.ctypes.data)


def msm(ctx, bases_arr: np.ndarray, scalars):
    """P::G1::msm(bases, scalars) -> affine tuple (or None)."""
    n = len(scalars)
    if bases_arr.shape[0] != n:
        raise ValueError(f"MSM: bases and scalars must have the same length, got {bases_arr.shape[0]} and {n}")
    sc = to_mont_array(scalars) if n else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1, 12), dtype=np.uint64)
    check(lib.zk_msm_g1(ctx.handle, _p(bases_arr), ZK_MEM_HOST, _p(sc), ZK_MEM_HOST, n, _p(out), ZK_MEM_HOST), "zk_msm_g1")
    return jacobian_to_affine_py(out)[0]


def msm_batched(ctx, bases_arr: np.ndarray, scalar_rows):
    rows = len(scalar_rows)
    n = bases_arr.shape[0]
    flat = [v for r in scalar_rows for v in r]
    assert len(flat) == rows * n
    sc = to_mont_array(flat) if flat else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((max(rows, 1), 12), dtype=np.uint64)
    check(lib.zk_msm_g1_batched(ctx.handle, _p(bases_arr), ZK_MEM_HOST, n, _p(sc), ZK_MEM_HOST, rows, _p(out), ZK_MEM_HOST),
          "zk_msm_g1_batched")
    return jacobian_to_affine_py(out[:rows])


def sparse_msm(ctx, all_bases_arr: np.ndarray, indices, scalars):
    """sparse_msm(all_bases, indices, scalars), src/crypto/polycommit/mod.rs:10-31."""
    if len(indices) != len(scalars):
        raise ValueError(f"Sparse MSM: indices and scalars must have the same length, got {len(indices)} and {len(scalars)}")
    k = len(indices)
    ia = np.array(list(indices) or [0], dtype=np.uint64)
    sc = to_mont_array(scalars) if k else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1, 12), dtype=np.uint64)
    check(lib.zk_msm_g1_gather(ctx.handle, _p(all_bases_arr), ZK_MEM_HOST, all_bases_arr.shape[0], _p(ia), _p(sc), ZK_MEM_HOST,
                               k, _p(out), ZK_MEM_HOST), "zk_msm_g1_gather")
    return jacobian_to_affine_py(out)[0]


def normalize(ctx, jac_arr: np.ndarray):
    n = jac_arr.shape[0]
    out = np.zeros((max(n, 1), 8), dtype=np.uint64)
    check(lib.zk_g1_normalize(ctx.handle, _p(jac_arr), ZK_MEM_HOST, n, _p(out), ZK_MEM_HOST), "zk_g1_normalize")
    return affine_from_array(out[:n])


def serialize_compressed(ctx, points) -> bytes:
    """ark-serialize compressed encoding of affine points ([(x, y) | None]), 32 bytes each."""
    arr = affine_to_array(points)
    out = np.zeros(max(len(points), 1) * 32, dtype=np.uint8)
    check(lib.zk_g1_compress(ctx.handle, _p(arr) if len(points) else None, ZK_MEM_HOST, len(points), _p(out), ZK_MEM_HOST),
          "zk_g1_compress")
    return out[:32 * len(points)].tobytes()


def deserialize_compressed(ctx, data: bytes):
    """Inverse of serialize_compressed; raises ZkError for an invalid encoding."""
    assert len(data) % 32 == 0
    n = len(data) // 32
    src = np.frombuffer(data, dtype=np.uint8).copy() if n else np.zeros(32, dtype=np.uint8)
    out = np.zeros((max(n, 1), 8), dtype=np.uint64)
    check(lib.zk_g1_decompress(ctx.handle, _p(src), ZK_MEM_HOST, n, _p(out), ZK_MEM_HOST), "zk_g1_decompress")
    return affine_from_array(out[:n])


def last_stats(ctx):
    w, k, mb = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    e, b = ctypes.c_uint64(), ctypes.c_uint64()
    check(lib.zk_msm_last_stats(ctx.handle, ctypes.byref(w), ctypes.byref(k), ctypes.byref(mb), ctypes.byref(e), ctypes.byref(b)),
          "zk_msm_last_stats")
    return {"window_bits": w.value, "windows": k.value, "max_bits": mb.value, "entries": e.value, "buckets": b.value}
