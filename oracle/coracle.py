"""ctypes wrapper of oracle/liboracle.so (TEST INFRASTRUCTURE ONLY; see pyoracle.py for the
rules on who may import this).  Values cross as Python ints in canonical form."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_char_p, c_int, c_uint32, c_uint64, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")
R_MOD = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001
_R = 1 << 256
_RINV = pow(_R, -1, R_MOD)
_M64 = (1 << 64) - 1


def build():
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return LIB_PATH


def _load():
    if not os.path.exists(LIB_PATH):
        build()
    return ctypes.CDLL(LIB_PATH)


lib = _load()


def mont(values, mod=R_MOD) -> np.ndarray:
    out = np.empty((max(len(values), 1), 4), dtype=np.uint64)
    for i, v in enumerate(values):
        m = (int(v) % mod) * _R % mod
        for k in range(4):
            out[i, k] = (m >> (64 * k)) & _M64
    return out


def unmont(arr, mod=R_MOD):
    rinv = _RINV if mod == R_MOD else pow(_R, -1, mod)
    a = np.asarray(arr, dtype=np.uint64).reshape(-1, 4)
    return [((int(r[0]) | int(r[1]) << 64 | int(r[2]) << 128 | int(r[3]) << 192) * rinv) % mod for r in a]


def _p(a):
    return c_void_p(a.ctypes.data)


def set_threads(t: int):
    lib.orc_set_threads(c_int(t))


class CProof:
    def __init__(self, msgs, chal, fin_t, fin, tail):
        self.round_messages, self.challenges, self.final_tables, self.final_eval, self.tail = msgs, chal, fin_t, fin, tail


def linear_prove_mont(label: bytes, n: int, tables_mont):
    """tables_mont: list of (2^n, 4) uint64 arrays already in wire form."""
    L = len(tables_mont)
    ptrs = (c_void_p * L)(*[_p(t) for t in tables_mont])
    msgs = np.zeros((max(n, 1) * (L + 1), 4), dtype=np.uint64)
    chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
    fin_t = np.zeros((L, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    tail = np.zeros((1, 4), dtype=np.uint64)
    lib.orc_linear_prove(c_char_p(label), c_uint32(n), c_uint32(L), ptrs, _p(msgs), _p(chal), _p(fin_t), _p(fin), _p(tail))
    m = unmont(msgs[: n * (L + 1)]) if n else []
    return CProof([m[r * (L + 1):(r + 1) * (L + 1)] for r in range(n)], unmont(chal[:n]) if n else [], unmont(fin_t),
                  unmont(fin)[0], unmont(tail)[0])


def linear_prove(label: bytes, tables):
    n = len(tables[0]).bit_length() - 1
    return linear_prove_mont(label, n, [mont(t) for t in tables])


def sparse_dense_prove_mont(label: bytes, n: int, idx: np.ndarray, vals_mont: np.ndarray, dense_mont: np.ndarray):
    nnz = int(idx.shape[0])
    idx = np.ascontiguousarray(idx, dtype=np.uint64)
    msgs = np.zeros((max(n, 1) * 3, 4), dtype=np.uint64)
    chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
    fin_t = np.zeros((2, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    tail = np.zeros((1, 4), dtype=np.uint64)
    lib.orc_sparse_dense_prove(c_char_p(label), c_uint32(n), c_uint64(nnz), _p(idx), _p(vals_mont), _p(dense_mont),
                               _p(msgs), _p(chal), _p(fin_t), _p(fin), _p(tail))
    m = unmont(msgs[: n * 3]) if n else []
    return CProof([m[r * 3:(r + 1) * 3] for r in range(n)], unmont(chal[:n]) if n else [], unmont(fin_t),
                  unmont(fin)[0], unmont(tail)[0])


def sparse_bool_prove(label: bytes, n: int, weights, positions, eq_point):
    flat = np.array([p for pos in positions for p in pos] or [0], dtype=np.uint64)
    cnt = np.array([len(p) for p in positions], dtype=np.uint64)
    msgs = np.zeros((max(n, 1) * 4, 4), dtype=np.uint64)
    chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    tail = np.zeros((1, 4), dtype=np.uint64)
    wm, pm = mont(weights), mont(eq_point)  # keep the arrays alive across the call
    lib.orc_sparse_bool_prove(c_char_p(label), c_uint32(n), c_uint32(len(weights)), _p(wm), _p(flat), _p(cnt),
                              _p(pm), _p(msgs), _p(chal), _p(fin), _p(tail))
    m = unmont(msgs[: n * 4]) if n else []
    return CProof([m[r * 4:(r + 1) * 4] for r in range(n)], unmont(chal[:n]) if n else [], None, unmont(fin)[0],
                  unmont(tail)[0])


def eq_table(point):
    out = np.zeros((1 << len(point), 4), dtype=np.uint64)
    pm = mont(point)
    lib.orc_eq_table(c_uint32(len(point)), _p(pm), _p(out))
    return unmont(out)


def fix_variables(evals, point):
    n = len(evals).bit_length() - 1
    out = np.zeros((1 << (n - len(point)), 4), dtype=np.uint64)
    em, pm = mont(evals), mont(point)
    lib.orc_fix_variables(c_uint32(n), _p(em), c_uint32(len(point)), _p(pm), _p(out))
    return unmont(out)


def fix_from_right(evals, point):
    n = len(evals).bit_length() - 1
    out = np.zeros((1 << (n - len(point)), 4), dtype=np.uint64)
    em, pm = mont(evals), mont(point)
    lib.orc_fix_from_right(c_uint32(n), _p(em), c_uint32(len(point)), _p(pm), _p(out))
    return unmont(out)


def mle_eval(evals, point):
    out = np.zeros((1, 4), dtype=np.uint64)
    em, pm = mont(evals), mont(point)
    lib.orc_mle_eval(c_uint32(len(point)), _p(em), _p(pm), _p(out))
    return unmont(out)[0]


# ---- G1 (g1.h): points cross as (n, 8) uint64 arrays {x, y} in Montgomery form mod q, zeros for infinity
Q_MOD = 0x30644E72E131A029B85045B68181585D97816A916871CA8D3C208C16D87CFD47


def affine_array(points) -> np.ndarray:
    """list of (x, y) tuples / None -> wire array."""
    flat = []
    for p in points:
        flat += [0, 0] if p is None else [p[0], p[1]]
    return mont(flat, Q_MOD).reshape(-1, 8) if points else np.zeros((0, 8), dtype=np.uint64)


def affine_tuples(arr):
    v = unmont(np.asarray(arr, dtype=np.uint64).reshape(-1, 4), Q_MOD)
    return [None if (v[2 * i] == 0 and v[2 * i + 1] == 0) else (v[2 * i], v[2 * i + 1]) for i in range(len(v) // 2)]


def g1_normalize(jac: np.ndarray):
    n = jac.reshape(-1, 12).shape[0]
    out = np.zeros((max(n, 1), 8), dtype=np.uint64)
    lib.orc_g1_normalize(c_uint64(n), _p(np.ascontiguousarray(jac)), _p(out))
    return affine_tuples(out[:n])


def g1_msm_mont(bases_arr: np.ndarray, scalars_mont: np.ndarray):
    """Bucket-method MSM over wire-form inputs on the configured threads -> affine tuple (None: infinity)."""
    n = int(bases_arr.reshape(-1, 8).shape[0])
    out = np.zeros((1, 12), dtype=np.uint64)
    lib.orc_g1_msm(c_uint64(n), _p(np.ascontiguousarray(bases_arr)), _p(np.ascontiguousarray(scalars_mont)), _p(out))
    return g1_normalize(out)[0]


def g1_msm(points, scalars):
    return g1_msm_mont(affine_array(points), mont(scalars))


def g1_msm_rows_mont(bases_arr: np.ndarray, scalars_mont: np.ndarray, n_rows: int):
    n = int(bases_arr.reshape(-1, 8).shape[0])
    out = np.zeros((max(n_rows, 1), 12), dtype=np.uint64)
    lib.orc_g1_msm_rows(c_uint64(n), c_uint64(n_rows), _p(np.ascontiguousarray(bases_arr)),
                        _p(np.ascontiguousarray(scalars_mont)), _p(out))
    return g1_normalize(out[:n_rows])


def g1_mul(point, k: int):
    out = np.zeros((1, 12), dtype=np.uint64)
    kc = np.array([(k >> (64 * i)) & _M64 for i in range(4)], dtype=np.uint64)
    b = affine_array([point])
    lib.orc_g1_mul(_p(b), _p(kc), _p(out))
    return g1_normalize(out)[0]


def gen_uniform_fr_mont(seed: int, stream: int, start: int, count: int) -> np.ndarray:
    """Element i = ChaCha20 block start+i of (seed, stream) as a 512-bit integer mod r, wire form (count, 4)."""
    out = np.empty((max(count, 1), 4), dtype=np.uint64)
    lib.orc_gen_uniform_fr(c_uint64(seed), c_uint64(stream), c_uint64(start), c_uint64(count), _p(out))
    return out[:count]


def gen_small_fr_mont(seed: int, stream: int, start: int, count: int, bits: int) -> np.ndarray:
    out = np.empty((max(count, 1), 4), dtype=np.uint64)
    lib.orc_gen_small_fr(c_uint64(seed), c_uint64(stream), c_uint64(start), c_uint64(count), c_int(bits), _p(out))
    return out[:count]
