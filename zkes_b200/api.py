"""Host-side mirror of the reference's interface for the proving hot path.

Class and method names follow the Rust crate (src/crypto/sumcheck, src/util/poly.rs,
src/util/transcript.rs) so tests read like the reference's own.  Every method forwards to the
C ABI in libzkb200.so; nothing here computes field arithmetic on the proving path."""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import numpy as np

from . import _lib
from ._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
from .field import from_mont_array, to_mont_array


def _ptr(a: np.ndarray) -> c_void_p:
    return c_void_p(a.ctypes.data)


class Context:
    """One per GPU: stream and scratch (zk_init / zk_free)."""

    def __init__(self, device: int = 0):
        h = c_void_p()
        check(lib.zk_init(device, ctypes.byref(h)), "zk_init")
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            lib.zk_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def launch_count(self) -> int:
        return int(lib.zk_launch_count(self.handle))

    def set_option(self, option: int, value: int):
        check(lib.zk_set_option(self.handle, option, value), "zk_set_option")

    def sync(self):
        check(lib.zk_device_sync(self.handle), "zk_device_sync")


class Transcript:
    """src/util/transcript.rs:13-46."""

    def __init__(self, label: bytes, _handle=None):
        self.handle = _handle if _handle is not None else lib.zk_transcript_new(label, len(label))

    def clone(self) -> "Transcript":
        return Transcript(b"", _handle=lib.zk_transcript_clone(self.handle))

    def __del__(self):
        if getattr(self, "handle", None):
            lib.zk_transcript_free(self.handle)
            self.handle = None

    def append_message(self, label: bytes, message: bytes):
        lib.zk_transcript_append_message(self.handle, label, len(label), message, len(message))

    def append_u64(self, label: bytes, value: int):
        lib.zk_transcript_append_u64(self.handle, label, len(label), value)

    def append_scalar(self, label: bytes, scalar: int):
        a = to_mont_array([scalar])
        lib.zk_transcript_append_scalar(self.handle, label, len(label), _ptr(a))

    def append_scalars(self, label: bytes, scalars):
        for s in scalars:
            self.append_scalar(label, s)

    def challenge_bytes(self, label: bytes, n: int) -> bytes:
        buf = ctypes.create_string_buffer(n)
        lib.zk_transcript_challenge_bytes(self.handle, label, len(label), buf, n)
        return buf.raw

    def challenge_scalar(self, label: bytes) -> int:
        out = np.zeros((1, 4), dtype=np.uint64)
        lib.zk_transcript_challenge_scalar(self.handle, label, len(label), _ptr(out))
        return from_mont_array(out)[0]

    def challenge_vector(self, label: bytes, n: int):
        return [self.challenge_scalar(label) for _ in range(n)]


class DenseMLPoly:
    """src/util/poly.rs:764-960.  Evaluations are held as Montgomery limbs, on the host
    (numpy (2^n, 4) uint64) or on the device (a raw device pointer plus length)."""

    def __init__(self, n: int, evaluations=None, *, mont: np.ndarray = None, device_ptr: int = None):
        self.n = n
        self.device_ptr = device_ptr
        if device_ptr is not None:
            self.mont = None
        elif mont is not None:
            self.mont = np.ascontiguousarray(mont, dtype=np.uint64).reshape(-1, 4)
        else:
            self.mont = to_mont_array(evaluations)

    @classmethod
    def from_evaluations(cls, evaluations):
        n = len(evaluations).bit_length() - 1
        assert 1 << n == len(evaluations), "Vector length must be a power of 2"
        return cls(n, evaluations)

    def __len__(self):
        return 1 << self.n if self.device_ptr is not None else self.mont.shape[0]

    @property
    def evaluations(self):
        return from_mont_array(self.mont)

    def evaluate_at_point(self, ctx: Context, point) -> int:
        """src/util/poly.rs:788-791 (evaluate_multilinear_extension, :622-652)."""
        assert len(point) == self.n, "invalid size of point"
        pt = to_mont_array(point) if self.n else np.zeros((1, 4), dtype=np.uint64)
        out = np.zeros((1, 4), dtype=np.uint64)
        src = c_void_p(self.device_ptr) if self.device_ptr is not None else _ptr(self.mont)
        mem = ZK_MEM_DEVICE if self.device_ptr is not None else ZK_MEM_HOST
        check(lib.zk_mle_eval(ctx.handle, self.n, src, mem, _ptr(pt), _ptr(out)), "zk_mle_eval")
        return from_mont_array(out)[0]

    def fix_variables(self, ctx: Context, partial_point) -> "DenseMLPoly":
        assert len(partial_point) <= self.n, "invalid size of partial point"
        k = len(partial_point)
        pt = to_mont_array(partial_point) if k else np.zeros((1, 4), dtype=np.uint64)
        out = np.zeros((1 << (self.n - k), 4), dtype=np.uint64)
        src = c_void_p(self.device_ptr) if self.device_ptr is not None else _ptr(self.mont)
        mem = ZK_MEM_DEVICE if self.device_ptr is not None else ZK_MEM_HOST
        check(lib.zk_fold_lsb(ctx.handle, self.n, src, mem, k, _ptr(pt), _ptr(out), ZK_MEM_HOST), "zk_fold_lsb")
        return DenseMLPoly(self.n - k, mont=out)


def evaluate_lagrange_basis(ctx: Context, r):
    """src/util/poly.rs:573-618 (and precompute_eq, :657-699)."""
    k = len(r)
    pt = to_mont_array(r) if k else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << k, 4), dtype=np.uint64)
    check(lib.zk_eq_table(ctx.handle, k, _ptr(pt), _ptr(out), ZK_MEM_HOST), "zk_eq_table")
    return from_mont_array(out)


def fix_variables_from_right(ctx: Context, poly: "DenseMLPoly", fixed_vars) -> "DenseMLPoly":
    """src/util/poly.rs:705-758."""
    assert len(fixed_vars) <= poly.n, "invalid size of partial point"
    k = len(fixed_vars)
    pt = to_mont_array(fixed_vars) if k else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << (poly.n - k), 4), dtype=np.uint64)
    src = c_void_p(poly.device_ptr) if poly.device_ptr is not None else _ptr(poly.mont)
    mem = ZK_MEM_DEVICE if poly.device_ptr is not None else ZK_MEM_HOST
    check(lib.zk_fix_from_right(ctx.handle, poly.n, src, mem, k, _ptr(pt), _ptr(out), ZK_MEM_HOST), "zk_fix_from_right")
    return DenseMLPoly(poly.n - k, mont=out)


def _i128_array(values):
    """Python integers -> (len, 2) u64 array holding Rust i128 values (two's complement, little-endian)."""
    out = np.empty((len(values), 2), dtype=np.uint64)
    for i, v in enumerate(values):
        assert -(1 << 127) <= v < (1 << 127), "value does not fit an i128"
        u = v & ((1 << 128) - 1)
        out[i, 0] = u & 0xFFFFFFFFFFFFFFFF
        out[i, 1] = u >> 64
    return out


def permute_evals_by_ranges(ctx: Context, evals, n: int, ranges, integers: bool = False):
    """src/basicblock/einsum.rs:142-198.  evals: field elements (canonical integers), or with integers=True
    the i128 witness values; ranges: (start, end) pairs of old variables in their new order."""
    assert len(evals) == 1 << n, "evals length must be 2^n"
    assert len(ranges) > 0, "ranges must not be empty"
    src = _i128_array(evals) if integers else to_mont_array(evals)
    out = np.zeros_like(src)
    rg = np.array([v for r in ranges for v in r], dtype=np.uint64)
    check(lib.zk_permute_by_ranges(ctx.handle, n, 16 if integers else 32, _ptr(src), ZK_MEM_HOST, len(ranges), _ptr(rg),
                                   _ptr(out), ZK_MEM_HOST), "zk_permute_by_ranges")
    if integers:
        res = []
        for lo, hi in out.tolist():
            u = (hi << 64) | lo
            res.append(u - (1 << 128) if u >> 127 else u)
        return res
    return from_mont_array(out)


def fix_variables_zkgpt(ctx: Context, num_vars: int, t_idx, r, q_bits: int = 0) -> "DenseMLPoly":
    """src/util/poly.rs:1378-1473: binds the len(r) low variables of the integer table t_idx (layout b + c * n).
    q_bits sizes the reference's lookup table and does not change the result; it is accepted and unused."""
    k = len(r)
    assert k <= num_vars and len(t_idx) == 1 << num_vars
    src = _i128_array(t_idx)
    pt = to_mont_array(r) if k else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << (num_vars - k), 4), dtype=np.uint64)
    check(lib.zk_fix_variables_int(ctx.handle, num_vars, _ptr(src), ZK_MEM_HOST, k, _ptr(pt), _ptr(out), ZK_MEM_HOST),
          "zk_fix_variables_int")
    return DenseMLPoly(num_vars - k, mont=out)


def range_aux_accumulate(ctx: Context, point, selection, beta_gamma: int, table_log: int, acc: "DenseMLPoly"):
    """src/dag/mod.rs:1314-1337 for one auxiliary selection polynomial: scatter-adds the Lagrange weights of
    `point` at the pairs' input indices into their table indices, returns the middle claim sum_t part[t] * t
    and adds beta_gamma * part to acc (a DenseMLPoly of table_log variables, updated in place)."""
    k = len(point)
    assert acc.n == table_log
    pt = to_mont_array(point) if k else np.zeros((1, 4), dtype=np.uint64)
    ii = np.ascontiguousarray(np.array([p[0] for p in selection] or [0], dtype=np.uint64))
    tt = np.ascontiguousarray(np.array([p[1] for p in selection] or [0], dtype=np.uint64))
    bg = to_mont_array([beta_gamma])
    mid = np.zeros((1, 4), dtype=np.uint64)
    check(lib.zk_range_aux_accumulate(ctx.handle, k, _ptr(pt), len(selection), _ptr(ii), _ptr(tt), ZK_MEM_HOST, _ptr(bg),
                                      table_log, _ptr(acc.mont), ZK_MEM_HOST, _ptr(mid)), "zk_range_aux_accumulate")
    return from_mont_array(mid)[0]


def range_table(ctx: Context, n: int, alpha: int) -> "DenseMLPoly":
    """range_dense(n).add_by_scalar(alpha) (src/util/poly.rs:1359-1366, 915-927)."""
    out = np.zeros((1 << n, 4), dtype=np.uint64)
    check(lib.zk_range_table(ctx.handle, n, _ptr(to_mont_array([alpha])), _ptr(out), ZK_MEM_HOST), "zk_range_table")
    return DenseMLPoly(n, mont=out)


class SumcheckProof:
    """src/crypto/sumcheck/prover.rs:9-14."""

    def __init__(self, final_eval, round_messages):
        self.final_eval = final_eval
        self.round_messages = round_messages


class SumcheckVerifier:
    """src/crypto/sumcheck/verifier.rs:7-70 (host arithmetic inside the library, no device needed)."""

    def __init__(self, num_var: int, num_poly: int, transcript: Transcript):
        transcript.append_u64(b"num_var", num_var)
        transcript.append_u64(b"num_poly", num_poly)
        self.num_var = num_var
        self.num_poly = num_poly

    def verify(self, transcript: Transcript, round_messages, claimed_sum):
        """(final running sum or None, challenges), as the reference returns them."""
        per = len(round_messages[0]) if round_messages else self.num_poly + 1
        if any(len(m) != per for m in round_messages):
            return None, []
        flat = to_mont_array([v for m in round_messages for v in m] or [0])
        claim = to_mont_array([claimed_sum])
        chal = np.zeros((max(len(round_messages), 1), 4), dtype=np.uint64)
        fin = np.zeros((1, 4), dtype=np.uint64)
        ok, failed = ctypes.c_int(0), ctypes.c_uint32(0)
        check(lib.zk_sumcheck_verify(transcript.handle, self.num_var, self.num_poly, _ptr(flat), len(round_messages), per,
                                     _ptr(claim), _ptr(chal), _ptr(fin), ctypes.byref(ok), ctypes.byref(failed)),
              "zk_sumcheck_verify")
        if not ok.value:
            return None, []
        return from_mont_array(fin)[0], from_mont_array(chal[: len(round_messages)])


class LinearSumcheckProver:
    """src/crypto/sumcheck/linear_prover.rs:13-191 on the GPU."""

    def __init__(self, num_var: int, num_polys: int, transcript: Transcript):
        transcript.append_u64(b"num_var", num_var)
        transcript.append_u64(b"num_poly", num_polys)
        self.num_var = num_var
        self.num_poly = num_polys
        self.challenges = []
        self.a_arrays = []  # after prove: a_arrays[i][0], the fully bound value of table i

    def prove(self, ctx: Context, instances, transcript: Transcript, fs_callback=None) -> SumcheckProof:
        assert len(instances) > 0, "Polynomials cannot be empty"
        assert len(instances) == self.num_poly, "Number of polynomials mismatch"
        for i, p in enumerate(instances):
            assert len(p) == 1 << self.num_var, f"Polynomial {i} has incorrect size"
        L, n = self.num_poly, self.num_var
        on_dev = instances[0].device_ptr is not None
        ptrs = (c_void_p * L)(*[c_void_p(p.device_ptr) if on_dev else _ptr(p.mont) for p in instances])
        msgs = np.zeros((max(n, 1), L + 1, 4), dtype=np.uint64)
        chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
        fin_t = np.zeros((L, 4), dtype=np.uint64)
        fin = np.zeros((1, 4), dtype=np.uint64)
        cb = _lib.FS_ROUND_FN(fs_callback) if fs_callback is not None else None
        check(lib.zk_sumcheck_linear_prove(ctx.handle, n, L, ptrs, ZK_MEM_DEVICE if on_dev else ZK_MEM_HOST,
                                           ctypes.cast(cb, c_void_p) if cb else None, None,
                                           None if cb else transcript.handle, _ptr(msgs), _ptr(chal), _ptr(fin_t),
                                           _ptr(fin)), "zk_sumcheck_linear_prove")
        self.challenges = from_mont_array(chal[:n])
        self.a_arrays = [[v] for v in from_mont_array(fin_t)]
        rm = [from_mont_array(msgs[r]) for r in range(n)]
        return SumcheckProof(from_mont_array(fin)[0], rm)


class SparseDenseSumcheckProver:
    """Product sumcheck of a sparse table (sorted non-zero entries) with a dense one.  Defined as
    LinearSumcheckProver (two tables) on [a.to_dense(), b]; header as linear_prover.rs:29-32."""

    def __init__(self, num_var: int, transcript: Transcript):
        transcript.append_u64(b"num_var", num_var)
        transcript.append_u64(b"num_poly", 2)
        self.num_var = num_var
        self.challenges = []
        self.a_arrays = []

    def prove(self, ctx: Context, indices, values, dense: DenseMLPoly, transcript: Transcript, *,
              device_ptrs=None) -> SumcheckProof:
        """indices: strictly increasing ints; values: canonical ints.  With device_ptrs =
        (idx_ptr, val_ptr, nnz) all three inputs are device buffers."""
        n = self.num_var
        assert len(dense) == 1 << n, "Polynomials have incorrect size"
        msgs = np.zeros((max(n, 1), 3, 4), dtype=np.uint64)
        chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
        fin_t = np.zeros((2, 4), dtype=np.uint64)
        fin = np.zeros((1, 4), dtype=np.uint64)
        if device_ptrs is not None:
            ip, vp, nnz = device_ptrs
            args = (c_void_p(ip), c_void_p(vp), c_void_p(dense.device_ptr), ZK_MEM_DEVICE)
        else:
            nnz = len(indices)
            ia = np.ascontiguousarray(np.array(list(indices), dtype=np.uint64))
            va = to_mont_array(values) if nnz else np.zeros((1, 4), dtype=np.uint64)
            args = (_ptr(ia) if nnz else None, _ptr(va), _ptr(dense.mont), ZK_MEM_HOST)
        check(lib.zk_sumcheck_sparse_dense_prove(ctx.handle, n, nnz, args[0], args[1], args[2], args[3], None, None,
                                                 transcript.handle, _ptr(msgs), _ptr(chal), _ptr(fin_t), _ptr(fin)),
              "zk_sumcheck_sparse_dense_prove")
        self.challenges = from_mont_array(chal[:n])
        self.a_arrays = [[v] for v in from_mont_array(fin_t)]
        return SumcheckProof(from_mont_array(fin)[0], [from_mont_array(msgs[r]) for r in range(n)])


class SparseBoolSumcheckProver:
    """src/crypto/sumcheck/linear_prover.rs:455-656."""

    def __init__(self, num_var: int, transcript: Transcript):
        transcript.append_u64(b"num_var", num_var)
        transcript.append_u64(b"num_poly", 3)
        self.num_var = num_var
        self.challenges = []

    def prove(self, ctx: Context, weights, positions, eq_challenge, transcript: Transcript) -> SumcheckProof:
        assert len(weights) == len(positions)
        assert len(eq_challenge) == self.num_var
        n = self.num_var
        w = to_mont_array(weights) if len(weights) else np.zeros((1, 4), dtype=np.uint64)
        flat = np.array([p for pos in positions for p in pos] or [0], dtype=np.uint64)
        cnt = np.array([len(p) for p in positions] or [0], dtype=np.uint64)
        pt = to_mont_array(eq_challenge) if n else np.zeros((1, 4), dtype=np.uint64)
        msgs = np.zeros((max(n, 1), 4, 4), dtype=np.uint64)
        chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
        fin = np.zeros((1, 4), dtype=np.uint64)
        check(lib.zk_sumcheck_sparse_bool_prove(ctx.handle, n, len(weights), _ptr(w), _ptr(flat), _ptr(cnt), _ptr(pt), None,
                                                None, transcript.handle, _ptr(msgs), _ptr(chal), _ptr(fin)),
              "zk_sumcheck_sparse_bool_prove")
        self.challenges = from_mont_array(chal[:n])
        return SumcheckProof(from_mont_array(fin)[0], [from_mont_array(msgs[r]) for r in range(n)])


class GeneralLinearSumcheckProver:
    """src/crypto/sumcheck/linear_prover.rs:193-438; Instance = (scalars, tables per term, eq)."""

    def __init__(self, num_var: int, num_polys: int, transcript: Transcript):
        transcript.append_u64(b"num_var", num_var)
        transcript.append_u64(b"num_poly", num_polys)
        self.num_var, self.num_poly = num_var, num_polys
        self.challenges = []
        self.a_arrays = []

    def prove(self, ctx: Context, instance, transcript: Transcript) -> SumcheckProof:
        scalars, arrays, eq = instance
        assert len(arrays) > 0 and len(scalars) > 0, "Polynomials cannot be empty"
        assert len(arrays[0]) == self.num_poly - 1, "Number of polynomials mismatch"
        assert len(scalars) == len(arrays), "Number of scalars mismatch"
        n, nf, nt = self.num_var, self.num_poly - 1, len(arrays)
        flat = [p for term in arrays for p in term]
        for i, p in enumerate(flat):
            assert len(p) == 1 << n, f"Polynomial {i} has incorrect size"
        ptrs = (c_void_p * max(len(flat), 1))(*[_ptr(p.mont) for p in flat])
        sc = to_mont_array(scalars)
        msgs = np.zeros((max(n, 1), self.num_poly + 1, 4), dtype=np.uint64)
        chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
        fin_t = np.zeros((max(nt * nf, 1), 4), dtype=np.uint64)
        fin = np.zeros((1, 4), dtype=np.uint64)
        check(lib.zk_sumcheck_general_prove(ctx.handle, n, self.num_poly, nt, _ptr(sc), ptrs, _ptr(eq.mont), ZK_MEM_HOST, None,
                                            None, transcript.handle, _ptr(msgs), _ptr(chal), _ptr(fin_t), _ptr(fin)),
              "zk_sumcheck_general_prove")
        self.challenges = from_mont_array(chal[:n])
        vals = from_mont_array(fin_t)
        self.a_arrays = [[[vals[j * nf + i]] for i in range(nf)] for j in range(nt)]
        return SumcheckProof(from_mont_array(fin)[0], [from_mont_array(msgs[r]) for r in range(n)])
