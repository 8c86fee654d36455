"""Multi-GPU host logic: one process per GPU (torch.distributed for the plumbing), the hypercube
cut on its top log2(world) variables.  The reference is single-process; these helpers have no
counterpart there."""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import numpy as np

from ._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
from .field import from_mont_array, to_mont_array


def log2_exact(world: int) -> int:
    lg = world.bit_length() - 1
    if world < 1 or (1 << lg) != world:
        raise ValueError(f"the number of ranks must be a power of two, got {world}")
    return lg


def shard_range(rank: int, world: int, num_var: int):
    """Index range [begin, end) of the 2^num_var table that `rank` owns (contiguous chunks: the top
    log2(world) variables select the rank, and they are the last ones the protocol binds)."""
    lg = log2_exact(world)
    if num_var < lg:
        raise ValueError(f"{num_var} variables cannot be sharded over {world} ranks")
    chunk = 1 << (num_var - lg)
    return rank * chunk, (rank + 1) * chunk


def shard_dense(table, rank: int, world: int):
    n = len(table).bit_length() - 1
    b, e = shard_range(rank, world, n)
    return table[b:e]


def shard_sparse(indices, values, rank: int, world: int, num_var: int):
    """Entries of a sorted sparse table that fall in the rank's range, indices made local."""
    b, e = shard_range(rank, world, num_var)
    idx, val = [], []
    for i, v in zip(indices, values):
        if b <= i < e:
            idx.append(i - b)
            val.append(v)
    return idx, val


def tail_tables(per_rank_values):
    """per_rank_values[r][i] = rank r's fully bound value of table i  ->  table i over the top variables."""
    world = len(per_rank_values)
    log2_exact(world)
    n_tables = len(per_rank_values[0])
    return [[per_rank_values[r][i] for r in range(world)] for i in range(n_tables)]


class Comm:
    """zk_comm over the ranks of an initialised torch.distributed process group."""

    def __init__(self, ctx, rank: int = None, world: int = None):
        import torch
        import torch.distributed as dist

        self.ctx = ctx
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        log2_exact(self.world)
        uid = (ctypes.c_uint8 * 128)()
        if self.rank == 0:
            check(lib.zk_comm_unique_id(uid), "zk_comm_unique_id")
        if self.world > 1:
            dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
            t = torch.tensor(list(uid), dtype=torch.uint8, device=dev)
            dist.broadcast(t, src=0)
            uid = (ctypes.c_uint8 * 128)(*t.cpu().tolist())
        h = c_void_p()
        check(lib.zk_comm_init(ctx.handle, self.rank, self.world, uid, ctypes.byref(h)), "zk_comm_init")
        self.handle = h

    @property
    def peer_exchange(self) -> bool:
        """True when the ranks mapped each other's exchange boxes (round messages then cross NVLink by
        peer stores inside one kernel per round instead of an NCCL all-gather)."""
        return bool(lib.zk_comm_peer_exchange(self.handle))

    def close(self):
        if self.handle:
            lib.zk_comm_free(self.ctx.handle, self.handle)
            self.handle = None


def _p(a):
    return c_void_p(a.ctypes.data)


def sharded_linear_prove(ctx, comm: Comm, num_var: int, local_tables, transcript):
    """Every rank passes its chunk of each table (DenseMLPoly) and an equal-state transcript whose
    header (num_var, num_poly) is already absorbed.  Returns (round_messages, challenges,
    final_table0, final_eval) as canonical ints, identical on all ranks."""
    L = len(local_tables)
    on_dev = local_tables[0].device_ptr is not None
    ptrs = (c_void_p * L)(*[c_void_p(t.device_ptr) if on_dev else _p(t.mont) for t in local_tables])
    msgs = np.zeros((max(num_var, 1), L + 1, 4), dtype=np.uint64)
    chal = np.zeros((max(num_var, 1), 4), dtype=np.uint64)
    fin_t = np.zeros((L, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    check(lib.zk_sumcheck_linear_prove_sharded(ctx.handle, comm.handle, num_var, L, ptrs, ZK_MEM_DEVICE if on_dev else ZK_MEM_HOST,
                                               None, None, transcript.handle, _p(msgs), _p(chal), _p(fin_t), _p(fin)),
          "zk_sumcheck_linear_prove_sharded")
    return ([from_mont_array(msgs[r]) for r in range(num_var)], from_mont_array(chal[:num_var]), from_mont_array(fin_t),
            from_mont_array(fin)[0])


def sharded_sparse_dense_prove(ctx, comm: Comm, num_var: int, local_idx, local_vals, local_dense, transcript):
    nnz = len(local_idx)
    ia = np.ascontiguousarray(np.array(list(local_idx) or [0], dtype=np.uint64))
    va = to_mont_array(local_vals) if nnz else np.zeros((1, 4), dtype=np.uint64)
    msgs = np.zeros((max(num_var, 1), 3, 4), dtype=np.uint64)
    chal = np.zeros((max(num_var, 1), 4), dtype=np.uint64)
    fin_t = np.zeros((2, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    check(lib.zk_sumcheck_sparse_dense_prove_sharded(ctx.handle, comm.handle, num_var, nnz, _p(ia), _p(va), _p(local_dense.mont),
                                                     ZK_MEM_HOST, None, None, transcript.handle, _p(msgs), _p(chal),
                                                     _p(fin_t), _p(fin)), "zk_sumcheck_sparse_dense_prove_sharded")
    return ([from_mont_array(msgs[r]) for r in range(num_var)], from_mont_array(chal[:num_var]), from_mont_array(fin_t),
            from_mont_array(fin)[0])


def sharded_sparse_bool_prove(ctx, comm: Comm, num_var: int, local_weights, local_positions, eq_challenge, transcript):
    """SparseBoolSumcheckProver::prove (linear_prover.rs:486-656) with the terms dealt to the ranks: this rank's
    weights and position lists in, the proof over all the terms out (the same on every rank)."""
    n = num_var
    w = to_mont_array(local_weights) if len(local_weights) else np.zeros((1, 4), dtype=np.uint64)
    flat = np.array([p for pos in local_positions for p in pos] or [0], dtype=np.uint64)
    cnt = np.array([len(p) for p in local_positions] or [0], dtype=np.uint64)
    pt = to_mont_array(eq_challenge) if n else np.zeros((1, 4), dtype=np.uint64)
    msgs = np.zeros((max(n, 1), 4, 4), dtype=np.uint64)
    chal = np.zeros((max(n, 1), 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    check(lib.zk_sumcheck_sparse_bool_prove_sharded(ctx.handle, comm.handle, n, len(local_weights), _p(w), _p(flat), _p(cnt),
                                                    _p(pt), None, None, transcript.handle, _p(msgs), _p(chal), _p(fin)),
          "zk_sumcheck_sparse_bool_prove_sharded")
    return [from_mont_array(msgs[r]) for r in range(n)], from_mont_array(chal[:n]), from_mont_array(fin)[0]


def sharded_msm(ctx, comm: Comm, local_bases_arr: np.ndarray, local_scalars):
    """sum over all ranks of MSM(local bases, local scalars) -> affine tuple, the same on every rank."""
    from . import curve
    n = len(local_scalars)
    sc = to_mont_array(local_scalars) if n else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1, 12), dtype=np.uint64)
    check(lib.zk_msm_g1_sharded(ctx.handle, comm.handle, _p(local_bases_arr), ZK_MEM_HOST, _p(sc), ZK_MEM_HOST, n, _p(out)),
          "zk_msm_g1_sharded")
    return curve.jacobian_to_affine_py(out)[0]


def sharded_fix_from_right(ctx, comm: Comm, n: int, local_evals, point):
    ev = to_mont_array(local_evals)
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    out = np.zeros((1 << (n - len(point)), 4), dtype=np.uint64)
    check(lib.zk_fix_from_right_sharded(ctx.handle, comm.handle, n, _p(ev), ZK_MEM_HOST, len(point), _p(pt), _p(out)),
          "zk_fix_from_right_sharded")
    return from_mont_array(out)


def sharded_kzh_setup(ctx, comm: Comm, dims: int, n: int, g, tau_x, tau_y, tau_z=None, alpha=None):
    from . import curve
    from .kzh import KZHSRS
    h = c_void_p()
    ga = curve.affine_to_array([g])
    tx, ty = to_mont_array(tau_x), to_mont_array(tau_y)
    tz = to_mont_array(tau_z) if tau_z is not None else None
    al = to_mont_array([alpha]) if alpha is not None else None
    check(lib.zk_kzh_srs_setup_sharded(ctx.handle, comm.rank, comm.world, dims, n, _p(ga), _p(tx), _p(ty),
                                       _p(tz) if tz is not None else None, _p(al) if al is not None else None,
                                       ctypes.byref(h)), "zk_kzh_srs_setup_sharded")
    return KZHSRS(ctx, dims, n, h)


def sharded_kzh_commit(ctx, comm: Comm, srs, local_evals, with_jacobian: bool = False):
    """-> (c affine, d_x affine list), identical on every rank; with_jacobian adds the raw d_x array
    that sharded_kzh_open takes."""
    from . import curve
    ev = to_mont_array(local_evals)
    c = np.zeros((1, 8), dtype=np.uint64)
    dx = np.zeros((1 << srs.x_log, 12), dtype=np.uint64)
    check(lib.zk_kzh_commit_sharded(ctx.handle, comm.handle, srs.handle, _p(ev), ZK_MEM_HOST, _p(c), _p(dx)),
          "zk_kzh_commit_sharded")
    res = (curve.affine_from_array(c)[0], curve.jacobian_to_affine_py(dx))
    return res + (dx,) if with_jacobian else res


def sharded_kzh_open(ctx, comm: Comm, srs, point, local_evals, d_x_jac=None):
    """kzh2_open / kzh3_open over x-row shards -> f_star (KZH2) or (d_y, c_y, f_star) (KZH3), on every rank."""
    from . import curve
    ev = to_mont_array(local_evals)
    pt = to_mont_array(point) if len(point) else np.zeros((1, 4), dtype=np.uint64)
    if srs.dims == 2:
        fs = np.zeros((1 << srs.y_log, 4), dtype=np.uint64)
        check(lib.zk_kzh_open_sharded(ctx.handle, comm.handle, srs.handle, _p(ev), ZK_MEM_HOST, _p(pt), len(point), None, None,
                                      None, _p(fs)), "zk_kzh_open_sharded")
        return from_mont_array(fs)
    dy = np.zeros((1 << srs.y_log, 12), dtype=np.uint64)
    cy = np.zeros((1, 8), dtype=np.uint64)
    fs = np.zeros((1 << srs.z_log, 4), dtype=np.uint64)
    check(lib.zk_kzh_open_sharded(ctx.handle, comm.handle, srs.handle, _p(ev), ZK_MEM_HOST, _p(pt), len(point), _p(d_x_jac),
                                  _p(dy), _p(cy), _p(fs)), "zk_kzh_open_sharded")
    return curve.jacobian_to_affine_py(dy), curve.affine_from_array(cy)[0], from_mont_array(fs)
