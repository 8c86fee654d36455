"""GPU parity at the sizes the benchmark configurations run at, against the C++ CPU oracle.

The small-case suites stop at 2^16 entries; the launches that are capped by the grid, the
two-folds-per-pass schedule over three table sizes, 32-bit entry positions near 2^26 and the
side stream only occur at these sizes.  Inputs come from the seeded generators of the library
(field elements) and of zkes_b200.synth (positions), so that both sides see identical bytes."""
import ctypes

import numpy as np
import pytest

import coracle
from zkes_b200 import synth
from zkes_b200._lib import ZK_MEM_DEVICE, check, lib
from zkes_b200.field import from_mont_array

pytestmark = pytest.mark.gpu
vp = ctypes.c_void_p


def dev_gen(ctx, kind, seed, stream, count, bits=8):
    import torch
    t = torch.empty((count, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    if kind == "uniform":
        check(lib.zk_gen_uniform_fr(ctx.handle, seed, stream, 0, count, t.data_ptr()), "zk_gen_uniform_fr")
    else:
        check(lib.zk_gen_small_fr(ctx.handle, seed, stream, 0, count, bits, t.data_ptr()), "zk_gen_small_fr")
    return t


def host_u64(t):
    return t.cpu().numpy().view(np.uint64)


def transcript(label, num_var, num_poly):
    tr = lib.zk_transcript_new(label, len(label))
    lib.zk_transcript_append_u64(tr, b"num_var", 7, num_var)
    lib.zk_transcript_append_u64(tr, b"num_poly", 8, num_poly)
    return tr


def tail_challenge(tr):
    out = np.zeros((1, 4), dtype=np.uint64)
    lib.zk_transcript_challenge_scalar(tr, b"after", 5, vp(out.ctypes.data))
    lib.zk_transcript_free(tr)
    return from_mont_array(out)[0]


def compare(n, L, msgs, chal, fin_t, fin, tail, want):
    got_msgs = from_mont_array(msgs.reshape(-1, 4))
    assert [got_msgs[r * (L + 1):(r + 1) * (L + 1)] for r in range(n)] == want.round_messages
    assert from_mont_array(chal) == want.challenges
    assert from_mont_array(fin_t) == want.final_tables
    assert from_mont_array(fin)[0] == want.final_eval
    assert tail == want.tail  # the transcripts end in the same state


@pytest.mark.parametrize("n,ell", [(20, 2), (18, 3), (21, 1)])
def test_linear_prover_benchmark_size(ctx, n, ell):
    """n = 20, two tables of uniform elements from seed 0: the dense configuration the reference's
    benches/sumcheck_prover.rs is modelled on (linear_prover.rs:43-191)."""
    coracle.set_threads(8)
    tables = [dev_gen(ctx, "uniform", 0, i, 1 << n) for i in range(ell)]
    ptrs = (vp * ell)(*[vp(t.data_ptr()) for t in tables])
    msgs = np.zeros((n, ell + 1, 4), dtype=np.uint64)
    chal = np.zeros((n, 4), dtype=np.uint64)
    fin_t = np.zeros((ell, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    tr = transcript(b"sumcheck_bench", n, ell)
    check(lib.zk_sumcheck_linear_prove(ctx.handle, n, ell, ptrs, ZK_MEM_DEVICE, None, None, tr, vp(msgs.ctypes.data),
                                       vp(chal.ctypes.data), vp(fin_t.ctypes.data), vp(fin.ctypes.data)), "linear_prove")
    want = coracle.linear_prove_mont(b"sumcheck_bench", n, [host_u64(t) for t in tables])
    compare(n, ell, msgs, chal, fin_t, fin, tail_challenge(tr), want)


@pytest.mark.parametrize("n,nnz_log", [(22, 16), (24, 18), (26, 20), (23, 21)])
def test_sparse_dense_benchmark_size(ctx, n, nnz_log):
    """Density 1/64 up to the benchmark's own size (n = 26, 2^20 int8 non-zeros, seed 1), and one denser
    case that leaves the entry form after a single round."""
    import torch
    coracle.set_threads(16)
    dense = dev_gen(ctx, "uniform", 1, 0, 1 << n)
    vals = dev_gen(ctx, "small", 1, 2, 1 << nnz_log)
    idx_host = synth.sparse_indices(1, n, 1 << nnz_log)
    idx = torch.from_numpy(idx_host.view(np.int64)).cuda()
    msgs = np.zeros((n, 3, 4), dtype=np.uint64)
    chal = np.zeros((n, 4), dtype=np.uint64)
    fin_t = np.zeros((2, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    tr = transcript(b"sumcheck_bench", n, 2)
    check(lib.zk_sumcheck_sparse_dense_prove(ctx.handle, n, 1 << nnz_log, vp(idx.data_ptr()), vp(vals.data_ptr()),
                                             vp(dense.data_ptr()), ZK_MEM_DEVICE, None, None, tr, vp(msgs.ctypes.data),
                                             vp(chal.ctypes.data), vp(fin_t.ctypes.data), vp(fin.ctypes.data)),
          "sparse_dense_prove")
    tail = tail_challenge(tr)
    dense_h, vals_h = host_u64(dense), host_u64(vals)
    del dense, vals
    torch.cuda.empty_cache()
    want = coracle.sparse_dense_prove_mont(b"sumcheck_bench", n, idx_host, vals_h, dense_h)
    compare(n, 2, msgs, chal, fin_t, fin, tail, want)
