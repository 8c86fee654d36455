"""Replay of the hot-path calls of a GPT-2-small inference proof.

The reference's `gpt2` bin (src/bin/gpt2.rs, src/dag/gpt2.rs:229-309) cannot run here: it needs the whole
Rust crate.  What this module does instead is issue, through the C ABI, the sequence of calls that the
bin's Dag::commit and Dag::prove make into the accelerated path, with the shapes of GPT-2-small at
sequence length 128 and synthetic values (the values do not change the work; the shapes do):

  commit   Dag::commit (dag/mod.rs:628-672): every Constant / Input / Auxiliary edge.  Per layer the four
           768 x 768 and two 768 x 3072 weight matrices padded to 2^20 and 2^22 evaluations, the bias and
           norm vectors, the 1.702 constant tensor of the GELU (dag/gpt2.rs:62-70, 2^19); the auxiliary
           selection polynomials of every lookup node as sparse commitments (all-ones, K = one entry per
           looked-up element, split into 5 blocks of 4 table bits: table_size_log 20 / table_commit_log 4
           of config.yaml, dag/mod.rs:553).
  prove    Dag::prove (dag/mod.rs:674-965) walks the nodes in reverse order.  Every einsum
           (basicblock/einsum.rs:468-582) folds each input on its free variables (DenseMLPoly::fix_variables
           below 2^18 entries, fix_variables_zkgpt on the i128 table from there on, after
           permute_evals_by_ranges where the layout asks for it), builds the eq table of the shared variables
           and runs LinearSumcheckProver with (inputs + 1) tables; element-wise blocks evaluate their input
           at the claim point (add.rs:89, scale.rs:83).  Then prove_range (dag/mod.rs:1275-1380): per
           auxiliary polynomial the scatter-add of Lagrange weights, one table sumcheck, and one
           SparseBoolSumcheckProver per auxiliary size over all the model's terms; finally one opening per
           claim (dag/mod.rs:876-936), dense and sparse.

Simplifications, stated so that the number is read as a trace and not as the bin: exp / sigmoid lookups
(two_pow tables) are counted as range nodes of the same size; the tiny per-row nodes of the layer norms
(2^7 elements) are left out; every committed dense polynomial gets one opening and every auxiliary
polynomial two (its boolean claim and its lookup claim); the commitment scheme is a parameter (KZH2 as the
benchmark configuration names it; the bin itself uses KZH3).  At N > 1 GPUs the independent items (commits
and openings) are dealt round-robin to the ranks with no exchange, as the reference's rayon loop deals the
openings to threads; the terms of each boolean-check sumcheck are dealt to the ranks in blocks (the partial
round messages are summed across the ranks); the other sumchecks share one transcript and run on every rank alike.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor

import ctypes
import time
from ctypes import c_void_p as vp

import numpy as np

from ._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
from .field import to_mont_array

R_MOD = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001
G2X = 1368015179489954701390400359078579693043519447331113978918064868415326638035
G2Y = 9918110051302171585080402603319702774565515993150576347155970296011118125764
TABLE_BLOCKS = 5      # table_size_log 20 in blocks of table_commit_log 4 (config.yaml)
TABLE_BLOCK_LOG = 4


def model_calls(seq_log=7, d_log=10, f_log=12, h_log=4, dh_log=6, layers=12):
    """The call list: (kind, args) tuples in prove order, plus the commit lists.  Variable counts: an
    activation (1, seq, 1024) has A = seq_log + d_log variables, an MLP activation (1, seq, 4096) FA, the
    attention scores (16, seq, seq) SC, a per-head tensor (16, seq, 64) V."""
    A, FA, SC, V = seq_log + d_log, seq_log + f_log, h_log + 2 * seq_log, h_log + seq_log + dh_log
    W, W1 = 2 * d_log, d_log + f_log
    prove, dense, lookups = [], [], []

    def fold(n, k):  # an input with 2^n entries bound on k variables: field fold below 2^18, integer fold from there on
        prove.append(("intfold" if n >= 18 else "fold", n, k))

    def einsum(inputs, eq_vars, rounds, permute=()):
        for n in permute:
            prove.append(("permute", n))
        for n, k in inputs:
            if k:
                fold(n, k)
        if eq_vars:
            prove.append(("eq", eq_vars))
        prove.append(("sumcheck", len(inputs) + 1, rounds))

    def lookup(n):  # a rescale / non-negativity / exp node over 2^n elements
        lookups.append(n)

    def layer_norm():  # dag/gpt2.rs:11-46 with llama_rms_norm (dag/llama.rs:319-380)
        einsum([(A, seq_log)], 0, d_log)                      # bsi->bs
        prove.append(("mle", A)); prove.append(("mle", A))    # sub, mask
        einsum([(A, 0), (A, 0)], A, A); lookup(A)             # x_sq = bsi,bsi->bsi, rescaled
        einsum([(A, seq_log)], 0, d_log)                      # sum of squares
        einsum([(A, d_log), (seq_log, 0)], seq_log, seq_log, permute=(A,)); lookup(A)  # h = bsi,bs->bsi
        einsum([(A, seq_log), (d_log, 0)], d_log, d_log); lookup(A)                    # out = bsi,i->bsi
        prove.append(("mle", A))                              # + bias

    for _ in range(layers):
        dense.extend([W] * 4 + [W1] * 2 + [d_log] * 8 + [f_log] + [FA])  # weights, biases / norm vectors, 1.702 tensor
        # ---- reverse order of the forward pass does not change the work: listed in forward order
        layer_norm()
        for _ in range(3):  # q, k, v = bsi,ij->bsj (+ bias)
            einsum([(A, seq_log), (W, d_log)], 0, d_log); lookup(A); prove.append(("mle", A))
        for _ in range(3):  # bshd->bhsd: no summed variable, the input is bound on all of its variables
            einsum([(V, V)], 0, 0, permute=(V,))
        einsum([(V, seq_log), (V, seq_log)], h_log, h_log + dh_log); lookup(SC)      # scores = bhsd,bhtd->bhst
        einsum([(SC, SC)], 0, 0); lookup(SC)                                          # bhst,z->bhst
        prove.append(("mle", SC)); lookup(SC)                                         # + softmax constant, exp
        einsum([(SC, seq_log), (V, dh_log)], h_log, h_log + seq_log, permute=(V,)); lookup(V)  # bhst,bhtd->bhsd
        einsum([(V, V)], 0, 0, permute=(V,))                                          # bhsd->bshd
        einsum([(A, seq_log), (W, d_log)], 0, d_log); lookup(A)                       # output projection
        prove.append(("mle", A)); prove.append(("mle", A))                            # + bias, + residual
        layer_norm()
        einsum([(A, seq_log), (W1, f_log)], 0, d_log); lookup(FA); prove.append(("mle", FA))   # h1
        einsum([(FA, 0), (FA, 0)], FA, FA); lookup(FA)                                # 1.702 x
        prove.append(("mle", FA)); lookup(FA)                                         # sigmoid: + constant, exp
        einsum([(FA, 0), (FA, 0)], FA, FA); lookup(FA)                                # x sigmoid(1.702 x)
        einsum([(FA, seq_log), (W1, d_log)], 0, f_log); lookup(A)                     # h2
        prove.append(("mle", A)); prove.append(("mle", A))
    layer_norm()
    dense.extend([d_log, d_log, 2 * seq_log, A])  # final norm vectors, attention mask, input
    return prove, dense, lookups


class _Buffers:
    """Synthetic device data, one buffer per size, reused by every call of that size."""

    def __init__(self, ctx, seed):
        import torch
        self.torch, self.ctx, self.seed = torch, ctx, seed
        self.field, self.ints, self.out = {}, {}, {}

    def fr(self, n, bits=16):
        if n not in self.field:
            t = self.torch.empty((1 << n, 4), dtype=self.torch.int64, device="cuda")
            self.torch.cuda.synchronize()
            check(lib.zk_gen_small_fr(self.ctx.handle, self.seed, 100 + n, 0, 1 << n, bits, t.data_ptr()), "zk_gen_small_fr")
            self.field[n] = t
        return self.field[n]

    def i128(self, n):
        if n not in self.ints:
            g = self.torch.Generator(device="cuda")
            g.manual_seed(self.seed * 1000 + n)
            lo = self.torch.randint(-(1 << 15), 1 << 15, (1 << n,), generator=g, device="cuda", dtype=self.torch.int64)
            self.ints[n] = self.torch.stack([lo, lo >> 63], dim=1).contiguous()  # two's complement, little-endian
        return self.ints[n]

    def scratch(self, n):
        if n not in self.out:
            self.out[n] = self.torch.empty((1 << n, 4), dtype=self.torch.int64, device="cuda")
        return self.out[n]


def run(ctx, comm=None, rank=0, world=1, seq_len=128, seed=4, dims=2, layers=12, open_threads=4):
    """Runs the trace and returns the JSON-ready report (seconds per phase, call counts)."""
    import torch

    from . import kzh

    seq_log = max(0, (seq_len - 1).bit_length())
    prove, dense, lookups = model_calls(seq_log=seq_log, layers=layers)
    buf = _Buffers(ctx, seed)
    h = ctx.handle
    rnd = np.random.default_rng(seed)

    def rand_fr(count):
        return to_mont_array([int(x) for x in rnd.integers(1, 1 << 62, size=count)])

    # ---- structured reference strings, one per polynomial size (the bin loads or builds one per size, gpt2.rs:266-285)
    t0 = time.perf_counter()
    sizes = sorted(set(dense) | {n + TABLE_BLOCK_LOG for n in lookups})
    srs = {}
    for n in sizes:
        if dims == 2:
            xl, yl = n // 2, n - n // 2
            logs = (xl, yl)
        else:
            k = n // 3
            logs = [(k, k, k), (k + 1, k, k), (k + 1, k + 1, k)][n % 3]
        taus = [[int(x) for x in rnd.integers(1, 1 << 62, size=1 << lg)] for lg in logs]
        srs[n] = kzh.KZHSRS.setup(ctx, dims, n, (G2X, G2Y), taus[0], taus[1], tau_z=taus[2] if dims == 3 else None,
                                  alpha=12345 if dims == 2 else None)
    ctx.sync()
    setup_s = time.perf_counter() - t0

    # ---- auxiliary selection polynomials: K = 2^n ones, position = table digit << n | element index.  The lists live
    # in pinned host memory, like the boolean sumchecks' below: each is committed once and opened twice, and a prover
    # that hands the same list to the library three times would register it once
    aux_pos, aux_pinned = {}, {}
    for n in sorted(set(lookups)):
        digits = rnd.integers(0, 1 << TABLE_BLOCK_LOG, size=1 << n, dtype=np.uint64)
        t = torch.empty((1 << n,), dtype=torch.int64, pin_memory=True)
        aux_pinned[n] = t  # keeps the pinned allocation alive
        aux_pos[n] = t.numpy().view(np.uint64)
        aux_pos[n][:] = (digits << np.uint64(n)) | np.arange(1 << n, dtype=np.uint64)

    # the position lists of the boolean sumchecks (one list per term, concatenated), in pinned host memory
    bool_terms = {}
    for n in lookups:
        bool_terms[n] = bool_terms.get(n, 0) + TABLE_BLOCKS
    bool_positions = {}
    for n, terms in bool_terms.items():
        t = torch.empty((terms << n,), dtype=torch.int64, pin_memory=True)
        t.view(terms, 1 << n).copy_(torch.from_numpy(aux_pos[n].view(np.int64)).unsqueeze(0).expand(terms, 1 << n))
        bool_positions[n] = t

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()
        ctx.sync()

    def mine(i):  # independent items are dealt round-robin to the ranks
        return i % world == rank

    # ---- commit phase
    commitments = {}
    c_out = np.zeros((1, 8), dtype=np.uint64)
    barrier()
    t0 = time.perf_counter()
    n_dense_commits = n_sparse_commits = 0
    for i, n in enumerate(dense):
        if not mine(i):
            continue
        dx = np.zeros((1 << srs[n].x_log, 12), dtype=np.uint64)
        check(lib.zk_kzh_commit(h, srs[n].handle, n, vp(buf.fr(n, 8).data_ptr()), ZK_MEM_DEVICE, vp(c_out.ctypes.data),
                                vp(dx.ctypes.data)), "zk_kzh_commit")
        commitments[("d", n)] = dx
        n_dense_commits += 1
    dense_commit_s = time.perf_counter() - t0  # each call returns its result on the host, so the split needs no sync
    item = len(dense)
    for n in lookups:
        for _ in range(TABLE_BLOCKS):
            if mine(item):
                m = n + TABLE_BLOCK_LOG
                dx = np.zeros((1 << srs[m].x_log, 12), dtype=np.uint64)
                check(lib.zk_sparse_kzh_commit(h, srs[m].handle, 1 << n, vp(aux_pos[n].ctypes.data), None,
                                               vp(c_out.ctypes.data), vp(dx.ctypes.data)), "zk_sparse_kzh_commit")
                commitments[("s", m)] = dx
                n_sparse_commits += 1
            item += 1
    barrier()
    commit_s = time.perf_counter() - t0

    # ---- prove phase: node proofs
    tr = lib.zk_transcript_new(b"gpt2_trace", 10)
    msgs = np.zeros((40, 5, 4), dtype=np.uint64)
    chal = np.zeros((40, 4), dtype=np.uint64)
    fin_t = np.zeros((4, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    point = rand_fr(40)
    counts = {}
    barrier()
    t0 = time.perf_counter()
    for call in prove:
        kind = call[0]
        counts[kind] = counts.get(kind, 0) + 1
        if kind == "fold":
            _, n, k = call
            check(lib.zk_fold_lsb(h, n, vp(buf.fr(n).data_ptr()), ZK_MEM_DEVICE, k, vp(point.ctypes.data),
                                  vp(buf.scratch(n).data_ptr()), ZK_MEM_DEVICE), "zk_fold_lsb")
        elif kind == "intfold":
            _, n, k = call
            check(lib.zk_fix_variables_int(h, n, vp(buf.i128(n).data_ptr()), ZK_MEM_DEVICE, k, vp(point.ctypes.data),
                                           vp(buf.scratch(n).data_ptr()), ZK_MEM_DEVICE), "zk_fix_variables_int")
        elif kind == "permute":
            _, n = call
            ranges = np.array([n // 2, n, 0, n // 2], dtype=np.uint64)  # the two halves of the variables swapped
            src = buf.i128(n) if n >= 18 else buf.fr(n)
            check(lib.zk_permute_by_ranges(h, n, 16 if n >= 18 else 32, vp(src.data_ptr()), ZK_MEM_DEVICE, 2, vp(ranges.ctypes.data),
                                           vp(buf.scratch(n).data_ptr()), ZK_MEM_DEVICE), "zk_permute_by_ranges")
        elif kind == "eq":
            _, k = call
            check(lib.zk_eq_table(h, k, vp(point.ctypes.data), vp(buf.scratch(max(k, 1)).data_ptr()), ZK_MEM_DEVICE), "zk_eq_table")
        elif kind == "mle":
            _, n = call
            check(lib.zk_mle_eval(h, n, vp(buf.fr(n).data_ptr()), ZK_MEM_DEVICE, vp(point.ctypes.data), vp(fin.ctypes.data)), "zk_mle_eval")
        elif kind == "sumcheck":
            _, ell, rounds = call
            lib.zk_transcript_append_u64(tr, b"num_var", 7, rounds)
            lib.zk_transcript_append_u64(tr, b"num_poly", 8, ell)
            tabs = (vp * ell)(*[vp(buf.fr(rounds).data_ptr() if i < ell - 1 else buf.scratch(max(rounds, 1)).data_ptr())
                                 for i in range(ell)])
            if rounds and ell > 1:  # the last table stands for the eq table: make it defined data
                buf.scratch(rounds).copy_(buf.fr(rounds))
            check(lib.zk_sumcheck_linear_prove(h, rounds, ell, tabs, ZK_MEM_DEVICE, None, None, tr, vp(msgs.ctypes.data),
                                               vp(chal.ctypes.data), vp(fin_t.ctypes.data), vp(fin.ctypes.data)),
                  "zk_sumcheck_linear_prove")
    ctx.sync()
    nodes_s = time.perf_counter() - t0

    # ---- prove_range (dag/mod.rs:1275-1380)
    t0 = time.perf_counter()
    acc = torch.zeros((1 << TABLE_BLOCK_LOG, 4), dtype=torch.int64, device="cuda")
    bg = rand_fr(1)
    mid = np.zeros((1, 4), dtype=np.uint64)
    dev_idx = {}
    for n in aux_pos:
        ii = torch.arange(1 << n, dtype=torch.int64, device="cuda")
        tt = torch.from_numpy((aux_pos[n] >> np.uint64(n)).view(np.int64)).cuda()
        dev_idx[n] = (ii, tt)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for n in lookups:
        ii, tt = dev_idx[n]
        for _ in range(TABLE_BLOCKS):
            check(lib.zk_range_aux_accumulate(h, n, vp(point.ctypes.data), 1 << n, vp(ii.data_ptr()), vp(tt.data_ptr()), ZK_MEM_DEVICE,
                                              vp(bg.ctypes.data), TABLE_BLOCK_LOG, vp(acc.data_ptr()), ZK_MEM_DEVICE,
                                              vp(mid.ctypes.data)), "zk_range_aux_accumulate")
    table = torch.empty((1 << TABLE_BLOCK_LOG, 4), dtype=torch.int64, device="cuda")
    check(lib.zk_range_table(h, TABLE_BLOCK_LOG, vp(bg.ctypes.data), vp(table.data_ptr()), ZK_MEM_DEVICE), "zk_range_table")
    lib.zk_transcript_append_u64(tr, b"num_var", 7, TABLE_BLOCK_LOG)
    lib.zk_transcript_append_u64(tr, b"num_poly", 8, 2)
    tabs = (vp * 2)(vp(acc.data_ptr()), vp(table.data_ptr()))
    check(lib.zk_sumcheck_linear_prove(h, TABLE_BLOCK_LOG, 2, tabs, ZK_MEM_DEVICE, None, None, tr, vp(msgs.ctypes.data),
                                       vp(chal.ctypes.data), vp(fin_t.ctypes.data), vp(fin.ctypes.data)), "zk_sumcheck_linear_prove")
    ctx.sync()
    range_s = time.perf_counter() - t0
    # one SparseBoolSumcheckProver per auxiliary size, over every term of the model (dag/mod.rs:1343-1351)
    t0 = time.perf_counter()
    for n, terms in sorted(bool_terms.items()):
        m = n + TABLE_BLOCK_LOG
        weights = rand_fr(terms)
        positions = bool_positions[n]
        n_pos = np.full(terms, 1 << n, dtype=np.uint64)
        bmsgs = np.zeros((m, 4, 4), dtype=np.uint64)
        bchal = np.zeros((m, 4), dtype=np.uint64)
        lib.zk_transcript_append_u64(tr, b"num_var", 7, m)
        lib.zk_transcript_append_u64(tr, b"num_poly", 8, 3)
        if world > 1 and comm is not None:
            # the terms are dealt to the ranks in contiguous blocks; the partial messages are summed across the ranks
            per = (terms + world - 1) // world
            lo, hi = min(terms, rank * per), min(terms, (rank + 1) * per)
            check(lib.zk_sumcheck_sparse_bool_prove_sharded(
                h, comm.handle, m, hi - lo, vp(weights[lo:].ctypes.data), vp(positions.data_ptr() + (lo << n) * 8),
                vp(n_pos.ctypes.data), vp(point.ctypes.data), None, None, tr, vp(bmsgs.ctypes.data), vp(bchal.ctypes.data),
                vp(fin.ctypes.data)), "zk_sumcheck_sparse_bool_prove_sharded")
        else:
            check(lib.zk_sumcheck_sparse_bool_prove(h, m, terms, vp(weights.ctypes.data), vp(positions.data_ptr()),
                                                    vp(n_pos.ctypes.data), vp(point.ctypes.data), None, None, tr,
                                                    vp(bmsgs.ctypes.data), vp(bchal.ctypes.data), vp(fin.ctypes.data)),
                  "zk_sumcheck_sparse_bool_prove")
    ctx.sync()
    bool_s = time.perf_counter() - t0

    # ---- openings (dag/mod.rs:876-936): one per dense commitment, two per auxiliary polynomial
    barrier()
    t0 = time.perf_counter()
    # The reference opens its commitments from a rayon loop (dag/mod.rs:893-936): the replay hands them to a few
    # host threads, each call on a lane of the context (ctypes releases the interpreter lock for the call).
    n_dense_open = n_sparse_open = 0

    def open_dense(n):
        if dims == 2:
            out = np.zeros((1 << srs[n].y_log, 4), dtype=np.uint64)
            check(lib.zk_kzh2_open(h, srs[n].handle, n, vp(buf.fr(n, 8).data_ptr()), ZK_MEM_DEVICE, vp(point.ctypes.data), n,
                                   vp(out.ctypes.data)), "zk_kzh2_open")
        else:
            s = srs[n]
            dy = np.zeros((1 << s.y_log, 12), dtype=np.uint64)
            cy = np.zeros((1, 8), dtype=np.uint64)
            fs = np.zeros((1 << s.z_log, 4), dtype=np.uint64)
            check(lib.zk_kzh3_open(h, s.handle, n, vp(buf.fr(n, 8).data_ptr()), ZK_MEM_DEVICE, vp(point.ctypes.data), n,
                                   vp(commitments[("d", n)].ctypes.data), vp(dy.ctypes.data), vp(cy.ctypes.data), vp(fs.ctypes.data)),
                  "zk_kzh3_open")

    def open_selection(n):
        m = n + TABLE_BLOCK_LOG
        s = srs[m]
        if dims == 2:
            out = np.zeros((1 << s.y_log, 4), dtype=np.uint64)
            check(lib.zk_sparse_kzh2_open(h, s.handle, 1 << n, vp(aux_pos[n].ctypes.data), None,
                                          vp(point.ctypes.data), m, vp(out.ctypes.data)), "zk_sparse_kzh2_open")
        else:
            dy = np.zeros((1 << s.y_log, 12), dtype=np.uint64)
            cy = np.zeros((1, 8), dtype=np.uint64)
            fs = np.zeros((1 << s.z_log, 4), dtype=np.uint64)
            check(lib.zk_sparse_kzh3_open(h, s.handle, 1 << n, vp(aux_pos[n].ctypes.data), None,
                                          vp(point.ctypes.data), m, vp(commitments[("s", m)].ctypes.data), vp(dy.ctypes.data),
                                          vp(cy.ctypes.data), vp(fs.ctypes.data)), "zk_sparse_kzh3_open")

    def run_all(fn, items):
        if open_threads <= 1 or len(items) < 2:
            for n in items:
                fn(n)
        else:
            for _ in pool.map(fn, items):  # re-raises a worker's exception
                pass

    pool = ThreadPoolExecutor(max_workers=open_threads) if open_threads > 1 else None
    dense_items = [n for i, n in enumerate(dense) if mine(i)]
    n_dense_open = len(dense_items)
    run_all(open_dense, dense_items)
    dense_open_s = time.perf_counter() - t0
    sel_items = []
    item = len(dense)
    for n in lookups:
        for _ in range(2 * TABLE_BLOCKS):
            if mine(item):
                sel_items.append(n)
            item += 1
    n_sparse_open = len(sel_items)
    run_all(open_selection, sel_items)
    if pool is not None:
        pool.shutdown()
    barrier()
    open_s = time.perf_counter() - t0
    lib.zk_transcript_free(tr)
    for s in srs.values():
        s.close()
    times = torch.tensor([commit_s, nodes_s, range_s, bool_s, open_s], dtype=torch.float64, device="cuda")
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    commit_s, nodes_s, range_s, bool_s, open_s = [float(x) for x in times.tolist()]
    prove_s = nodes_s + range_s + bool_s + open_s
    del buf
    torch.cuda.empty_cache()
    return {
        "metric": "gpt2_small_prove_trace_seconds", "value": prove_s, "unit": "s", "higher_is_better": False, "n_gpus": world,
        "what": "trace replay of the hot-path calls of a GPT-2-small proof (shapes of the reference's DAG, synthetic values), "
                "not a run of the reference's gpt2 bin",
        "config": f"12 layers, d_model 768 (padded 1024), d_ff 3072 (4096), 12 heads (16), sequence length {seq_len}, "
                  f"KZH{dims}, lookups in 5 blocks of 4 table bits; seed {seed}",
        "commit_s": commit_s, "commit_breakdown_s": {"dense": dense_commit_s, "selection": commit_s - dense_commit_s},
        "prove_s": prove_s,
        "prove_breakdown_s": {"node_proofs": nodes_s, "range_preprocessing_and_table_sumcheck": range_s,
                              "sparse_bool_sumchecks": bool_s, "openings": open_s},
        "openings_breakdown_s": {"dense": dense_open_s, "selection": open_s - dense_open_s},
        "opening_threads": open_threads,
        "srs_setup_s": setup_s,
        "calls": {"dense_commits": len(dense), "sparse_commits": TABLE_BLOCKS * len(lookups), "node_calls": counts,
                  "range_accumulates": TABLE_BLOCKS * len(lookups), "sparse_bool_proves": len(bool_terms),
                  "sparse_bool_terms": {str(n + TABLE_BLOCK_LOG): t for n, t in sorted(bool_terms.items())},
                  "dense_openings": len(dense), "sparse_openings": 2 * TABLE_BLOCKS * len(lookups),
                  "this_rank": {"dense_commits": n_dense_commits, "sparse_commits": n_sparse_commits,
                                "dense_openings": n_dense_open, "sparse_openings": n_sparse_open}},
        "parallelism": "1 GPU" if world == 1 else f"commits and openings dealt round-robin to {world} GPUs (no exchange); "
                                                  "the terms of the boolean-check sumchecks dealt to the ranks (partial messages summed); "
                                                  "node proofs and lookup preprocessing on every rank (one shared transcript)",
    }
