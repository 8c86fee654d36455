"""Worker for the multi-rank tests (launched by torch.distributed.run, one process per rank).

  mode "gloo": CPU emulation of the sharded protocol with the oracle's arithmetic and the
               product's sharding helpers, exchanged over gloo; checks equality with the
               single-process oracle proof.
  mode "nccl": the CUDA library's sharded provers on one GPU per rank against the oracle.
  mode "gloo-faults": failures injected on the host among CPU ranks (a rank that never posts its share, a
               share damaged on the way, a rank that rejects its arguments): every rank must come back with
               an error status instead of waiting on, the communicator must stay retired until it is made
               anew, and a fresh one must prove correctly.
  mode "nccl-faults": the same contract through the CUDA library on 2+ GPUs: one rank rejects its arguments
               before launching anything, the other's bounded device-side wait runs out (ZK_ERR_TIMEOUT), both
               then see ZK_ERR_COMM until the communicator is made anew."""
import os
import random
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import pyoracle as o  # noqa: E402
from zkes_b200 import dist as zd  # noqa: E402


def problem(n, nnz, seed):
    rnd = random.Random(seed)
    idx = sorted(rnd.sample(range(1 << n), nnz))
    vals = [o.fr_from_int(rnd.randrange(-128, 128)) for _ in idx]
    dense = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    f = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
    return idx, vals, dense, f


def emulate_sharded_linear(tables, rank, world, label, replicate_entries=0):
    """The sharded protocol with big-integer arithmetic: local partial messages, all-gather, sum,
    replicated transcript, local folds, then the gathered tail.  With replicate_entries, once all ranks
    together hold at most that many entries per table the chunks are gathered (rank order = table order)
    and every rank runs the remaining rounds on the whole table."""
    n = len(tables[0]).bit_length() - 1
    L = len(tables)
    local = [zd.shard_dense(t, rank, world) for t in tables]
    tr = o.Transcript(label)
    tr.append_u64(b"num_var", n)
    tr.append_u64(b"num_poly", L)
    helper = o.LinearSumcheckProver.__new__(o.LinearSumcheckProver)
    helper.num_poly = L
    msgs, chals = [], []
    n_local = n - zd.log2_exact(world)
    for _ in range(n_local):
        if replicate_entries and len(local[0]) * world <= replicate_entries:
            whole = []
            for t in local:
                parts = [None] * world
                dist.all_gather_object(parts, t)
                whole.append([v for part in parts for v in part])
            while len(whole[0]) > 1:
                helper.a_arrays = whole
                msg = helper._round_message()
                for m in msg:
                    tr.append_scalar(b"round_message", m)
                ch = tr.challenge_scalar(b"challenge")
                msgs.append(msg)
                chals.append(ch)
                whole = [o.fix_variables(t, [ch]) for t in whole]
            final = 1
            for t in whole:
                final = final * t[0] % o.R_MOD
            return msgs, chals, [t[0] for t in whole], final
        helper.a_arrays = local
        part = helper._round_message()
        gathered = [None] * world
        dist.all_gather_object(gathered, part)
        msg = [sum(g[c] for g in gathered) % o.R_MOD for c in range(L + 1)]
        for m in msg:
            tr.append_scalar(b"round_message", m)
        ch = tr.challenge_scalar(b"challenge")
        msgs.append(msg)
        chals.append(ch)
        local = [o.fix_variables(t, [ch]) for t in local]
    finals = [None] * world
    dist.all_gather_object(finals, [t[0] for t in local])
    tail = zd.tail_tables(finals)
    for _ in range(n - n_local):
        helper.a_arrays = tail
        msg = helper._round_message()
        for m in msg:
            tr.append_scalar(b"round_message", m)
        ch = tr.challenge_scalar(b"challenge")
        msgs.append(msg)
        chals.append(ch)
        tail = [o.fix_variables(t, [ch]) for t in tail]
    final = 1
    for t in tail:
        final = final * t[0] % o.R_MOD
    return msgs, chals, [t[0] for t in tail], final


def emulate_sharded_sbool(weights, positions, eq_challenge, rank, world, label):
    """The boolean-check prover with its terms dealt to the ranks (rank r holds terms r, r + world, ...), in big
    integers: partial round messages over the local terms, all-gather, sum, replicated transcript, local folds;
    the final value is summed the same way (linear_prover.rs:529-656 run on a share of the terms)."""
    n = len(eq_challenge)
    tr = o.Transcript(label)
    tr.append_u64(b"num_var", n)
    tr.append_u64(b"num_poly", 3)
    terms = [(w, sorted((p, 1) for p in pos)) for w, pos in zip(weights[rank::world], positions[rank::world])]
    eq = o.evaluate_lagrange_basis(eq_challenge)

    def summed(vals):
        parts = [None] * world
        dist.all_gather_object(parts, vals)
        return [sum(p[c] for p in parts) % o.R_MOD for c in range(len(vals))]

    msgs, chals = [], []
    for _ in range(n):
        t = [0, 0, 0, 0]
        for w, entries in terms:
            for rest, v0, v1 in o._pair_walk(entries):
                e0, e1 = eq[2 * rest], eq[2 * rest + 1]
                for c in range(4):
                    aux = v0 + c * (v1 - v0)
                    t[c] += w * aux * (aux - 1) * (e0 + c * (e1 - e0))
        msg = summed([x % o.R_MOD for x in t])
        for m in msg:
            tr.append_scalar(b"round_message", m)
        ch = tr.challenge_scalar(b"challenge")
        msgs.append(msg)
        chals.append(ch)
        eq = o.fix_variables(eq, [ch])
        terms = [(w, [(rest, (v0 + ch * (v1 - v0)) % o.R_MOD) for rest, v0, v1 in o._pair_walk(entries)
                      if (v0 + ch * (v1 - v0)) % o.R_MOD]) for w, entries in terms]
    inner = 0
    for w, entries in terms:
        v = entries[0][1] if entries and entries[0][0] == 0 else 0
        inner += w * v * (v - 1)
    fin = summed([(eq[0] if eq else 0) * inner % o.R_MOD])[0]
    return msgs, chals, fin, tr


class ExchangeError(Exception):
    def __init__(self, status):
        super().__init__(status)
        self.status = status


class HostBox:
    """CPU stand-in for the ranks' exchange boxes with the rules of the library's communicator: a share is
    posted under its exchange number, a wait for the others' shares is bounded, and the first failure
    retires the box on the rank that saw it (every later exchange fails at once)."""

    def __init__(self, store, name, rank, world, wait_s=1.5):
        self.store, self.name, self.rank, self.world, self.wait_s = store, name, rank, world, wait_s
        self.xseq = 0
        self.poisoned = False

    def exchange_sum(self, vals, skip_post=False, damage=False):
        import datetime
        import pickle
        if self.poisoned:
            raise ExchangeError("COMM")
        self.xseq += 1
        mine = [(v + 1) % o.R_MOD for v in vals] if damage else list(vals)
        if not skip_post:
            self.store.set(f"{self.name}/x{self.xseq}/{self.rank}", pickle.dumps(mine))
        total = [0] * len(vals)
        for r in range(self.world):
            key = f"{self.name}/x{self.xseq}/{r}"
            try:
                self.store.wait([key], datetime.timedelta(seconds=self.wait_s))
            except Exception:
                self.poisoned = True
                raise ExchangeError("TIMEOUT")
            share = vals if r == self.rank and not skip_post and not damage else pickle.loads(self.store.get(key))
            total = [(a + b) % o.R_MOD for a, b in zip(total, share)]
        return total


def boxed_sharded_linear(box, tables, rank, world, label, fault=None):
    """The sharded protocol over a HostBox.  fault = (kind, rank, round): "skip" (the rank never posts that
    round's share), "damage" (its share arrives changed), "args" (it rejects its arguments before round 0).
    Returns ("OK", proof parts) or raises ExchangeError with the status the library would return."""
    from zkes_b200 import SumcheckVerifier, Transcript
    if box.poisoned:
        raise ExchangeError("COMM")
    n = len(tables[0]).bit_length() - 1
    L = len(tables)
    try:
        if fault and fault[0] == "args" and fault[1] == rank:
            raise ExchangeError("ARG")
        local = [zd.shard_dense(t, rank, world) for t in tables]
        tr = o.Transcript(label)
        tr.append_u64(b"num_var", n)
        tr.append_u64(b"num_poly", L)
        helper = o.LinearSumcheckProver.__new__(o.LinearSumcheckProver)
        helper.num_poly = L
        msgs, chals = [], []
        n_local = n - zd.log2_exact(world)
        for rnd_i in range(n_local):
            helper.a_arrays = local
            part = helper._round_message()
            hit = fault and fault[1] == rank and fault[2] == rnd_i
            msg = box.exchange_sum(part, skip_post=bool(hit and fault[0] == "skip"), damage=bool(hit and fault[0] == "damage"))
            for m in msg:
                tr.append_scalar(b"round_message", m)
            ch = tr.challenge_scalar(b"challenge")
            msgs.append(msg)
            chals.append(ch)
            local = [o.fix_variables(t, [ch]) for t in local]
        finals = [box.exchange_sum([t[0] if r == rank else 0 for r in range(world) for t in local])]
        per_rank = [finals[0][r * L:(r + 1) * L] for r in range(world)]
        tail = zd.tail_tables(per_rank)
        for _ in range(n - n_local):
            helper.a_arrays = tail
            msg = helper._round_message()
            for m in msg:
                tr.append_scalar(b"round_message", m)
            ch = tr.challenge_scalar(b"challenge")
            msgs.append(msg)
            chals.append(ch)
            tail = [o.fix_variables(t, [ch]) for t in tail]
        final = 1
        for t in tail:
            final = final * t[0] % o.R_MOD
        # the library's self-check of a sharded prove: every summed message continues the round before it
        vt = Transcript(label)
        res, _ = SumcheckVerifier(n, L, vt).verify(vt, msgs, (msgs[0][0] + msgs[0][1]) % o.R_MOD)
        if res is None or res != final:
            raise ExchangeError("COMM")
        return msgs, chals, final
    except ExchangeError:
        box.poisoned = True
        raise


def gloo_faults(rank, world):
    store = dist.distributed_c10d._get_default_store()
    n = 6
    idx, vals, dense, f = problem(n, 20, 9)
    t = o.Transcript(b"faults")
    p = o.LinearSumcheckProver(n, 2, t)
    want = p.prove([dense, f], t)

    def run(box, fault=None):
        try:
            got = boxed_sharded_linear(box, [dense, f], rank, world, b"faults", fault)
            assert got[0] == want.round_messages and got[1] == p.challenges and got[2] == want.final_eval
            return "OK"
        except ExchangeError as e:
            return e.status

    victim = world - 1
    for case, fault in enumerate([("skip", victim, 2), ("damage", victim, 1), ("args", victim, 0)]):
        box = HostBox(store, f"case{case}", rank, world)
        assert run(box) == "OK"                      # a healthy prove first
        st = run(box, fault)
        statuses = [None] * world
        dist.all_gather_object(statuses, st)
        assert all(s != "OK" for s in statuses), (fault, statuses)   # nobody returns a proof, nobody hangs
        if fault[0] == "args":
            assert statuses[victim] == "ARG" and all(s == "TIMEOUT" for r, s in enumerate(statuses) if r != victim)
        if fault[0] == "damage":
            assert all(s == "COMM" for s in statuses), statuses        # the round chain breaks on every rank alike
        assert run(box) == "COMM"                    # retired: fails at once, on every rank
        dist.barrier()
        fresh = HostBox(store, f"case{case}-fresh", rank, world)
        assert run(fresh) == "OK"


def nccl_faults(rank, world, local_rank):
    import ctypes
    import numpy as np
    from zkes_b200 import Context, DenseMLPoly, Transcript
    from zkes_b200._lib import (ZK_ERR_ARG, ZK_ERR_COMM, ZK_ERR_TIMEOUT, ZK_MEM_HOST, ZK_OPT_EXCHANGE_WAIT_MS, ZkError, lib)
    ctx = Context(local_rank)
    ctx.set_option(ZK_OPT_EXCHANGE_WAIT_MS, 400)
    comm = zd.Comm(ctx)
    assert comm.peer_exchange, "the ranks could not map each other's boxes: the bounded wait is the peer path's"
    n = 13  # all local rounds in the resident kernel, exchanged through the boxes (no NCCL collective on the path)
    idx, vals, dense, f = problem(n, 50, 5)
    ot = o.Transcript(b"faults")
    op = o.LinearSumcheckProver(n, 2, ot)
    want = op.prove([dense, f], ot)
    local = [DenseMLPoly.from_evaluations(zd.shard_dense(tb, rank, world)) for tb in (dense, f)]

    def prove(c):
        t = Transcript(b"faults")
        t.append_u64(b"num_var", n)
        t.append_u64(b"num_poly", 2)
        return zd.sharded_linear_prove(ctx, c, n, local, t)

    msgs, chals, _, fin = prove(comm)
    assert msgs == want.round_messages and fin == want.final_eval
    dist.barrier()
    # the last rank rejects its arguments (no table pointers) and launches nothing; the others wait, bounded
    if rank == world - 1:
        rc = lib.zk_sumcheck_linear_prove_sharded(ctx.handle, comm.handle, n, 0, None, ZK_MEM_HOST, None, None, None, None,
                                                  None, None, None)
        assert rc == ZK_ERR_ARG, rc
    else:
        try:
            prove(comm)
            raise AssertionError("a prove with a rank missing returned a proof")
        except ZkError as e:
            assert e.code == ZK_ERR_TIMEOUT, e
    try:  # retired on every rank: nothing is launched, the status comes back at once
        prove(comm)
        raise AssertionError("a retired communicator proved")
    except ZkError as e:
        assert e.code == ZK_ERR_COMM, e
    dist.barrier()
    comm.close()
    comm = zd.Comm(ctx)
    msgs, chals, _, fin = prove(comm)  # a communicator made anew works, and the context was never lost
    assert msgs == want.round_messages and chals == op.challenges and fin == want.final_eval
    comm.close()
    ctx.close()


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "gloo-faults":
        dist.init_process_group("gloo")
        gloo_faults(rank, world)
    elif mode == "nccl-faults":
        local_rank = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        nccl_faults(rank, world, local_rank)
    elif mode == "gloo":
        dist.init_process_group("gloo")
        for n, nnz, seed in [(5, 7, 1), (7, 30, 2)]:
            idx, vals, dense, f = problem(n, nnz, seed)
            a = [0] * (1 << n)
            for i, v in zip(idx, vals):
                a[i] = v
            # the sparse helper and the dense one describe the same shard
            li, lv = zd.shard_sparse(idx, vals, rank, world, n)
            la = zd.shard_dense(a, rank, world)
            assert [la[i] for i in li] == lv and sum(1 for v in la if v) == sum(1 for v in lv if v)
            got = emulate_sharded_linear([a, dense], rank, world, b"sharded")
            t = o.Transcript(b"sharded")
            p = o.LinearSumcheckProver(n, 2, t)
            pr = p.prove([a, dense], t)
            assert got[0] == pr.round_messages and got[1] == p.challenges and got[3] == pr.final_eval
            got3 = emulate_sharded_linear([a, dense, f], rank, world, b"sharded")
            t = o.Transcript(b"sharded")
            p = o.LinearSumcheckProver(n, 3, t)
            pr = p.prove([a, dense, f], t)
            assert got3[0] == pr.round_messages and got3[3] == pr.final_eval
            for entries in (1 << n, 8):  # gathered at once; gathered after some sharded rounds
                rep = emulate_sharded_linear([a, dense, f], rank, world, b"sharded", replicate_entries=entries)
                assert rep[0] == pr.round_messages and rep[1] == p.challenges and rep[3] == pr.final_eval
                assert rep[2] == [x[0] for x in p.a_arrays]
        # the boolean-check prover with its terms dealt to the ranks (with fewer terms than ranks, some hold none)
        for bn, terms, k in [(3, 1, 4), (5, 3, 9), (7, 2 * world + 1, 40)]:
            rnd = random.Random(bn * 31 + terms)
            w = [rnd.randrange(o.R_MOD) for _ in range(terms)]
            pos = [rnd.sample(range(1 << bn), k) for _ in range(terms)]
            pt = [rnd.randrange(o.R_MOD) for _ in range(bn)]
            msgs, chals, fin, tr = emulate_sharded_sbool(w, pos, pt, rank, world, b"range")
            ot = o.Transcript(b"range")
            op = o.SparseBoolSumcheckProver(bn, ot)
            opr = op.prove(w, pos, pt, ot)
            assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
            assert tr.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
    else:
        local_rank = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from zkes_b200 import Context, DenseMLPoly, Transcript
        ctx = Context(local_rank)
        comm = zd.Comm(ctx)
        from zkes_b200._lib import ZK_OPT_PEER_EXCHANGE, ZK_OPT_REPLICATE_LOG
        if rank == 0:
            print("peer exchange mapped:", comm.peer_exchange, flush=True)
        # the round messages cross the ranks through peer memory (1, when the boxes could be mapped) or NCCL (0)
        for peer in (1, 0):
          ctx.set_option(ZK_OPT_PEER_EXCHANGE, peer)
          # 0: every local round sharded; 8: sharded rounds, then the tables are gathered with a challenge still
          # to bind; 18 (the default): gathered at once at these sizes
          for replicate_log in (0, 8, 18):
              ctx.set_option(ZK_OPT_REPLICATE_LOG, replicate_log)
              for n, nnz, seed in [(3, 2, 1), (6, 9, 2), (11, 100, 3), (13, 3000, 4)]:
                  if n < zd.log2_exact(world):
                      continue
                  idx, vals, dense, f = problem(n, nnz, seed)
                  a = [0] * (1 << n)
                  for i, v in zip(idx, vals):
                      a[i] = v
                  for tables in ([a, dense], [dense, f, a], [f]):
                      t = Transcript(b"sharded")
                      t.append_u64(b"num_var", n)
                      t.append_u64(b"num_poly", len(tables))
                      local = [DenseMLPoly.from_evaluations(zd.shard_dense(tb, rank, world)) for tb in tables]
                      msgs, chals, fin_t, fin = zd.sharded_linear_prove(ctx, comm, n, local, t)
                      ot = o.Transcript(b"sharded")
                      op = o.LinearSumcheckProver(n, len(tables), ot)
                      opr = op.prove(tables, ot)
                      assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
                      assert fin_t == [x[0] for x in op.a_arrays]
                      assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
                  t = Transcript(b"sharded")
                  t.append_u64(b"num_var", n)
                  t.append_u64(b"num_poly", 2)
                  li, lv = zd.shard_sparse(idx, vals, rank, world, n)
                  ld = DenseMLPoly.from_evaluations(zd.shard_dense(dense, rank, world))
                  msgs, chals, fin_t, fin = zd.sharded_sparse_dense_prove(ctx, comm, n, li, lv, ld, t)
                  ot = o.Transcript(b"sharded")
                  op, opr = o.sparse_dense_prove(n, idx, vals, dense, ot)
                  assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
        # ---- large enough for the sharded launch to hand over at 2^14 gathered entries to the launch that runs the rest
        # of the rounds ahead of their challenges on every rank (defaults: peer exchange, replication at 2^18)
        ctx.set_option(ZK_OPT_PEER_EXCHANGE, 1)
        ctx.set_option(ZK_OPT_REPLICATE_LOG, 18)
        n = 15 + zd.log2_exact(world) - 1
        idx, vals, dense, f = problem(n, 4000, 9)
        a = [0] * (1 << n)
        for i, v in zip(idx, vals):
            a[i] = v
        for tables in ([a, dense], [dense, f, a]):
            t = Transcript(b"sharded")
            t.append_u64(b"num_var", n)
            t.append_u64(b"num_poly", len(tables))
            local = [DenseMLPoly.from_evaluations(zd.shard_dense(tb, rank, world)) for tb in tables]
            msgs, chals, fin_t, fin = zd.sharded_linear_prove(ctx, comm, n, local, t)
            ot = o.Transcript(b"sharded")
            op = o.LinearSumcheckProver(n, len(tables), ot)
            opr = op.prove(tables, ot)
            assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
            assert fin_t == [x[0] for x in op.a_arrays]
            assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
        t = Transcript(b"sharded")
        t.append_u64(b"num_var", n)
        t.append_u64(b"num_poly", 2)
        li, lv = zd.shard_sparse(idx, vals, rank, world, n)
        ld = DenseMLPoly.from_evaluations(zd.shard_dense(dense, rank, world))
        msgs, chals, fin_t, fin = zd.sharded_sparse_dense_prove(ctx, comm, n, li, lv, ld, t)
        ot = o.Transcript(b"sharded")
        op, opr = o.sparse_dense_prove(n, idx, vals, dense, ot)
        assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
        # ---- the boolean-check prover with its terms dealt to the ranks (a rank may hold none), through peer memory
        # and through NCCL
        for peer in (1, 0):
            ctx.set_option(ZK_OPT_PEER_EXCHANGE, peer)
            for bn, terms, k in [(4, 1, 5), (6, 3, 10), (9, 5, 100), (12, 2 * world + 1, 700), (0, 2, 1)]:
                rnd = random.Random(bn * 31 + terms)
                w = [rnd.randrange(o.R_MOD) for _ in range(terms)]
                pos = [rnd.sample(range(1 << bn), min(k, 1 << bn)) for _ in range(terms)]
                pt = [rnd.randrange(o.R_MOD) for _ in range(bn)]
                t = Transcript(b"range")
                t.append_u64(b"num_var", bn)
                t.append_u64(b"num_poly", 3)
                msgs, chals, fin = zd.sharded_sparse_bool_prove(ctx, comm, bn, w[rank::world], pos[rank::world], pt, t)
                ot = o.Transcript(b"range")
                op = o.SparseBoolSumcheckProver(bn, ot)
                opr = op.prove(w, pos, pt, ot)
                assert msgs == opr.round_messages and chals == op.challenges and fin == opr.final_eval
                assert t.challenge_scalar(b"after") == ot.challenge_scalar(b"after")
        ctx.set_option(ZK_OPT_PEER_EXCHANGE, 1)
        # ---- MSM by point range, KZH commit by x-rows, fix_from_right over the top variables
        from zkes_b200 import curve
        rnd = random.Random(77)
        pts = [o.g1_mul(o.G1_GEN, rnd.randrange(1, o.R_MOD)) for _ in range(16 * world)]
        sc = [rnd.randrange(o.R_MOD) if i % 3 else o.fr_from_int(rnd.randrange(-128, 128)) for i in range(len(pts))]
        b, e = rank * 16, (rank + 1) * 16
        got = zd.sharded_msm(ctx, comm, curve.affine_to_array(pts[b:e]), sc[b:e])
        assert got == o.g1_msm(pts, sc)
        for dims, n in ((2, 6), (3, 7)):
            if dims == 2:
                xl, yl = o.kzh2_degrees(n)
                d = o.gen_uniform_fr(5, 0, 0, 2 + (1 << xl) + (1 << yl))
                tx, ty, alpha = d[1:1 + (1 << xl)], d[1 + (1 << xl):1 + (1 << xl) + (1 << yl)], d[-1]
                osrs = o.KZH2SRS(n, d[0], tx, ty, alpha)
                srs = zd.sharded_kzh_setup(ctx, comm, 2, n, osrs.g, tx, ty, alpha=alpha)
                full = osrs.h_xy
            else:
                xl, yl, zl = o.kzh3_degrees(n)
                d = o.gen_uniform_fr(6, 0, 0, 1 + (1 << xl) + (1 << yl) + (1 << zl))
                tx = d[1:1 + (1 << xl)]
                ty = d[1 + (1 << xl):1 + (1 << xl) + (1 << yl)]
                tz = d[1 + (1 << xl) + (1 << yl):]
                osrs = o.KZH3SRS(n, d[0], tx, ty, tz)
                srs = zd.sharded_kzh_setup(ctx, comm, 3, n, osrs.g, tx, ty, tau_z=tz)
                full = osrs.h_xyz
            lo, hi = zd.shard_range(rank, world, n)
            assert srs.read(0, 0, hi - lo) == full[lo:hi]
            f = [rnd.randrange(o.R_MOD) if i % 2 else o.fr_from_int(rnd.randrange(-128, 128)) for i in range(1 << n)]
            c, dx, dx_jac = zd.sharded_kzh_commit(ctx, comm, srs, f[lo:hi], with_jacobian=True)
            oc, odx = (o.kzh2_commit if dims == 2 else o.kzh3_commit)(osrs, f)
            assert c == oc and dx == odx
            full_pt = [rnd.randrange(o.R_MOD) for _ in range(n)]
            if dims == 2:
                assert zd.sharded_kzh_open(ctx, comm, srs, full_pt, f[lo:hi]) == o.kzh2_open(osrs, full_pt, odx, f)[1]
            else:
                dy, cy, fs = zd.sharded_kzh_open(ctx, comm, srs, full_pt, f[lo:hi], dx_jac)
                _, ody, ocy, ofs = o.kzh3_open(osrs, full_pt, odx, f)
                assert dy == ody and cy == ocy and fs == ofs
            pt = [rnd.randrange(o.R_MOD) for _ in range(xl)]
            got = zd.sharded_fix_from_right(ctx, comm, n, f[lo:hi], pt)
            assert got == o.fix_variables_from_right(f, pt)
            srs.close()
        comm.close()
        ctx.close()
    dist.barrier()
    if rank == 0:
        print("sharded worker ok:", mode, "world", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
