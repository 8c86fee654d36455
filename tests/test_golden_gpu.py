"""GPU path against the committed golden vectors (tests/golden/sumcheck.json) and the device
input generators against the oracle's."""
import ctypes
import json
import os

import numpy as np
import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, LinearSumcheckProver, SparseDenseSumcheckProver, Transcript

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "sumcheck.json")))


def ints(xs):
    return [int(x, 16) for x in xs]


def test_linear_golden(ctx):
    for case in GOLD["linear"]:
        tables = [ints(t) for t in case["tables"]]
        n = len(tables[0]).bit_length() - 1
        t = Transcript(case["label"].encode())
        p = LinearSumcheckProver(n, len(tables), t)
        pr = p.prove(ctx, [DenseMLPoly.from_evaluations(x) for x in tables], t)
        assert pr.round_messages == [ints(m) for m in case["round_messages"]]
        assert p.challenges == ints(case["challenges"])
        assert pr.final_eval == int(case["final_eval"], 16)
        assert t.challenge_scalar(b"after") == int(case["tail"], 16)


def test_sparse_dense_golden(ctx):
    for case in GOLD["sparse_dense"]:
        t = Transcript(b"sd_sumcheck")
        p = SparseDenseSumcheckProver(case["n"], t)
        pr = p.prove(ctx, case["idx"], ints(case["vals"]), DenseMLPoly.from_evaluations(ints(case["dense"])), t)
        assert pr.round_messages == [ints(m) for m in case["round_messages"]]
        assert pr.final_eval == int(case["final_eval"], 16)
        assert t.challenge_scalar(b"after") == int(case["tail"], 16)


def test_device_generators(ctx):
    import torch
    from zkes_b200._lib import check, lib
    from zkes_b200.field import from_mont_array

    buf = torch.zeros((1000, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_uniform_fr(ctx.handle, 7, 3, 5, 4, ctypes.c_void_p(buf.data_ptr())), "gen")
    assert from_mont_array(buf[:4].cpu().numpy().view(np.uint64)) == ints(GOLD["poly"]["uniform_seed7"])
    check(lib.zk_gen_small_fr(ctx.handle, 7, 3, 5, 8, 8, ctypes.c_void_p(buf.data_ptr())), "gen")
    assert from_mont_array(buf[:8].cpu().numpy().view(np.uint64)) == ints(GOLD["poly"]["small_seed7_bits8"])
    check(lib.zk_gen_uniform_fr(ctx.handle, 11, 0, 100, 1000, ctypes.c_void_p(buf.data_ptr())), "gen")
    assert from_mont_array(buf.cpu().numpy().view(np.uint64)) == o.gen_uniform_fr(11, 0, 100, 1000)
    check(lib.zk_gen_small_fr(ctx.handle, 11, 1, 0, 1000, 16, ctypes.c_void_p(buf.data_ptr())), "gen")
    got = from_mont_array(buf.cpu().numpy().view(np.uint64))
    assert got == o.gen_small_fr(11, 1, 0, 1000, 16)
    assert all(v < (1 << 15) or o.R_MOD - v <= (1 << 15) for v in got)
