"""zk_fold_lsb_static: the fold for hosts that cannot allocate device memory (its scratch is a
static device array inside the library).  Checked through the C ABI against zk_fold_lsb,
bit for bit, on two calls in a row that reuse the shared scratch with different sizes."""
import ctypes
import random

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_fold_matches_allocating_fold(ctx):
    import torch

    from zkes_b200._lib import ZK_ERR_ARG, ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
    from zkes_b200.field import R_MOD, to_mont_array

    rnd = random.Random(2024)
    vp = ctypes.c_void_p
    for n, k in [(12, 5), (9, 9), (16, 3), (6, 0), (7, 1)]:  # consecutive calls share the scratch
        evals = to_mont_array([rnd.randrange(R_MOD) for _ in range(1 << n)])
        point = to_mont_array([rnd.randrange(R_MOD) for _ in range(max(k, 1))])
        want = np.zeros((1 << (n - k), 4), dtype=np.uint64)
        check(lib.zk_fold_lsb(ctx.handle, n, vp(evals.ctypes.data), ZK_MEM_HOST, k, vp(point.ctypes.data),
                              vp(want.ctypes.data), ZK_MEM_HOST), "zk_fold_lsb")
        d_in = torch.from_numpy(evals.view(np.int64)).cuda()
        d_out = torch.zeros((1 << (n - k), 4), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        check(lib.zk_fold_lsb_static(n, vp(d_in.data_ptr()), k, vp(point.ctypes.data), vp(d_out.data_ptr()), vp(stream)),
              "zk_fold_lsb_static")
        torch.cuda.synchronize()
        got = d_out.cpu().numpy().view(np.uint64)
        assert np.array_equal(got, want), (n, k)
    # beyond the static maximum: a clear error, nothing launched
    big = torch.zeros((1 << 17, 4), dtype=torch.int64, device="cuda")
    out = torch.zeros((1 << 16, 4), dtype=torch.int64, device="cuda")
    rc = lib.zk_fold_lsb_static(17, vp(big.data_ptr()), 1, vp(point.ctypes.data), vp(out.data_ptr()), None)
    assert rc == ZK_ERR_ARG
    assert b"static scratch limit" in lib.zk_last_error()
