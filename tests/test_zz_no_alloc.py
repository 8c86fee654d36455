"""zk_fold_lsb_static: the fold for hosts that cannot allocate device memory (its scratch is a
static device array inside the library).  Checked through the C ABI, bit for bit, against
zk_fold_lsb and against the CPU oracle's fix_variables, on calls in a row that reuse the shared
scratch with different sizes; from the second call on the device's free memory must not move
(the first call on a device may load the library's code and the array with it)."""
import ctypes
import random

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_fold_matches_allocating_fold(ctx):
    import torch

    from zkes_b200._lib import ZK_ERR_ARG, ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib
    from zkes_b200.field import R_MOD, to_mont_array

    import coracle

    rnd = random.Random(2024)
    vp = ctypes.c_void_p
    for call, (n, k) in enumerate( [(12, 5), (9, 9), (16, 3), (6, 0), (7, 1)]):  # consecutive calls share the scratch
        ev = [rnd.randrange(R_MOD) for _ in range(1 << n)]
        pt = [rnd.randrange(R_MOD) for _ in range(max(k, 1))]
        evals, point = to_mont_array(ev), to_mont_array(pt)
        expected = to_mont_array(coracle.fix_variables(ev, pt[:k]))  # DenseMLPoly::fix_variables, util/poly.rs:842-887
        want = np.zeros((1 << (n - k), 4), dtype=np.uint64)
        check(lib.zk_fold_lsb(ctx.handle, n, vp(evals.ctypes.data), ZK_MEM_HOST, k, vp(point.ctypes.data),
                              vp(want.ctypes.data), ZK_MEM_HOST), "zk_fold_lsb")
        d_in = torch.from_numpy(evals.view(np.int64)).cuda()
        d_out = torch.zeros((1 << (n - k), 4), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        free_before = torch.cuda.mem_get_info()[0]
        check(lib.zk_fold_lsb_static(n, vp(d_in.data_ptr()), k, vp(point.ctypes.data), vp(d_out.data_ptr()), vp(stream)),
              "zk_fold_lsb_static")
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        if call > 0:  # nothing was allocated: cudaMemGetInfo's free bytes are where they were
            assert free_after == free_before, (n, k, free_before, free_after)
        got = d_out.cpu().numpy().view(np.uint64)
        assert np.array_equal(got, expected), (n, k)
        assert np.array_equal(got, want), (n, k)
    # beyond the static maximum: a clear error, nothing launched
    big = torch.zeros((1 << 17, 4), dtype=torch.int64, device="cuda")
    out = torch.zeros((1 << 16, 4), dtype=torch.int64, device="cuda")
    rc = lib.zk_fold_lsb_static(17, vp(big.data_ptr()), 1, vp(point.ctypes.data), vp(out.data_ptr()), None)
    assert rc == ZK_ERR_ARG
    assert b"static scratch limit" in lib.zk_last_error()
