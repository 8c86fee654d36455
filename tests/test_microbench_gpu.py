"""The integer-throughput probes run and report sane numbers."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [0, 2, 3, 4])
def test_microbench_runs(ctx, kind):
    from zkes_b200._lib import check, lib

    ms = ctypes.c_float()
    ops = ctypes.c_double()
    check(lib.zk_microbench(ctx.handle, kind, 148 * 8, 256, 2000, ctypes.byref(ms), ctypes.byref(ops)), "zk_microbench")
    assert ms.value > 0 and ops.value > 0
    print(f"kind {kind}: {ops.value / ms.value / 1e9:.2f} Tops/s ({ms.value:.3f} ms)")
