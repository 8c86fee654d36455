"""The CUDA library's sharded provers on 2 (and 4) GPUs, one process per GPU over NCCL, against
the oracle.  Skipped when the box has a single GPU."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_nccl_sharded_provers(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "sharded_worker.py"), "nccl"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "sharded worker ok" in r.stdout


def test_nccl_rank_failure_contract():
    """One rank of two rejects its arguments and launches nothing; the other's device-side wait is bounded and
    returns ZK_ERR_TIMEOUT; both then get ZK_ERR_COMM until the communicator is made anew, after which the
    prove matches the oracle again.  No kernel is made to fault or hang: the wait simply runs out."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29655", os.path.join(ROOT, "tests", "sharded_worker.py"), "nccl-faults"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "sharded worker ok" in r.stdout
