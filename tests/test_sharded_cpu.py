"""Multi-rank logic on CPU: sharding helpers, and a world-size-2 gloo run of the sharded protocol
(tests/sharded_worker.py) that must reproduce the single-process oracle proof."""
import os
import subprocess
import sys

import pytest

from zkes_b200 import dist as zd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_helpers():
    assert zd.shard_range(0, 1, 5) == (0, 32)
    assert zd.shard_range(3, 4, 5) == (24, 32)
    assert zd.shard_sparse([1, 9, 17, 31], [5, 6, 7, 8], 1, 2, 5) == ([1, 15], [7, 8])
    assert zd.shard_dense(list(range(8)), 1, 4) == [2, 3]
    assert zd.tail_tables([[1, 2], [3, 4]]) == [[1, 3], [2, 4]]
    with pytest.raises(ValueError):
        zd.shard_range(0, 3, 5)
    with pytest.raises(ValueError):
        zd.shard_range(0, 8, 2)


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_sharded_protocol(world):
    port = 29500 + world + (os.getpid() % 1000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "sharded_worker.py"), "gloo"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "sharded worker ok" in r.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_injected_failures(world):
    """A rank that never posts its share, a share damaged on the way, a rank that rejects its arguments: every
    rank returns an error status (nobody waits on, nobody returns a proof), the communicator stays retired,
    a fresh one proves correctly."""
    port = 29700 + world + (os.getpid() % 1000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "sharded_worker.py"), "gloo-faults"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "sharded worker ok" in r.stdout
