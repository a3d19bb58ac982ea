"""Multi-GPU parity: 2 (or more) ranks, one per GPU, sharded max with allreduce(max) and row-sharded
matmuls with allgather, checked against the CPU oracle on every rank. Skipped on a one-GPU box."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_sharded_workloads_on_all_gpus(gpu):
    n = gpu.driver.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4 if n < 8 else 8
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", "29731", os.path.join(HERE, "multi_rank_worker.py")], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-4000:]
    assert r.stdout.count(" ok") == world
    print("\n".join(l for l in r.stdout.splitlines() if "multi" in l))      # whether the box had an NVLink multicast mapping to offer
