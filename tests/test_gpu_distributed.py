"""Multi-GPU DistributedUtils test: launches tests/dp_worker.py on 2 GPUs (one process per GPU, NCCL)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 8])
def test_data_parallel_n_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29531 + world), os.path.join(ROOT, "tests", "dp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and f"dp_worker ok {world}" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_single_worker_backend_runs_the_same_code_path():
    """One worker: collectives are identities, DistributedOptimizer == the plain rule (optimizer.jl:8-25)."""
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29532")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "dp_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "dp_worker ok 1" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
