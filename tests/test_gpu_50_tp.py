"""Tensor-parallel decoders on 2, 4 and 8 GPUs of one box against the CPU oracle.  Skipped on a
single-GPU box; the sharding arithmetic itself is covered on CPU ranks by tests/test_tp_plan.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(HERE, "tp_check.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500)
    sys.stdout.write(r.stdout[-3000:])
    assert r.returncode == 0, r.stderr[-3000:]
