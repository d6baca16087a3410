"""Data-parallel update paths on two GPUs, when the box has them (one process per GPU)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_sharded_update_equals_allreduce_update_on_two_ranks():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "dp_check.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "DP_CHECK OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
