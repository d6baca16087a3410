"""Data-parallel update paths and the loss of a rank, on two GPUs when the box has them (one process
per GPU; skipped on a one-GPU box)."""
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


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_a_rank_that_leaves_between_steps_is_survived():
    """rank_failure_check.py: the peer exits cleanly between steps; the survivor's next collective is
    ended by the watchdog with ANL_ERR_COMM, further collectives refuse, a new communicator recovers."""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    # every rank also arms its own 120 s alarm; the launcher is killed with its whole process group if
    # it overstays, so nothing can be left holding a GPU
    p = subprocess.Popen([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29534", os.path.join(here, "rank_failure_check.py")],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, start_new_session=True)
    try:
        out, err = p.communicate(timeout=200)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, 9)
        out, err = p.communicate()
        raise AssertionError(("timed out", out[-2000:], err[-2000:]))
    assert "RANK_FAILURE OK" in out, (out[-2000:], err[-2000:])
