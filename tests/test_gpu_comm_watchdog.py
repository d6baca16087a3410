"""The collective watchdog, exercised without any GPU fault: the stall is a host callback that
holds the communication stream back, the dead communicator is one this process aborted itself."""
import time

import numpy as np
import pytest

from anneal_b200.device import Device, DeviceError
from anneal_b200.uop import dtypes

pytestmark = pytest.mark.gpu


def test_wait_without_pending_work_returns_at_once():
    dev = Device(0)
    try:
        dev.comm_set_timeout(50)
        dev.comm_wait()
        dev.synchronize()
    finally:
        dev.close()


def test_stalled_collective_stream_times_out_and_poisons_the_communicator():
    """No NCCL communicator is attached while the stream is stalled: ncclCommAbort drains the
    device before it returns, and a host callback cannot be cut short the way a kernel waiting for
    a peer is, so with a real communicator the call would last as long as the injected stall."""
    dev = Device(0)
    try:
        buf = dev.buffer(dtypes.float32, 1024).upload(np.ones(1024, np.float32))
        dev.comm_set_timeout(40)
        dev.comm_inject_delay(1500)
        t0 = time.perf_counter()
        with pytest.raises(DeviceError, match="did not finish within 40 ms"):
            dev.synchronize()
        waited = time.perf_counter() - t0
        assert 0.03 <= waited < 1.0                      # gave up at the deadline, not after the stall
        with pytest.raises(DeviceError, match="aborted"):
            dev.allreduce_sum(buf)
        time.sleep(max(0.0, 1.7 - (time.perf_counter() - t0)))   # let the callback return
        dev.comm_set_timeout(0)
        dev.synchronize()
        assert np.array_equal(buf.download(), np.ones(1024, np.float32))
        dev.comm_init(0, 1, dev.comm_unique_id())        # a fresh communicator lifts the refusal
        dev.allreduce_sum(buf)
        dev.synchronize()
    finally:
        dev.close()


def test_abort_on_request():
    dev = Device(0)
    try:
        dev.comm_init(0, 1, dev.comm_unique_id())
        dev.comm_abort()
        buf = dev.buffer(dtypes.float32, 16)
        with pytest.raises(DeviceError, match="aborted"):
            dev.allreduce_sum(buf)
    finally:
        dev.close()
