"""anl_sum_f32_static — the entry point for callers that cannot allocate (their own pool owns the
device, or they cannot afford the allocator's synchronisation). Collected last on purpose.

It must agree with the existing route for the same reduction (a scheduled SUM run through anl_run,
whose split kernels borrow pool scratch) on two calls in a row: the second call sees the first
call's partials in the shared array and must not be affected by them."""
import ctypes as C

import numpy as np
import pytest

from anneal_b200 import realize as R, workloads as W
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes

pytestmark = pytest.mark.gpu


def _static_sum(cuda, xbuf, n, outbuf):
    err = C.create_string_buffer(256)
    # queued on the device's own stream: ordered after the upload of x, before the download of out
    rc = cuda.L.anl_sum_f32_static(xbuf.device_ptr, n, outbuf.device_ptr, cuda.stream, err, 256)
    return rc, err.value.decode()


def test_static_sum_matches_scheduled_sum_twice(cuda):
    out = cuda.buffer(dtypes.float32, 1)
    for n, seed in ((1 << 21, 1), (300_000, 2)):        # second call is shorter: fewer partials than the stale ones
        data = W.normal(9, seed, n)
        R.reset()
        x = Tensor.new_leaf((n,))
        items, out_ids = R.build_schedule([x.sum()])
        xbuf = cuda.buffer(dtypes.float32, n).upload(data)
        want = cuda.run(items, {x.node.idx: xbuf})[out_ids[0]][0]
        rc, msg = _static_sum(cuda, xbuf, n, out)
        assert rc == 0, msg
        cuda.synchronize()
        got = out.download()[0]
        mags = float(np.abs(data.astype(np.float64)).sum())
        assert abs(float(got) - float(want)) <= 1e-5 * mags, (n, got, want)
        assert abs(float(got) - float(data.astype(np.float64).sum())) <= 1e-5 * mags
        xbuf.release()
    out.release()


def test_static_sum_rejects_sizes_beyond_the_maximum(cuda):
    out = cuda.buffer(dtypes.float32, 1)
    x = cuda.buffer(dtypes.float32, 16)
    for n in (0, (1 << 30) + 1):
        rc, msg = _static_sum(cuda, x, n, out)
        assert rc == 7 and "outside" in msg, (rc, msg)
    x.release()
    out.release()
