"""Shared helpers: run one schedule on the CPU oracle and on the CUDA device and compare."""
import numpy as np

from anneal_b200 import realize as R
from anneal_b200.realize import leaf_inputs


def schedule(tensors):
    items, out_ids = R.build_schedule(tensors)
    return items, out_ids, leaf_inputs(tensors)


def rel_err(got, want, floor=None):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max() if want.size else 1.0
    if floor is not None:
        scale = max(scale, floor)
    if scale == 0:
        scale = 1.0
    return float(np.abs(got - want).max() / scale) if want.size else 0.0


def elementwise_err(got, want, floor=None):
    """max over elements of |got - want| / max(|want|, floor); the floor defaults to the root mean
    square of ``want``: an entry that cancels to nearly zero is held to the accuracy of a typical
    entry of its buffer instead of to a relative error no finite-precision sum can meet."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    if not want.size:
        return 0.0
    if floor is None:
        floor = float(np.sqrt(np.mean(want * want)))
    floor = max(floor, 1e-30)
    return float((np.abs(got - want) / np.maximum(np.abs(want), floor)).max())


#: the per-element bound is this many times the bound on the max-normalised error: the floor is the
#: RMS, typically a third to a fifth of the largest magnitude
ELEMENTWISE_SLACK = 4.0


def compare(cuda, oracle, tensors, tol, binding=None, what=""):
    """Every final output of the schedule, CUDA against oracle: the largest error relative to the
    output's largest magnitude must be within ``tol``, and every element's error relative to
    max(its own magnitude, the output's RMS) within ``ELEMENTWISE_SLACK * tol``."""
    items, out_ids, inputs = schedule(tensors)
    want = oracle.run(items, inputs, binding)
    got = cuda.run(items, inputs, binding)
    assert set(got) == set(want), (sorted(got), sorted(want))
    worst = 0.0
    for k in want:
        assert got[k].shape == want[k].shape, (what, k, got[k].shape, want[k].shape)
        assert np.isfinite(want[k]).all(), f"{what}: oracle produced non-finite values"
        e = rel_err(got[k], want[k])
        worst = max(worst, e)
        assert e <= tol, f"{what}: buffer {k}: rel err {e:.3e} > {tol:.1e}"
        pe = elementwise_err(got[k], want[k])
        assert pe <= ELEMENTWISE_SLACK * tol, f"{what}: buffer {k}: element err {pe:.3e} > {ELEMENTWISE_SLACK * tol:.1e}"
    return worst, {k: got[k] for k in got}, want, out_ids
