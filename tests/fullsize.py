"""Kernel-by-kernel parity at benchmark size.

The CPU oracle cannot run a 3 TFLOP step, but it can evaluate any one kernel at a few thousand of
its output positions (``OracleExecutor.sample_item``): a contraction with K terms then costs n*K.
The device runs the whole schedule once with every output kept (no slot shared, so nothing is
overwritten and every fused launch still has to produce each kernel's buffer); each kernel is then
checked on its own: the oracle is given the DEVICE's values of that kernel's inputs and must
reproduce the device's values of its output at the sampled positions.  An error in any kernel —
a wrong tile, a dropped k-block, an operand read with the wrong major-ness — shows in that kernel's
row, and errors do not compound from kernel to kernel.
"""
import dataclasses

import numpy as np


def unaliased(items):
    """Copies of ``items`` in which no output shares a slot: the device returns all of them."""
    out = []
    for it in items:
        bufs = [dataclasses.replace(b) for b in it.bufs]
        bufs[0].slot = -1
        out.append(dataclasses.replace(it, bufs=bufs))
    return out


def sample_positions(shape, n, rng):
    """n positions of a row-major output: corners, tile edges of the contraction kernels (multiples
    of 128 and 256 and their neighbours) and uniformly drawn ones."""
    total = int(np.prod(shape)) if len(shape) else 1
    if total <= n:
        return np.arange(total, dtype=np.int64)
    picks = [0, total - 1]
    if len(shape) >= 2:
        rows, cols = int(np.prod(shape[:-1])), int(shape[-1])
        edge_r = sorted({r for b in (0, 127, 128, 255, 256, rows // 2, rows - 129, rows - 1) for r in (b,) if 0 <= r < rows})
        edge_c = sorted({c for b in (0, 31, 32, 127, 128, 255, 256, cols // 2, cols - 33, cols - 1) for c in (b,) if 0 <= c < cols})
        picks += [r * cols + c for r in edge_r for c in edge_c]
    picks = np.array(picks, dtype=np.int64)
    rest = rng.integers(0, total, size=max(n - picks.size, 0), dtype=np.int64)
    return np.unique(np.concatenate([picks, rest]))


def elementwise_error(got, want, floor):
    """max over elements of |got - want| / max(|want|, floor)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float((np.abs(got - want) / np.maximum(np.abs(want), floor)).max()) if want.size else 0.0


#: how many modelled standard deviations of legitimate device-versus-oracle difference are allowed
#: on top of the stated tolerance (see ``OracleExecutor.sample_item(noise=True)``)
NOISE_SIGMAS = 6.0


def check_every_kernel(cuda, oracle, items, inputs, tol, binding=None, samples=4096, seed=0, tol_of=None):
    """Runs ``items`` on the device keeping every output, then checks each kernel against the oracle
    at sampled positions.  Per element

        |device - oracle| <= tol * max(|oracle|, floor) + NOISE_SIGMAS * sigma

    floor = the root mean square of the oracle's sampled values of that kernel (an element that
    cancels to nearly zero is held to the accuracy of a typical element of its buffer); sigma = the
    oracle's model of how far two valid evaluations of this element differ (another order of
    additions in a REDUCE, another approximation of exp2, an f16 rounding tipped by either).  For a
    well-conditioned kernel sigma is far below tol * floor and the check is the stated tolerance;
    for a sum whose terms cancel — the row statistics of a softmax gradient that are zero in exact
    arithmetic — it is what makes a comparison possible at all.  Returns the device's values and a
    list of (kernel, worst error relative to max(|oracle|, floor), worst ratio of the noise
    allowance to the tolerance term): a ratio well below 1 says the check was the stated tolerance."""
    keep = unaliased(items)
    got = cuda.run(keep, inputs, binding)
    known = dict(inputs)
    known.update(got)
    rng = np.random.default_rng(seed)
    report = []
    for k, it in enumerate(keep):
        ob = it.bufs[0]
        dev_out = got[ob.uop_idx]
        assert np.isfinite(dev_out).all(), f"kernel {k}: device produced non-finite values"
        sym = list(binding.values())[0] if binding else 0          # the one bound extent (0 marks it in a shape)
        shape = tuple(sym if s == 0 else s for s in ob.shape)
        pos = sample_positions(shape, samples, rng)
        idx, want, sigma = oracle.sample_item(it, known, pos, binding, noise=True)
        assert np.isfinite(want).all(), f"kernel {k}: oracle produced non-finite values"
        w = want.astype(np.float64)
        floor = max(float(np.sqrt(np.mean(w * w))), 1e-30)
        t = tol_of(k, it) if tol_of else tol
        d = np.abs(dev_out[idx].astype(np.float64) - w)
        allowed = t * np.maximum(np.abs(w), floor) + NOISE_SIGMAS * sigma
        worst = int(np.argmax(d / allowed))
        scale = np.maximum(np.abs(w), floor)
        report.append((k, float((d / scale).max()), float((NOISE_SIGMAS * sigma / (t * scale)).max())))
        assert (d <= allowed).all(), (f"kernel {k} (output {ob.shape}, {len(it.bufs) - 1} inputs): |device - oracle| = {d[worst]:.3e} at position {idx[worst]} "
                                      f"(oracle {w[worst]:.6e}, floor {floor:.3e}, sigma {sigma[worst]:.3e}) exceeds {allowed[worst]:.3e}; {idx.size} sampled outputs")
    return report, got
