"""Parameter updates attached to gradient outputs, where they interact with launch fusion and with
captured replays; and the launch shape of caller-supplied kernels."""
import numpy as np
import pytest

from anneal_b200 import nn, realize as R, workloads as W
from anneal_b200.device import Device, GradientTarget
from anneal_b200.gradient import backward
from anneal_b200.tensor import Tensor, broadcast_to
from anneal_b200.uop import dtypes
from util import schedule

pytestmark = pytest.mark.gpu


def _gain_graph(n, c, x, g, w):
    """Outputs: the gradient of sum(x * w) with respect to the gain vector w (a column sum, ready at
    once) and dx of sum(softmax(x * w) * g), five per-row kernels that all read w and fuse into one
    row-chain launch — so the LAST reader of the parameter sits inside the chain."""
    xt = Tensor.new_leaf((n, c)).set_data(x)
    gt = Tensor.new_leaf((n, c)).set_data(g)
    wt = Tensor.new_leaf((c,)).set_data(w)
    wb = broadcast_to(wt, (n, c))
    gw = backward(xt.mul(wb).sum(), [wt])[wt]
    y = nn.softmax_rows(xt.mul(wb))
    dx = backward(y.mul(gt).sum(), [xt])[xt]
    return [gw, dx], xt, gt, wt


def test_update_waits_for_a_last_reader_inside_a_row_chain():
    n, c, lr = 256, 512, 0.25
    x, g, w = W.normal(11, 1, n * c), W.normal(11, 2, n * c), W.normal(11, 3, c)
    res = []
    for flags in (0, Device.NO_ROW_CHAIN):
        dev = Device(0, flags)
        try:
            R.reset()
            ts, xt, gt, wt = _gain_graph(n, c, x, g, w)
            items, out_ids = R.build_schedule(ts)
            master = dev.buffer(dtypes.float32, c).upload(w)
            grad = dev.buffer(dtypes.float32, c)
            k0 = dev.stats()["kernels_launched"]
            out = dev.run(items, {xt.node.idx: x, gt.node.idx: g, wt.node.idx: master},
                          placed={out_ids[0]: GradientTarget(grad, master, None, lr, 1.0)})
            launches = dev.stats()["kernels_launched"] - k0
            dev.synchronize()
            res.append((master.download(), grad.download(), out[out_ids[1]], launches, len(items)))
        finally:
            dev.close()
    (w_chain, g_chain, dx_chain, l_chain, n_items), (w_plain, g_plain, dx_plain, l_plain, _) = res
    assert l_chain < l_plain, (l_chain, l_plain)                   # the chain did fuse
    want = w - np.float32(lr) * x.reshape(n, c).sum(0, dtype=np.float64).astype(np.float32)
    assert np.abs(w_chain - want).max() < 1e-3 * np.abs(want).max()
    assert np.array_equal(w_chain, w_plain)                        # the update ran, once, in both
    assert np.array_equal(g_chain, g_plain)
    # every kernel of the chain read the parameter before it changed
    assert np.abs(dx_chain - dx_plain).max() <= 1e-5 * np.abs(dx_plain).max()


def test_replay_picks_up_a_changed_learning_rate(cuda):
    """The rate and the scale of an attached update are kernel arguments inside the captured graph;
    a replay that is handed other values must apply those, like an eager run."""
    n, c = 128, 256
    x, w = W.normal(12, 1, n * c), W.normal(12, 2, c)
    xt = Tensor.new_leaf((n, c)).set_data(x)
    wt = Tensor.new_leaf((c,)).set_data(w)
    gw = backward(xt.mul(broadcast_to(wt, (n, c))).sum(), [wt])[wt]
    items, out_ids = R.build_schedule([gw])
    master = cuda.buffer(dtypes.float32, c).upload(w)
    grad = cuda.buffer(dtypes.float32, c)
    colsum = x.reshape(n, c).sum(0, dtype=np.float64)
    want = w.astype(np.float64)
    for lr, scale in ((0.1, 1.0), (0.2, 1.0), (0.2, 0.5)):
        cuda.replay(items, {xt.node.idx: x, wt.node.idx: master}, placed={out_ids[0]: GradientTarget(grad, master, None, lr, scale)})
        cuda.synchronize()
        want = want - lr * scale * colsum
        got = master.download()
        assert np.abs(got - want).max() < 1e-4 * np.abs(want).max(), (lr, scale)
    master.release()
    grad.release()


def test_pre_rendered_kernel_uses_all_three_launch_dimensions(cuda):
    """A caller-supplied kernel is launched with the workgroup counts and the local size it came
    with, in x, y and z (backend/webgpu/executor.go:366 dispatches all three counts)."""
    from anneal_b200.schedule import Buffer, ExecItem
    src = ('extern "C" __global__ void main_kernel(float* out, const float* in) {'
           ' int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y * blockDim.y + threadIdx.y, z = blockIdx.z * blockDim.z + threadIdx.z;'
           ' int i = (z * 12 + y) * 40 + x; if (x < 40 && y < 12 && z < 6) out[i] = in[i] + (float)(100 * z + y); }')
    n = 40 * 12 * 6
    it = ExecItem(None, [Buffer(910001, n, (n,), dtypes.float32), Buffer(910002, n, (n,), dtypes.float32)],
                  source=src, local_size=(8, 4, 2), grid=(5, 3, 3))
    x = np.arange(n, dtype=np.float32)
    out = cuda.run([it], {910002: x})[910001].reshape(6, 12, 40)
    want = x.reshape(6, 12, 40) + (100 * np.arange(6)[:, None, None] + np.arange(12)[None, :, None])
    assert np.array_equal(out, want.astype(np.float32))


def test_device_stats_hook_reports_what_a_realize_launched(cuda):
    """The device-side companion of the schedule's stats hook: launches, tensor-core contractions,
    kernels that ran inside a contraction's epilogue, bytes moved, per realize."""
    from anneal_b200 import realize as RR
    R.reset()
    R.MATERIALIZE_CONTRACTION_OPERANDS = "auto"
    seen = []
    RR.DEFAULT_EXECUTOR = cuda
    RR.DEVICE_STATS_HOOK = seen.append
    try:
        m = W.WideMLP(batch=512, width=256, classes=136, depth=2)
        x, y = m.make_inputs()
        g = m.graph(x, y)
        RR.realize(*g.targets())
    finally:
        RR.DEVICE_STATS_HOOK = None
        RR.DEFAULT_EXECUTOR = None
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    assert len(seen) == 1
    st = seen[0]
    assert st["gemm_launched"] == 8 and st["epilogues_fused"] == 5 and st["colsums_fused"] == 2
    assert st["kernels_launched"] > st["gemm_launched"] and st["h2d_bytes"] > 0 and st["d2h_bytes"] > 0
    assert np.isfinite(g.loss.data).all()


def test_captured_step_runs_leaf_kernels_beside_the_contractions():
    """Inside a captured graph the scalar loss and the bias-gradient finishes — small kernels whose
    output no later kernel reads — go to the side stream; launched one by one they stay in order on
    the main stream. Both give the same losses and parameters, bit for bit, step by step."""
    from anneal_b200.train import ResidentTrainer
    res = []
    for use_graph in (True, False):
        dev = Device(0)
        try:
            R.reset()
            m = W.WideMLP(batch=512, width=512, classes=136, depth=3)
            x, y = m.make_inputs()
            tr = ResidentTrainer(dev, m, 0.05, use_graph=use_graph, resident_inputs=True)
            tr.load_batch(x, y)
            losses = []
            for _ in range(5):
                tr.step()
                losses.append(tr.loss())
            res.append((losses, tr.parameters(), dev.stats()["side_launches"]))
        finally:
            dev.close()
    (lg, pg, ng), (le, pe, ne) = res
    assert ng >= 3 and ne == 0, (ng, ne)
    assert lg == le
    for a, b in zip(pg, pe):
        assert np.array_equal(a, b)
