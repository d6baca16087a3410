"""Tensor-core contraction path: every operand layout, ragged edges, against the oracle."""
import numpy as np
import pytest

from anneal_b200 import workloads as W
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes
from util import compare, schedule

pytestmark = pytest.mark.gpu
F16 = 2e-3


def hleaf(shape, seed):
    n = int(np.prod(shape))
    return Tensor.new_leaf(shape, dtypes.float16).set_data(W.normal(11, seed, n) * np.float32(0.5))


def gemm_count(cuda, fn):
    before = cuda.stats()["gemm_launched"]
    fn()
    return cuda.stats()["gemm_launched"] - before


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 328, 136), (64, 1000, 520), (384, 72, 2048),
                                   (512, 512, 320), (1000, 328, 136), (2304, 1000, 520)])
@pytest.mark.parametrize("layout", ["KK", "KM", "MM", "MK"])
def test_gemm_layouts(cuda, oracle, M, N, K, layout):
    # A is [M,K] (K-major) or stored [K,M] (M-major); B is [N,K] (K-major) or stored [K,N] (N-major)
    a = hleaf((M, K), 1) if layout[0] == "K" else hleaf((K, M), 1).permute((1, 0))
    b = hleaf((N, K), 2).permute((1, 0)) if layout[1] == "K" else hleaf((K, N), 2)
    out = a.matmul(b)
    n = gemm_count(cuda, lambda: compare(cuda, oracle, [out], F16, what=f"gemm {layout} {M}x{N}x{K}"))
    assert n == 1, "contraction was not routed to the tensor-core kernel"


def test_linear_forward_backward_routes_to_gemm(cuda, oracle):
    from anneal_b200 import realize as R
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.WideMLP(batch=256, width=128, classes=72, depth=2)
        x, y = m.make_inputs()
        g = m.graph(x, y)
        n = gemm_count(cuda, lambda: compare(cuda, oracle, g.targets(), F16, what="wide mlp"))
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    assert n == 8      # 3 forward, 2 input-gradient, 3 weight-gradient contractions


# ── f32 contractions: the FP32-pipe tiled kernel ────────────────────────────────────────────────
F32 = 1e-5


def fleaf(shape, seed):
    n = int(np.prod(shape))
    return Tensor.new_leaf(shape, dtypes.float32).set_data(W.normal(12, seed, n) * np.float32(0.5))


@pytest.mark.parametrize("M,N,K", [(512, 640, 136), (515, 601, 131), (2048, 1024, 64), (130, 2100, 1000)])
@pytest.mark.parametrize("layout", ["KK", "KM", "MM", "MK"])
def test_gemm_f32_layouts(cuda, oracle, M, N, K, layout):
    a = fleaf((M, K), 1) if layout[0] == "K" else fleaf((K, M), 1).permute((1, 0))
    b = fleaf((N, K), 2).permute((1, 0)) if layout[1] == "K" else fleaf((K, N), 2)
    out = a.matmul(b)
    n = gemm_count(cuda, lambda: compare(cuda, oracle, [out], F32, what=f"gemm f32 {layout} {M}x{N}x{K}"))
    assert n == 1, "f32 contraction was not routed to the tiled kernel"


def test_gemm_f32_small_stays_on_generated_kernel(cuda, oracle):
    out = fleaf((64, 784), 1).matmul(fleaf((128, 784), 2).permute((1, 0)))
    n = gemm_count(cuda, lambda: compare(cuda, oracle, [out], F32, what="small f32 matmul"))
    assert n == 0


@pytest.mark.parametrize("b,gemms", [(1, 5), (3, 5), (17, 5), (32, 5), (300, 5), (2100, 5)])
def test_gemm_f32_symbolic_batch(cuda, oracle, b, gemms):
    """The bound batch is M of the forward/input-gradient contractions and K of the weight-gradient
    ones; one compiled plan serves every binding and picks the kernel per launch: the few-row and
    few-term kernels up to 32 rows (one pass over the weights for all rows), the tensor-core kernel in
    3 x TF32 form from there on.

    The tiled kernel accumulates with fused multiply-adds, the oracle rounds the product first, so a
    hidden pre-activation within rounding distance of zero can land on the other side of the ReLU
    and switch that unit's gradient on or off for one sample.  Hidden units with such a sample are
    left out of the comparison of the first layer's gradients; everything else is continuous in the
    pre-activation and is compared in full."""
    from anneal_b200 import realize as R
    from util import rel_err, schedule
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.DynMLP(din=512, hidden=1024, dout=256, max_batch=4096)
        x, y = m.inputs(b)
        out, loss, grads, ins = m.graph(b, x, y)
        items, out_ids, inputs = schedule([out] + grads)
        before = cuda.stats()["gemm_launched"]
        got = cuda.run(items, inputs, {"n": b})
        n = cuda.stats()["gemm_launched"] - before
        want = oracle.run(items, inputs, {"n": b})
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    assert n == gemms
    z = x.reshape(b, 512).astype(np.float64) @ m.params[0].value.reshape(1024, 512).astype(np.float64).T + m.params[1].value
    steady = ~(np.abs(z) < 1e-5).any(axis=0)            # hidden units whose ReLU masks do not hang on rounding
    assert steady.sum() >= 1000
    o_id, dw1, db1, dw2, db2 = out_ids
    for k in (o_id, dw2, db2):
        assert rel_err(got[k], want[k]) <= 2e-5, (b, k)
    assert rel_err(got[dw1].reshape(1024, 512)[steady], want[dw1].reshape(1024, 512)[steady]) <= 2e-5
    assert rel_err(got[db1][steady], want[db1][steady]) <= 2e-5


# ── large f32 contractions: the tensor-core kernel in 3 x TF32 form ──────────────────────────────
@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (2100, 1000, 1031), (515, 1000, 20001), (64, 2048, 1024), (100, 1000, 700)])
@pytest.mark.parametrize("layout", ["KK", "KM", "MM", "MK"])
def test_gemm_f32_on_tensor_cores(cuda, M, N, K, layout):
    """Against float64 on a sample of rows: the split into TF32 halves plus chunked f32 accumulation
    stays within 1e-5 of the largest output (a tenth of the 1e-4 the contract allows a contraction; the
    FP32-pipe kernel, which the same device runs when it is opened with NO_TF32X3, is at 1e-6 for
    K = 1000 and at 5e-6 for K = 20000), at every operand layout, ragged edges and a K of many chunks."""
    from anneal_b200 import realize as R
    from anneal_b200.device import Device
    R.reset()
    a = fleaf((M, K), 1) if layout[0] == "K" else fleaf((K, M), 1).permute((1, 0))
    b = fleaf((N, K), 2).permute((1, 0)) if layout[1] == "K" else fleaf((K, N), 2)
    out = a.matmul(b)
    items, out_ids, inputs = schedule([out])
    before = cuda.stats()
    y = cuda.run(items, inputs)[out_ids[0]].reshape(M, N)
    after = cuda.stats()
    assert after["gemm_launched"] - before["gemm_launched"] == 1
    # two operand splits and the contraction, plus the sum over K slices where the tiles are few and K is long
    assert after["kernels_launched"] - before["kernels_launched"] in (3, 4)
    la = [v for k, v in inputs.items() if v.size == M * K][0]
    lb = [v for k, v in inputs.items() if v.size == N * K and v is not la][0]
    am = la.reshape(M, K) if layout[0] == "K" else la.reshape(K, M).T
    bm = lb.reshape(N, K) if layout[1] == "K" else lb.reshape(K, N).T
    rows = np.random.default_rng(5).choice(M, size=48, replace=False)
    rows[0], rows[1] = 0, M - 1
    ref = am[rows].astype(np.float64) @ bm.astype(np.float64).T
    scale = np.abs(ref).max()
    err = np.abs(y[rows] - ref).max() / scale
    plain = Device(0, flags=Device.NO_TF32X3)
    try:
        g0 = plain.stats()["kernels_launched"]
        y32 = plain.run(items, inputs)[out_ids[0]].reshape(M, N)
        assert plain.stats()["kernels_launched"] - g0 == 1
    finally:
        plain.close()
    err32 = np.abs(y32[rows] - ref).max() / scale
    assert err <= 1e-5 and err32 <= 1e-5, (err, err32)
    # the two routes agree everywhere, not only on the sampled rows (each within its own 1e-5 of the exact product)
    assert np.abs(y - y32).max() / scale <= 2e-5
    # and a replay gives the same bits
    assert np.array_equal(cuda.run(items, inputs)[out_ids[0]].reshape(M, N), y)
