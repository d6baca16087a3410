"""The caller stand-in builds the same graph shapes as the reference's tensor API: structural checks
in the form of tensor/tensor_test.go:111-420 and tensor/nn/nn_test.go:38-200 (ops at the root, source
counts, result shapes and dtypes, parameter counts) — no device needed."""
import pytest

from anneal_b200 import nn, realize as R
from anneal_b200.tensor import Tensor
from anneal_b200.uop import Op, dtypes


@pytest.fixture(autouse=True)
def fresh_arena():
    R.reset()
    yield
    R.reset()


def leaf(*shape, dtype=dtypes.float32):
    return Tensor.new_leaf(tuple(shape), dtype)


@pytest.mark.parametrize("name,op", [("neg", Op.NEG), ("exp2", Op.EXP2), ("log2", Op.LOG2), ("sin", Op.SIN),
                                      ("sqrt", Op.SQRT), ("recip", Op.RECIPROCAL), ("trunc", Op.TRUNC)])
def test_unary_ops(name, op):                       # tensor_test.go:111-137
    y = getattr(leaf(2, 3), name)()
    assert y.node.op == op and len(y.node.src) == 1 and tuple(y.shape) == (2, 3)


def test_derived_unary():                           # tensor_test.go:139-150: exp = exp2(x / ln 2), log = log2(x) * ln 2
    x = leaf(3)
    assert x.exp().node.op == Op.EXP2
    assert x.log().node.op == Op.MUL


@pytest.mark.parametrize("name,op", [("add", Op.ADD), ("sub", Op.SUB), ("mul", Op.MUL), ("maximum", Op.MAX)])
def test_binary_ops(name, op):                      # tensor_test.go:154-178
    z = getattr(leaf(2, 3), name)(leaf(2, 3))
    assert tuple(z.shape) == (2, 3)
    if name != "sub":                               # the reference's Sub is a node of its own; here it may be add(neg)
        assert z.node.op == op and len(z.node.src) == 2


def test_comparisons_produce_bool():                # tensor_test.go:180-195
    x, y = leaf(4), leaf(4)
    lt, eq = x.cmplt(y), x.cmpeq(y)
    assert lt.dtype == dtypes.bool and lt.node.op == Op.CMPLT
    assert eq.dtype == dtypes.bool


def test_where_has_three_sources():                 # tensor_test.go:197-207
    w = Tensor.where(leaf(3, dtype=dtypes.bool), leaf(3), leaf(3))
    assert w.node.op == Op.WHERE and len(w.node.src) == 3


def test_movement_shapes():                         # tensor_test.go:270-333
    assert tuple(leaf(2, 3, 4).reshape((6, 4)).shape) == (6, 4)
    assert tuple(leaf(1, 3).expand((5, 3)).shape) == (5, 3)
    assert tuple(leaf(2, 3, 4).permute((2, 0, 1)).shape) == (4, 2, 3)
    p = leaf(2, 3).pad(((1, 1), (0, 2)))
    assert p.node.op == Op.PAD and tuple(p.shape) == (4, 5)
    s = leaf(4, 6).shrink(((1, 3), (2, 5)))
    assert s.node.op == Op.SHRINK and tuple(s.shape) == (2, 3)
    assert tuple(leaf(3, 4).flip((True, False)).shape) == (3, 4)
    assert tuple(leaf(2, 3).transpose().shape) == (3, 2)
    assert tuple(leaf(2, 3, 4).flatten().shape) == (24,)


def test_reductions():                              # tensor_test.go:335-375
    x = leaf(2, 3, 4)
    assert tuple(x.sum([1]).shape) == (2, 4)
    assert tuple(x.sum([1], keepdim=True).shape) == (2, 1, 4)
    assert tuple(leaf(2, 3).sum().shape) == ()
    assert tuple(leaf(2, 3).max([0]).shape) == (3,)
    assert tuple(leaf(4, 5).mean([1]).shape) == (4,)


def test_matmul_shapes():                           # tensor_test.go:377-405
    assert tuple(leaf(2, 3).matmul(leaf(3, 4)).shape) == (2, 4)
    with pytest.raises(Exception):
        leaf(2, 3).matmul(leaf(4, 5))


def test_cast_changes_dtype_only():                 # tensor_test.go:407-420
    y = leaf(2, 3).cast(dtypes.float16)
    assert y.dtype == dtypes.float16 and tuple(y.shape) == (2, 3)


def test_activations_and_linear():                  # nn_test.go:38-103
    assert nn.relu(leaf(3, 4)).node.op == Op.MAX
    assert tuple(nn.sigmoid(leaf(5)).shape) == (5,) and tuple(nn.tanh(leaf(5)).shape) == (5,)
    lin = nn.Linear(8, 4, bias=False)
    assert tuple(lin.forward(leaf(3, 8)).shape) == (3, 4) and len(lin.params()) == 1
    lin_b = nn.Linear(8, 4, bias=True)
    assert tuple(lin_b.forward(leaf(3, 8)).shape) == (3, 4) and len(lin_b.params()) == 2


def test_conv2d_and_pool_shapes():                  # nn_test.go:143-176, maxpool_test.go
    conv = nn.Conv2d(3, 8, (3, 3), stride=(1, 1), pad=(1, 1), bias=True)
    y = conv.forward(leaf(2, 3, 16, 16))
    assert tuple(y.shape) == (2, 8, 16, 16) and len(conv.params()) == 2
    valid = nn.Conv2d(1, 4, (3, 3), bias=False)
    assert tuple(valid.forward(leaf(1, 1, 8, 8)).shape) == (1, 4, 6, 6) and len(valid.params()) == 1
    assert tuple(nn.max_pool2d(leaf(2, 8, 16, 16), 2, 2, 2, 2).shape) == (2, 8, 8, 8)
