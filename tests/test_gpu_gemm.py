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
