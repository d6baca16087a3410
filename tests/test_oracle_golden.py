"""The CPU oracle pinned against the known-answer vectors of the reference's own tests
(tests/golden/reference_vectors.json; each case cites the reference file and lines)."""
import json
import os

import numpy as np
import pytest

from anneal_b200 import nn, realize as R
from anneal_b200.gradient import backward
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes, quantize
from oracle import binding

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))


@pytest.fixture(autouse=True)
def use_oracle(oracle):
    R.DEFAULT_EXECUTOR = oracle
    yield
    R.DEFAULT_EXECUTOR = None


def leaf(shape, data, dtype=dtypes.float32):
    return Tensor.new_leaf(shape, dtype).set_data(np.asarray(data, dtype=np.float32))


def build(case):
    g = case["graph"]
    if g == "exp2":
        return leaf((len(case["x"]),), case["x"]).exp2()
    if g == "add":
        return leaf((4,), case["x"]).add(leaf((4,), case["y"]))
    if g == "sum_all":
        return leaf((8,), case["x"]).sum()
    if g == "sum_axis0_4x4":
        return leaf((4, 4), case["x"]).sum([0])
    if g == "max_all":
        return leaf((4,), case["x"]).max()
    if g == "log2_exp2":
        return leaf((4,), case["x"]).exp2().log2()
    if g == "matmul_2x3_3x2":
        a = leaf((2, 3), case["x"]).reshape((2, 3, 1)).expand((2, 3, 2))
        b = leaf((3, 2), case["y"]).reshape((1, 3, 2)).expand((2, 3, 2))
        return a.mul(b).sum([1])
    if g == "mse_2x3_3x2":
        a = leaf((2, 3), case["x"]).reshape((2, 3, 1)).expand((2, 3, 2))
        b = leaf((3, 2), case["w"]).reshape((1, 3, 2)).expand((2, 3, 2))
        d = a.mul(b).sum([1]).sub(leaf((2, 2), case["t"]))
        return d.mul(d).mean()
    if g == "grad_sum_exp2":
        x = leaf((4,), case["x"])
        return backward(x.exp2().sum(), [x])[x]
    raise KeyError(g)


@pytest.mark.parametrize("case", GOLD["value_oracles"], ids=lambda c: c["graph"] + "@" + c["ref"].split(":")[1])
def test_value_oracles(case):
    t = build(case)
    R.realize(t)
    assert np.allclose(t.data, np.asarray(case["want"], dtype=np.float32), atol=case["tol"], rtol=0), (t.data, case["want"])


@pytest.mark.parametrize("case", GOLD["padded_reduce"], ids=lambda c: c["ref"].split(":")[1])
def test_padded_reduce_uses_the_reduce_identity(case):
    x = leaf(tuple(case["shape"]), case["x"]).pad(case["pad"])
    y = x.max([case["axis"]]) if case["op"] == "max" else x.sum([case["axis"]])
    R.realize(y)
    assert list(y.data) == case["want"]


def test_sgd_quadratic_trajectory():
    c = GOLD["sgd_trajectory"]
    p = nn.Parameter((c["n"],))
    p.value[:] = c["p0"]
    for step in range(c["steps"]):
        assert np.allclose(p.value, c["p"][step], atol=c["tol"])
        R.reset()
        pl = p.load()
        d = pl.sub(leaf((c["n"],), [c["target"]] * c["n"]))
        g = backward(d.mul(d).sum(), [pl])[pl]
        R.realize(g)
        assert np.allclose(g.data, c["grad"][step], atol=c["tol"])
        p.sgd_step(g.data, c["lr"])
    assert np.allclose(p.value, c["p"][c["steps"]], atol=c["tol"])


def ref_maxpool(data, N, C, H, W, kH, kW, sH, sW):
    oH, oW = (H - kH) // sH + 1, (W - kW) // sW + 1
    x = data.reshape(N, C, H, W)
    out = np.empty((N, C, oH, oW), dtype=np.float32)
    for i in range(oH):
        for j in range(oW):
            out[:, :, i, j] = x[:, :, i * sH:i * sH + kH, j * sW:j * sW + kW].max(axis=(2, 3))
    return out.reshape(-1)


@pytest.mark.parametrize("case", GOLD["maxpool"]["cases"], ids=str)
def test_maxpool_forward_exact(case):
    N, C, H, W, kH, kW, sH, sW, neg = case
    data = np.arange(1, N * C * H * W + 1, dtype=np.float32) * (-1 if neg else 1)
    out = nn.max_pool2d(leaf((N, C, H, W), data), kH, kW, sH, sW)
    R.realize(out)
    assert np.array_equal(out.data, ref_maxpool(data, N, C, H, W, kH, kW, sH, sW))


def test_f16_cast_round_trip_is_bit_exact():
    v = GOLD["f16_cast_roundtrip"]["x"]
    x = leaf((len(v),), v, dtypes.float16)
    y = x.cast(dtypes.float32).cast(dtypes.float16)
    R.realize(y)
    assert np.array_equal(y.data, np.asarray(v, dtype=np.float32))


def test_bf16_round_trip_truncates():
    v = np.asarray(GOLD["bf16_roundtrip"]["x"], dtype=np.float32)
    x = leaf((v.size,), v, dtypes.bfloat16)
    y = x.cast(dtypes.float32).cast(dtypes.bfloat16)
    R.realize(y)
    assert np.array_equal(y.data, (v.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32))


def test_bf16_add_matches_truncation_model():
    rng = np.random.default_rng(17)
    a, b = (rng.random(512) * 2 - 1).astype(np.float32), (rng.random(512) * 2 - 1).astype(np.float32)
    tr = lambda v: (np.asarray(v, np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    z = leaf((512,), a, dtypes.bfloat16).add(leaf((512,), b, dtypes.bfloat16))
    R.realize(z)
    assert np.abs(z.data - tr(tr(a) + tr(b))).max() <= 1e-6


@pytest.mark.parametrize("bits,want", GOLD["f32_to_f16_bits"]["cases"] + GOLD["backend_f32_to_f16_bits"]["cases"])
def test_f32_to_f16_known_answers(bits, want):
    f = np.array([bits], dtype=np.uint32).view(np.float32)[0]
    assert binding.lib().orc_f32_to_f16_bits(float(f) if f == f else f) == want or (f != f and bits == 0x7F800001)
    if f == f:   # the frontend's quantiser (numpy RTNE) agrees on every non-NaN case
        q = quantize(np.array([f], np.float32), dtypes.float16)
        assert np.array([q[0]], np.float32).astype(np.float16).view(np.uint16)[0] == want


@pytest.mark.parametrize("bits,want", GOLD["f16_to_f32_bits"]["cases"] + GOLD["backend_f16_to_f32_bits"]["cases"])
def test_f16_to_f32_known_answers(bits, want):
    assert np.array([bits], dtype=np.uint16).view(np.float16).astype(np.float32).view(np.uint32)[0] == want


def test_f16_arithmetic_is_rounded_per_op():
    # 2049 is not representable in f16: 2048 + 1 rounds to even (2048), and (2048+1)+1 stays 2048,
    # while an f32 evaluation would give 2050
    x = leaf((1,), [2048.0], dtypes.float16)
    one = Tensor.full((1,), 1.0, dtypes.float16)
    y = x.add(one).add(one)
    R.realize(y)
    assert y.data[0] == 2048.0
    # inside an f16 reduction the body is widened: sum of 2048 ones from 2048 reaches 4096 exactly
    v = leaf((2049,), [2048.0] + [1.0] * 2048, dtypes.float16)
    s = v.sum()
    R.realize(s)
    assert s.data[0] == 4096.0


def test_max_identity_is_minus_flt_max_not_inf():
    # an empty-support max (every element padded away) yields -FLT_MAX, the WGSL literal the
    # reference emits (codegen/wgsl.go:373-379), not -inf
    x = leaf((2,), [1.0, 2.0]).shrink(((0, 1),)).pad(((0, 0),))
    y = leaf((1, 2), [1.0, 2.0]).pad(((0, 0), (2, 0))).shrink(((0, 1), (0, 2))).max([1])
    R.realize(y)
    assert y.data[0] == np.float32(-3.4028234663852886e38)


def test_bulk_f16_bytes():
    """float32sToF16Bytes of the backend (backend/webgpu/conversion_test.go:79-99): little-endian
    half bit patterns, through the oracle's converter and the frontend's quantiser."""
    c = GOLD["backend_bulk_f16"]
    x = np.asarray(c["x"], np.float32)
    assert x.astype(np.float16).tobytes() == bytes(c["bytes"])
    bits = [binding.lib().orc_f32_to_f16_bits(float(v)) for v in x]
    assert np.asarray(bits, np.uint16).tobytes() == bytes(c["bytes"])


def symbolic_add_run(run):
    """out[i] = a[i] + b[i] over a symbolic extent (backend/webgpu/symbolic_test.go:27-152), built
    with the frontend: two [n, 1] inputs whose outermost size is bound per call."""
    from anneal_b200 import uop as U
    n = run["n"]
    var = U.Var("n", 1, 1024)
    a = Tensor.new_symbolic_batch_input(var, (1,)).set_data(np.arange(n, dtype=np.float32) * run["a_scale"])
    b = Tensor.new_symbolic_batch_input(var, (1,)).set_data(np.arange(n, dtype=np.float32) * run["b_scale"])
    out = a.add(b)
    R.realize_with_binding({"n": n}, out)
    want = np.arange(n, dtype=np.float32) * run["a_scale"] + np.arange(n, dtype=np.float32) * run["b_scale"]
    assert out.data.shape == (n,)
    assert np.abs(out.data - want).max() <= GOLD["symbolic_add"]["tol"]


@pytest.mark.parametrize("run", GOLD["symbolic_add"]["runs"], ids=lambda r: f"n={r['n']}")
def test_symbolic_add_known_answers(run):
    symbolic_add_run(run)


def reference_test_data(n, offset):
    """testData of the reference's gradient tests (tensor/gradient_test.go:540-551), in float32."""
    d = np.empty(n, np.float32)
    for i in range(n):
        v = np.float32(0.5) + np.float32(i) * np.float32(0.3) + np.float32(offset)
        if v > np.float32(2.5):
            v = np.float32(0.5) + np.float32(i % 4) * np.float32(0.3)
        d[i] = v
    return d


def gradient_check(case):
    """Backward of sum(f(x)) realized on the executor in use, against the closed-form derivative at
    the reference's inputs and tolerance (absolute, as the reference compares)."""
    n = case["n"]
    xd = reference_test_data(n, case["offset"]).astype(np.float64)
    x = leaf((n,), xd)
    f = case["f"]
    ln2 = np.log(2.0)
    if f in ("add", "mul"):
        yd = reference_test_data(n, case["offset_y"]).astype(np.float64)
        y = leaf((n,), yd)
        loss = (x.add(y) if f == "add" else x.mul(y)).sum()
        g = backward(loss, [x, y])
        R.realize(g[x], g[y])
        want = (np.ones(n), np.ones(n)) if f == "add" else (yd, xd)
        assert np.abs(g[x].data - want[0]).max() <= case["tol"]
        assert np.abs(g[y].data - want[1]).max() <= case["tol"]
        return
    build_f = {"neg": lambda t: t.neg(), "exp2": lambda t: t.exp2(), "log2": lambda t: t.log2(), "sin": lambda t: t.sin(),
               "sqrt": lambda t: t.sqrt(), "recip": lambda t: t.recip(), "exp": lambda t: t.exp(), "log": lambda t: t.log(),
               "diamond": lambda t: t.mul(t).add(t)}[f]
    want = {"neg": -np.ones(n), "exp2": ln2 * 2.0 ** xd, "log2": 1.0 / (xd * ln2), "sin": np.cos(xd), "sqrt": 0.5 / np.sqrt(xd),
            "recip": -1.0 / xd ** 2, "exp": np.exp(xd), "log": 1.0 / xd, "diamond": 2.0 * xd + 1.0}[f]
    g = backward(build_f(x).sum(), [x])[x]
    R.realize(g)
    assert np.abs(g.data - want).max() <= case["tol"], (f, g.data, want)


@pytest.mark.parametrize("case", GOLD["gradient_checks"]["cases"], ids=lambda c: c["f"])
def test_gradient_known_answers(case):
    gradient_check(case)


def structured_gradient_check(case):
    """The reference's structured gradient tests (broadcast, matmul, linear layer, two-layer MLP, a
    hand-built 2x2 convolution, a partial sum), rebuilt with the frontend from the same primitives,
    at its inputs; Backward realized on the executor in use against the closed form in float64."""
    from anneal_b200.tensor import broadcast_to
    td = lambda shape, off: reference_test_data(int(np.prod(shape)), off)
    tol, graph = case["tol"], case["graph"]

    def check(grads, want):
        R.realize(*[grads[t] for t, _, _ in want])
        for t, name, w in want:
            assert np.abs(grads[t].data - np.asarray(w, np.float64).reshape(-1)).max() <= tol[name], (graph, name)

    if graph == "broadcast":
        wd, xd = td((1, 3), 0), td((2, 3), 1)
        w, x = leaf((1, 3), wd), leaf((2, 3), xd)
        g = backward(w.expand((2, 3)).add(x).sum(), [w])
        check(g, [(w, "w", np.full(3, 2.0))])
    elif graph == "matmul":
        xd, wd = td((2, 3), 0).astype(np.float64).reshape(2, 3), td((3, 4), 0.2).astype(np.float64).reshape(3, 4)
        x, w = leaf((2, 3), xd), leaf((3, 4), wd)
        g = backward(x.matmul(w).sum(), [x, w])
        ones = np.ones((2, 4))
        check(g, [(x, "x", ones @ wd.T), (w, "w", xd.T @ ones)])
    elif graph == "linear":
        xd, wd, bd = td((2, 4), 0).astype(np.float64).reshape(2, 4), td((3, 4), 0.1), td((3,), 0.5)
        x, w, b = leaf((2, 4), xd), leaf((3, 4), wd), leaf((3,), bd)
        y = x.matmul(w.permute((1, 0)))
        g = backward(y.add(broadcast_to(b, y.shape)).sum(), [w, b])
        check(g, [(w, "w", np.ones((2, 3)).T @ xd), (b, "b", np.full(3, 2.0))])
    elif graph == "mlp":
        xd = td((2, 4), 0).astype(np.float64).reshape(2, 4)
        w1d, w2d = td((3, 4), 0.1).astype(np.float64).reshape(3, 4), td((2, 3), 0.2).astype(np.float64).reshape(2, 3)
        x, w1, w2 = leaf((2, 4), xd), leaf((3, 4), w1d), leaf((2, 3), w2d)
        h1 = x.matmul(w1.permute((1, 0)))
        out = h1.maximum(Tensor.full(h1.shape, 0.0)).matmul(w2.permute((1, 0)))
        g = backward(out.sum(), [w1, w2])
        h = xd @ w1d.T
        dh = (np.ones((2, 2)) @ w2d) * (h > 0)
        check(g, [(w1, "w1", dh.T @ xd), (w2, "w2", np.ones((2, 2)).T @ np.maximum(h, 0))])
    elif graph == "conv2d":
        N, Cin, H, W, Cout, kH, kW = 1, 1, 4, 4, 2, 2, 2
        Ho, Wo = H - kH + 1, W - kW + 1
        xd, wd = td((N, Cin, H, W), 0).astype(np.float64).reshape(N, Cin, H, W), td((Cout, Cin, kH, kW), 0.1)
        x, weight = leaf((N, Cin, H, W), xd), leaf((Cout, Cin, kH, kW), wd)
        out = None
        for ki in range(kH):
            for kj in range(kW):
                patch = x.shrink(((0, N), (0, Cin), (ki, ki + Ho), (kj, kj + Wo)))
                pmat = patch.reshape((N, Cin, Ho * Wo)).permute((0, 2, 1))
                wslice = weight.shrink(((0, Cout), (0, Cin), (ki, ki + 1), (kj, kj + 1))).reshape((Cout, Cin)).permute((1, 0))
                contrib = pmat.matmul(wslice).permute((0, 2, 1)).reshape((N, Cout, Ho, Wo))
                out = contrib if out is None else out.add(contrib)
        g = backward(out.sum(), [weight])
        want = np.empty((Cout, Cin, kH, kW))
        for ki in range(kH):
            for kj in range(kW):
                want[:, :, ki, kj] = xd[0, :, ki:ki + Ho, kj:kj + Wo].sum(axis=(1, 2))[None, :]
        check(g, [(weight, "weight", want)])
    elif graph == "reduce_sum":
        x = leaf((2, 3), td((2, 3), 0))
        g = backward(x.sum([1]).sum(), [x])
        check(g, [(x, "x", np.ones(6))])
    else:
        raise KeyError(graph)


@pytest.mark.parametrize("case", GOLD["structured_gradients"]["cases"], ids=lambda c: c["graph"])
def test_structured_gradient_known_answers(case):
    structured_gradient_check(case)


def maxpool_backward_check(case):
    """d/dx of sum(MaxPool2D(x)^2) at x = (i+1)*0.1 (tensor/nn/maxpool_test.go:131-215): without ties
    every window hands 2*max to its arg-max; all elements are compared, not only the first four."""
    N, C, H, W, kH, kW, sH, sW = case
    data = (np.arange(1, N * C * H * W + 1, dtype=np.float32) * np.float32(0.1))
    x = leaf((N, C, H, W), data)
    out = nn.max_pool2d(x, kH, kW, sH, sW)
    g = backward(out.mul(out).sum(), [x])[x]
    R.realize(g)
    xd = data.astype(np.float64).reshape(N, C, H, W)
    want = np.zeros_like(xd)
    for i in range((H - kH) // sH + 1):
        for j in range((W - kW) // sW + 1):
            win = xd[:, :, i * sH:i * sH + kH, j * sW:j * sW + kW].reshape(N, C, -1)
            am = win.argmax(-1)
            for n in range(N):
                for c in range(C):
                    di, dj = divmod(int(am[n, c]), kW)
                    want[n, c, i * sH + di, j * sW + dj] += 2.0 * win[n, c, am[n, c]]
    assert np.abs(g.data - want.reshape(-1)).max() <= GOLD["maxpool_backward"]["tol"]


@pytest.mark.parametrize("case", GOLD["maxpool_backward"]["cases"], ids=str)
def test_maxpool_backward_known_answers(case):
    maxpool_backward_check(case)


def maxpool_tie_check(case):
    """Tied maxima share the adjoint equally (tensor/nn/maxpool_test.go:217-305)."""
    x = leaf(tuple(case["shape"]), case["x"])
    out = nn.max_pool2d(x, case["k"][0], case["k"][1], case["s"][0], case["s"][1])
    g = backward(out.sum(), [x])[x]
    R.realize(g)
    assert np.abs(g.data - np.asarray(case["want"], np.float64)).max() <= GOLD["maxpool_ties"]["tol"]


@pytest.mark.parametrize("case", GOLD["maxpool_ties"]["cases"], ids=lambda c: str(c["shape"]))
def test_maxpool_ties_split_equally(case):
    maxpool_tie_check(case)


def test_cnn_schedule_with_and_without_im2col_buffers_agree_bit_for_bit(oracle):
    """A convolution's im2col as an expression inside the contraction (the reference's schedule) and
    as a buffer written first (the operand-materialising rule) are the same f32 operations in the
    same order; the GPU trajectory test relies on it to keep the oracle's 100 steps affordable."""
    from anneal_b200 import realize as R, workloads as W
    from util import schedule
    res = []
    for mat in (False, True):
        R.reset()
        R.MATERIALIZE_CONTRACTION_OPERANDS = mat
        try:
            m = W.SmallCNN(batch=4, hw=12)
            items, out_ids, inputs = schedule(m.graph().targets())
        finally:
            R.MATERIALIZE_CONTRACTION_OPERANDS = False
        out = oracle.run(items, inputs)
        res.append([out[k] for k in out_ids])
    assert len(res[0]) == 7
    for a, b in zip(*res):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
