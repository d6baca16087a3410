"""Scheduler structure: the facts the reference's own tests and SPEC pin about kernel lists."""
import numpy as np
import pytest

from anneal_b200 import nn, realize as R, schedule as S, workloads as W
from anneal_b200.gradient import backward
from anneal_b200.tensor import Tensor
from anneal_b200.uop import Op, dtypes
from anneal_b200 import uop as U


def kernels(tensors, **kw):
    items, _ = S.create_schedule([t.node for t in tensors], **kw)
    return items


def test_epilogue_fusion_kernel_counts():
    # SPEC.md:28 — matmul+bias 2→1, matmul+bias+relu 2→1 with fusion on
    x, w, b = Tensor.new_leaf((4, 8)), Tensor.new_leaf((8, 3)), Tensor.new_leaf((3,))
    y = x.matmul(w).add(b.reshape((1, 3)).expand((4, 3)))
    assert len(kernels([y])) == 1 and len(kernels([y], fusion=False)) == 2
    assert len(kernels([nn.relu(y)])) == 1 and len(kernels([nn.relu(y)], fusion=False)) == 2


def test_fusion_respects_the_buffer_budget():
    x = Tensor.new_leaf((4, 8))
    y = x.sum([1])
    z = y
    for _ in range(8):
        z = z.add(Tensor.new_leaf((4,)))
    assert len(kernels([z])) == 2            # 9 inputs + output would exceed 8 buffers
    assert len(kernels([z], max_bufs=16)) == 1


def test_fusion_on_and_off_agree(oracle):
    # schedule/fusion_oracle_test.go:85-127 — identical values either way
    rng = np.random.default_rng(0)
    x = Tensor.new_leaf((6, 10)).set_data(rng.standard_normal(60))
    w = Tensor.new_leaf((10, 5)).set_data(rng.standard_normal(50))
    b = Tensor.new_leaf((5,)).set_data(rng.standard_normal(5))
    y = nn.relu(x.matmul(w).add(b.reshape((1, 5)).expand((6, 5))))
    res = []
    for f in (True, False):
        items, out = S.create_schedule([y.node], fusion=f)
        res.append(oracle.run(items, R.leaf_inputs([y]))[out[y.node.idx]])
    assert np.array_equal(res[0], res[1])


def test_param_order_and_output_first():
    # schedule/kernels.go:132-143 — PARAM 0 is the output, inputs follow in depth-first order
    a, b = Tensor.new_leaf((3,)), Tensor.new_leaf((3,))
    it = kernels([b.sub(a)])[0]
    assert [x.uop_idx for x in it.bufs[1:]] == [b.node.idx, a.node.idx]
    assert it.bufs[0].slot == -1


def test_memory_plan_shares_slots_for_disjoint_lifetimes():
    x = Tensor.new_leaf((4, 4))
    a = x.sum([1])
    b = a.reshape((4, 1)).expand((4, 4)).mul(x).sum([1])
    c = b.reshape((4, 1)).expand((4, 4)).mul(x).sum([1])
    d = c.reshape((4, 1)).expand((4, 4)).mul(x).sum([1])
    items = kernels([d])
    slots = [it.bufs[0].slot for it in items]
    assert slots[-1] == -1 and slots[0] == slots[2] and slots[0] != slots[1]


def test_size_one_dims_become_constants_not_ranges():
    x = Tensor.new_leaf((1, 5))
    it = kernels([x.exp2()])[0]
    ranges = [n for n in U.toposort(it.ast) if n.op == Op.RANGE]
    assert len(ranges) == 1 and ranges[0].arg.size == 5


def test_keepdim_reduce_reports_kept_shape_but_node_drops_axis():
    x = Tensor.new_leaf((3, 4))
    s = x.sum([1], keepdim=True)
    assert s.shape == (3, 1)
    from anneal_b200.gradient import node_shape
    assert node_shape(s.node, {}) == (3,)


def test_materialize_makes_contraction_operands_buffers():
    m = W.WideMLP(batch=8, width=16, classes=4, depth=2)
    g = m.graph()
    plain = S.create_schedule([t.node for t in g.targets()])[0]
    nodes = S.materialize_contraction_operands([t.node for t in g.targets()])
    mat = S.create_schedule(nodes, keep_contractions=True)[0]

    def dense(it):
        end = it.ast.src[0]
        return S._is_dense_contraction(end.src[0].src[1])
    assert sum(dense(it) for it in mat) == 8 and sum(dense(it) for it in plain) < 8


def test_gradients_match_finite_differences(oracle):
    # tensor/gradient_test.go:500-534 — central differences, eps 1e-3
    R.DEFAULT_EXECUTOR = oracle
    rng = np.random.default_rng(3)
    x0 = rng.standard_normal(12).astype(np.float32)

    def f(xv, want_grad):
        R.reset()
        x = Tensor.new_leaf((3, 4)).set_data(xv)
        y = nn.softmax_rows(x.mul(x)).mul(x.exp2()).max([1]).sum()
        if want_grad:
            g = backward(y, [x])[x]
            R.realize(g)
            return g.data
        R.realize(y)
        return float(y.data[0])
    g = f(x0, True)
    for i in range(12):
        e = np.zeros(12, np.float32)
        e[i] = 1e-3
        fd = (f(x0 + e, False) - f(x0 - e, False)) / 2e-3
        assert abs(fd - g[i]) < 5e-3 * max(1.0, abs(fd)), (i, fd, g[i])
    R.DEFAULT_EXECUTOR = None


def test_jit_replays_without_rescheduling(oracle, monkeypatch):
    # tensor/jit_test.go:481 TestJITSkipsScheduling
    R.DEFAULT_EXECUTOR = oracle
    calls = []
    orig = S.create_schedule
    monkeypatch.setattr(S, "create_schedule", lambda *a, **k: (calls.append(1), orig(*a, **k))[1])
    jit = R.JIT()
    outs = []
    for step in range(3):
        x = Tensor.new_leaf((4,)).set_data(np.arange(4) + step)
        y = x.exp2().sum()
        jit.realize(y)
        outs.append(float(y.data[0]))
    assert len(calls) == 1 and jit.stats() == (1, 2)
    assert np.allclose(outs, [np.exp2(np.arange(4) + s).sum() for s in range(3)])
    # a structurally different graph re-captures
    x = Tensor.new_leaf((4,)).set_data(np.arange(4))
    jit.realize(x.exp2().max())
    assert jit.stats()[0] == 2
    R.DEFAULT_EXECUTOR = None


def test_realize_without_backend_reports_it():
    R.DEFAULT_EXECUTOR = None
    with pytest.raises(R.RealizeError, match="no backend registered"):
        R.realize(Tensor.new_leaf((2,)).exp2())


def test_movement_ops_dissolve_into_one_kernel(oracle):
    """schedule/schedule_test.go:613-807: a movement op followed by an elementwise op (or a
    reduction) is one kernel — reshape, permute, expand, shrink, pad, flip, a scalar sum, a sum over
    a permuted tensor; the reference only counts kernels and checks their structure, here the values
    are checked against numpy as well."""
    def data(shape):
        return (np.arange(1, int(np.prod(shape)) + 1, dtype=np.float32) * np.float32(0.25))

    cases = [
        ((32,), lambda t: t.reshape((4, 8)).neg(), lambda a: -a.reshape(4, 8)),
        ((3, 4), lambda t: t.permute((1, 0)).sin(), lambda a: np.sin(a.T)),
        ((1, 4), lambda t: t.expand((3, 4)).sqrt(), lambda a: np.sqrt(np.broadcast_to(a, (3, 4)))),
        ((4, 8), lambda t: t.shrink(((0, 2), (2, 6))).recip(), lambda a: 1.0 / a[0:2, 2:6]),
        ((4,), lambda t: t.pad(((2, 2),)).exp2(), lambda a: np.exp2(np.pad(a, (2, 2)))),
        ((4, 4), lambda t: t.flip((True, False)).log2(), lambda a: np.log2(a[::-1])),
        ((4, 8), lambda t: t.sum([0, 1]), lambda a: a.sum()),
        ((3, 4), lambda t: t.permute((1, 0)).sum([0]), lambda a: a.T.sum(0)),
    ]
    for shape, build, ref in cases:
        R.reset()
        x = Tensor.new_leaf(shape).set_data(data(shape))
        y = build(x)
        items, out = S.create_schedule([y.node])
        assert len(items) == 1, (shape, len(items))
        got = oracle.run(items, R.leaf_inputs([y]))[out[y.node.idx]]
        want = np.asarray(ref(data(shape).astype(np.float64).reshape(shape)), np.float64).reshape(-1)
        assert np.allclose(got, want, rtol=1e-6, atol=1e-6), (shape, got, want)


def test_row_major_strides_known_answers():
    """schedule/index_sint_test.go:69-143: strides[i] = product of the dims to the right; a symbolic
    (outermost) dim takes the product of the concrete tail and contributes nothing itself."""
    for dims, want in (((4,), [1]), ((2, 3), [3, 1]), ((2, 3, 5), [15, 5, 1]), ((2, 3, 5, 7), [105, 35, 7, 1]),
                       ((4, 1, 3), [3, 3, 1])):
        assert S._strides(dims) == want
    n = U.Var("n", 1, 64)
    assert S._strides((n, 16)) == [16, 1]
    assert S._strides((U.Var("m", 1, 32), 4, 8)) == [32, 8, 1]
    assert S._strides((U.Var("k", 1, 8),)) == [1]


def test_stats_hook_reports_each_scheduling_run():
    """schedule/stats.go:14-18: the hook is called once per successful CreateSchedule with the graph size,
    the kernel count and the number of reduce kernels spliced into their consumers."""
    from anneal_b200 import schedule as S, workloads as W
    seen = []
    S.STATS_HOOK = seen.append
    try:
        R.reset()
        m = W.MLP(batch=8, dims=(16, 12, 10))
        items, _ = R.build_schedule(m.graph().targets())
    finally:
        S.STATS_HOOK = None
    assert len(seen) == 1
    st = seen[0]
    assert st.kernels == len(items) and st.uops > st.kernels and st.fused >= 1 and st.pass_name == "memory_plan"
    R.reset()
    R.build_schedule(W.MLP(batch=8, dims=(16, 12, 10)).graph().targets())
    assert len(seen) == 1               # cleared hook: no further calls
