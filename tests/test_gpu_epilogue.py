"""A contraction, the elementwise kernel behind it and a bias gradient as ONE launch of the two-CTA
tcgen05 kernel: the consumer's generated code in the epilogue, the contraction itself still stored
when anything else reads it, partial column sums finished by a small kernel.  The schedule is what
the reference would schedule; the fusion happens at launch and must not change a value the
separate launches produce, except for the order in which a bias gradient's f16 addends are summed
in f32."""
import numpy as np
import pytest

from anneal_b200 import realize as R, workloads as W
from anneal_b200.device import Device
from anneal_b200.realize import leaf_inputs
from anneal_b200.train import ResidentTrainer
from fullsize import check_every_kernel, unaliased
from util import rel_err

pytestmark = pytest.mark.gpu


def _wide(batch, width, classes, depth):
    R.reset()
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.WideMLP(batch=batch, width=width, classes=classes, depth=depth)
        x, y = m.make_inputs()
        g = m.graph(x, y)
        items, out_ids = R.build_schedule(g.targets())
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    return m, items, out_ids, leaf_inputs(g.targets())


@pytest.mark.parametrize("batch,width,classes", [(512, 256, 136), (520, 384, 200), (768, 512, 1000)])
def test_fused_launches_equal_separate_launches(batch, width, classes):
    """Ragged rows (520 = 2 pair tiles + 8 rows), ragged columns (136, 200 and 1000 are not multiples
    of the 256-wide tile), tiles narrower than one tile (136)."""
    m, items, out_ids, inputs = _wide(batch, width, classes, 2)
    keep = unaliased(items)
    res = []
    for flags in (0, Device.NO_EPILOGUE_FUSION):
        dev = Device(0, flags)
        try:
            s0 = dev.stats()
            got = dev.run(keep, inputs)
            s1 = dev.stats()
            res.append((got, {k: s1[k] - s0[k] for k in ("kernels_launched", "epilogues_fused", "colsums_fused", "gemm_launched")}))
        finally:
            dev.close()
    (fused, sf), (plain, sp) = res
    assert sp["epilogues_fused"] == 0 and sp["colsums_fused"] == 0
    # per layer: bias+GELU behind the forward contraction, the GELU-backward product behind the
    # input-gradient contraction; plus the logits' bias add; and one bias gradient per hidden layer
    assert sf["epilogues_fused"] == 2 + 2 + 1, sf
    assert sf["colsums_fused"] == 2, sf
    assert sf["gemm_launched"] == sp["gemm_launched"]
    assert sf["kernels_launched"] == sp["kernels_launched"] - 5, (sf, sp)      # 5 consumers gone; each bias gradient is still one (smaller) launch
    bias_grads = {it.bufs[0].uop_idx for it in keep if len(it.bufs[0].shape) == 1 and it.bufs[0].uop_idx in out_ids}
    where = {it.bufs[0].uop_idx: (n, it.bufs[0].shape) for n, it in enumerate(keep)}
    for k in plain:
        if k in bias_grads:
            assert rel_err(fused[k], plain[k]) <= 1e-3, (k, rel_err(fused[k], plain[k]))
        elif not np.array_equal(fused[k], plain[k]):
            n, shape = where[k]
            bad = np.argwhere(fused[k].reshape(shape) != plain[k].reshape(shape))
            raise AssertionError(f"kernel {n} output {shape}: {len(bad)} of {fused[k].size} values differ; rows {bad[:, 0].min()}..{bad[:, 0].max()}, "
                                 f"columns {bad[:, -1].min()}..{bad[:, -1].max()}; first {bad[0]}: fused {fused[k].reshape(shape)[tuple(bad[0])]} separate {plain[k].reshape(shape)[tuple(bad[0])]}; "
                                 f"distinct rows {len(np.unique(bad[:, 0]))}, distinct columns {len(np.unique(bad[:, -1]))}")


def test_fused_launches_against_the_oracle(cuda, oracle):
    m, items, out_ids, inputs = _wide(520, 384, 200, 2)
    e0 = cuda.stats()["epilogues_fused"]
    report, kept = check_every_kernel(cuda, oracle, items, inputs, 2e-3, samples=1 << 20)      # every element
    assert cuda.stats()["epilogues_fused"] - e0 == 5
    # without the buffers kept, the contraction's own output is not stored where only the consumer reads it
    got = cuda.run(items, inputs)
    for k in out_ids:
        assert np.array_equal(got[k], kept[k]), k


def test_fused_training_steps_follow_the_unfused_trajectory():
    """Resident training through the captured graph, fused and unfused: the losses agree to f16
    rounding of the bias gradients (every other value is identical step by step until those
    roundings feed back)."""
    res = []
    for flags in (0, Device.NO_EPILOGUE_FUSION):
        dev = Device(0, flags)
        try:
            R.reset()
            m = W.WideMLP(batch=512, width=512, classes=136, depth=3)
            x, y = m.make_inputs()
            tr = ResidentTrainer(dev, m, 0.05, use_graph=True, resident_inputs=True)
            tr.load_batch(x, y)
            losses = []
            for _ in range(6):
                tr.step()
                losses.append(tr.loss())
            res.append((losses, tr.parameters(), dev.stats()["epilogues_fused"]))
        finally:
            dev.close()
    (lf, pf, nf), (lp, pp, npl) = res
    assert nf > 0 and npl == 0
    assert lf[0] == lp[0]
    assert np.abs(np.array(lf) - np.array(lp)).max() <= 2e-3 * abs(lp[0])
    assert lf[-1] < lf[0]
    for a, b in zip(pf, pp):
        assert rel_err(a, b) <= 2e-3


def test_timed_out_barrier_is_reported_once_and_replays_recover(cuda):
    """The state a contraction leaves when a bounded barrier wait runs out (status code set, tile
    counter not signed off) is injected from the host; nothing on the GPU waits or fails.  The next
    call that waits for the device reports it; after that, eager runs and graph replays give the
    right answer again."""
    m, items, out_ids, inputs = _wide(512, 256, 136, 2)
    want = cuda.run(items, inputs)
    first = cuda.replay(items, inputs)
    for k in want:
        assert np.array_equal(first[k], want[k])
    cuda._check(cuda.L.anl_gemm_inject_status(cuda.h, 13, 77))
    from anneal_b200.device import DeviceError
    with pytest.raises(DeviceError, match="timed out on a barrier"):
        cuda.replay(items, inputs)
    again = cuda.replay(items, inputs)
    for k in want:
        assert np.array_equal(again[k], want[k])
    cuda._check(cuda.L.anl_gemm_inject_status(cuda.h, 3, 5))
    with pytest.raises(DeviceError, match="timed out on a barrier"):
        cuda.synchronize()
    eager = cuda.run(items, inputs)
    for k in want:
        assert np.array_equal(eager[k], want[k])
