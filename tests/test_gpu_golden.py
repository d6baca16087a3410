"""The CUDA device against the known-answer vectors of the reference's own tests.

The same cases pin the CPU oracle in test_oracle_golden.py; here every one of them goes through the
C ABI to the GPU, so the device is checked against the reference's literal expectations directly and
not only against the oracle. Tolerances are the ones the reference's tests state (each case carries
its own; exact where the reference compares exactly)."""
import numpy as np
import pytest

import test_oracle_golden as G
from anneal_b200 import realize as R, tensor as tensor_mod
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes

pytestmark = pytest.mark.gpu
GOLD = G.GOLD


@pytest.fixture(autouse=True)
def use_cuda(cuda):
    R.DEFAULT_EXECUTOR = cuda
    yield
    R.DEFAULT_EXECUTOR = None


@pytest.mark.parametrize("case", GOLD["value_oracles"], ids=lambda c: c["graph"] + "@" + c["ref"].split(":")[1])
def test_value_oracles(case):
    G.test_value_oracles(case)


@pytest.mark.parametrize("case", GOLD["padded_reduce"], ids=lambda c: c["ref"].split(":")[1])
def test_padded_reduce_uses_the_reduce_identity(case):
    G.test_padded_reduce_uses_the_reduce_identity(case)


def test_sgd_quadratic_trajectory():
    G.test_sgd_quadratic_trajectory()


@pytest.mark.parametrize("case", GOLD["maxpool"]["cases"], ids=str)
def test_maxpool_forward_exact(case):
    G.test_maxpool_forward_exact(case)


def test_f16_cast_round_trip_is_bit_exact():
    G.test_f16_cast_round_trip_is_bit_exact()


def test_bf16_round_trip_truncates():
    G.test_bf16_round_trip_truncates()


def test_bf16_add_matches_truncation_model():
    G.test_bf16_add_matches_truncation_model()


def test_f32_to_f16_known_answers_on_upload():
    """The f32 -> f16 bit patterns of the reference's two conversion tests (the uop package's and the
    backend's own copy, backend/webgpu/conversion_test.go:8-51), through the device's own conversion: values travel as f32, are rounded to f16 storage on
    upload, and come back widened. NaN inputs must stay NaN; everything else is compared bit for
    bit against the expected f16 pattern widened to f32."""
    cases = GOLD["f32_to_f16_bits"]["cases"] + GOLD["backend_f32_to_f16_bits"]["cases"]
    src = np.array([c[0] for c in cases], dtype=np.uint32).view(np.float32)
    want = np.array([c[1] for c in cases], dtype=np.uint16).view(np.float16).astype(np.float32)
    # set_data would quantise on the host first; hand the raw f32 values to the device instead
    x = Tensor.new_leaf((src.size,), dtypes.float16)
    x.data = src.copy()
    tensor_mod.LEAF_DATA[x.node.idx] = x.data
    y = x.cast(dtypes.float32)
    R.realize(y)
    nan = np.isnan(want)
    assert np.isnan(y.data[nan]).all()
    assert np.array_equal(y.data[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_bulk_f16_values_survive_the_round_trip(cuda):
    """backend/webgpu/conversion_test.go:79-99: 0, 1, 2 and 65504 are exact in f16; stored in an
    f16 buffer and read back they are unchanged."""
    x = np.asarray(GOLD["backend_bulk_f16"]["x"], np.float32)
    buf = cuda.buffer(dtypes.float16, x.size)
    buf.upload(x)
    assert np.array_equal(buf.download(), x)
    buf.release()


def test_symbolic_add_compiles_once_for_both_extents(cuda):
    """backend/webgpu/symbolic_test.go:27-152: one symbolic kernel, dispatched at n = 8 and at
    n = 128 with the reference's inputs; exact results, and the second extent compiles nothing."""
    runs = GOLD["symbolic_add"]["runs"]
    G.symbolic_add_run(runs[0])
    compiles = cuda.stats()["nvrtc_compiles"]
    R.reset()
    G.symbolic_add_run(runs[1])
    assert cuda.stats()["nvrtc_compiles"] == compiles


@pytest.mark.parametrize("case", GOLD["gradient_checks"]["cases"], ids=lambda c: c["f"])
def test_gradient_known_answers(case):
    G.gradient_check(case)


@pytest.mark.parametrize("case", GOLD["structured_gradients"]["cases"], ids=lambda c: c["graph"])
def test_structured_gradient_known_answers(case):
    G.structured_gradient_check(case)


@pytest.mark.parametrize("case", GOLD["maxpool_backward"]["cases"], ids=str)
def test_maxpool_backward_known_answers(case):
    G.maxpool_backward_check(case)


@pytest.mark.parametrize("case", GOLD["maxpool_ties"]["cases"], ids=lambda c: str(c["shape"]))
def test_maxpool_ties_split_equally(case):
    G.maxpool_tie_check(case)


def test_f16_arithmetic_is_rounded_per_op():
    G.test_f16_arithmetic_is_rounded_per_op()


def test_max_identity_is_minus_flt_max_not_inf():
    G.test_max_identity_is_minus_flt_max_not_inf()


def test_empty_schedule_returns_nothing(cuda):
    """backend/webgpu/executor.go:27-29: no items, no outputs, no error."""
    import ctypes as C
    from anneal_b200 import kir
    assert not cuda.run([], {})
    blob = kir.serialize([])                  # the same through the C entry point itself
    n = C.c_int(7)
    rc = cuda.L.anl_run(cuda.h, blob, len(blob), None, 0, None, 0, None, 0, None, C.byref(n))
    assert rc == 0 and n.value == 0


def test_unknown_input_keys_are_ignored(cuda, oracle):
    """backend/webgpu/executor.go:161-165: inputs are looked up by the buffers' ids; keys that no
    buffer names are skipped silently, and the caller's arrays are left untouched."""
    x = Tensor.new_leaf((5,), dtypes.float32).set_data(np.arange(5, dtype=np.float32))
    y = x.add(x)
    items, out_ids = R.build_schedule([y])
    inputs = R.leaf_inputs([y])
    keep = {k: v.copy() for k, v in inputs.items()}
    inputs[0xFFFFFF] = np.ones(3, np.float32)
    got = cuda.run(items, inputs)
    assert np.array_equal(got[out_ids[0]], np.arange(5, dtype=np.float32) * 2)
    for k, v in keep.items():
        assert np.array_equal(inputs[k], v)
