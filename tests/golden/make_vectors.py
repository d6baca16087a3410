"""Writes tests/golden/reference_vectors.json.

The reference cannot be executed here (no Go toolchain), so the fixture is the set of known-answer
vectors that are literal in the reference's own test sources, transcribed with the file and line
they come from. Each case names a small graph the tests rebuild with the frontend, its inputs and
the expected output with the reference's own tolerance.
"""
import json
import math
import os

LN2 = math.log(2.0)

cases = {
    "source": "georgebuilds/anneal test files; see `ref` on each case",
    "value_oracles": [
        {"ref": "backend/webgpu/webgpu_test.go:84-103", "graph": "exp2", "x": [0, 1, 2, 3], "want": [1, 2, 4, 8], "tol": 1e-5},
        {"ref": "backend/webgpu/webgpu_test.go:107-127", "graph": "add", "x": [1, 2, 3, 4], "y": [10, 20, 30, 40], "want": [11, 22, 33, 44], "tol": 1e-5},
        {"ref": "backend/webgpu/webgpu_test.go:131-153", "graph": "sum_all", "x": [1, 2, 3, 4, 5, 6, 7, 8], "want": [36], "tol": 1e-3},
        {"ref": "backend/webgpu/webgpu_test.go:157-180", "graph": "sum_axis0_4x4", "x": list(range(1, 17)), "want": [28, 32, 36, 40], "tol": 1e-3},
        {"ref": "backend/webgpu/webgpu_test.go:188-210", "graph": "max_all", "x": [-5, -3, -1, -4], "want": [-1], "tol": 1e-5},
        {"ref": "backend/webgpu/webgpu_test.go:214-231", "graph": "log2_exp2", "x": [0.5, 1.0, 1.5, 2.0], "want": [0.5, 1.0, 1.5, 2.0], "tol": 1e-5},
        {"ref": "backend/webgpu/webgpu_test.go:235-266", "graph": "matmul_2x3_3x2", "x": [1, 2, 3, 4, 5, 6], "y": [7, 8, 9, 10, 11, 12], "want": [58, 64, 139, 154], "tol": 1e-2},
        {"ref": "backend/webgpu/webgpu_test.go:262-272", "graph": "exp2", "x": [1, 2, 3, 4], "want": [2, 4, 8, 16], "tol": 1e-5},
        {"ref": "backend/webgpu/webgpu_test.go:278-321", "graph": "mse_2x3_3x2", "x": [1, 2, 3, 4, 5, 6], "w": [0.1, 0.2, 0.3, 0.4, 0.5, 0.6], "t": [1.0, 2.0, 3.0, 4.0], "want": [2.8625], "tol": 1e-3},
        {"ref": "backend/webgpu/webgpu_test.go:327-359", "graph": "grad_sum_exp2", "x": [0, 1, 2, 3], "want": [LN2 * 1, LN2 * 2, LN2 * 4, LN2 * 8], "tol": 1e-4},
    ],
    "padded_reduce": [
        {"ref": "schedule/schedule_test.go:809-835", "op": "max", "shape": [4], "pad": [[2, 2]], "axis": 0, "x": [-3, -1, -4, -2], "want": [-1]},
        {"ref": "schedule/schedule_test.go:837-858", "op": "sum", "shape": [4], "pad": [[1, 1]], "axis": 0, "x": [1, 2, 3, 4], "want": [10]},
        {"ref": "schedule/schedule_test.go:860-881", "op": "max", "shape": [3], "pad": [[3, 3]], "axis": 0, "x": [5, 2, 8], "want": [8]},
        {"ref": "schedule/schedule_test.go:883-915", "op": "sum", "shape": [2, 3], "pad": [[1, 1], [0, 0]], "axis": 0, "x": [1, 2, 3, 4, 5, 6], "want": [5, 7, 9]},
    ],
    "sgd_trajectory": {"ref": "tensor/nn/train_test.go:71-144", "lr": 0.1, "n": 4, "steps": 4, "p0": 3.0, "target": 1.0, "tol": 1e-4,
                       "p": [3.0, 2.6, 2.28, 2.024, 1.8192], "grad": [4.0, 3.2, 2.56, 2.048]},
    "maxpool": {"ref": "tensor/nn/maxpool_test.go:16-111", "tol": 0,
                "cases": [[1, 1, 4, 4, 2, 2, 2, 2, False], [1, 1, 4, 4, 2, 2, 1, 1, False], [1, 1, 8, 8, 2, 2, 2, 2, False],
                          [1, 1, 8, 8, 4, 4, 4, 4, False], [1, 1, 8, 6, 3, 2, 2, 1, False], [1, 1, 4, 4, 2, 2, 2, 2, True],
                          [2, 3, 8, 8, 2, 2, 2, 2, False]]},
    "f16_cast_roundtrip": {"ref": "backend/webgpu/f16_test.go:268-296", "x": [0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -3.5, 0.00390625]},
    "bf16_roundtrip": {"ref": "backend/webgpu/f16_test.go:352-378", "x": [0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -3.5, 0.015625]},
    "f32_to_f16_bits": {"ref": "uop/dtype_conversion_test.go:8-63", "cases": [
        [0x00000000, 0x0000], [0x80000000, 0x8000], [0x3F800000, 0x3C00], [0xBF800000, 0xBC00], [0x40000000, 0x4000],
        [0x3F000000, 0x3800], [0x3E800000, 0x3400], [0x477FE000, 0x7BFF], [0x38800000, 0x0400],
        [0x3F801000, 0x3C00], [0x3F802000, 0x3C01], [0x3F803000, 0x3C02], [0x3F805000, 0x3C02],
        [0x33800000, 0x0001], [0x35800000, 0x0010], [0x38802000, 0x0401], [0x387FE000, 0x0400], [0x33000000, 0x0000],
        [0x477FF000, 0x7C00], [0x501502F9, 0x7C00], [0xD01502F9, 0xFC00],
        [0x7F800000, 0x7C00], [0xFF800000, 0xFC00], [0x7FC00000, 0x7E00], [0x7F800001, 0x7C01], [0x3F808000, 0x3C04]]},
    "f16_to_f32_bits": {"ref": "uop/dtype_conversion_test.go:65-99", "cases": [
        [0x0000, 0x00000000], [0x8000, 0x80000000], [0x3C00, 0x3F800000], [0xBC00, 0xBF800000], [0x7BFF, 0x477FE000],
        [0x0400, 0x38800000], [0x0001, 0x33800000], [0x7C00, 0x7F800000], [0xFC00, 0xFF800000]]},
    # the backend's own copy of the conversion (backend/webgpu/executor.go), tested with its own table
    "backend_f32_to_f16_bits": {"ref": "backend/webgpu/conversion_test.go:8-51", "cases": [
        [0x00000000, 0x0000], [0x80000000, 0x8000], [0x3F800000, 0x3C00], [0xBF800000, 0xBC00], [0x477FE000, 0x7BFF],
        [0x38800000, 0x0400], [0x3F801000, 0x3C00], [0x3F802000, 0x3C01], [0x3F803000, 0x3C02], [0x3F805000, 0x3C02],
        [0x33800000, 0x0001], [0x33000000, 0x0000], [0x477FF000, 0x7C00], [0x501502F9, 0x7C00],
        [0x7F800000, 0x7C00], [0x7FC00000, 0x7E00], [0x7F800001, 0x7C01]]},
    "backend_f16_to_f32_bits": {"ref": "backend/webgpu/conversion_test.go:53-77", "cases": [[0x3C00, 0x3F800000], [0x0001, 0x33800000]]},
    "backend_bulk_f16": {"ref": "backend/webgpu/conversion_test.go:79-99", "x": [0.0, 1.0, 2.0, 65504.0],
                         "bytes": [0x00, 0x00, 0x00, 0x3C, 0x00, 0x40, 0xFF, 0x7B]},
    # one compiled symbolic kernel out[i] = a[i] + b[i] dispatched at n = 8 and n = 128
    "symbolic_add": {"ref": "backend/webgpu/symbolic_test.go:27-152", "tol": 1e-5,
                     "runs": [{"n": 8, "a_scale": 1.0, "b_scale": 2.0}, {"n": 128, "a_scale": 0.5, "b_scale": 1.5}]},
    # gradient of sum(f(x)) for the primitive rules, inputs from the reference's testData helper
    # (tensor/gradient_test.go:540-551: 0.5 + 0.3 i + offset, wrapped to 0.5 + 0.3 (i % 4) above 2.5);
    # the reference compares Backward with central differences of its evaluator at these tolerances,
    # the expectation recorded here is the derivative's closed form
    "gradient_checks": {"ref": "tensor/gradient_test.go:555-704", "data": "testData(shape, offset), tensor/gradient_test.go:540-551", "cases": [
        {"f": "neg", "n": 3, "offset": 0.0, "tol": 1e-4, "ref": "tensor/gradient_test.go:555-565"},
        {"f": "exp2", "n": 3, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:567-577"},
        {"f": "log2", "n": 3, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:579-589"},
        {"f": "sin", "n": 4, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:591-601"},
        {"f": "sqrt", "n": 3, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:603-613"},
        {"f": "recip", "n": 3, "offset": 1.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:615-625"},
        {"f": "exp", "n": 3, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:631-641"},
        {"f": "log", "n": 3, "offset": 0.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:645-655"},
        {"f": "add", "n": 3, "offset": 0.0, "offset_y": 1.0, "tol": 1e-4, "ref": "tensor/gradient_test.go:659-672"},
        {"f": "mul", "n": 3, "offset": 0.0, "offset_y": 1.0, "tol": 1e-3, "ref": "tensor/gradient_test.go:674-687"},
        {"f": "diamond", "n": 3, "offset": 0.5, "tol": 1e-3, "ref": "tensor/gradient_test.go:691-702"}]},
    # the same comparison for the structured graphs: tolerances are the reference's, inputs testData with
    # the listed offsets, expectations the closed forms worked out in float64 by the test
    "structured_gradients": {"data": "testData(shape, offset), tensor/gradient_test.go:540-551", "cases": [
        {"graph": "broadcast", "ref": "tensor/gradient_test.go:730-744", "tol": {"w": 1e-3}},
        {"graph": "matmul", "ref": "tensor/gradient_test.go:748-762", "tol": {"x": 5e-3, "w": 5e-3}},
        {"graph": "linear", "ref": "tensor/gradient_test.go:766-794", "tol": {"w": 5e-3, "b": 3e-3}},
        {"graph": "mlp", "ref": "tensor/gradient_test.go:798-829", "tol": {"w1": 5e-3, "w2": 5e-3}},
        {"graph": "conv2d", "ref": "tensor/gradient_test.go:833-878", "tol": {"weight": 5e-3}},
        {"graph": "reduce_sum", "ref": "tensor/gradient_test.go:882-893", "tol": {"x": 5e-4}}]},
    # max-pool backward: data (i+1)*0.1, loss = sum(pool(x)^2); the reference checks the first four
    # elements against central differences at 1e-3, the tests check every element against the closed form
    "maxpool_backward": {"ref": "tensor/nn/maxpool_test.go:131-215", "tol": 1e-3,
                         "cases": [[1, 1, 4, 4, 2, 2, 2, 2], [1, 1, 4, 4, 2, 2, 1, 1], [1, 1, 6, 6, 3, 3, 3, 3], [8, 4, 4, 4, 2, 2, 2, 2]]},
    # ties split the adjoint equally (literal inputs and expectations)
    "maxpool_ties": {"ref": "tensor/nn/maxpool_test.go:217-305", "tol": 1e-5, "cases": [
        {"shape": [1, 1, 2, 2], "k": [2, 2], "s": [2, 2], "x": [3, 3, 1, 2], "want": [0.5, 0.5, 0, 0]},
        {"shape": [1, 1, 1, 9], "k": [1, 9], "s": [1, 9], "x": [5, 5, 5, 0, 0, 0, 0, 0, 0],
         "want": [1 / 3, 1 / 3, 1 / 3, 0, 0, 0, 0, 0, 0]}]},
    "beam_test_inputs": {"ref": "codegen/beam.go:410-420", "formula": "((j + i*17) % 13 + 1) * 0.01"},
}

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(out, "w") as f:
        json.dump(cases, f, indent=1)
    print(out)
