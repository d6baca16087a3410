"""The C-ABI library loads without a GPU and exports every symbol include/anneal_cuda.h declares;
the renderer and NVRTC work on the CPU box (no kernel is launched here)."""
import ctypes
import os
import re

import numpy as np
import pytest

from anneal_b200 import build, device, nn, realize as R, workloads as W
from anneal_b200.tensor import Tensor
from anneal_b200.uop import dtypes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return device.load_library()


def test_header_and_library_agree(lib):
    hdr = open(os.path.join(ROOT, "include", "anneal_cuda.h")).read()
    declared = set(re.findall(r"\b(anl_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(device.ABI_SYMBOLS), declared ^ set(device.ABI_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_open_without_gpu_fails_cleanly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    assert lib.anl_open(0, 0, ctypes.byref(h)) != 0 and not h.value
    with pytest.raises(device.DeviceError):
        device.Device(0)


def test_malformed_blob_is_rejected(lib):
    src = ctypes.create_string_buffer(64)
    n = ctypes.c_size_t()
    k, b, o = ctypes.c_int(), ctypes.c_int(), ctypes.c_int64()
    note = ctypes.create_string_buffer(64)
    for blob in (b"", b"NOPE\0\0\0\0", b"KIR1\x01\0\0\0\x05"):
        rc = lib.anl_lower(None, blob, len(blob), 0, None, src, 64, ctypes.byref(n), ctypes.byref(k), ctypes.byref(b), ctypes.byref(o), note, 64)
        assert rc != 0


def _lower_all(tensors):
    items, _ = R.build_schedule(tensors)
    out = []
    for i in range(len(items)):
        r = device.lower(items, i)
        device.compile_check(r["source"])
        out.append(r)
    return items, out


def test_elementwise_uses_128_bit_accesses_when_provable():
    x = Tensor.new_leaf((64, 512))
    b = Tensor.new_leaf((512,))
    _, low = _lower_all([x.add(b.reshape((1, 512)).expand((64, 512))).exp2()])
    assert low[0]["class"] == "elementwise" and "V=4" in low[0]["note"]
    assert "ldv_<float, 4>" in low[0]["source"] and "stv_<float, 4>" in low[0]["source"]
    # a transposed read cannot be vectorised
    _, low = _lower_all([x.permute((1, 0)).exp2()])
    assert "V=1" in low[0]["note"]


def test_index_arithmetic_is_canonicalised():
    # reshape/expand/permute chains arrive as div/mod trees (schedule/index.go:231-293); the load of a
    # matmul operand must come out as a plain affine index
    a, b = Tensor.new_leaf((37, 53)), Tensor.new_leaf((53, 29))
    _, low = _lower_all([a.matmul(b)])
    body = low[0]["source"][low[0]["source"].index('extern "C"'):]
    assert re.search(r"data1\[\(r\d+ \* 53 \+ r\d+\)\]", body), body


def test_f16_reduce_accumulates_in_f32_and_narrows_once():
    # codegen/f16_codegen_test.go: "var acc0: f32" for an f16 matmul
    a, b = Tensor.new_leaf((8, 16), dtypes.float16), Tensor.new_leaf((16, 8), dtypes.float16)
    _, low = _lower_all([a.matmul(b)])
    src = low[0]["source"]
    assert re.search(r"float acc\d+ = 0.0f;", src) and "__float2half_rn(acc" in src and "__half2float(data1[" in src


def test_max_identity_and_scalar_reduce():
    x = Tensor.new_leaf((8,))
    _, low = _lower_all([x.max()])
    assert "__int_as_float(0xff7fffff)" in low[0]["source"]


def test_pad_guarded_load_is_clamped():
    x = Tensor.new_leaf((4,))
    _, low = _lower_all([x.pad(((2, 2),)).sum([0])])
    assert "clampi_(" in low[0]["source"]


def test_symbolic_kernel_takes_the_bound_as_argument():
    m = W.DynMLP(din=32, hidden=48, dout=16, max_batch=64)
    out, loss, grads, _ = m.graph(8)
    items, low = _lower_all([out] + grads)
    assert any("const int n0" in r["source"] for r in low)
    assert all(it.sym_vars == ["n"] for it in items if any(0 in b.shape for b in it.bufs))


def test_all_benchmark_configs_render_and_compile():
    for build_graph in (lambda: W.MLP().graph().targets(), lambda: W.SmallCNN(batch=2, hw=8, c1=2, c2=3).graph().targets(),
                        lambda: W.SoftmaxFwdBwd(16, 128).graph(True)[0]):
        R.reset()
        _lower_all(build_graph())
    R.reset()
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.WideMLP(batch=64, width=64, classes=72, depth=2)
        items, low = _lower_all(m.graph().targets())
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    assert any("row-broadcast" in r["note"] for r in low)


def test_opts_change_the_launch_shape():
    x = Tensor.new_leaf((300, 700))
    items, _ = R.build_schedule([x.sum([1])])
    base = device.lower(items, 0)
    forced = device.lower(items, 0, [128, 4, 0, 0, 0])
    assert forced["block"] == 128 and "lanes=4" in forced["note"] and base["note"] != forced["note"]
    split = device.lower(R.build_schedule([Tensor.new_leaf((1 << 20,)).sum()])[0], 0)
    assert split["class"] == "reduce_split"


def test_f16_elementwise_kernels_pair_their_arithmetic():
    """All-f16 elementwise kernels are rendered in __half2 (two outputs per instruction); a kernel
    with an f32 value in it keeps the one-element form. Both must compile for sm_100a."""
    from anneal_b200 import nn
    R.reset()
    x = Tensor.new_leaf((64, 256), dtypes.float16)
    b = Tensor.new_leaf((256,), dtypes.float16)
    from anneal_b200.tensor import broadcast_to
    items, _ = R.build_schedule([nn.gelu_tanh(x.add(broadcast_to(b, (64, 256))))])
    low = device.lower(items, 0)
    assert "paired f16" in low["note"] and "__hmul2" in low["source"] and "h2_ex2_" in low["source"]
    assert "* 0x1p+0f" not in low["source"]                   # multiplications by one are folded
    device.compile_check(low["source"])
    # a comparison and a select stay paired: masks and a bitwise select
    R.reset()
    y = Tensor.new_leaf((64, 256), dtypes.float16)
    z = Tensor.new_leaf((64, 256), dtypes.float16)
    items, _ = R.build_schedule([y.maximum(z).mul(y)])
    low = device.lower(items, 0)
    assert "paired f16" in low["note"]
    device.compile_check(low["source"])
    # mixed precision: not paired
    R.reset()
    w = Tensor.new_leaf((64, 256), dtypes.float32)
    items, _ = R.build_schedule([w.mul(w).exp()])
    low = device.lower(items, 0)
    assert "paired" not in low["note"]
    device.compile_check(low["source"])


def test_contraction_is_reported_with_symbolic_extents():
    """`lower` says when the device would route an item to a contraction kernel: f32 with the bound
    batch as M (forward) or as K (weight gradient)."""
    R.reset()
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.DynMLP(din=64, hidden=128, dout=32, max_batch=4096)
        out, loss, grads, _ = m.graph(8)
        items, _ = R.build_schedule([out] + grads)
        notes = [device.lower(items, i)["note"] for i in range(len(items))]
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    assert any("contraction f32 M=n N=128 K=64" in n for n in notes)
    assert any("contraction f32 M=128 N=64 K=n" in n for n in notes)


def test_row_chain_sweeps_wide_rows_in_chunks():
    """A softmax forward+backward whose rows are a multiple of 4 x 512 elements is rendered with one
    128-bit load per operand and chunk and a 128-bit store; narrower rows keep the one-element
    form. Both compile for sm_100a."""
    R.reset()
    s = W.SoftmaxFwdBwd(8, 4096)
    ts, _ = s.graph()
    items, _ = R.build_schedule(ts)
    wide = device.lower_chain(items, 0, len(items))["source"]
    assert wide.count("ldv_<float, 4>") >= 7 and "stv_<float, 4>" in wide
    device.compile_check(wide)
    R.reset()
    s = W.SoftmaxFwdBwd(8, 320)
    ts, _ = s.graph()
    items, _ = R.build_schedule(ts)
    narrow = device.lower_chain(items, 0, len(items))["source"]
    assert "ldv_<float, 4>(" not in narrow.split("row_chain(")[1]
    device.compile_check(narrow)


def test_damaged_blobs_never_crash_the_library():
    """Truncated and bit-damaged schedules must come back as a status from `anl_lower` and
    `anl_lower_chain` (parser + code generator), never as a crash: the helper runs in a child
    process so that a segmentation fault shows up as its exit code."""
    import os
    import subprocess
    import sys
    helper = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kir_fuzz.py")
    for seed in (1, 2):
        r = subprocess.run([sys.executable, helper, str(seed), "4000"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, (seed, r.returncode, r.stderr[-400:])
        assert "rejected=" in r.stdout


def test_contraction_kernel_sources_compile_with_and_without_a_fused_consumer(lib):
    """The two-CTA tcgen05 kernel is compiled at run time; every variant the wide MLP needs — the three
    operand layouts, the bias + GELU consumer, the logits' bias add, the GELU-backward product —
    must get through NVRTC for sm_100a on a box without a GPU."""
    R.reset()
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    try:
        m = W.WideMLP(batch=512, width=256, classes=136, depth=2)
        items, _ = R.build_schedule(m.graph().targets())
    finally:
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
    plain = fused = 0
    layouts = set()
    for i in range(len(items)):
        try:
            r = device.lower_gemm(items, i)
        except device.DeviceError:
            continue
        plain += 1
        layouts.add(r["note"].split(" M=")[0])
        device.compile_check(r["source"])
        try:
            f = device.lower_gemm(items, i, fuse_next=True)
        except device.DeviceError:
            continue
        fused += 1
        assert "void epi8_(" in f["source"] and "#define CFG_EPI 1" in f["source"]
        # the consumer's operand loads live in a function of their own, so that the kernel can issue them ahead
        assert "void epi8_load_(" in f["source"] and re.search(r"#define EPI_NRAW [12]\b", f["source"])
        device.compile_check(f["source"])
    assert plain == 7 and fused == 5, (plain, fused)
    assert layouts == {"gemm tcgen05 A:K B:K", "gemm tcgen05 A:K B:MN", "gemm tcgen05 A:MN B:MN"}
    # the tunables are compile-time constants of the source
    tuned = device.lower_gemm(items, 0, opts=device.gemm_opts(tile_n=128, stages=4, group_m=-1, stream_stores=1))["source"]
    for line in ("#define CFG_BNT 128", "#define CFG_STAGES 4", "#define CFG_GROUP_M 0", "#define CFG_STREAM_STORES 1"):
        assert line in tuned
    device.compile_check(tuned)


def test_f32_contraction_kernel_sources_compile_in_3xtf32_form(lib):
    """Large f32 contractions take the two-CTA kernel with f32 operands split into TF32 halves (the split
    pre-pass hands every operand layout over k-contiguous); the source must get through NVRTC for
    sm_100a on a box without a GPU."""
    from anneal_b200.tensor import Tensor
    from anneal_b200.uop import dtypes
    seen = set()
    for layout in ("KK", "KM", "MK", "MM"):
        R.reset()
        M, N, K = 2048, 1024, 1024
        a = Tensor.new_leaf((M, K), dtypes.float32) if layout[0] == "K" else Tensor.new_leaf((K, M), dtypes.float32).permute((1, 0))
        b = Tensor.new_leaf((N, K), dtypes.float32).permute((1, 0)) if layout[1] == "K" else Tensor.new_leaf((K, N), dtypes.float32)
        items, _ = R.build_schedule([a.matmul(b)])
        r = device.lower_gemm(items, 0)
        assert "3xTF32" in r["note"] and "#define CFG_TF32 1" in r["source"] and "kind::tf32" in r["source"]
        assert "#define CFG_A_MN 0" in r["source"] and "#define CFG_B_MN 0" in r["source"]
        seen.add(r["note"].split(" M=")[0])
        device.compile_check(r["source"])
    assert len(seen) == 4, seen
    # a small one stays on the FP32 pipes
    R.reset()
    items, _ = R.build_schedule([Tensor.new_leaf((512, 640), dtypes.float32).matmul(Tensor.new_leaf((640, 136), dtypes.float32))])
    with pytest.raises(device.DeviceError):
        device.lower_gemm(items, 0)
