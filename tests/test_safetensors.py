"""Checkpoint format, after tensor/safetensors/safetensors_test.go: round trips, write fidelity,
dtype conversions on load and the error messages."""
import json
import struct

import numpy as np
import pytest

from anneal_b200 import nn, safetensors as st


def _param(shape, values):
    p = nn.Parameter(shape)
    p.value[:] = np.asarray(values, dtype=np.float32).reshape(-1)
    return p


def _write(path, entries, metadata=None):
    """entries: name -> (dtype string, shape, raw bytes)"""
    header, data, off = {}, b"", 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dt, shape, raw) in entries.items():
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        data += raw
        off += len(raw)
    h = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(h)) + h + data)


def test_round_trip_and_write_fidelity(tmp_path):
    f = tmp_path / "ck.safetensors"
    a = {"l2.weight": _param((2, 3), [1, 2, 3, 4, 5, 6]), "l1.bias": _param((3,), [0.5, -0.25, 1e-8])}
    st.save(str(f), a)
    blob = f.read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    assert hlen % 8 == 0                                     # header padded with spaces to 8 bytes
    header = json.loads(blob[8:8 + hlen])
    assert list(header) == ["l1.bias", "l2.weight"]          # lexicographic order
    assert header["l1.bias"] == {"dtype": "F32", "shape": [3], "data_offsets": [0, 12]}
    assert header["l2.weight"]["data_offsets"] == [12, 36]
    assert blob[8 + hlen:8 + hlen + 12] == np.array([0.5, -0.25, 1e-8], "<f4").tobytes()
    b = {"l2.weight": nn.Parameter((2, 3)), "l1.bias": nn.Parameter((3,))}
    st.load(str(f), b)
    for k in a:
        assert np.array_equal(a[k].value, b[k].value)


def test_load_converts_other_dtypes(tmp_path):
    f = tmp_path / "multi.safetensors"
    _write(f, {
        "f64": ("F64", (2,), np.array([1.5, -2.25], "<f8").tobytes()),
        "f16": ("F16", (3,), np.array([1.0, -0.5, 65504.0], "<f2").tobytes()),
        "bf16": ("BF16", (2,), np.array([0x3F80, 0xC000], "<u2").tobytes()),      # 1.0, -2.0
        "i8": ("I8", (2,), np.array([-3, 7], "i1").tobytes()),
        "u16": ("U16", (1,), np.array([65535], "<u2").tobytes()),
        "i64": ("I64", (1,), np.array([1 << 24], "<i8").tobytes()),
        "bool": ("BOOL", (3,), bytes([0, 1, 2])),
    }, metadata={"format": "pt"})
    e = st.load_entries(str(f))
    assert "__metadata__" not in e
    assert e["f64"][1].tolist() == [1.5, -2.25]
    assert e["f16"][1].tolist() == [1.0, -0.5, 65504.0]
    assert e["bf16"][1].tolist() == [1.0, -2.0]
    assert e["i8"][1].tolist() == [-3.0, 7.0]
    assert e["u16"][1].tolist() == [65535.0]
    assert e["i64"][1].tolist() == [float(1 << 24)]
    assert e["bool"][1].tolist() == [0.0, 1.0, 1.0]
    assert all(v[1].dtype == np.float32 for v in e.values())


def test_errors(tmp_path):
    f = tmp_path / "bad.safetensors"
    _write(f, {"big": ("I32", (1,), np.array([(1 << 24) + 1], "<i4").tobytes())})
    with pytest.raises(st.SafetensorsError, match="not exactly representable"):
        st.load_entries(str(f))
    _write(f, {"q": ("F8_E4M3", (1,), b"\x00")})
    with pytest.raises(st.SafetensorsError, match="unsupported dtype F8_E4M3"):
        st.load_entries(str(f))
    _write(f, {"w": ("F32", (2, 2), np.zeros(4, "<f4").tobytes())})
    with pytest.raises(st.SafetensorsError, match=r"shape mismatch: file has \[2 2\], parameter expects \[4\]"):
        st.load(str(f), {"w": nn.Parameter((4,))})
    with pytest.raises(st.SafetensorsError, match="'b' not found"):
        st.load(str(f), {"b": nn.Parameter((1,))})
    _write(f, {"w": ("F32", (3,), np.zeros(2, "<f4").tobytes())})
    with pytest.raises(st.SafetensorsError, match="expects 12 bytes, got 8"):
        st.load_entries(str(f))
    with pytest.raises(st.SafetensorsError, match="open"):
        st.load_entries(str(tmp_path / "missing.safetensors"))
