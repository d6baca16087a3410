"""safetensors checkpoints for ``nn.Parameter`` maps, after tensor/safetensors/safetensors.go.

Layout: 8-byte little-endian header length, that many bytes of JSON (tensor name →
``{"dtype", "shape", "data_offsets"}``, padded with spaces to a multiple of 8), then
the raw little-endian tensor bytes. ``save`` always writes F32 in lexicographic name
order (safetensors.go:70-146); ``load`` converts F64, F16, BF16, integer and BOOL
tensors to float32 with the reference's rules (safetensors.go:21-35) and reports a
missing tensor, a shape mismatch or an unsupported dtype with the reference's
messages. A ``__metadata__`` entry is ignored.

The caller owns the names (a ``dict`` from name to Parameter), as in the reference.
For device-resident training, ``ResidentTrainer.save_checkpoint`` / ``load_checkpoint``
move the f32 master weights through this format.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Tuple

import numpy as np

MAX_EXACT_INT = 1 << 24      # largest |integer| a float32 holds exactly (safetensors.go:57-60)

_NP = {"F32": "<f4", "F64": "<f8", "F16": "<f2", "I8": "i1", "I16": "<i2", "I32": "<i4", "I64": "<i8",
       "U8": "u1", "U16": "<u2", "U32": "<u4", "U64": "<u8", "BOOL": "u1", "BF16": "<u2"}


class SafetensorsError(ValueError):
    pass


def _gofmt(shape) -> str:
    """A shape printed the way Go's %v prints a slice, so messages read like the reference's."""
    return "[" + " ".join(str(int(d)) for d in shape) + "]"


def save(path: str, params: Dict[str, "object"]) -> None:
    """Write every parameter's ``value`` as F32; names sorted for a deterministic file."""
    header: Dict[str, dict] = {}
    chunks: List[bytes] = []
    off = 0
    for name in sorted(params):
        p = params[name]
        data = np.ascontiguousarray(p.value, dtype="<f4").reshape(-1)
        n = int(np.prod(p.shape)) if len(p.shape) else 1
        if data.size != n:
            raise SafetensorsError(f"safetensors: tensor {name!r}: value has {data.size} elements, shape {_gofmt(p.shape)} expects {n}")
        raw = data.tobytes()
        header[name] = {"dtype": "F32", "shape": [int(d) for d in p.shape], "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hdr = json.dumps(header, separators=(",", ":"), sort_keys=True).encode("utf-8")
    if len(hdr) % 8:
        hdr += b" " * (8 - len(hdr) % 8)
    try:
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(hdr)))
            f.write(hdr)
            for c in chunks:
                f.write(c)
    except OSError as e:
        raise SafetensorsError(f"safetensors: create {path!r}: {e}") from e


def _to_f32(name: str, dtype: str, raw: bytes, shape) -> np.ndarray:
    if dtype not in _NP:
        raise SafetensorsError(f"safetensors: tensor {name!r}: unsupported dtype {dtype}")
    count = int(np.prod(shape)) if len(shape) else 1
    a = np.frombuffer(raw, dtype=_NP[dtype])
    if a.size != count:
        raise SafetensorsError(f"safetensors: tensor {name!r}: dtype {dtype} shape {_gofmt(shape)} expects "
                               f"{count * np.dtype(_NP[dtype]).itemsize} bytes, got {len(raw)}")
    if dtype == "BF16":
        return (a.astype(np.uint32) << np.uint32(16)).view(np.float32)
    if dtype == "BOOL":
        return (a != 0).astype(np.float32)
    if dtype in ("I32", "I64", "U32", "U64"):
        big = np.abs(a.astype(np.float64)) > MAX_EXACT_INT
        if big.any():
            v = a[big][0]
            raise SafetensorsError(f"safetensors: tensor {name!r}: integer value {int(v)} is not exactly representable as float32")
    return a.astype(np.float32)


def load_entries(path: str) -> Dict[str, Tuple[Tuple[int, ...], np.ndarray]]:
    """Every tensor of the file as (shape, float32 data)."""
    try:
        with open(path, "rb") as f:
            blob = f.read()
    except OSError as e:
        raise SafetensorsError(f"safetensors: open {path!r}: {e}") from e
    if len(blob) < 8:
        raise SafetensorsError("safetensors: read header length: file shorter than 8 bytes")
    (hlen,) = struct.unpack("<Q", blob[:8])
    if 8 + hlen > len(blob):
        raise SafetensorsError(f"safetensors: read header ({hlen} bytes): unexpected end of file")
    try:
        header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    except ValueError as e:
        raise SafetensorsError(f"safetensors: parse header JSON: {e}") from e
    data = blob[8 + hlen:]
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (a, b) = ent["dtype"], tuple(int(d) for d in ent["shape"]), ent["data_offsets"]
        except (KeyError, TypeError, ValueError) as e:
            raise SafetensorsError(f"safetensors: parse entry {name!r}: {e}") from e
        if a < 0 or b < a or b > len(data):
            raise SafetensorsError(f"safetensors: tensor {name!r} data_offsets [{a},{b}] out of range (data buffer is {len(data)} bytes)")
        out[name] = (shape, _to_f32(name, dtype, data[a:b], shape))
    return out


def load(path: str, into: Dict[str, "object"]) -> None:
    """Restore ``value`` of every parameter in ``into``; the file must hold each name with the same shape."""
    entries = load_entries(path)
    for name, p in into.items():
        if name not in entries:
            raise SafetensorsError(f"safetensors: tensor {name!r} not found in {path!r}")
        shape, data = entries[name]
        if tuple(shape) != tuple(p.shape):
            raise SafetensorsError(f"safetensors: tensor {name!r} shape mismatch: file has {_gofmt(shape)}, parameter expects {_gofmt(p.shape)}")
        p.value[:] = data
