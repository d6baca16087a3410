"""ctypes binding of the C oracle (oracle/kir_oracle.c). Test infrastructure only.

``OracleExecutor`` has the calling convention of the reference's
``backend.Executor`` / ``SymbolicExecutor`` (backend/device.go:10-37): inputs
and outputs are float32 arrays keyed by buffer id, and only final outputs (not
read by a later kernel) are returned.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libkir_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "kir_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_load.restype = C.c_void_p
        L.orc_load.argtypes = [C.c_char_p, C.c_size_t]
        L.orc_error.restype = C.c_char_p
        L.orc_error.argtypes = [C.c_void_p]
        L.orc_set_input.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_void_p, C.c_int64]
        L.orc_bind.argtypes = [C.c_void_p, C.c_char_p, C.c_int64]
        L.orc_run.argtypes = [C.c_void_p, C.c_int]
        L.orc_run_item.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_run_item_sampled.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_buffer_elems.restype = C.c_int64
        L.orc_buffer_elems.argtypes = [C.c_void_p, C.c_uint32]
        L.orc_get_buffer.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_int64]
        L.orc_free.argtypes = [C.c_void_p]
        L.orc_f32_to_f16_bits.restype = C.c_uint16
        L.orc_f32_to_f16_bits.argtypes = [C.c_float]
        L.orc_f16_round.restype = C.c_float
        L.orc_f16_round.argtypes = [C.c_float]
        _lib = L
    return _lib


class OracleError(RuntimeError):
    pass


class OracleExecutor:
    def __init__(self, threads: Optional[int] = None):
        self.threads = threads or (os.cpu_count() or 1)

    def run(self, items, inputs: Dict[int, np.ndarray], binding: Optional[Dict[str, int]] = None,
            want_all: bool = False) -> Dict[int, np.ndarray]:
        from anneal_b200 import kir
        if not items:
            return {}
        L = lib()
        blob = kir.serialize(items)
        h = L.orc_load(blob, len(blob))
        try:
            err = L.orc_error(h)
            if err:
                raise OracleError(err.decode())
            dt = {}
            for it in items:
                for b in it.bufs:
                    dt[b.uop_idx] = b.dtype.code
            for k, v in inputs.items():
                if k not in dt:
                    continue
                a = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
                L.orc_set_input(h, k, dt[k], a.ctypes.data, a.size)
            for k, v in (binding or {}).items():
                L.orc_bind(h, k.encode(), int(v))
            if L.orc_run(h, self.threads):
                raise OracleError(L.orc_error(h).decode())
            read = {b.uop_idx for it in items for b in it.bufs[1:]}
            out = {}
            for it in items:
                ob = it.bufs[0]
                if ob.uop_idx in read and ob.slot >= 0 and not want_all:
                    continue
                n = L.orc_buffer_elems(h, ob.uop_idx)
                a = np.empty(n, dtype=np.float32)
                L.orc_get_buffer(h, ob.uop_idx, a.ctypes.data, n)
                out[ob.uop_idx] = a
            return out
        finally:
            L.orc_free(h)

    def sample_item(self, item, inputs: Dict[int, np.ndarray], flat, binding: Optional[Dict[str, int]] = None, noise: bool = False):
        """The values kernel ``item`` stores at the flat output positions ``flat`` (row-major over its
        output), given float32 arrays for every buffer it reads. A benchmark-size contraction is
        checked this way on a few thousand outputs: n*K terms instead of M*N*K. Returns the positions
        in ascending order and the values at them; with ``noise`` also the modelled standard deviation
        of each value's rounding error (first-order propagation of independent roundings), which
        is what tells a sum whose terms cancel from a wrong result."""
        from anneal_b200 import kir
        L = lib()
        blob = kir.serialize([item])
        h = L.orc_load(blob, len(blob))
        try:
            err = L.orc_error(h)
            if err:
                raise OracleError(err.decode())
            for b in item.bufs[1:]:
                if b.uop_idx not in inputs:
                    raise OracleError(f"sample_item: no data for input buffer {b.uop_idx}")
                a = np.ascontiguousarray(inputs[b.uop_idx], dtype=np.float32).reshape(-1)
                L.orc_set_input(h, b.uop_idx, b.dtype.code, a.ctypes.data, a.size)
            for k, v in (binding or {}).items():
                L.orc_bind(h, k.encode(), int(v))
            idx = np.ascontiguousarray(np.sort(np.asarray(flat, dtype=np.int64)))
            out = np.empty(idx.size, dtype=np.float32)
            sigma = np.zeros(idx.size, dtype=np.float64) if noise else None
            if L.orc_run_item_sampled(h, 0, idx.ctypes.data, idx.size, out.ctypes.data, sigma.ctypes.data if noise else None, self.threads):
                raise OracleError(L.orc_error(h).decode())
            return (idx, out, sigma) if noise else (idx, out)
        finally:
            L.orc_free(h)

    def run_symbolic(self, items, inputs, binding):
        return self.run(items, inputs, binding)

    def close(self):
        pass
