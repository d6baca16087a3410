"""ctypes binding of libanneal_cuda.so: the CUDA device behind anneal's
``backend.Executor`` / ``SymbolicExecutor`` / ``Benchmarker`` interfaces
(backend/device.go:10-37).

``Device.run`` and ``Device.run_symbolic`` take and return float32 arrays keyed
by buffer id, like the reference's ``Run`` / ``RunSymbolic``; only final outputs
come back. There is no CPU fallback: if the library or a GPU is missing the
constructor raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import kir

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libanneal_cuda.so")


class DeviceError(RuntimeError):
    """Raised with the backend's message, prefixed ``cuda:`` the way the reference
    prefixes ``webgpu:`` (backend/webgpu/executor.go:102)."""


class _Input(C.Structure):
    _fields_ = [("uop_idx", C.c_uint32), ("data", C.c_void_p), ("elems", C.c_int64), ("resident", C.c_void_p)]


class _Binding(C.Structure):
    _fields_ = [("name", C.c_char_p), ("value", C.c_int64)]


class _Output(C.Structure):
    _fields_ = [("uop_idx", C.c_uint32), ("data", C.POINTER(C.c_float)), ("elems", C.c_int64), ("resident", C.c_void_p),
                ("allreduce", C.c_int), ("sgd_master", C.c_void_p), ("sgd_param", C.c_void_p), ("sgd_lr", C.c_float),
                ("sgd_scale", C.c_float)]


class _Bench(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("min_us", "median_us", "max_us", "mean_us", "stddev_us", "cv")]


class _Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("kernels_launched", "gemm_launched", "nvrtc_compiles", "nvrtc_cache_hits",
                                          "lower_cache_hits", "h2d_bytes", "d2h_bytes", "graph_replays",
                                          "graph_captures", "device_allocs", "epilogues_fused", "colsums_fused", "side_launches")]


class _Prof(C.Structure):
    _fields_ = [("klass", C.c_int), ("launches", C.c_int), ("total_ms", C.c_double), ("flops", C.c_double)]


class _Beam(C.Structure):
    _fields_ = [("opts", C.c_int * 4), ("base_us", C.c_double), ("best_us", C.c_double), ("tried", C.c_int),
                ("rejected", C.c_int), ("from_cache", C.c_int)]


class _Info(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("sm_major", C.c_int), ("sm_minor", C.c_int), ("sm_count", C.c_int),
                ("total_mem", C.c_size_t), ("has_f16", C.c_int), ("has_bf16", C.c_int), ("has_tcgen05", C.c_int)]


_lib = None


def load_library():
    """dlopen the in-tree library; fails loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise DeviceError(f"cuda: {LIB_PATH} is missing; run `python -m anneal_b200.build`")
    L = C.CDLL(LIB_PATH)
    vp, i, u8p = C.c_void_p, C.c_int, C.c_char_p
    L.anl_open.argtypes = [i, C.c_uint, C.POINTER(vp)]
    L.anl_close.argtypes = [vp]
    L.anl_close.restype = None
    L.anl_last_error.argtypes = [vp]
    L.anl_last_error.restype = C.c_char_p
    L.anl_device_info.argtypes = [vp, C.POINTER(_Info)]
    L.anl_get_stats.argtypes = [vp, C.POINTER(_Stats)]
    L.anl_synchronize.argtypes = [vp]
    L.anl_gemm_inject_status.argtypes = [vp, i, i]
    L.anl_gemm_set_defaults.argtypes = [vp, C.POINTER(i)]
    L.anl_stream.argtypes = [vp]
    L.anl_stream.restype = vp
    L.anl_run.argtypes = [vp, u8p, C.c_size_t, C.POINTER(_Input), i, C.POINTER(_Binding), i,
                          C.POINTER(_Output), i, C.POINTER(_Output), C.POINTER(i)]
    L.anl_outputs_free.argtypes = [C.POINTER(_Output), i]
    L.anl_outputs_free.restype = None
    L.anl_lower.argtypes = [vp, u8p, C.c_size_t, i, C.POINTER(i), C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t),
                            C.POINTER(i), C.POINTER(i), C.POINTER(C.c_int64), C.c_char_p, C.c_size_t]
    L.anl_lower_chain.argtypes = [u8p, C.c_size_t, i, i, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
    L.anl_lower_gemm.argtypes = [vp, u8p, C.c_size_t, i, i, C.POINTER(i), C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
    L.anl_compile_check.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
    L.anl_benchmark.argtypes = [vp, u8p, C.c_size_t, i, C.POINTER(i), i, i, C.POINTER(_Bench)]
    L.anl_graph_create.argtypes = [vp, u8p, C.c_size_t, C.POINTER(vp)]
    L.anl_graph_replay.argtypes = [vp, C.POINTER(_Input), i, C.POINTER(_Binding), i,
                                   C.POINTER(_Output), i, C.POINTER(_Output), C.POINTER(i)]
    L.anl_graph_release.argtypes = [vp]
    L.anl_graph_release.restype = None
    L.anl_buffer_create.argtypes = [vp, i, C.c_int64, C.POINTER(vp)]
    L.anl_buffer_upload.argtypes = [vp, vp, C.c_int64]
    L.anl_buffer_upload_begin.argtypes = [vp, vp, C.c_int64]
    L.anl_buffer_upload_begin_stored.argtypes = [vp, vp, C.c_int64]
    L.anl_buffer_upload_commit.argtypes = [vp]
    L.anl_buffer_download.argtypes = [vp, vp, C.c_int64]
    L.anl_buffer_download_begin.argtypes = [vp, vp, C.c_int64]
    L.anl_buffer_download_wait.argtypes = [vp]
    L.anl_buffer_release.argtypes = [vp]
    L.anl_buffer_release.restype = None
    L.anl_buffer_view.argtypes = [vp, C.c_int64, C.c_int64, C.POINTER(vp)]
    L.anl_buffer_device_ptr.argtypes = [vp]
    L.anl_buffer_device_ptr.restype = vp
    L.anl_buffer_elems.argtypes = [vp]
    L.anl_buffer_elems.restype = C.c_int64
    L.anl_sgd_step.argtypes = [vp, vp, vp, vp, C.c_float, C.c_float]
    L.anl_comm_unique_id.argtypes = [C.c_char_p]
    L.anl_comm_init.argtypes = [vp, i, i, C.c_char_p]
    L.anl_allreduce_sum.argtypes = [vp, vp]
    L.anl_allgather.argtypes = [vp, vp]
    L.anl_comm_destroy.argtypes = [vp]
    L.anl_comm_set_timeout.argtypes = [vp, i]
    L.anl_comm_wait.argtypes = [vp]
    L.anl_comm_abort.argtypes = [vp]
    L.anl_comm_inject_delay.argtypes = [vp, i]
    L.anl_timer_start.argtypes = [vp]
    L.anl_timer_stop.argtypes = [vp, C.POINTER(C.c_float)]
    L.anl_profile_enable.argtypes = [vp, i]
    L.anl_profile_read.argtypes = [vp, C.POINTER(_Prof), i, C.POINTER(i)]
    L.anl_sum_f32_static.argtypes = [vp, C.c_int64, vp, vp, C.c_char_p, C.c_size_t]
    L.anl_beam_search.argtypes = [vp, u8p, C.c_size_t, i, i, i, C.c_char_p, C.POINTER(_Beam)]
    L.anl_host_alloc.argtypes = [C.c_size_t, C.POINTER(vp)]
    L.anl_host_free.argtypes = [vp]
    L.anl_host_free.restype = None
    _lib = L
    return L


#: every symbol include/anneal_cuda.h declares
ABI_SYMBOLS = [
    "anl_open", "anl_close", "anl_device_info", "anl_last_error", "anl_get_stats", "anl_run", "anl_outputs_free",
    "anl_lower", "anl_lower_chain", "anl_compile_check", "anl_benchmark", "anl_graph_create", "anl_graph_replay", "anl_graph_release",
    "anl_buffer_create", "anl_buffer_upload", "anl_buffer_upload_begin", "anl_buffer_upload_begin_stored", "anl_buffer_upload_commit", "anl_buffer_download", "anl_buffer_release", "anl_buffer_device_ptr",
    "anl_buffer_elems", "anl_buffer_view", "anl_sgd_step", "anl_comm_unique_id", "anl_comm_init", "anl_allreduce_sum", "anl_allgather",
    "anl_comm_destroy", "anl_comm_set_timeout", "anl_comm_wait", "anl_comm_abort", "anl_comm_inject_delay", "anl_host_alloc", "anl_host_free", "anl_synchronize", "anl_timer_start", "anl_timer_stop",
    "anl_profile_enable", "anl_profile_read", "anl_sum_f32_static", "anl_beam_search", "anl_stream", "anl_lower_gemm", "anl_gemm_inject_status", "anl_buffer_download_begin", "anl_buffer_download_wait", "anl_gemm_set_defaults",
]

KERNEL_CLASSES = {0: "elementwise", 1: "reduce", 2: "reduce_split", 3: "gemm", 4: "raw"}


#: include/anneal_cuda.h ANL_NUM_OPTS
NUM_OPTS = 11


def _opts(opts):
    """{block_threads, reduce_lanes, vector_width, split, debug_bounds, tile_n, stages, group_m,
    stream_stores, single_cta, whole_tail} as the C array the library expects, shorter lists padded with 0."""
    if not opts:
        return None
    return (C.c_int * NUM_OPTS)(*(list(opts) + [0] * NUM_OPTS)[:NUM_OPTS])


def gemm_opts(tile_n=0, stages=0, group_m=0, stream_stores=0, single_cta=0, whole_tail=0):
    """An opts list that only sets the contraction kernel's tunables."""
    return [0, 0, 0, 0, 0, tile_n, stages, group_m, stream_stores, single_cta, whole_tail]


def lower(items, index: int = 0, opts: Optional[Sequence[int]] = None):
    """CUDA C for one item, with its kernel class and launch shape. Needs no GPU
    (the counterpart of codegen.RenderWGSL, codegen/wgsl.go:36-39)."""
    L = load_library()
    blob = kir.serialize(items)
    cap = 1 << 16
    note = C.create_string_buffer(512)
    n = C.c_size_t()
    klass, block, opb = C.c_int(), C.c_int(), C.c_int64()
    o = _opts(opts)
    while True:
        src = C.create_string_buffer(cap)
        rc = L.anl_lower(None, blob, len(blob), index, o, src, cap, C.byref(n), C.byref(klass), C.byref(block),
                         C.byref(opb), note, 512)
        if rc or n.value < cap:
            break
        cap = n.value + 1
    if rc:
        raise DeviceError(f"cuda: lower: {note.value.decode()} (status {rc})")
    return {"source": src.value.decode(), "class": KERNEL_CLASSES.get(klass.value, "?"), "block": block.value,
            "outputs_per_block": opb.value, "note": note.value.decode()}


def lower_chain(items, first: int, count: int) -> dict:
    """CUDA C of items[first:first+count] fused into one row-chain kernel; raises if they do not qualify."""
    L = load_library()
    blob = kir.serialize(items)
    cap = 1 << 18
    src = C.create_string_buffer(cap)
    note = C.create_string_buffer(512)
    n = C.c_size_t()
    rc = L.anl_lower_chain(blob, len(blob), first, count, src, cap, C.byref(n), note, 512)
    if rc:
        raise DeviceError(f"cuda: lower_chain: {note.value.decode()} (status {rc})")
    return {"source": src.value.decode(), "note": note.value.decode()}


def lower_gemm(items, index: int, fuse_next: bool = False, opts: Optional[Sequence[int]] = None) -> dict:
    """Source of the two-CTA tcgen05 kernel for contraction items[index], with items[index+1] in its
    epilogue when ``fuse_next``; raises if the item does not take that kernel or the pair does not fuse."""
    L = load_library()
    blob = kir.serialize(items)
    cap = 1 << 18
    src = C.create_string_buffer(cap)
    note = C.create_string_buffer(512)
    n = C.c_size_t()
    rc = L.anl_lower_gemm(None, blob, len(blob), index, 1 if fuse_next else 0, _opts(opts), src, cap, C.byref(n), note, 512)
    if rc:
        raise DeviceError(f"cuda: lower_gemm: {note.value.decode()} (status {rc})")
    return {"source": src.value.decode(), "note": note.value.decode()}


def compile_check(source: str) -> str:
    """NVRTC-compile for sm_100a without a GPU; returns the log, raises on error."""
    L = load_library()
    log = C.create_string_buffer(1 << 16)
    rc = L.anl_compile_check(source.encode(), log, 1 << 16)
    if rc:
        raise DeviceError("cuda: compile failed: " + log.value.decode())
    return log.value.decode()


class GradientTarget:
    """Where a gradient output goes and what happens right behind it: optional all-reduce across
    ranks, optional SGD update of its parameter (master f32 + storage copy)."""

    def __init__(self, grad, master=None, param=None, lr: float = 0.0, scale: float = 1.0, allreduce=False):
        # allreduce: False/0 none, True/1 all-reduce then update everywhere, 2 reduce-scatter, update the
        # rank's own shard, all-gather the new parameter values
        self.grad, self.master, self.param, self.lr, self.scale, self.allreduce = grad, master, param, lr, scale, int(allreduce)


class ResidentBuffer:
    """A device buffer that outlives a run: parameters, master weights, gradients."""

    def __init__(self, dev: "Device", dtype, elems: int, _handle=None):
        self.dev, self.dtype, self.elems = dev, dtype, int(elems)
        if _handle is None:
            _handle = C.c_void_p()
            dev._check(dev.L.anl_buffer_create(dev.h, dtype.code, self.elems, C.byref(_handle)))
        self.h = _handle

    def view(self, offset: int, elems: int) -> "ResidentBuffer":
        """A window of this buffer (offset a multiple of 128 elements); no copy."""
        h = C.c_void_p()
        self.dev._check(self.dev.L.anl_buffer_view(self.h, int(offset), int(elems), C.byref(h)))
        return ResidentBuffer(self.dev, self.dtype, elems, h)

    def upload(self, data):
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        self.dev._check(self.dev.L.anl_buffer_upload(self.h, a.ctypes.data, a.size))
        return self

    def upload_begin(self, data: np.ndarray):
        """Start copying `data` (contiguous, ideally pinned) on the copy stream; the buffer keeps
        its contents until `upload_commit`.  The array is held until then.  float32 data is
        converted to the storage dtype at the commit; a float16 array is accepted for an f16 buffer
        and moves as it is (half the bytes, no conversion pass)."""
        if not data.flags["C_CONTIGUOUS"]:
            raise ValueError("upload_begin: a contiguous array is required (no hidden copy may outlive the call)")
        if data.dtype == np.float16 and self.dtype.code == 10:      # ANL_F16
            self._staged = data
            self.dev._check(self.dev.L.anl_buffer_upload_begin_stored(self.h, data.ctypes.data, data.size))
            return self
        if data.dtype != np.float32:
            raise ValueError("upload_begin: float32 data, or float16 data for an f16 buffer, is required")
        self._staged = data
        self.dev._check(self.dev.L.anl_buffer_upload_begin(self.h, data.ctypes.data, data.size))
        return self

    def upload_commit(self):
        self.dev._check(self.dev.L.anl_buffer_upload_commit(self.h))
        return self

    def download(self) -> np.ndarray:
        a = np.empty(self.elems, dtype=np.float32)
        self.dev._check(self.dev.L.anl_buffer_download(self.h, a.ctypes.data, a.size))
        return a

    def download_begin(self, host: np.ndarray):
        """Queue a read-back of the first ``host.size`` values into ``host`` (float32, contiguous,
        pinned) behind the work already queued; returns at once. ``download_wait`` completes it."""
        if host.dtype != np.float32 or not host.flags["C_CONTIGUOUS"]:
            raise ValueError("download_begin: a contiguous float32 array is required")
        self._dl = host
        self.dev._check(self.dev.L.anl_buffer_download_begin(self.h, host.ctypes.data, host.size))
        return self

    def download_wait(self):
        self.dev._check(self.dev.L.anl_buffer_download_wait(self.h))
        return self._dl

    @property
    def device_ptr(self) -> int:
        return self.dev.L.anl_buffer_device_ptr(self.h)

    def release(self):
        if self.h:
            self.dev.L.anl_buffer_release(self.h)
            self.h = None


class Device:
    """``cuda.Open()``: the B200 executor."""

    DEBUG_BOUNDS = 1
    NO_GEMM = 2
    BEAM = 4
    NO_ROW_CHAIN = 8
    TAIL_SPLIT = 16
    NO_EPILOGUE_FUSION = 32
    NO_TF32X3 = 64

    def __init__(self, ordinal: Optional[int] = None, flags: int = 0):
        self.L = load_library()
        if ordinal is None:
            ordinal = int(os.environ.get("ANNEAL_CUDA_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        if os.environ.get("ANNEAL_CUDA_DEBUG_BOUNDS") == "1":
            flags |= self.DEBUG_BOUNDS
        if os.environ.get("ANNEAL_BEAM") == "1":      # the reference's switch (codegen/beam.go:471)
            flags |= self.BEAM
        h = C.c_void_p()
        rc = self.L.anl_open(ordinal, flags, C.byref(h))
        if rc:
            raise DeviceError(f"cuda: open device {ordinal}: no usable sm_100 GPU (status {rc})")
        self.h = h
        self._blobs: Dict[int, bytes] = {}
        self._graphs: Dict[int, C.c_void_p] = {}

    # ── plumbing ──────────────────────────────────────────────────────────
    def _check(self, rc: int):
        if rc:
            raise DeviceError(self.L.anl_last_error(self.h).decode())

    def _blob(self, items) -> bytes:
        # a JIT replays the same frozen list object; serialise it once
        key = id(items)
        ent = self._blobs.get(key)
        if ent is None or ent[0] is not items:
            ent = (items, kir.serialize(items))
            self._blobs[key] = ent
        return ent[1]

    @staticmethod
    def _inputs(inputs):
        keep = []
        arr = (_Input * max(len(inputs), 1))()
        for k, (idx, v) in enumerate(inputs.items()):
            if isinstance(v, ResidentBuffer):
                arr[k] = _Input(idx, None, v.elems, v.h)
            else:
                a = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
                keep.append(a)
                arr[k] = _Input(idx, a.ctypes.data, a.size, None)
        return arr, len(inputs), keep

    @staticmethod
    def _binds(binding):
        binding = binding or {}
        arr = (_Binding * max(len(binding), 1))()
        for k, (n, v) in enumerate(binding.items()):
            arr[k] = _Binding(n.encode(), int(v))
        return arr, len(binding)

    @staticmethod
    def _placed(placed, allreduce=()):
        placed = placed or {}
        keep = []
        arr = (_Output * max(len(placed), 1))()
        for k, (idx, v) in enumerate(placed.items()):
            if isinstance(v, GradientTarget):
                arr[k] = _Output(idx, None, v.grad.elems, v.grad.h, int(v.allreduce),
                                 v.master.h if v.master is not None else None, v.param.h if v.param is not None else None,
                                 v.lr, v.scale)
            elif isinstance(v, ResidentBuffer):
                arr[k] = _Output(idx, None, v.elems, v.h, 1 if idx in allreduce else 0, None, None, 0.0, 0.0)
            else:
                assert v.dtype == np.float32 and v.flags["C_CONTIGUOUS"]
                keep.append(v)
                arr[k] = _Output(idx, v.ctypes.data_as(C.POINTER(C.c_float)), v.size, None, 0, None, None, 0.0, 0.0)
        return arr, len(placed), keep

    def _collect(self, outs, n, placed):
        res = {}
        placed = placed or {}
        for k in range(n):
            o = outs[k]
            if o.uop_idx in placed:
                res[o.uop_idx] = placed[o.uop_idx]
            else:
                res[o.uop_idx] = np.ctypeslib.as_array(o.data, shape=(max(o.elems, 0),)).copy() if o.elems else np.empty(0, np.float32)
        self.L.anl_outputs_free(outs, n)
        return res

    # ── Executor / SymbolicExecutor ───────────────────────────────────────
    def run(self, items, inputs, binding=None, placed=None, allreduce=()):
        """``allreduce``: ids of placed resident outputs to sum across ranks as soon as they are
        produced, overlapped with the rest of the schedule."""
        if not items:
            return {}
        blob = self._blob(items)
        ia, ni, keep_i = self._inputs(inputs)
        ba, nb = self._binds(binding)
        pa, npl, keep_p = self._placed(placed, allreduce)
        cap = len(items)
        outs = (_Output * cap)()
        n = C.c_int(cap)
        self._check(self.L.anl_run(self.h, blob, len(blob), ia, ni, ba, nb, pa, npl, outs, C.byref(n)))
        return self._collect(outs, n.value, placed)

    def run_symbolic(self, items, inputs, binding):
        return self.run(items, inputs, binding)

    def replay(self, items, inputs, binding=None, placed=None, allreduce=()):
        """Run through a CUDA graph captured on first use of this item list."""
        if not items:
            return {}
        key = id(items)
        g = self._graphs.get(key)
        if g is None or g[0] is not items:
            blob = self._blob(items)
            h = C.c_void_p()
            self._check(self.L.anl_graph_create(self.h, blob, len(blob), C.byref(h)))
            g = (items, h)
            self._graphs[key] = g
        ia, ni, keep_i = self._inputs(inputs)
        ba, nb = self._binds(binding)
        pa, npl, keep_p = self._placed(placed, allreduce)
        cap = len(items)
        outs = (_Output * cap)()
        n = C.c_int(cap)
        self._check(self.L.anl_graph_replay(g[1], ia, ni, ba, nb, pa, npl, outs, C.byref(n)))
        return self._collect(outs, n.value, placed)

    # ── Benchmarker ───────────────────────────────────────────────────────
    def benchmark(self, item, warmup: int = 2, iterations: int = 5, opts: Optional[Sequence[int]] = None):
        blob = kir.serialize([item])
        r = _Bench()
        o = _opts(opts)
        self._check(self.L.anl_benchmark(self.h, blob, len(blob), 0, o, warmup, iterations, C.byref(r)))
        return {n: getattr(r, n) for n, _ in _Bench._fields_}

    def beam_search(self, item, width: int = 4, depth: int = 4, cache_path: Optional[str] = None):
        """codegen.BeamSearch for one kernel; returns the winning transform and its timing."""
        blob = kir.serialize([item])
        r = _Beam()
        self._check(self.L.anl_beam_search(self.h, blob, len(blob), 0, width, depth,
                                           cache_path.encode() if cache_path else None, C.byref(r)))
        return {"opts": list(r.opts), "base_us": r.base_us, "best_us": r.best_us, "tried": r.tried,
                "rejected": r.rejected, "from_cache": bool(r.from_cache)}

    # ── residency / optimiser / data parallel ────────────────────────────
    def buffer(self, dtype, elems) -> ResidentBuffer:
        return ResidentBuffer(self, dtype, elems)

    def sgd_step(self, master: ResidentBuffer, param: ResidentBuffer, grad: ResidentBuffer, lr: float, grad_scale: float = 1.0):
        self._check(self.L.anl_sgd_step(self.h, master.h, param.h, grad.h, lr, grad_scale))

    def comm_unique_id(self) -> bytes:
        b = C.create_string_buffer(128)
        if self.L.anl_comm_unique_id(b):
            raise DeviceError("nccl: cannot create a unique id")
        return b.raw

    def comm_init(self, rank: int, nranks: int, uid: bytes):
        self._check(self.L.anl_comm_init(self.h, rank, nranks, uid))

    def allreduce_sum(self, buf: ResidentBuffer):
        self._check(self.L.anl_allreduce_sum(self.h, buf.h))

    def allgather(self, buf: ResidentBuffer):
        """In place: every rank's 1/nranks shard of ``buf`` gathered into all ranks' copies."""
        self._check(self.L.anl_allgather(self.h, buf.h))

    def comm_set_timeout(self, milliseconds: int):
        """Longest a collective may stay unfinished before the watchdog aborts the communicator."""
        self._check(self.L.anl_comm_set_timeout(self.h, int(milliseconds)))

    def comm_wait(self):
        self._check(self.L.anl_comm_wait(self.h))

    def comm_abort(self):
        self._check(self.L.anl_comm_abort(self.h))

    def comm_inject_delay(self, milliseconds: int):
        """Test aid: a host callback holds the communication stream back (no GPU work involved)."""
        self._check(self.L.anl_comm_inject_delay(self.h, int(milliseconds)))

    def timer_start(self):
        self._check(self.L.anl_timer_start(self.h))

    def timer_stop(self) -> float:
        """Milliseconds between timer_start and now on the compute stream (CUDA events)."""
        ms = C.c_float()
        self._check(self.L.anl_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def profile(self, on: bool):
        self._check(self.L.anl_profile_enable(self.h, 1 if on else 0))

    def profile_read(self):
        arr = (_Prof * 8)()
        n = C.c_int()
        self._check(self.L.anl_profile_read(self.h, arr, 8, C.byref(n)))
        return {KERNEL_CLASSES.get(arr[k].klass, str(arr[k].klass)): {"launches": arr[k].launches, "total_ms": arr[k].total_ms,
                                                                       "flops": arr[k].flops} for k in range(n.value)}

    def gemm_defaults(self, **kw):
        """Device-wide tunables of the contraction kernel (see ``gemm_opts``); no arguments: heuristics."""
        self._check(self.L.anl_gemm_set_defaults(self.h, _opts(gemm_opts(**kw)) if kw else None))

    @property
    def stream(self) -> int:
        """The cudaStream_t handle the device queues on (for callers that launch work of their own)."""
        return self.L.anl_stream(self.h)

    def synchronize(self):
        self._check(self.L.anl_synchronize(self.h))

    def info(self):
        i = _Info()
        self._check(self.L.anl_device_info(self.h, C.byref(i)))
        return {"name": i.name.decode(), "sm": f"{i.sm_major}.{i.sm_minor}", "sm_count": i.sm_count,
                "total_mem": i.total_mem, "tcgen05": bool(i.has_tcgen05)}

    def stats(self):
        s = _Stats()
        self._check(self.L.anl_get_stats(self.h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in _Stats._fields_}

    def close(self):
        if getattr(self, "h", None):
            for _, g in self._graphs.values():
                self.L.anl_graph_release(g)
            self._graphs.clear()
            self.L.anl_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def pinned_array(n: int, dtype=np.float32) -> np.ndarray:
    """float32 (or float16) array in page-locked host memory (lives until process exit)."""
    L = load_library()
    p = C.c_void_p()
    dt = np.dtype(dtype)
    if dt not in (np.dtype(np.float32), np.dtype(np.float16)):
        raise ValueError("pinned_array: float32 or float16")
    if L.anl_host_alloc(n * dt.itemsize, C.byref(p)):
        raise DeviceError("cuda: pinned host allocation failed")
    raw = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n * dt.itemsize,))
    return raw.view(dt)
