"""``realize`` / ``realize_with_binding`` / ``JIT``: where the tensor graph meets
the device.

Mirrors tensor/realize.go:26-116 and tensor/jit.go:47-246. An executor is any
object with ``run(items, inputs) -> {buffer id: float32 array}``,
``run_symbolic(items, inputs, binding)`` and ``close()`` — the shape of the
reference's ``backend.Executor`` / ``SymbolicExecutor`` (backend/device.go:10-37);
``anneal_b200.device.Device`` is the CUDA one.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

from . import uop as U
from .uop import Op
from .tensor import Tensor, LEAF_DATA
from . import schedule as S

#: the registered device (tensor/realize.go:17 ``DefaultExecutor``)
DEFAULT_EXECUTOR = None
#: ask the scheduler to turn expression operands of contractions into buffers
MATERIALIZE_CONTRACTION_OPERANDS = False


class RealizeError(RuntimeError):
    pass


def leaf_inputs(tensors: Sequence[Tensor]) -> Dict[int, np.ndarray]:
    """Host data of every BUFFER leaf reachable from ``tensors``
    (tensor/realize.go:122-145)."""
    out = {}
    seen = set()
    stack = [t.node for t in tensors]
    while stack:
        u = stack.pop()
        if u.idx in seen:
            continue
        seen.add(u.idx)
        if u.op == Op.BUFFER:
            d = LEAF_DATA.get(u.idx)
            if d is not None:
                out[u.idx] = d
            continue
        stack.extend(u.src)
    return out


def reset() -> None:
    """Start a fresh compilation unit (a new arena per training step in the
    reference, examples/mlp.go:111)."""
    LEAF_DATA.clear()
    U.reset_intern()


#: buffers one fused kernel may bind when scheduling for the CUDA device.  The reference's 8
#: (schedule/schedule.go:217-229) is WebGPU's storage-buffer limit; a CUDA kernel takes hundreds of
#: pointers.  None keeps the reference's value.
FUSION_BUFFER_CAP = None


def build_schedule(tensors: Sequence[Tensor]):
    """MATERIALIZE_CONTRACTION_OPERANDS: False — the reference's schedule; True — every contraction
    operand that is an expression becomes a buffer; "auto" — decided per operand by what it costs
    (schedule.materialize_contraction_operands)."""
    nodes = [t.node for t in tensors]
    mode = MATERIALIZE_CONTRACTION_OPERANDS
    if mode:
        nodes = S.materialize_contraction_operands(nodes, by_cost=(mode == "auto"))
    items, out_map = S.create_schedule(nodes, max_bufs=FUSION_BUFFER_CAP, keep_contractions=bool(mode), outputs_first=bool(mode))
    return items, [out_map[n.idx] for n in nodes]


#: Device-side companion of schedule.STATS_HOOK (the reference feeds its dashboard's compiler panel from
#: that hook, tui/dashboard.go:68-80): if set, called after every realize / replay with what the device
#: did for it — kernels launched, how many of them contractions on the tensor-core kernels, elementwise
#: kernels and bias gradients that ran inside a contraction's epilogue, graph replays, compiles, bytes
#: moved each way.  Same threading rule as the schedule hook.
DEVICE_STATS_HOOK = None
_DEVICE_COUNTERS = ("kernels_launched", "gemm_launched", "epilogues_fused", "colsums_fused", "side_launches", "graph_replays", "graph_captures",
                    "nvrtc_compiles", "h2d_bytes", "d2h_bytes")


def _with_device_stats(executor, call):
    if DEVICE_STATS_HOOK is None or not hasattr(executor, "stats"):
        return call()
    before = executor.stats()
    out = call()
    after = executor.stats()
    DEVICE_STATS_HOOK({k: after[k] - before[k] for k in _DEVICE_COUNTERS if k in after})
    return out


def _assign(tensors, out_ids, outputs):
    for t, oid in zip(tensors, out_ids):
        if oid not in outputs:
            raise RealizeError(f"tensor: realize: executor returned no data for buffer {oid}")
        t.data = outputs[oid]


def realize(*tensors: Tensor) -> None:
    if not tensors:
        return
    if DEFAULT_EXECUTOR is None:
        raise RealizeError("tensor: realize: no backend registered")
    items, out_ids = build_schedule(tensors)
    try:
        outputs = _with_device_stats(DEFAULT_EXECUTOR, lambda: DEFAULT_EXECUTOR.run(items, leaf_inputs(tensors)))
    except Exception as e:  # wrap with the caller's prefix (tensor/realize.go:70)
        raise RealizeError(f"tensor: realize: {e}") from e
    _assign(tensors, out_ids, outputs)


def realize_with_binding(binding: Dict[str, int], *tensors: Tensor) -> None:
    if not tensors:
        return
    if DEFAULT_EXECUTOR is None or not hasattr(DEFAULT_EXECUTOR, "run_symbolic"):
        raise RealizeError("tensor: realize: backend does not support symbolic shapes")
    items, out_ids = build_schedule(tensors)
    try:
        outputs = _with_device_stats(DEFAULT_EXECUTOR, lambda: DEFAULT_EXECUTOR.run_symbolic(items, leaf_inputs(tensors), dict(binding)))
    except Exception as e:
        raise RealizeError(f"tensor: realize: {e}") from e
    _assign(tensors, out_ids, outputs)


def _dfs_leaves(tensors: Sequence[Tensor]) -> List[U.UOp]:
    """BUFFER leaves in pre-order depth-first encounter order: the positional
    key a JIT replay uses to map new leaves onto captured ones (tensor/jit.go:303-327)."""
    seen, out = set(), []
    stack = [t.node for t in reversed(tensors)]
    while stack:
        u = stack.pop()
        if u.idx in seen:
            continue
        seen.add(u.idx)
        if u.op == Op.BUFFER:
            out.append(u)
            continue
        stack.extend(reversed(u.src))
    return out


def _structure_key(tensors: Sequence[Tensor]) -> int:
    """Position-independent hash of the expression: two graphs built by the same
    code over different leaves hash alike (uop/uop.go:231-253 StructuralKeys)."""
    memo: Dict[int, int] = {}
    leaf_no: Dict[int, int] = {}
    for t in tensors:
        for u in U.toposort(t.node):
            if u.op == Op.BUFFER:
                leaf_no.setdefault(u.idx, len(leaf_no))
                memo[u.idx] = hash(("leaf", leaf_no[u.idx], u.dtype.code, tuple(str(s) for s in u.arg)))
            else:
                memo[u.idx] = hash((u.op, u.dtype.code, tuple(memo[s.idx] for s in u.src), U._hashable(u.arg)))
    return hash(tuple(memo[t.node.idx] for t in tensors))


class JIT:
    """Capture the schedule of a realize call once, replay it for structurally
    identical graphs without scheduling (tensor/jit.go:47-246). The frozen item
    list is handed to the executor unchanged, so a device that keys compiled
    kernels and CUDA graphs on the item list replays them."""

    def __init__(self):
        self.items = None
        self.symbolic = False
        self.cap_leaves: List[int] = []
        self.leaf_sizes: List[int] = []
        self.out_ids: List[int] = []
        self.key = None
        self.captures = 0
        self.replays = 0

    def stats(self):
        return self.captures, self.replays

    def _capture(self, tensors, leaves, binding):
        items, out_ids = build_schedule(tensors)
        ex = DEFAULT_EXECUTOR
        if ex is None:
            raise RealizeError("tensor: realize: no backend registered")
        inputs = leaf_inputs(tensors)
        outputs = ex.run(items, inputs) if binding is None else ex.run_symbolic(items, inputs, dict(binding))
        _assign(tensors, out_ids, outputs)
        self.items, self.out_ids = items, out_ids
        self.symbolic = binding is not None
        self.cap_leaves = [u.idx for u in leaves]
        self.leaf_sizes = [int(np.prod([s for s in u.arg if isinstance(s, int)])) for u in leaves]
        self.key = _structure_key(tensors)
        self.captures += 1

    def _matches(self, tensors, leaves, symbolic):
        if self.items is None or self.symbolic != symbolic or len(leaves) != len(self.cap_leaves):
            return False
        if not symbolic:
            sizes = [int(np.prod([s for s in u.arg if isinstance(s, int)])) for u in leaves]
            if sizes != self.leaf_sizes:
                return False
        return _structure_key(tensors) == self.key

    def _replay(self, tensors, leaves, binding):
        inputs = {}
        for cap, u in zip(self.cap_leaves, leaves):
            d = LEAF_DATA.get(u.idx)
            if d is not None:
                inputs[cap] = d
        ex = DEFAULT_EXECUTOR
        outputs = _with_device_stats(ex, lambda: ex.run(self.items, inputs) if binding is None else ex.run_symbolic(self.items, inputs, dict(binding)))
        _assign(tensors, self.out_ids, outputs)
        self.replays += 1

    def realize(self, *tensors: Tensor) -> None:
        if not tensors:
            return
        leaves = _dfs_leaves(tensors)
        if self._matches(tensors, leaves, False):
            self._replay(tensors, leaves, None)
        else:
            self._capture(tensors, leaves, None)

    def realize_with_binding(self, binding: Dict[str, int], *tensors: Tensor) -> None:
        if not tensors:
            return
        leaves = _dfs_leaves(tensors)
        if self._matches(tensors, leaves, True):
            self._replay(tensors, leaves, binding)
        else:
            self._capture(tensors, leaves, binding)
