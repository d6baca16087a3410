"""UOp IR used by the host-side stand-in for anneal's frontend.

The numeric opcode values are the ones anneal's ``uop.Op`` enum assigns
(uop/ops.go:12-157, an ``iota`` list) so that a kernel serialised here has the
same opcodes a Go ``backend/cuda`` binding would emit from ``item.Ast``.
Only the ops that survive scheduling, plus the tensor-graph ops the scheduler
consumes, are named.

Nodes are immutable and interned on ``(op, dtype, src, arg, tag)``; the ops
that carry identity (buffers, ranges, uniques) are never interned, as in
uop/uop.go:90-100.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from typing import Any, Optional, Tuple


class Op:
    DEFINE_VAR = 0
    PARAM = 7
    SINK = 13
    INDEX = 18
    STORE = 20
    CAST = 22
    BITCAST = 23
    EXP2 = 24
    LOG2 = 25
    SIN = 26
    SQRT = 27
    RECIPROCAL = 28
    NEG = 29
    TRUNC = 30
    ADD = 31
    MUL = 32
    SHL = 33
    SHR = 34
    IDIV = 35
    MAX = 36
    MOD = 37
    CMPLT = 38
    CMPNE = 39
    CMPEQ = 40
    XOR = 41
    OR = 42
    AND = 43
    SUB = 45
    FDIV = 46
    POW = 47
    WHERE = 48
    MULACC = 49
    RANGE = 51
    END = 53
    CONST = 56
    # tensor-graph-only ops (never serialised)
    CONTIGUOUS = 64
    BUFFERIZE = 67
    BUFFER = 69
    RESHAPE = 74
    PERMUTE = 75
    EXPAND = 76
    PAD = 77
    SHRINK = 78
    FLIP = 79
    REDUCE_AXIS = 81
    REDUCE = 82


OP_NAMES = {v: k for k, v in vars(Op).items() if not k.startswith("_")}

UNARY = {Op.EXP2, Op.LOG2, Op.SIN, Op.SQRT, Op.RECIPROCAL, Op.NEG, Op.TRUNC}
BINARY = {Op.ADD, Op.MUL, Op.SHL, Op.SHR, Op.IDIV, Op.MAX, Op.MOD, Op.CMPLT, Op.CMPNE,
          Op.CMPEQ, Op.XOR, Op.OR, Op.AND, Op.SUB, Op.FDIV, Op.POW}
MOVEMENT = {Op.RESHAPE, Op.PERMUTE, Op.EXPAND, Op.PAD, Op.SHRINK, Op.FLIP}

# ops that always allocate a fresh node (uop/uop.go:90-100)
_NO_INTERN = {Op.BUFFER, Op.RANGE}


@dataclass(frozen=True)
class DType:
    """Scalar dtype; ``code`` is the wire id used by the kernel-IR format."""
    name: str
    code: int
    bits: int
    kind: str  # 'f', 'i', 'u', 'b', 'v'
    priority: int

    def __repr__(self):
        return self.name

    @property
    def is_float(self):
        return self.kind == "f"

    @property
    def is_int(self):
        return self.kind in ("i", "u")

    @property
    def is_unsigned(self):
        return self.kind == "u"

    @property
    def is_bool(self):
        return self.kind == "b"


class dtypes:
    void = DType("void", 0, 0, "v", -1)
    bool = DType("bool", 1, 1, "b", 0)
    int8 = DType("int8", 2, 8, "i", 1)
    uint8 = DType("uint8", 3, 8, "u", 2)
    int16 = DType("int16", 4, 16, "i", 3)
    uint16 = DType("uint16", 5, 16, "u", 4)
    int32 = DType("int32", 6, 32, "i", 5)
    uint32 = DType("uint32", 7, 32, "u", 6)
    int64 = DType("int64", 8, 64, "i", 7)
    uint64 = DType("uint64", 9, 64, "u", 8)
    float16 = DType("float16", 10, 16, "f", 11)
    bfloat16 = DType("bfloat16", 11, 16, "f", 12)
    float32 = DType("float32", 12, 32, "f", 13)
    float64 = DType("float64", 13, 64, "f", 14)
    index = DType("index", 14, 32, "i", 5)


DTYPE_BY_CODE = {d.code: d for d in vars(dtypes).values() if isinstance(d, DType)}


def least_upper_dtype(a: DType, b: DType) -> DType:
    """Smallest dtype both promote to (uop/dtype.go:616-636). f16 with bf16
    meets at f32; ints promote to any float."""
    if a is b:
        return a
    if {a, b} == {dtypes.float16, dtypes.bfloat16}:
        return dtypes.float32
    if a.is_float or b.is_float:
        fa = [d for d in (a, b) if d.is_float]
        return max(fa, key=lambda d: d.priority)
    return a if a.priority >= b.priority else b


def quantize(v, dt: DType):
    """Round a float32 array to the values representable in ``dt``
    (uop/dtype.go:476-487): f16 by round-to-nearest-even, bf16 by truncating the
    low 16 bits."""
    import numpy as np
    v = np.asarray(v, dtype=np.float32)
    if dt is dtypes.float16:
        with np.errstate(over="ignore"):
            return v.astype(np.float16).astype(np.float32)
    if dt is dtypes.bfloat16:
        return (v.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    return v


@dataclass(frozen=True)
class Var:
    """A symbolic dimension (``DefineVar`` in the reference, uop/uop.go:346):
    an opaque integer in [vmin, vmax] bound at dispatch time."""
    name: str
    vmin: int
    vmax: int

    def __repr__(self):
        return f"Var({self.name})"


@dataclass(frozen=True)
class RangeArg:
    """Payload of a RANGE node (uop/uop.go:296-330)."""
    id: int
    size: int
    axis: int  # 0 loop, 1 reduce (uop/uop.go:288-295)
    symbolic: bool = False
    sym_param: int = 0
    var_name: str = ""


AXIS_LOOP, AXIS_REDUCE = 0, 1

_counter = itertools.count()
_intern: dict = {}


class UOp:
    __slots__ = ("op", "dtype", "src", "arg", "tag", "idx")

    def __init__(self, op, dtype, src, arg, tag, idx):
        self.op, self.dtype, self.src, self.arg, self.tag, self.idx = op, dtype, src, arg, tag, idx

    def __repr__(self):
        a = "" if self.arg is None else f" {self.arg!r}"
        return f"<{OP_NAMES.get(self.op, self.op)}#{self.idx}{a} {self.dtype}>"


def _hashable(x):
    if isinstance(x, list):
        return tuple(_hashable(i) for i in x)
    if isinstance(x, float):
        # distinguish 0.0 / -0.0 and make NaN hashable-equal
        return ("f", math.copysign(1.0, x), x if x == x else "nan")
    return x


def new(op: int, dtype: DType, src: Tuple["UOp", ...] = (), arg: Any = None, tag: Any = None) -> UOp:
    src = tuple(src)
    if op in _NO_INTERN:
        return UOp(op, dtype, src, arg, tag, next(_counter))
    key = (op, dtype, tuple(s.idx for s in src), _hashable(arg), _hashable(tag))
    u = _intern.get(key)
    if u is None:
        u = UOp(op, dtype, src, arg, tag, next(_counter))
        _intern[key] = u
    return u


def const(dtype: DType, v) -> UOp:
    if dtype.is_float:
        v = float(v)
    elif dtype.is_bool:
        v = bool(v)
    else:
        v = int(v)
    return new(Op.CONST, dtype, (), v)


def reset_intern() -> None:
    """Drop the intern table (the analogue of starting a fresh arena per training
    step, examples/mlp.go:111)."""
    _intern.clear()


def toposort(root: UOp, stop=None):
    """Sources-before-users order of everything reachable from root. ``stop(u)``
    true means: list u but do not descend into it."""
    seen, order = set(), []
    stack = [(root, 0)]
    while stack:
        u, i = stack.pop()
        if u.idx in seen:
            continue
        if stop is not None and i == 0 and stop(u):
            seen.add(u.idx)
            order.append(u)
            continue
        if i < len(u.src):
            stack.append((u, i + 1))
            c = u.src[i]
            if c.idx not in seen:
                stack.append((c, 0))
        else:
            seen.add(u.idx)
            order.append(u)
    return order
