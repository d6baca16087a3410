"""Kernel-IR wire format: how a schedule crosses the C boundary.

One blob carries a list of ``ExecItem`` (schedule/exec.go:6-32): per item the
kernel AST as a flat node table in sources-before-users order (the last node is
the SINK), the buffer table, the symbolic-variable names and an optional
pre-rendered source with its launch shape. A node mirrors the reference's
``uopNode`` (uop/uop.go:39-45) with the ``arg`` union flattened:

    file   := "KIR1" u32 n_items item*
    item   := u32 n_nodes, u32 n_srcs, u32 n_bufs, u32 n_sym, u32 source_len,
              u32 local[3], u32 grid[3],
              node[n_nodes], u32 srcs[n_srcs], buf[n_bufs], sym[n_sym], source bytes
    node   := u16 op, u8 dtype, u8 flags, u32 nsrc, u32 src_off, u32 aux, i64 arg     (24 bytes)
    buf    := u32 uop_idx, i32 slot, u8 dtype, u8 rank, u16 0, i64 size, i64 shape[rank]
    sym    := u16 len, bytes

    CONST  : arg = f64 bits (float dtypes) | i64 | 0/1
    RANGE  : arg = size, aux = range id, flags = axis | symbolic<<3 | sym_param<<4
    PARAM  : arg = parameter number
    REDUCE : aux = opcode of the combining op
    SINK   : arg = number of parameters

All integers little-endian. Opcodes are ``uop.Op`` values, dtypes ``DType.code``.
"""
from __future__ import annotations

import struct
from typing import List

from . import uop as U
from .uop import Op
from .schedule import ExecItem

MAGIC = b"KIR1"


def _node_fields(n: U.UOp):
    flags, aux, arg = 0, 0, 0
    if n.op == Op.CONST:
        if n.dtype.is_float:
            arg = struct.unpack("<q", struct.pack("<d", float(n.arg)))[0]
        else:
            arg = int(n.arg)
    elif n.op == Op.RANGE:
        ra = n.arg
        arg, aux = ra.size, ra.id
        flags = (ra.axis & 7) | ((1 if ra.symbolic else 0) << 3) | ((ra.sym_param & 15) << 4)
    elif n.op == Op.PARAM:
        arg = int(n.arg)
    elif n.op == Op.REDUCE:
        aux = int(n.arg)
    elif n.op == Op.SINK:
        arg = int(n.arg)
    return flags, aux, arg


def serialize_item(it: ExecItem) -> bytes:
    nodes = U.toposort(it.ast) if it.ast is not None else []
    pos = {n.idx: i for i, n in enumerate(nodes)}
    srcs: List[int] = []
    recs = []
    for n in nodes:
        flags, aux, arg = _node_fields(n)
        recs.append(struct.pack("<HBBIIIq", n.op, n.dtype.code, flags, len(n.src), len(srcs), aux, arg))
        srcs.extend(pos[s.idx] for s in n.src)
    src_b = it.source.encode() if it.source else b""
    out = [struct.pack("<5I3I3I", len(nodes), len(srcs), len(it.bufs), len(it.sym_vars), len(src_b),
                       *it.local_size, *it.grid)]
    out.extend(recs)
    out.append(struct.pack(f"<{len(srcs)}I", *srcs))
    for b in it.bufs:
        out.append(struct.pack("<IiBBHq", b.uop_idx, b.slot, b.dtype.code, len(b.shape), 0, b.size))
        out.append(struct.pack(f"<{len(b.shape)}q", *b.shape))
    for s in it.sym_vars:
        sb = s.encode()
        out.append(struct.pack("<H", len(sb)) + sb)
    out.append(src_b)
    return b"".join(out)


def serialize(items: List[ExecItem]) -> bytes:
    return MAGIC + struct.pack("<I", len(items)) + b"".join(serialize_item(i) for i in items)


def dump(it: ExecItem) -> str:
    """Readable listing of one kernel, for debugging and docs."""
    nodes = U.toposort(it.ast)
    pos = {n.idx: i for i, n in enumerate(nodes)}
    lines = []
    for i, n in enumerate(nodes):
        a = "" if n.arg is None else f" {n.arg}"
        lines.append(f"%{i} = {U.OP_NAMES.get(n.op, n.op)}:{n.dtype}{a} ({', '.join('%' + str(pos[s.idx]) for s in n.src)})")
    for j, b in enumerate(it.bufs):
        lines.append(f"buf{j}: id={b.uop_idx} {b.dtype} shape={b.shape} slot={b.slot}")
    return "\n".join(lines)
