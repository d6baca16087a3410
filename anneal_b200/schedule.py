"""Tensor graph → ordered list of kernels (``ExecItem``).

Restates the rules of anneal's rangeify scheduler so that the kernels handed to
the device have the reference's shape:

* realize points are the sink sources, CONTIGUOUS and every REDUCE_AXIS
  (schedule/rangeify.go:195-218); everything else is inlined into each consumer;
* movement ops dissolve into index arithmetic with no simplification
  (schedule/index.go:30-225), PAD becoming ``WHERE(valid, inner, fill)`` whose
  fill is the enclosing reduce's identity;
* a REDUCE_AXIS kernel with exactly one consumer that is a reduce-free kernel is
  spliced into that consumer (schedule/schedule.go:122-287) subject to a buffer
  budget;
* kernels are ordered by their buffer dependencies and intermediates share
  slots by greedy interval colouring (schedule/kernels.go:173-463).

One rule is added for the CUDA device and is off unless asked for
(``materialize_contraction_operands``): operands of a SUM-of-products that are
not plain views of a buffer are first materialised through CONTIGUOUS, so the
contraction reaches the device as a dense GEMM over buffers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from . import uop as U
from .uop import Op, dtypes, RangeArg, AXIS_LOOP, AXIS_REDUCE
from .gradient import node_shape

#: epilogue fusion on/off (schedule/schedule.go:120 ``FusionEnabled``)
FUSION_ENABLED = True
#: buffers a fused kernel may bind, output included (schedule/schedule.go:217-229)
MAX_KERNEL_BUFFERS = 8


@dataclass
class CompilerStats:
    """schedule/stats.go:3-12: what one scheduling run produced."""
    uops: int            # nodes of the tensor-level graph that was scheduled
    kernels: int         # kernels in the schedule
    fused: int           # reduce kernels spliced into their consumer (schedule/schedule.go:122-287)
    pass_name: str = "memory_plan"


#: schedule/stats.go:14-18: if set, called by create_schedule after each successful run, synchronously
#: in the caller's thread; set before training, clear (None) when done; not safe for concurrent change
STATS_HOOK = None


@dataclass
class Buffer:
    """schedule/exec.go:6-13."""
    uop_idx: int
    size: int          # elements; 0 when a dimension is symbolic
    shape: Tuple[int, ...]  # 0 marks the symbolic dimension
    dtype: U.DType
    slot: int = -1


@dataclass
class ExecItem:
    """schedule/exec.go:14-32. ``source``/``local_size``/``grid`` play the role of
    the reference's pre-rendered ``WGSL``/``LocalSize``/``WorkgroupCount``."""
    ast: Optional[U.UOp]
    bufs: List[Buffer]
    sym_vars: List[str] = field(default_factory=list)
    source: str = ""
    local_size: Tuple[int, int, int] = (1, 1, 1)
    grid: Tuple[int, int, int] = (1, 1, 1)


class _Ctx:
    def __init__(self):
        self.next_id = 0
        self.sym_params = 0
        self.reduce_ranges: List[U.UOp] = []

    def start_kernel(self):
        self.sym_params = 0
        self.reduce_ranges = []

    def new_range(self, size, axis) -> U.UOp:
        rid = self.next_id
        self.next_id += 1
        if isinstance(size, U.Var):
            p = self.sym_params
            self.sym_params += 1
            r = U.new(Op.RANGE, dtypes.index, (), RangeArg(rid, 0, axis, True, p, size.name))
        elif size == 1:
            return U.const(dtypes.index, 0)
        else:
            r = U.new(Op.RANGE, dtypes.index, (), RangeArg(rid, int(size), axis))
        if axis == AXIS_REDUCE:
            self.reduce_ranges.append(r)
        return r


def _ic(v: int) -> U.UOp:
    return U.const(dtypes.index, v)


def _strides(shape):
    """Row-major strides; a symbolic (outermost) dim does not contribute
    (schedule/index.go:296-312)."""
    st, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        st[i] = acc
        if isinstance(shape[i], int):
            acc *= shape[i]
    return st


def _flat_index(indices, shape) -> U.UOp:
    if not indices:
        return _ic(0)
    if len(indices) == 1:
        return indices[0]
    res = None
    for r, s in zip(indices, _strides(shape)):
        term = r if s == 1 else U.new(Op.MUL, dtypes.index, (r, _ic(s)))
        res = term if res is None else U.new(Op.ADD, dtypes.index, (res, term))
    return res


def _unflat_index(flat, shape):
    """flat → per-dim indices: ``(flat / stride) % size`` for every static dim,
    modulo included on the last one; a symbolic dim keeps the bare quotient
    (schedule/index.go:259-293, 340-373)."""
    if not shape:
        return []
    if len(shape) == 1:
        return [flat]
    out = []
    for sz, st in zip(shape, _strides(shape)):
        d = flat if st == 1 else U.new(Op.IDIV, dtypes.index, (flat, _ic(st)))
        out.append(d if isinstance(sz, U.Var) else U.new(Op.MOD, dtypes.index, (d, _ic(sz))))
    return out


def identity_const(rop: int, dt: U.DType) -> U.UOp:
    """Identity of a reduce op as a CONST; 0 when there is no reduce context
    (schedule/index.go:375-431). MAX over floats is -inf here and is clamped to
    -FLT_MAX where the constant is rendered."""
    if rop == Op.MUL:
        v = 1.0 if dt.is_float else (True if dt.is_bool else 1)
    elif rop == Op.MAX:
        if dt.is_float:
            v = -math.inf
        elif dt.is_bool:
            v = False
        elif dt.is_unsigned:
            v = 0
        else:
            v = -(1 << (min(dt.bits, 64) - 1))
    else:
        v = 0.0 if dt.is_float else (False if dt.is_bool else 0)
    return U.const(dt, v)


class _Indexer:
    """Threads output indices through one kernel's subgraph."""

    def __init__(self, ctx: _Ctx, shapes, realized: Dict[int, U.UOp], root: U.UOp):
        self.ctx, self.shapes, self.realized, self.root = ctx, shapes, realized, root
        self.memo = {}

    def run(self, u: U.UOp, idx: Sequence[U.UOp], fill: int) -> U.UOp:
        key = (u.idx, tuple(i.idx for i in idx), fill)
        r = self.memo.get(key)
        if r is None:
            r = self._run(u, list(idx), fill)
            self.memo[key] = r
        return r

    def _run(self, u, idx, fill):
        op = u.op
        if u is not self.root and u.idx in self.realized:
            return U.new(Op.INDEX, u.dtype, (self.realized[u.idx], *idx))
        if op == Op.BUFFER:
            return U.new(Op.INDEX, u.dtype, (u, *idx))
        if op in (Op.CONST, Op.RANGE):
            return u
        if op == Op.RESHAPE:
            src_sh = self.shapes[u.src[0].idx]
            flat = _flat_index(idx, tuple(u.arg))
            return self.run(u.src[0], _unflat_index(flat, src_sh), fill)
        if op == Op.PERMUTE:
            si = [None] * len(u.arg)
            for i, p in enumerate(u.arg):
                si[p] = idx[i]
            return self.run(u.src[0], si, fill)
        if op == Op.EXPAND:
            src_sh = self.shapes[u.src[0].idx]
            si = [_ic(0) if (isinstance(s, int) and s == 1) else idx[i] for i, s in enumerate(src_sh)]
            return self.run(u.src[0], si, fill)
        if op == Op.SHRINK:
            si = [i if lo == 0 else U.new(Op.ADD, dtypes.index, (i, _ic(lo)))
                  for i, (lo, _) in zip(idx, u.arg)]
            return self.run(u.src[0], si, fill)
        if op == Op.PAD:
            src_sh = self.shapes[u.src[0].idx]
            si, conds = [], []
            for r, (lo, hi), sz in zip(idx, u.arg, src_sh):
                if lo != 0:
                    si.append(U.new(Op.SUB, dtypes.index, (r, _ic(lo))))
                    conds.append(U.new(Op.CMPLT, dtypes.bool, (_ic(lo - 1), r)))
                else:
                    si.append(r)
                if hi != 0:
                    conds.append(U.new(Op.CMPLT, dtypes.bool, (r, _ic(lo + sz))))
            inner = self.run(u.src[0], si, fill)
            if not conds:
                return inner
            valid = conds[0]
            for c in conds[1:]:
                valid = U.new(Op.AND, dtypes.bool, (valid, c))
            return U.new(Op.WHERE, u.dtype, (valid, inner, identity_const(fill, u.dtype)))
        if op == Op.FLIP:
            src_sh = self.shapes[u.src[0].idx]
            si = [U.new(Op.SUB, dtypes.index, (_ic(s - 1), i)) if f else i
                  for i, f, s in zip(idx, u.arg, src_sh)]
            return self.run(u.src[0], si, fill)
        if op == Op.CONTIGUOUS:
            return self.run(u.src[0], idx, fill)
        if op == Op.REDUCE_AXIS:
            rop, axes = u.arg
            src_sh = self.shapes[u.src[0].idx]
            rr = {ax: self.ctx.new_range(src_sh[ax], AXIS_REDUCE) for ax in axes}
            full, o = [], 0
            for i in range(len(src_sh)):
                if i in rr:
                    full.append(rr[i])
                else:
                    full.append(idx[o])
                    o += 1
            body = self.run(u.src[0], full, rop)
            return U.new(Op.REDUCE, u.dtype, (body, *[rr[a] for a in axes]), rop)
        # elementwise: the reduce context ends here (schedule/index.go:207-224)
        srcs = [s if s.op in (Op.CONST, Op.RANGE) else self.run(s, idx, 0) for s in u.src]
        return U.new(op, u.dtype, tuple(srcs), u.arg, u.tag)


@dataclass
class _Kernel:
    node: U.UOp                 # the realized tensor-graph node
    placeholder: U.UOp          # BUFFERIZE marker used by readers
    body: U.UOp
    out_ranges: List[U.UOp]
    red_ranges: List[U.UOp]
    removable: bool
    shape: tuple
    reads: set = field(default_factory=set)   # idx of BUFFER / placeholder nodes read
    has_reduce: bool = False
    fused_into: Optional[int] = None


def _body_nodes(body: U.UOp):
    return U.toposort(body, stop=lambda n: n.op in (Op.BUFFER, Op.BUFFERIZE))


def _substitute(root: U.UOp, subs: Dict[int, U.UOp]) -> U.UOp:
    out: Dict[int, U.UOp] = {}
    for n in _body_nodes(root):
        if n.idx in subs:
            out[n.idx] = subs[n.idx]
            continue
        if n.op in (Op.BUFFER, Op.BUFFERIZE) or not n.src:
            out[n.idx] = n
            continue
        srcs = tuple(out[s.idx] for s in n.src)
        out[n.idx] = n if all(a is b for a, b in zip(srcs, n.src)) else U.new(n.op, n.dtype, srcs, n.arg, n.tag)
    return out[root.idx]


def _is_view_of_buffer(u: U.UOp, realized) -> bool:
    while u.op in U.MOVEMENT:
        u = u.src[0]
    return u.op == Op.BUFFER or u.idx in realized or u.op in (Op.CONTIGUOUS, Op.REDUCE_AXIS)


#: an operand expression is written to a buffer when it would otherwise be evaluated at least this
#: many times per element (once per output column, or row, of the contraction it feeds)
MATERIALIZE_MIN_REUSE = 8

_GATHER_OPS = None


def _is_gather(o: U.UOp) -> bool:
    """True when the expression only moves data: movement ops, PAD and sums of such slices (the
    im2col a convolution builds from K padded slices, tensor/nn/nn.go:256-276).  On this device a
    gather costs one guarded load per use — the generator resolves which slice is live — so writing
    it out (K times the input's size) and reading it back is the dearer option."""
    global _GATHER_OPS
    if _GATHER_OPS is None:
        _GATHER_OPS = set(U.MOVEMENT) | {Op.ADD, Op.CONST, Op.BUFFER, Op.CONTIGUOUS, Op.REDUCE_AXIS}
    stack, seen = [o], set()
    while stack:
        u = stack.pop()
        if u.idx in seen:
            continue
        seen.add(u.idx)
        if u.op not in _GATHER_OPS:
            return False
        if u.op in (Op.BUFFER, Op.CONTIGUOUS, Op.REDUCE_AXIS):
            continue                       # a buffer (or a kernel of its own): the expression ends here
        stack.extend(u.src)
    return True


def materialize_contraction_operands(roots: List[U.UOp], by_cost: bool = False) -> List[U.UOp]:
    """Rewrite the graph so that the operands of a ``SUM(MUL(a, b))`` are views of buffers.

    ``by_cost`` decides per operand instead of wrapping all of them: an expression is written to a
    buffer when the contraction would re-evaluate it at least MATERIALIZE_MIN_REUSE times per
    element (the other operand's free extent: every output column needs the same row of A) and it
    does arithmetic; a pure gather stays an expression (see ``_is_gather``), and so does anything
    feeding a matrix-vector product, where nothing is re-used.

    An operand that is an expression (an activation of the previous layer's output, a masked
    adjoint) is wrapped in CONTIGUOUS *below* its movement ops, at the point where it still has its
    own un-broadcast shape, so that it is computed once instead of once per multiply — and every
    other consumer of that expression reads the same buffer instead of recomputing it. Not part of
    the reference scheduler; its only existing use of CONTIGUOUS as a materialisation barrier is
    tensor/gradient_ruleset.go:309-312."""
    sink = U.new(Op.SINK, dtypes.void, tuple(roots))
    topo = U.toposort(sink)[:-1]
    chosen = set()
    shapes: Dict[int, tuple] = {}
    for u in topo:
        node_shape(u, shapes)
    for u in topo:
        if u.op == Op.REDUCE_AXIS and u.arg[0] == Op.ADD and u.src[0].op == Op.MUL:
            # a contraction multiplies two operands broadcast along different axes: both reach the
            # MUL through an EXPAND (tensor/reduce.go:143-165); a plain sum of products does not
            operands, expanded = [], []
            for o in u.src[0].src:
                ex = False
                while o.op in U.MOVEMENT:
                    ex = ex or o.op == Op.EXPAND
                    o = o.src[0]
                operands.append(o)
                expanded.append(ex)
            if all(expanded):
                out_elems = math.prod(d for d in node_shape(u, shapes) if isinstance(d, int)) or 1
                for o in operands:
                    if o.op in (Op.BUFFER, Op.CONTIGUOUS, Op.REDUCE_AXIS, Op.CONST):
                        continue
                    if by_cost:
                        own = math.prod(d for d in node_shape(o, shapes) if isinstance(d, int)) or 1
                        k = math.prod(node_shape(u.src[0], shapes)[a] for a in u.arg[1] if isinstance(node_shape(u.src[0], shapes)[a], int)) or 1
                        reuse = max(1, out_elems * k // max(own, 1))      # times each element of this operand is multiplied
                        if reuse < MATERIALIZE_MIN_REUSE or _is_gather(o):
                            continue
                    chosen.add(o.idx)
    if not chosen:
        return list(roots)
    out: Dict[int, U.UOp] = {}
    for u in topo:
        srcs = tuple(out[s.idx] for s in u.src)
        v = u if all(a is b for a, b in zip(srcs, u.src)) else U.new(u.op, u.dtype, srcs, u.arg, u.tag)
        if u.idx in chosen:
            v = U.new(Op.CONTIGUOUS, v.dtype, (v,))
        out[u.idx] = v
    return [out[r.idx] for r in roots]


def _is_dense_contraction(body: U.UOp) -> bool:
    return (body.op == Op.REDUCE and body.arg == Op.ADD and body.src[0].op == Op.MUL
            and all(o.op == Op.INDEX for o in body.src[0].src))


def create_schedule(outputs: Sequence[U.UOp], max_bufs: Optional[int] = None,
                    fusion: Optional[bool] = None, keep_contractions: bool = False,
                    outputs_first: bool = False) -> Tuple[List[ExecItem], Dict[int, int]]:
    """Schedule the tensor-graph nodes ``outputs``.

    Returns the ordered items and a map from each output node's idx to the
    ``uop_idx`` of the buffer that holds it (the reference matches outputs to
    tensors by schedule order instead, tensor/realize.go:152-181).

    ``keep_contractions`` leaves a dense SUM-of-products over two buffers as a kernel of its own
    instead of splicing it into an elementwise consumer, so that it reaches the device as a plain
    GEMM (used together with ``materialize_contraction_operands``). ``outputs_first`` lets a ready
    kernel that produces a requested output run before other ready kernels, so gradients finish as
    early as the dependencies allow and their all-reduce can overlap the rest of the backward pass."""
    import sys
    sys.setrecursionlimit(max(sys.getrecursionlimit(), 100000))
    max_bufs = MAX_KERNEL_BUFFERS if max_bufs is None else max_bufs
    fusion = FUSION_ENABLED if fusion is None else fusion
    sink = U.new(Op.SINK, dtypes.void, tuple(outputs))
    topo = U.toposort(sink)[:-1]
    shapes: Dict[int, tuple] = {}
    for u in topo:
        node_shape(u, shapes)

    realize = {o.idx for o in outputs}
    for u in topo:
        if u.op in (Op.CONTIGUOUS, Op.REDUCE_AXIS):
            realize.add(u.idx)

    ctx = _Ctx()
    placeholders: Dict[int, U.UOp] = {}
    kernels: Dict[int, _Kernel] = {}       # keyed by placeholder idx
    order: List[int] = []
    for u in topo:
        if u.idx not in realize:
            continue
        ctx.start_kernel()
        out_shape = shapes[u.idx]
        out_ranges = [ctx.new_range(s, AXIS_LOOP) for s in out_shape]
        body = _Indexer(ctx, shapes, placeholders, u).run(u, out_ranges, 0)
        ph = U.new(Op.BUFFERIZE, u.dtype, (), u.idx)
        k = _Kernel(u, ph, body, out_ranges, list(ctx.reduce_ranges), u.op == Op.REDUCE_AXIS, out_shape)
        for n in _body_nodes(body):
            if n.op in (Op.BUFFER, Op.BUFFERIZE):
                k.reads.add(n.idx)
            if n.op == Op.REDUCE:
                k.has_reduce = True
        placeholders[u.idx] = ph
        kernels[ph.idx] = k
        order.append(ph.idx)

    # ── epilogue fusion ───────────────────────────────────────────────────
    if fusion:
        consumers: Dict[int, List[int]] = {}
        for kid in order:
            for r in kernels[kid].reads:
                if r in kernels:
                    consumers.setdefault(r, []).append(kid)
        for o in outputs:
            consumers.setdefault(placeholders[o.idx].idx, []).append(-1)
        reads_in_reduce: Dict[int, set] = {}
        for kid in order:
            s = set()
            for n in _body_nodes(kernels[kid].body):
                if n.op == Op.REDUCE:
                    s |= {m.idx for m in _body_nodes(n.src[0]) if m.op == Op.BUFFERIZE}
            reads_in_reduce[kid] = s
        cur = {kid: set(kernels[kid].reads) for kid in order}
        for kid in order:
            k = kernels[kid]
            if not k.removable:
                continue
            cons = consumers.get(kid, [])
            if len(cons) != 1 or cons[0] == -1:
                continue
            c = kernels[cons[0]]
            if keep_contractions and _is_dense_contraction(k.body):
                # a consumer that only re-indexes the contraction (a permuted copy of a weight
                # gradient) folds into it and leaves a contraction; anything else stays separate
                if not (c.body.op == Op.INDEX and c.body.src[0].idx == kid):
                    continue
            if c.has_reduce or kid in reads_in_reduce[cons[0]]:
                continue
            combined = (cur[cons[0]] - {kid}) | cur[kid]
            if len(combined) + 1 > max_bufs:
                continue
            k.fused_into = cons[0]
            cur[cons[0]] = combined
        for kid in order:
            k = kernels[kid]
            if k.fused_into is not None:
                continue
            producers = [p for p in order if kernels[p].fused_into == kid]
            if not producers:
                continue
            prod_set = set(producers)
            out: Dict[int, U.UOp] = {}
            for n in _body_nodes(k.body):
                if n.op == Op.INDEX and n.src[0].idx in prod_set:
                    p = kernels[n.src[0].idx]
                    subs = {pr.idx: out[i.idx] for pr, i in zip(p.out_ranges, n.src[1:]) if pr.op == Op.RANGE}
                    out[n.idx] = _substitute(p.body, subs)
                    continue
                if n.op in (Op.BUFFER, Op.BUFFERIZE) or not n.src:
                    out[n.idx] = n
                    continue
                srcs = tuple(out[s.idx] for s in n.src)
                out[n.idx] = n if all(a is b for a, b in zip(srcs, n.src)) else U.new(n.op, n.dtype, srcs, n.arg, n.tag)
            k.body = out[k.body.idx]
            extra = [r for p in producers for r in kernels[p].red_ranges]
            k.red_ranges = sorted(k.red_ranges + extra, key=lambda r: r.idx)
            k.reads = set()
            for n in _body_nodes(k.body):
                if n.op in (Op.BUFFER, Op.BUFFERIZE):
                    k.reads.add(n.idx)

    live = [kid for kid in order if kernels[kid].fused_into is None]

    # ── buffers, PARAM numbering, kernel ASTs ─────────────────────────────
    out_buf: Dict[int, U.UOp] = {}
    for kid in live:
        k = kernels[kid]
        out_buf[kid] = U.new(Op.BUFFER, k.node.dtype, (), tuple(k.shape))

    def buf_desc(b: U.UOp) -> Buffer:
        sh = tuple(0 if isinstance(s, U.Var) else int(s) for s in b.arg)
        size = 0 if any(isinstance(s, U.Var) for s in b.arg) else int(math.prod(sh))
        return Buffer(b.idx, size, sh, b.dtype)

    items: List[ExecItem] = []
    deps: List[set] = []
    for kid in live:
        k = kernels[kid]
        body = _substitute(k.body, {p: out_buf[p] for p in k.reads if p in out_buf})
        ob = out_buf[kid]
        store_dst = U.new(Op.INDEX, dtypes.void, (ob, *k.out_ranges))
        store = U.new(Op.STORE, dtypes.void, (store_dst, body))
        end = U.new(Op.END, dtypes.void, (store, *k.out_ranges, *k.red_ranges))
        # input buffers in depth-first encounter order (schedule/kernels.go:12-25, 124-143)
        seen, inputs = set(), []

        def visit(n):
            stack = [n]
            while stack:
                m = stack.pop()
                if m.idx in seen:
                    continue
                seen.add(m.idx)
                if m.op == Op.BUFFER:
                    if m is not ob:
                        inputs.append(m)
                    continue
                stack.extend(reversed(m.src))
        visit(end)
        pmap = {ob.idx: U.new(Op.PARAM, ob.dtype, (), 0)}
        for j, b in enumerate(inputs):
            pmap[b.idx] = U.new(Op.PARAM, b.dtype, (), j + 1)
        ast_end = _substitute_bufs(end, pmap)
        ast = U.new(Op.SINK, dtypes.void, (ast_end,), 1 + len(inputs))
        sym = {}
        for r in list(k.out_ranges) + list(k.red_ranges):
            if r.op == Op.RANGE and r.arg.symbolic:
                sym[r.arg.sym_param] = r.arg.var_name
        sym_vars = [sym[i] for i in range(len(sym))] if sym else []
        items.append(ExecItem(ast, [buf_desc(ob)] + [buf_desc(b) for b in inputs], sym_vars))
        deps.append({b.idx for b in inputs})

    # ── order by dependencies (stable Kahn) ───────────────────────────────
    writer = {it.bufs[0].uop_idx: i for i, it in enumerate(items)}
    n = len(items)
    indeg = [0] * n
    users: List[List[int]] = [[] for _ in range(n)]
    for i in range(n):
        for b in deps[i]:
            w = writer.get(b)
            if w is not None and w != i:
                users[w].append(i)
                indeg[i] += 1
    wanted = {out_buf[placeholders[o.idx].idx].idx for o in outputs}
    # among ready producers of requested outputs the smallest goes first: a bias gradient's tiny
    # all-reduce then hides under the weight-gradient contraction instead of queueing behind its
    # 33 MB all-reduce at the very end of the step
    prio = ((lambda i: (0, items[i].bufs[0].size, i) if items[i].bufs[0].uop_idx in wanted else (1, 0, i))
            if outputs_first else (lambda i: (0, 0, i)))
    ready = sorted((i for i in range(n) if indeg[i] == 0), key=prio)
    ordered = []
    while ready:
        i = ready.pop(0)
        ordered.append(items[i])
        for j in users[i]:
            indeg[j] -= 1
            if indeg[j] == 0:
                ready.append(j)
        ready.sort(key=prio)
    assert len(ordered) == n, "schedule: dependency cycle"
    out_map_ids = {out_buf[placeholders[o.idx].idx].idx for o in outputs}
    memory_plan(ordered, out_map_ids)
    out_map = {o.idx: out_buf[placeholders[o.idx].idx].idx for o in outputs}
    if STATS_HOOK is not None:
        STATS_HOOK(CompilerStats(len(topo), len(ordered), sum(1 for k in kernels.values() if k.fused_into is not None)))
    return ordered, out_map


def _substitute_bufs(root: U.UOp, pmap: Dict[int, U.UOp]) -> U.UOp:
    out: Dict[int, U.UOp] = {}
    for n in U.toposort(root):
        if n.op == Op.BUFFER:
            out[n.idx] = pmap[n.idx]
            continue
        if not n.src:
            out[n.idx] = n
            continue
        srcs = tuple(out[s.idx] for s in n.src)
        out[n.idx] = n if all(a is b for a, b in zip(srcs, n.src)) else U.new(n.op, n.dtype, srcs, n.arg, n.tag)
    return out[root.idx]


def memory_plan(items: List[ExecItem], keep: Optional[set] = None) -> None:
    """Greedy slot sharing for intermediates; leaves and final outputs keep
    slot -1 (schedule/kernels.go:365-463). ``keep`` names requested outputs that a
    later kernel also reads: they keep slot -1 too, so the device hands them back
    (the reference would alias them away, tensor/realize.go:147-151)."""
    keep = keep or set()
    written = {it.bufs[0].uop_idx: i for i, it in enumerate(items)}
    last_read: Dict[int, int] = {}
    for i, it in enumerate(items):
        for b in it.bufs[1:]:
            if b.uop_idx in written and b.uop_idx not in keep:
                last_read[b.uop_idx] = max(last_read.get(b.uop_idx, -1), i)
    inter = sorted((written[b], b) for b in last_read)
    slots: List[int] = []
    slot_of: Dict[int, int] = {}
    for first, b in inter:
        for s, lr in enumerate(slots):
            if lr < first:
                slots[s] = last_read[b]
                slot_of[b] = s
                break
        else:
            slot_of[b] = len(slots)
            slots.append(last_read[b])
    for it in items:
        it.bufs[0].slot = slot_of.get(it.bufs[0].uop_idx, -1)
