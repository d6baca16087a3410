"""Reverse-mode autodiff over the tensor graph.

Same driver and rule set as the reference's ``tensor.Backward``
(tensor/gradient.go:45-121, tensor/gradient_ruleset.go:68-326): a reverse
topological walk, one rule per forward op, adjoints of shared nodes summed with
ADD. The rules only call ordinary tensor ops, so gradient kernels are scheduled
exactly like forward kernels. Nothing here touches the device.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

from . import uop as U
from .uop import Op, dtypes
from .tensor import Tensor, LN2, has_symbolic


def node_shape(u: U.UOp, cache: Dict[int, tuple]) -> tuple:
    """Shape of a tensor-graph node (schedule/rangeify.go:60-147)."""
    if u.idx in cache:
        return cache[u.idx]
    op = u.op
    if op == Op.CONST:
        sh = ()
    elif op == Op.BUFFER:
        sh = tuple(u.arg)
    elif op in (Op.RESHAPE, Op.EXPAND):
        sh = tuple(u.arg)
    elif op == Op.PERMUTE:
        s = node_shape(u.src[0], cache)
        sh = tuple(s[p] for p in u.arg)
    elif op == Op.PAD:
        s = node_shape(u.src[0], cache)
        sh = tuple(d + a + b for d, (a, b) in zip(s, u.arg))
    elif op == Op.SHRINK:
        sh = tuple(b - a for a, b in u.arg)
    elif op == Op.REDUCE_AXIS:
        s = node_shape(u.src[0], cache)
        axes = set(u.arg[1])
        sh = tuple(d for i, d in enumerate(s) if i not in axes)
    elif u.src:
        sh = node_shape(u.src[0], cache)
    else:
        sh = ()
    cache[u.idx] = sh
    return sh


def backward(loss: Tensor, params: List[Tensor]) -> Dict[Tensor, Tensor]:
    """Gradients of ``loss`` w.r.t. each leaf in ``params`` (absent if unreachable)."""
    if loss is None or not params:
        return {}
    topo = U.toposort(loss.node)
    shapes: Dict[int, tuple] = {loss.node.idx: loss.shape}
    for u in topo:
        node_shape(u, shapes)

    adj: Dict[int, Tensor] = {loss.node.idx: Tensor.full(shapes[loss.node.idx], 1.0, loss.dtype)}
    for u in reversed(topo):
        a = adj.get(u.idx)
        if a is None:
            continue
        rule = _RULES.get(u.op)
        if rule is None:
            continue
        node_t = Tensor(u, shapes[u.idx], u.dtype)
        srcs = [Tensor(s, shapes[s.idx], s.dtype) for s in u.src]
        contribs = rule(u, node_t, a, srcs)
        if contribs is None:
            continue
        for s, g in zip(u.src, contribs):
            if g is None or not s.dtype.is_float:
                continue
            adj[s.idx] = adj[s.idx].add(g) if s.idx in adj else g
    return {p: adj[p.node.idx] for p in params if p.node.idx in adj}


def _k(a: Tensor, v: float) -> Tensor:
    return Tensor.full(a.shape, v, a.dtype)


def _r_neg(u, n, adj, s): return [adj.neg()]
def _r_exp2(u, n, adj, s): return [adj.mul(n).mul(_k(adj, LN2))]
def _r_log2(u, n, adj, s): return [adj.div(s[0].mul(_k(adj, LN2)))]
def _r_sin(u, n, adj, s): return [adj.mul(s[0].add(_k(adj, math.pi / 2)).sin())]
def _r_sqrt(u, n, adj, s): return [adj.div(_k(adj, 2.0).mul(n))]
def _r_recip(u, n, adj, s): return [adj.neg().mul(n).mul(n)]


def _r_cast(u, n, adj, s):
    if s[0].dtype.is_float:
        return [adj.cast(U.least_upper_dtype(adj.dtype, s[0].dtype))]
    return None


def _r_add(u, n, adj, s): return [adj, adj]
def _r_sub(u, n, adj, s): return [adj, adj.neg()]
def _r_mul(u, n, adj, s): return [adj.mul(s[1]), adj.mul(s[0])]


def _r_fdiv(u, n, adj, s):
    r = s[1].recip()
    return [adj.div(s[1]), adj.neg().mul(s[0]).mul(r).mul(r)]


def _r_max(u, n, adj, s):
    """max(a,b): the first operand wins ties (gradient_ruleset.go:159-167)."""
    z = _k(adj, 0.0)
    e0 = s[0].cmpeq(n)
    g0 = Tensor.where(e0, adj, z)
    not_tied = Tensor.where(e0, z, adj)
    g1 = Tensor.where(s[1].cmpeq(n), not_tied, z)
    return [g0, g1]


def _r_mulacc(u, n, adj, s): return [adj.mul(s[1]), adj.mul(s[0]), adj]


def _r_where(u, n, adj, s):
    z = _k(adj, 0.0)
    return [None, Tensor.where(s[0], adj, z), Tensor.where(s[0], z, adj)]


def _r_reshape(u, n, adj, s): return [adj.reshape(s[0].shape)]


def _r_expand(u, n, adj, s):
    """Sum over the broadcast axes, then restore the source shape
    (gradient_ruleset.go:207-233)."""
    axes = [i for i, d in enumerate(s[0].shape) if isinstance(d, int) and d == 1]
    g = adj
    if axes:
        g = g.sum(axes, keepdim=True)
    return [g.reshape(s[0].shape)]


def _r_permute(u, n, adj, s):
    inv = [0] * len(u.arg)
    for i, p in enumerate(u.arg):
        inv[p] = i
    return [adj.permute(inv)]


def _r_pad(u, n, adj, s):
    return [adj.shrink([(a, a + d) for (a, _), d in zip(u.arg, s[0].shape)])]


def _r_shrink(u, n, adj, s):
    return [adj.pad([(a, d - b) for (a, b), d in zip(u.arg, s[0].shape)])]


def _r_flip(u, n, adj, s): return [adj.flip([f != 0 for f in u.arg])]


#: The reference materialises the adjoint in front of a max-reduce's backward only because the fused
#: kernel would otherwise bind more buffers than WebGPU allows (gradient_ruleset.go:309-312).  A CUDA
#: kernel takes hundreds of pointers; with this off the adjoint stays an expression of its consumer.
MAX_REDUCE_BARRIER = True


def _r_contiguous(u, n, adj, s): return [adj]


def _r_reduce(u, n, adj, s):
    """SUM: broadcast the adjoint back. MAX: route it to the arg-max positions,
    splitting ties equally, with the adjoint materialised first
    (gradient_ruleset.go:285-323)."""
    rop, axes = u.arg
    src_sh = s[0].shape
    keep = tuple(1 if i in axes else d for i, d in enumerate(src_sh))
    if rop == Op.ADD:
        return [adj.reshape(keep).expand(src_sh)]
    if rop == Op.MAX:
        adj_m = adj.contiguous() if MAX_REDUCE_BARRIER else adj
        node_e = n.reshape(keep).expand(src_sh)
        adj_e = adj_m.reshape(keep).expand(src_sh)
        mask = s[0].cmpeq(node_e)
        ties = mask.cast(adj_m.dtype).sum(list(axes), keepdim=True).expand(src_sh)
        return [Tensor.where(mask, adj_e.div(ties), Tensor.full(src_sh, 0.0, adj_m.dtype))]
    return None


_RULES = {
    Op.NEG: _r_neg, Op.EXP2: _r_exp2, Op.LOG2: _r_log2, Op.SIN: _r_sin, Op.SQRT: _r_sqrt,
    Op.RECIPROCAL: _r_recip, Op.CAST: _r_cast, Op.BITCAST: _r_cast,
    Op.ADD: _r_add, Op.SUB: _r_sub, Op.MUL: _r_mul, Op.FDIV: _r_fdiv, Op.MAX: _r_max,
    Op.MULACC: _r_mulacc, Op.WHERE: _r_where,
    Op.RESHAPE: _r_reshape, Op.EXPAND: _r_expand, Op.PERMUTE: _r_permute, Op.PAD: _r_pad,
    Op.SHRINK: _r_shrink, Op.FLIP: _r_flip, Op.CONTIGUOUS: _r_contiguous,
    Op.REDUCE_AXIS: _r_reduce,
}
