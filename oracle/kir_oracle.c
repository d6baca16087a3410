/*
 * CPU oracle for anneal's scheduled kernels.  TEST INFRASTRUCTURE ONLY: it is
 * the checker the CUDA path is compared with and the timed CPU baseline; no
 * product code links, loads or calls it.
 *
 * It interprets the kernel-IR blob (the serialised []schedule.ExecItem) with
 * the semantics of the WGSL the reference generates, which is the only
 * specification of the arithmetic the reference has (its backend hands that
 * text to a GPU driver through un-vendored third-party modules):
 *
 *   iteration space, store index ........ codegen/lower.go:175-550
 *   flat load index from buffer shape ... codegen/lower.go:584-652
 *   reductions: one accumulator per REDUCE, nested loops in source order,
 *     ascending, f32 accumulator for f16/bf16 with the whole body widened
 *     and one narrowing at the end ....... codegen/lower.go:654-719, 158-171
 *   op table, i32 truncating / and % ..... codegen/wgsl.go:240-312
 *   literals: a float constant is (float)v, an f16 one (half)(float)v,
 *     +-inf clamp to +-FLT_MAX / +-65504 .. codegen/wgsl.go:314-355
 *   reduce identities: 0, 1, -FLT_MAX .... codegen/wgsl.go:357-396
 *   f16 round-to-nearest-even, bf16 by truncation at the store
 *     ..................................... uop/dtype.go:392-487, codegen/wgsl.go:228-229
 *   values cross the boundary as f32 and are quantised on upload
 *     ..................................... backend/webgpu/executor.go:161-179, 457-466
 *
 * WHERE evaluates only the selected branch, so a PAD's guarded load is never
 * performed out of range (WGSL clamps such reads; the value is discarded
 * either way, schedule/index.go:101-134).  Sub-expressions that do not depend
 * on the innermost ranges, reductions included, are re-used until one of the
 * ranges they read changes: the values are identical to recomputing them per
 * element and full-size schedules stay tractable.
 *
 * Difference-noise model (sampled evaluation only, optional): beside each value the evaluator can
 * carry the variance of the difference a second, equally valid evaluation would show.  Two
 * implementations of these kernels legitimately differ in three places only: the order in which a
 * REDUCE adds its terms (each partial sum rounds to f32, unit roundoff 2^-24), the approximation of
 * exp2 / log2 / sin and of the f16-class reciprocal and division (a few f32 units), and — as a
 * consequence — an f16 rounding that such a small difference tips to the neighbouring value (from
 * there on it is a difference of whole f16 units, which later roundings pass on unchanged).
 * Everything else (f16 and f32 add, sub, mul, compare, select) rounds identically everywhere and
 * only propagates what it is given, to first order.  A comparison can then tell "differs by more
 * than the stated tolerance" from "is a sum whose terms cancel, so that any two orders of addition
 * differ by this much" — the row statistics of a softmax gradient that are zero in exact arithmetic
 * are the case in point.  The model is not part of the reference; it changes no value.
 *
 * Parity status: pinned by the known-answer vectors that are literal in the
 * reference's own tests (backend/webgpu/webgpu_test.go:84-359,
 * schedule/schedule_test.go:809-915, tensor/nn/train_test.go:71-144,
 * tensor/nn/maxpool_test.go:16-111, backend/webgpu/f16_test.go); the
 * reference itself cannot be executed where this was written (no Go toolchain).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum {
    OP_PARAM = 7, OP_SINK = 13, OP_INDEX = 18, OP_STORE = 20, OP_CAST = 22, OP_BITCAST = 23,
    OP_EXP2 = 24, OP_LOG2 = 25, OP_SIN = 26, OP_SQRT = 27, OP_RECIP = 28, OP_NEG = 29, OP_TRUNC = 30,
    OP_ADD = 31, OP_MUL = 32, OP_SHL = 33, OP_SHR = 34, OP_IDIV = 35, OP_MAX = 36, OP_MOD = 37,
    OP_CMPLT = 38, OP_CMPNE = 39, OP_CMPEQ = 40, OP_XOR = 41, OP_OR = 42, OP_AND = 43, OP_SUB = 45,
    OP_FDIV = 46, OP_POW = 47, OP_WHERE = 48, OP_MULACC = 49, OP_RANGE = 51, OP_END = 53, OP_CONST = 56,
    OP_REDUCE = 82
};
enum { DT_VOID = 0, DT_BOOL = 1, DT_I32 = 6, DT_U32 = 7, DT_F16 = 10, DT_BF16 = 11, DT_F32 = 12, DT_F64 = 13, DT_INDEX = 14 };
/* compute classes */
enum { C_F32, C_F16, C_INT, C_UINT, C_BOOL };

typedef union { float f; int32_t i; uint32_t u; } val;

typedef struct {
    uint16_t op; uint8_t dtype, flags; uint32_t nsrc, src_off, aux; int64_t arg;
} __attribute__((packed)) raw_node;

typedef struct {
    int op, dtype, nsrc, cls, widen;
    const uint32_t *src;
    int64_t arg; uint32_t aux; int flags;
    int ndep; int *dep;          /* indices (into item->ranges) of the ranges this node reads */
    int range_slot;              /* RANGE: index into item->ranges */
    val cval;                    /* CONST: value in this node's compute class */
} node;

typedef struct { uint32_t id; int slot, dtype, rank; int64_t size; int64_t shape[8]; } bufdesc;

typedef struct {
    int n_nodes, n_bufs, n_sym, n_ranges;
    node *nodes; bufdesc *bufs; char **sym; int *range_node; uint32_t *srcpool;
} item;

typedef struct { uint32_t id; int dtype; int64_t elems; val *data; int owned; } buffer;

typedef struct {
    int n_items; item *items;
    int n_buf; buffer *bufs; int cap_buf;
    int n_bind; char bind_name[16][64]; int64_t bind_val[16];
    char err[256];
} orc;

/* ── f16 conversions (uop/dtype.go:392-474): round-to-nearest-even from double ── */
static float f16_round_d(double d) {
    if (d != d) return NAN;
    double a = fabs(d);
    if (a == 0.0) return (float)d;
    if (isinf(a)) return (float)d;
    int e; frexp(a, &e);            /* a = m * 2^e, m in [0.5,1) → exponent of leading bit = e-1 */
    int lead = e - 1;
    int q = lead < -14 ? -24 : lead - 10;   /* quantum exponent */
    double s = ldexp(a, -q);
    double r = nearbyint(s);                /* default rounding mode is RTNE */
    double out = ldexp(r, q);
    if (out >= 65520.0) out = INFINITY;     /* rounds past max finite (65504) */
    return (float)(d < 0 ? -out : out);
}
static float f16_round_f(float f) { return f16_round_d((double)f); }
static float bf16_trunc(float f) { uint32_t u; memcpy(&u, &f, 4); u &= 0xFFFF0000u; memcpy(&f, &u, 4); return f; }

static int dtype_class(int dt) {
    switch (dt) {
    case DT_F16: return C_F16;
    case DT_BOOL: return C_BOOL;
    case DT_F32: case DT_BF16: case DT_F64: case DT_VOID: return C_F32;
    case DT_U32: case 3: case 5: case 9: return C_UINT;
    default: return C_INT;
    }
}

/* ── blob parsing ── */
static int parse(orc *o, const uint8_t *p, size_t len) {
    const uint8_t *end = p + len;
    if (len < 8 || memcmp(p, "KIR1", 4)) { snprintf(o->err, sizeof o->err, "oracle: bad magic"); return 1; }
    uint32_t n; memcpy(&n, p + 4, 4); p += 8;
    o->n_items = (int)n; o->items = calloc(n ? n : 1, sizeof(item));
    for (uint32_t k = 0; k < n; k++) {
        item *it = &o->items[k];
        uint32_t h[11];
        if (p + 44 > end) goto trunc;
        memcpy(h, p, 44); p += 44;
        it->n_nodes = h[0]; it->n_bufs = h[2]; it->n_sym = h[3];
        uint32_t n_srcs = h[1], src_len = h[4];
        if (p + (size_t)it->n_nodes * 24 + (size_t)n_srcs * 4 > end) goto trunc;
        it->nodes = calloc(it->n_nodes ? it->n_nodes : 1, sizeof(node));
        it->srcpool = malloc((n_srcs ? n_srcs : 1) * 4);
        const raw_node *rn = (const raw_node *)p; p += (size_t)it->n_nodes * 24;
        memcpy(it->srcpool, p, (size_t)n_srcs * 4); p += (size_t)n_srcs * 4;
        for (int i = 0; i < it->n_nodes; i++) {
            raw_node r; memcpy(&r, &rn[i], 24);
            node *nd = &it->nodes[i];
            nd->op = r.op; nd->dtype = r.dtype; nd->flags = r.flags; nd->nsrc = r.nsrc;
            nd->src = it->srcpool + r.src_off; nd->aux = r.aux; nd->arg = r.arg;
            nd->cls = dtype_class(r.dtype);
            for (int s = 0; s < nd->nsrc; s++)
                if (nd->src[s] >= (uint32_t)i) { snprintf(o->err, sizeof o->err, "oracle: node %d not in topological order", i); return 1; }
        }
        it->bufs = calloc(it->n_bufs ? it->n_bufs : 1, sizeof(bufdesc));
        for (int b = 0; b < it->n_bufs; b++) {
            if (p + 20 > end) goto trunc;
            bufdesc *bd = &it->bufs[b];
            int32_t slot; memcpy(&bd->id, p, 4); memcpy(&slot, p + 4, 4);
            bd->slot = slot; bd->dtype = p[8]; bd->rank = p[9]; memcpy(&bd->size, p + 12, 8); p += 20;
            if (bd->rank > 8) { snprintf(o->err, sizeof o->err, "oracle: rank > 8"); return 1; }
            if (p + 8 * bd->rank > end) goto trunc;
            memcpy(bd->shape, p, 8 * bd->rank); p += 8 * bd->rank;
        }
        it->sym = calloc(it->n_sym ? it->n_sym : 1, sizeof(char *));
        for (int s = 0; s < it->n_sym; s++) {
            uint16_t l; if (p + 2 > end) goto trunc;
            memcpy(&l, p, 2); p += 2;
            it->sym[s] = calloc(l + 1, 1); memcpy(it->sym[s], p, l); p += l;
        }
        p += src_len;
    }
    return 0;
trunc:
    snprintf(o->err, sizeof o->err, "oracle: truncated blob");
    return 1;
}

/* ── static analysis per item: range table, dependency sets, widening, constants ── */
static void mark_widen(item *it, int i) {
    node *n = &it->nodes[i];
    if (n->widen) return;
    n->widen = 1;
    if (n->op == OP_INDEX) return;     /* index arithmetic is integer; the load itself widens */
    for (int s = 0; s < n->nsrc; s++) mark_widen(it, n->src[s]);
}

static val const_value(const node *n) {
    val v; v.u = 0;
    if (n->dtype == DT_F16 || n->dtype == DT_F32 || n->dtype == DT_BF16 || n->dtype == DT_F64) {
        double d; memcpy(&d, &n->arg, 8);
        int f16 = (n->dtype == DT_F16);
        if (isinf(d)) v.f = (float)((d < 0 ? -1.0 : 1.0) * (f16 ? 65504.0 : (double)3.4028234663852886e38f));
        else if (d != d) v.f = NAN;
        else { v.f = (float)d; if (f16 && !n->widen) v.f = f16_round_f(v.f); }
    } else if (n->dtype == DT_BOOL) v.i = n->arg != 0;
    else v.i = (int32_t)n->arg;
    return v;
}

static void analyse(item *it) {
    int nr = 0;
    for (int i = 0; i < it->n_nodes; i++) if (it->nodes[i].op == OP_RANGE) nr++;
    it->n_ranges = nr; it->range_node = calloc(nr ? nr : 1, sizeof(int));
    nr = 0;
    for (int i = 0; i < it->n_nodes; i++)
        if (it->nodes[i].op == OP_RANGE) { it->nodes[i].range_slot = nr; it->range_node[nr++] = i; }
    for (int i = 0; i < it->n_nodes; i++) {
        node *n = &it->nodes[i];
        if (n->op == OP_REDUCE && n->dtype == DT_F16) mark_widen(it, n->src[0]);
    }
    unsigned char *mask = calloc((size_t)it->n_nodes * (nr ? nr : 1), 1);
    for (int i = 0; i < it->n_nodes; i++) {
        node *n = &it->nodes[i];
        unsigned char *m = mask + (size_t)i * (nr ? nr : 1);
        if (n->op == OP_RANGE) m[n->range_slot] = 1;
        for (int s = 0; s < n->nsrc; s++) {
            unsigned char *ms = mask + (size_t)n->src[s] * (nr ? nr : 1);
            for (int r = 0; r < nr; r++) m[r] |= ms[r];
        }
        if (n->op == OP_REDUCE)        /* a REDUCE binds its own ranges */
            for (int s = 1; s < n->nsrc; s++)
                if (it->nodes[n->src[s]].op == OP_RANGE) m[it->nodes[n->src[s]].range_slot] = 0;
        int c = 0; for (int r = 0; r < nr; r++) c += m[r];
        n->ndep = c; n->dep = malloc((c ? c : 1) * sizeof(int));
        c = 0; for (int r = 0; r < nr; r++) if (m[r]) n->dep[c++] = r;
        if (n->op == OP_CONST) n->cval = const_value(n);
    }
    free(mask);
}

/* ── evaluation ── */
typedef struct {
    const orc *o; const item *it;
    val **bufdata; int64_t *bufelems; int64_t (*strides)[8];
    int32_t *rval; uint64_t *rver;      /* per range: current value, version */
    val *cache; uint64_t *cver;         /* per node: cached value and the version sum it was computed at */
    double *nvar, *qvar;                /* per node, when not NULL: modelled variance of the difference between two valid
                                           evaluations: the part that is still continuous, and the part that f16 roundings
                                           have already turned into whole-unit differences */
} ectx;

static inline uint64_t dep_version(const ectx *c, const node *n) {
    uint64_t s = 1;
    for (int d = 0; d < n->ndep; d++) s += c->rver[n->dep[d]];
    return s;
}

static val eval(ectx *c, int i);

static inline float as_f(const node *n, val v) {
    switch (n->cls) { case C_F32: case C_F16: return v.f; case C_UINT: return (float)v.u; default: return (float)v.i; }
}

static inline float fin(const node *n, double r) {
    /* result of a float op in the node's compute type */
    if (n->cls == C_F16 && !n->widen) return f16_round_d(r);
    return (float)r;
}

static int64_t range_bound(const ectx *c, const node *r) {
    if (r->flags & 8) {
        int p = (r->flags >> 4) & 15;
        const char *name = p < c->it->n_sym ? c->it->sym[p] : "";
        for (int b = 0; b < c->o->n_bind; b++)
            if (!strcmp(c->o->bind_name[b], name)) return c->o->bind_val[b];
        return 0;
    }
    return r->arg;
}

#define U32 5.9604644775390625e-08   /* 2^-24 */
#define U16 4.8828125e-04            /* 2^-11 */
/* variance an approximated function adds: two f32 units of its result */
static inline double approx_var(double r) { return (2.0 * U32 * r) * (2.0 * U32 * r); }
/* an f16 rounding of r whose argument carries variance v.  A difference well below one unit tips
 * the rounding to the neighbouring value with probability ~ sigma / ulp and then counts a whole
 * unit: variance sigma * ulp.  A difference of a unit or more comes through as it is, plus the two
 * roundings' own variance. */
static inline double f16_tip_var(double v, double r) {
    double a = fabs(r) < 6.103515625e-05 ? 6.103515625e-05 : fabs(r);     /* below 2^-14 the spacing stays 2^-24 */
    double ulp = 2.0 * U16 * a, sg = sqrt(v);
    return sg < ulp ? sg * ulp : v + ulp * ulp / 6.0;
}
static inline int rounds_f16(const node *n) { return n->cls == C_F16 && !n->widen; }
static inline double nv(const ectx *c, int i) { return c->nvar ? c->nvar[i] : 0.0; }
static inline double qv(const ectx *c, int i) { return c->qvar ? c->qvar[i] : 0.0; }

static val eval_reduce(ectx *c, const node *n) {
    const item *it = c->it;
    int rop = (int)n->aux;
    int isf = (n->cls == C_F32 || n->cls == C_F16);
    val acc;
    if (isf) acc.f = rop == OP_MUL ? 1.0f : rop == OP_MAX ? -3.4028234663852886e38f : 0.0f;
    else if (n->cls == C_UINT) acc.u = rop == OP_MUL ? 1u : 0u;
    else acc.i = rop == OP_MUL ? 1 : rop == OP_MAX ? INT32_MIN : 0;
    int nr = n->nsrc - 1, slots[8]; int64_t bound[8]; int nl = 0;
    for (int s = 0; s < nr && nl < 8; s++) {
        const node *r = &it->nodes[n->src[1 + s]];
        if (r->op != OP_RANGE) continue;
        slots[nl] = r->range_slot; bound[nl] = range_bound(c, r); nl++;
    }
    double vacc = 0.0, qacc = 0.0;
    for (int l = 0; l < nl; l++) if (bound[l] <= 0) goto done;
    for (int l = 0; l < nl; l++) { c->rval[slots[l]] = 0; c->rver[slots[l]]++; }
    for (;;) {
        val e = eval(c, n->src[0]);
        if (isf) {
            float x = e.f;
            if (c->nvar) {
                double ve = c->nvar[n->src[0]], qe = c->qvar[n->src[0]];
                if (rop == OP_ADD) { double r = (double)acc.f + (double)x; vacc += ve + (U32 * r) * (U32 * r) / 3.0; qacc += qe; }
                else if (rop == OP_MUL) { vacc = vacc * (double)x * (double)x + ve * (double)acc.f * (double)acc.f; qacc = qacc * (double)x * (double)x + qe * (double)acc.f * (double)acc.f; }
                else { if (ve > vacc) vacc = ve; if (qe > qacc) qacc = qe; }
            }
            if (rop == OP_ADD) acc.f = acc.f + x;
            else if (rop == OP_MUL) acc.f = acc.f * x;
            else if (rop == OP_MAX) acc.f = (x != x || acc.f != acc.f) ? (x != x ? acc.f : x) : (acc.f < x ? x : acc.f);
            else acc.f = acc.f + x;
        } else if (n->cls == C_UINT) {
            if (rop == OP_ADD) acc.u += e.u; else if (rop == OP_MUL) acc.u *= e.u; else if (rop == OP_MAX) acc.u = acc.u < e.u ? e.u : acc.u; else acc.u += e.u;
        } else {
            if (rop == OP_ADD) acc.i += e.i; else if (rop == OP_MUL) acc.i *= e.i; else if (rop == OP_MAX) acc.i = acc.i < e.i ? e.i : acc.i; else acc.i += e.i;
        }
        int l = nl - 1;
        while (l >= 0) {
            c->rval[slots[l]]++; c->rver[slots[l]]++;
            if (c->rval[slots[l]] < bound[l]) break;
            c->rval[slots[l]] = 0; l--;
        }
        if (l < 0) break;
    }
done:
    if (n->dtype == DT_F16) { acc.f = f16_round_f(acc.f); qacc += f16_tip_var(vacc, (double)acc.f); vacc = 0.0; }   /* f16(acc): the single narrowing */
    if (c->nvar) { c->nvar[n - c->it->nodes] = vacc; c->qvar[n - c->it->nodes] = qacc; }
    return acc;
}

static val eval_index(ectx *c, const node *n) {
    const item *it = c->it;
    const node *p = &it->nodes[n->src[0]];
    int pi = (int)p->arg;
    int nd = n->nsrc - 1;
    int64_t flat = 0;
    if (nd == 1) flat = eval(c, n->src[1]).i;
    else for (int d = 0; d < nd; d++) flat += (int64_t)eval(c, n->src[1 + d]).i * c->strides[pi][d];
    val v; v.u = 0;
    if (flat < 0 || flat >= c->bufelems[pi]) return v;   /* WGSL: out-of-range reads are defined and discarded */
    return c->bufdata[pi][flat];
}

static val eval(ectx *c, int i) {
    const node *n = &c->it->nodes[i];
    if (n->op == OP_CONST) return n->cval;
    if (n->op == OP_RANGE) { val v; v.i = c->rval[n->range_slot]; return v; }
    uint64_t ver = dep_version(c, n);
    if (c->cver[i] == ver) return c->cache[i];
    val r; r.u = 0;
    const uint32_t *s = n->src;
    const node *nodes = c->it->nodes;
    int isf = (n->cls == C_F32 || n->cls == C_F16);
    switch (n->op) {
    case OP_INDEX: r = eval_index(c, n); break;
    case OP_REDUCE: r = eval_reduce(c, n); break;
    case OP_WHERE: r = eval(c, s[0]).i ? eval(c, s[1]) : eval(c, s[2]); if (n->cls == C_F16 && !n->widen) r.f = f16_round_f(r.f); break;
    case OP_CAST: {
        const node *sn = &nodes[s[0]]; val a = eval(c, s[0]);
        if (isf) { float x = as_f(sn, a); r.f = (n->cls == C_F16 && !n->widen) ? f16_round_f(x) : x; }
        else if (n->cls == C_BOOL) r.i = (sn->cls == C_F32 || sn->cls == C_F16) ? (a.f != 0.0f) : (a.i != 0);
        else if (n->cls == C_UINT) r.u = (sn->cls == C_F32 || sn->cls == C_F16) ? (uint32_t)a.f : a.u;
        else r.i = (sn->cls == C_F32 || sn->cls == C_F16) ? (int32_t)a.f : a.i;
        break; }
    case OP_BITCAST: r = eval(c, s[0]); break;
    case OP_EXP2: r.f = fin(n, exp2f(eval(c, s[0]).f)); break;
    case OP_LOG2: r.f = fin(n, log2f(eval(c, s[0]).f)); break;
    case OP_SIN: r.f = fin(n, sinf(eval(c, s[0]).f)); break;
    case OP_SQRT: r.f = fin(n, n->cls == C_F16 && !n->widen ? sqrt((double)eval(c, s[0]).f) : (double)sqrtf(eval(c, s[0]).f)); break;
    case OP_RECIP: { float x = eval(c, s[0]).f; r.f = fin(n, n->cls == C_F16 && !n->widen ? 1.0 / (double)x : (double)(1.0f / x)); break; }
    case OP_NEG: if (isf) { float x = eval(c, s[0]).f; r.f = (n->cls == C_F16 && !n->widen) ? -f16_round_f(x) : -x; } else r.i = -eval(c, s[0]).i; break;
    case OP_TRUNC: r.f = truncf(eval(c, s[0]).f); break;
    case OP_ADD: case OP_SUB: case OP_MUL: case OP_FDIV: case OP_MAX: case OP_POW: {
        val a = eval(c, s[0]), b = eval(c, s[1]);
        if (isf) {
            if (n->cls == C_F16 && !n->widen) {
                /* an operand shared with an f16 reduction carries its widened (f32) value: it is
                 * narrowed where f16 code uses it */
                double x = f16_round_f(a.f), y = f16_round_f(b.f), z;
                switch (n->op) { case OP_ADD: z = x + y; break; case OP_SUB: z = x - y; break; case OP_MUL: z = x * y; break;
                                 case OP_FDIV: z = x / y; break; case OP_MAX: z = (x != x) ? y : (y != y) ? x : (x < y ? y : x); break; default: z = pow(x, y); }
                r.f = f16_round_d(z);
            } else {
                float x = a.f, y = b.f;
                switch (n->op) { case OP_ADD: r.f = x + y; break; case OP_SUB: r.f = x - y; break; case OP_MUL: r.f = x * y; break;
                                 case OP_FDIV: r.f = x / y; break; case OP_MAX: r.f = (x != x) ? y : (y != y) ? x : (x < y ? y : x); break; default: r.f = powf(x, y); }
            }
        } else if (n->cls == C_UINT) {
            switch (n->op) { case OP_ADD: r.u = a.u + b.u; break; case OP_SUB: r.u = a.u - b.u; break; case OP_MUL: r.u = a.u * b.u; break; case OP_MAX: r.u = a.u < b.u ? b.u : a.u; break; default: r.u = 0; }
        } else {
            switch (n->op) { case OP_ADD: r.i = (int32_t)((uint32_t)a.i + (uint32_t)b.i); break; case OP_SUB: r.i = (int32_t)((uint32_t)a.i - (uint32_t)b.i); break;
                             case OP_MUL: r.i = (int32_t)((uint32_t)a.i * (uint32_t)b.i); break; case OP_MAX: r.i = a.i < b.i ? b.i : a.i; break; default: r.i = 0; }
        }
        break; }
    case OP_MULACC: { /* (s0 + (s1 * s2)), codegen/wgsl.go:303-304 */
        val a = eval(c, s[0]), b = eval(c, s[1]), d = eval(c, s[2]);
        if (isf) { if (n->cls == C_F16 && !n->widen) r.f = f16_round_d((double)f16_round_f(a.f) + (double)f16_round_d((double)f16_round_f(b.f) * (double)f16_round_f(d.f))); else { float m = b.f * d.f; r.f = a.f + m; } }
        else r.i = a.i + b.i * d.i;
        break; }
    case OP_IDIV: { val a = eval(c, s[0]), b = eval(c, s[1]);
        if (n->cls == C_UINT) r.u = b.u ? a.u / b.u : 0; else r.i = (b.i == 0 || (a.i == INT32_MIN && b.i == -1)) ? 0 : a.i / b.i; break; }
    case OP_MOD: { val a = eval(c, s[0]), b = eval(c, s[1]);
        if (isf) r.f = fin(n, fmodf(a.f, b.f));
        else if (n->cls == C_UINT) r.u = b.u ? a.u % b.u : 0; else r.i = (b.i == 0 || (a.i == INT32_MIN && b.i == -1)) ? 0 : a.i % b.i; break; }
    case OP_SHL: r.u = eval(c, s[0]).u << (eval(c, s[1]).u & 31); break;
    case OP_SHR: if (n->cls == C_UINT) r.u = eval(c, s[0]).u >> (eval(c, s[1]).u & 31); else r.i = eval(c, s[0]).i >> (eval(c, s[1]).u & 31); break;
    case OP_AND: r.u = eval(c, s[0]).u & eval(c, s[1]).u; break;
    case OP_OR: r.u = eval(c, s[0]).u | eval(c, s[1]).u; break;
    case OP_XOR: r.u = eval(c, s[0]).u ^ eval(c, s[1]).u; break;
    case OP_CMPLT: case OP_CMPNE: case OP_CMPEQ: {
        const node *sn = &nodes[s[0]]; val a = eval(c, s[0]), b = eval(c, s[1]);
        if (sn->cls == C_F32 || sn->cls == C_F16) r.i = n->op == OP_CMPLT ? a.f < b.f : n->op == OP_CMPNE ? a.f != b.f : a.f == b.f;
        else if (sn->cls == C_UINT) r.i = n->op == OP_CMPLT ? a.u < b.u : n->op == OP_CMPNE ? a.u != b.u : a.u == b.u;
        else r.i = n->op == OP_CMPLT ? a.i < b.i : n->op == OP_CMPNE ? a.i != b.i : a.i == b.i;
        break; }
    default: break;
    }
    if (c->nvar && isf && n->op != OP_REDUCE) {
        /* first-order propagation; operand values come from the cache the evaluation above filled */
        double v = 0.0, q = 0.0, rr = (double)r.f;
        #define VAL(k) ((double)as_f(&nodes[s[k]], c->cache[s[k]]))
        #define CVAL(k) (nodes[s[k]].op == OP_CONST ? (double)as_f(&nodes[s[k]], nodes[s[k]].cval) : nodes[s[k]].op == OP_RANGE ? (double)c->rval[nodes[s[k]].range_slot] : VAL(k))
        /* LIN1(d): one operand with derivative d; LIN2(da, db): two */
        #define LIN1(d) do { double d_ = (d); v = d_ * d_ * nv(c, s[0]); q = d_ * d_ * qv(c, s[0]); } while (0)
        #define LIN2(da, db) do { double a_ = (da), b_ = (db); v = a_ * a_ * nv(c, s[0]) + b_ * b_ * nv(c, s[1]); q = a_ * a_ * qv(c, s[0]) + b_ * b_ * qv(c, s[1]); } while (0)
        switch (n->op) {
        case OP_INDEX: break;
        case OP_WHERE: { int k = eval(c, s[0]).i ? 1 : 2; v = nv(c, s[k]); q = qv(c, s[k]); break; }
        case OP_CAST: { const node *sn = &nodes[s[0]]; if (sn->cls == C_F32 || sn->cls == C_F16) LIN1(1.0); break; }
        case OP_BITCAST: case OP_NEG: case OP_TRUNC: LIN1(1.0); break;
        case OP_EXP2: LIN1(0.6931471805599453 * rr); v += approx_var(rr); break;
        case OP_LOG2: { double a = CVAL(0); LIN1(a != 0.0 ? 1.0 / (a * 0.6931471805599453) : 0.0); v += approx_var(rr) + (2.0 * U32) * (2.0 * U32); break; }
        case OP_SIN: LIN1(1.0); v += approx_var(rr) + (2.0 * U32) * (2.0 * U32); break;
        case OP_SQRT: LIN1(rr != 0.0 ? 0.5 / rr : 0.0); break;
        case OP_RECIP: LIN1(rr * rr); if (rounds_f16(n)) v += approx_var(rr); break;
        case OP_ADD: case OP_SUB: LIN2(1.0, 1.0); break;
        case OP_MUL: { double a = CVAL(0), b = CVAL(1); LIN2(b, a); break; }
        case OP_FDIV: { double a = CVAL(0), b = CVAL(1); if (b != 0.0) LIN2(1.0 / b, a / (b * b)); if (rounds_f16(n)) v += approx_var(rr); break; }
        case OP_MAX: { double a = nv(c, s[0]) + qv(c, s[0]), b = nv(c, s[1]) + qv(c, s[1]); int k = a > b ? 0 : 1; v = nv(c, s[k]); q = qv(c, s[k]); break; }
        case OP_MULACC: { double b = CVAL(1), d = CVAL(2); v = nv(c, s[0]) + d * d * nv(c, s[1]) + b * b * nv(c, s[2]); q = qv(c, s[0]) + d * d * qv(c, s[1]) + b * b * qv(c, s[2]); break; }
        default: LIN1(1.0); v += approx_var(rr); break;
        }
        if (rounds_f16(n) && v > 0.0) { q += f16_tip_var(v, rr); v = 0.0; }
        #undef LIN1
        #undef LIN2
        #undef VAL
        #undef CVAL
        if (!(v == v) || v > 1e300) v = 1e300;
        if (!(q == q) || q > 1e300) q = 1e300;
        c->nvar[i] = v; c->qvar[i] = q;
    }
    c->cache[i] = r; c->cver[i] = ver;
    return r;
}

static buffer *find_buf(orc *o, uint32_t id) {
    for (int i = 0; i < o->n_buf; i++) if (o->bufs[i].id == id) return &o->bufs[i];
    return NULL;
}

static buffer *get_buf(orc *o, uint32_t id, int dtype, int64_t elems) {
    buffer *b = find_buf(o, id);
    if (b) {
        if (b->elems < elems) { b->data = realloc(b->data, (size_t)elems * sizeof(val)); memset(b->data + b->elems, 0, (size_t)(elems - b->elems) * sizeof(val)); b->elems = elems; }
        return b;
    }
    if (o->n_buf == o->cap_buf) { o->cap_buf = o->cap_buf ? o->cap_buf * 2 : 64; o->bufs = realloc(o->bufs, o->cap_buf * sizeof(buffer)); }
    b = &o->bufs[o->n_buf++];
    b->id = id; b->dtype = dtype; b->elems = elems; b->data = calloc(elems ? elems : 1, sizeof(val)); b->owned = 1;
    return b;
}

static int64_t sym_value(const orc *o, const item *it) {
    for (int s = 0; s < it->n_sym; s++)
        for (int b = 0; b < o->n_bind; b++)
            if (!strcmp(o->bind_name[b], it->sym[s])) return o->bind_val[b];
    return -1;
}

static int64_t resolved_elems(const orc *o, const item *it, const bufdesc *bd) {
    int has0 = 0; int64_t p = 1;
    for (int d = 0; d < bd->rank; d++) { if (bd->shape[d] == 0) has0 = 1; else p *= bd->shape[d]; }
    if (!has0) return bd->rank ? p : (bd->size ? bd->size : 1);
    int64_t v = sym_value(o, it);
    if (v < 0) for (int b = 0; b < o->n_bind; b++) v = o->bind_val[b];   /* a leaf read by a static kernel of a symbolic schedule */
    return v < 0 ? 0 : p * v;
}

static int run_item(orc *o, const item *it, int threads) {
    if (it->n_nodes == 0) { snprintf(o->err, sizeof o->err, "oracle: item without AST"); return 1; }
    const node *sink = &it->nodes[it->n_nodes - 1];
    if (sink->op != OP_SINK) { snprintf(o->err, sizeof o->err, "oracle: last node is not SINK"); return 1; }
    const node *end = &it->nodes[sink->src[0]];
    const node *store = &it->nodes[end->src[0]];
    int body = store->src[1];
    /* loop ranges: END.src[1:] that are loop-axis RANGE nodes, in order (codegen/lower.go:196-222) */
    int lslots[16], nl = 0; int64_t lsize[16];
    ectx proto; memset(&proto, 0, sizeof proto); proto.o = o; proto.it = it;
    for (int s = 1; s < end->nsrc; s++) {
        const node *r = &it->nodes[end->src[s]];
        if (r->op == OP_RANGE && (r->flags & 7) != 1 && nl < 16) {
            lslots[nl] = r->range_slot; lsize[nl] = range_bound(&proto, r); nl++;
        }
    }
    int64_t total = 1; for (int l = 0; l < nl; l++) total *= lsize[l];
    /* bind buffers */
    val *bufdata[64]; int64_t bufelems[64]; int64_t strides[64][8];
    if (it->n_bufs > 64) { snprintf(o->err, sizeof o->err, "oracle: too many buffers"); return 1; }
    for (int b = 0; b < it->n_bufs; b++) {
        const bufdesc *bd = &it->bufs[b];
        int64_t elems = resolved_elems(o, it, bd);
        buffer *bf = b == 0 ? get_buf(o, bd->id, bd->dtype, elems > total ? elems : total) : find_buf(o, bd->id);
        if (!bf) { snprintf(o->err, sizeof o->err, "oracle: input buffer %u has no data", bd->id); return 1; }
        if (b == 0) bf->dtype = bd->dtype;
        bufdata[b] = bf->data; bufelems[b] = bf->elems;
        int64_t st = 1;
        for (int d = bd->rank - 1; d >= 0; d--) { strides[b][d] = st; st *= (bd->shape[d] ? bd->shape[d] : 1); }
    }
    /* data pointers may have moved if get_buf realloc'd the table: re-read */
    for (int b = 0; b < it->n_bufs; b++) { buffer *bf = find_buf(o, it->bufs[b].id); bufdata[b] = bf->data; bufelems[b] = bf->elems; }
    int out_dt = it->bufs[0].dtype;
    val *out = bufdata[0];
    int nthreads = threads > 0 ? threads : 1;
    if (total < 256) nthreads = 1;
    int failed = 0;
#pragma omp parallel num_threads(nthreads)
    {
#ifdef _OPENMP
        int tid = omp_get_thread_num(), nt = omp_get_num_threads();
#else
        int tid = 0, nt = 1;
#endif
        ectx c = proto;
        c.bufdata = bufdata; c.bufelems = bufelems; c.strides = strides;
        c.rval = calloc(it->n_ranges ? it->n_ranges : 1, sizeof(int32_t));
        c.rver = calloc(it->n_ranges ? it->n_ranges : 1, sizeof(uint64_t));
        c.cache = calloc(it->n_nodes, sizeof(val));
        c.cver = calloc(it->n_nodes, sizeof(uint64_t));
        int64_t lo = total * tid / nt, hi = total * (tid + 1) / nt;
        int32_t cur[16];
        int64_t rem = lo;
        for (int l = nl - 1; l >= 0; l--) { cur[l] = (int32_t)(rem % lsize[l]); rem /= lsize[l]; }
        for (int l = 0; l < nl; l++) { c.rval[lslots[l]] = cur[l]; c.rver[lslots[l]] = 1; }
        for (int64_t g = lo; g < hi; g++) {
            val v = eval(&c, body);
            const node *bn = &it->nodes[body];
            int body_is_float = (bn->cls == C_F32 || bn->cls == C_F16);
            if (out_dt == DT_F16 || out_dt == DT_BF16 || (out_dt == DT_F32 && !body_is_float)) {
                float fv = as_f(bn, v);
                if (out_dt == DT_F16) fv = f16_round_f(fv);          /* narrowing at the store */
                else if (out_dt == DT_BF16) fv = bf16_trunc(fv);     /* bitcast & 0xFFFF0000, codegen/wgsl.go:228-229 */
                memcpy(&out[g], &fv, 4);
            } else {
                out[g] = v;
            }
            for (int l = nl - 1; l >= 0; l--) {
                cur[l]++; c.rver[lslots[l]]++;
                if (cur[l] < lsize[l]) { c.rval[lslots[l]] = cur[l]; break; }
                cur[l] = 0; c.rval[lslots[l]] = 0;
            }
        }
        free(c.rval); free(c.rver); free(c.cache); free(c.cver);
    }
    return failed;
}

/* ── public entry points (bound with ctypes by the tests and the bench's cpu_baseline leg) ── */
orc *orc_load(const uint8_t *blob, size_t len) {
    orc *o = calloc(1, sizeof(orc));
    if (parse(o, blob, len)) return o;
    for (int i = 0; i < o->n_items; i++) analyse(&o->items[i]);
    return o;
}
const char *orc_error(const orc *o) { return o->err; }
int orc_num_items(const orc *o) { return o->n_items; }

/* data arrives as float32 whatever the storage dtype and is quantised to it (backend/webgpu/executor.go:161-179) */
int orc_set_input(orc *o, uint32_t id, int dtype, const float *data, int64_t n) {
    buffer *b = get_buf(o, id, dtype, n);
    b->dtype = dtype;
#pragma omp parallel for schedule(static) if (n > (1 << 16))
    for (int64_t i = 0; i < n; i++) {
        if (dtype == DT_F16) b->data[i].f = f16_round_f(data[i]);
        else if (dtype == DT_BF16) b->data[i].f = bf16_trunc(data[i]);
        else b->data[i].f = data[i];     /* non-float buffers travel bit-reinterpreted */
    }
    return 0;
}
int orc_bind(orc *o, const char *name, int64_t v) {
    for (int b = 0; b < o->n_bind; b++) if (!strcmp(o->bind_name[b], name)) { o->bind_val[b] = v; return 0; }
    if (o->n_bind == 16) return 1;
    snprintf(o->bind_name[o->n_bind], 64, "%s", name); o->bind_val[o->n_bind++] = v;
    return 0;
}
int orc_run(orc *o, int threads) {
    if (o->err[0]) return 1;
    for (int i = 0; i < o->n_items; i++) if (run_item(o, &o->items[i], threads)) return 1;
    return 0;
}
int orc_run_item(orc *o, int i, int threads) {
    if (o->err[0] || i < 0 || i >= o->n_items) return 1;
    return run_item(o, &o->items[i], threads);
}
/* Value of the STORE body of item i, narrowed as the store narrows it, at the given flat output
 * positions (row-major over the kernel's loop ranges, codegen/lower.go:196-222), without touching
 * the output buffer.  A contraction with K terms then costs n*K instead of M*N*K, which lets a
 * benchmark-size kernel be compared on a few thousand outputs.  Every input buffer must hold data
 * (orc_set_input, or an earlier kernel).  Positions should arrive sorted: sub-expressions that do
 * not read the ranges that changed are re-used, exactly as in a full run.  `noise_sigma`, when not
 * NULL, receives for each position the modelled standard deviation of the difference between two
 * valid evaluations of the kernel (see the header). */
int orc_run_item_sampled(orc *o, int i, const int64_t *flat, int64_t n, float *out, double *noise_sigma, int threads) {
    if (o->err[0] || i < 0 || i >= o->n_items) return 1;
    const item *it = &o->items[i];
    if (it->n_nodes == 0) { snprintf(o->err, sizeof o->err, "oracle: item without AST"); return 1; }
    const node *sink = &it->nodes[it->n_nodes - 1];
    if (sink->op != OP_SINK) { snprintf(o->err, sizeof o->err, "oracle: last node is not SINK"); return 1; }
    const node *end = &it->nodes[sink->src[0]];
    const node *store = &it->nodes[end->src[0]];
    int body = store->src[1];
    int lslots[16], nl = 0; int64_t lsize[16];
    ectx proto; memset(&proto, 0, sizeof proto); proto.o = o; proto.it = it;
    for (int s = 1; s < end->nsrc; s++) {
        const node *r = &it->nodes[end->src[s]];
        if (r->op == OP_RANGE && (r->flags & 7) != 1 && nl < 16) { lslots[nl] = r->range_slot; lsize[nl] = range_bound(&proto, r); nl++; }
    }
    int64_t total = 1; for (int l = 0; l < nl; l++) total *= lsize[l];
    for (int64_t k = 0; k < n; k++) if (flat[k] < 0 || flat[k] >= total) { snprintf(o->err, sizeof o->err, "oracle: sampled position outside the output"); return 1; }
    val *bufdata[64]; int64_t bufelems[64]; int64_t strides[64][8];
    if (it->n_bufs > 64) { snprintf(o->err, sizeof o->err, "oracle: too many buffers"); return 1; }
    val dummy; dummy.u = 0;
    for (int b = 0; b < it->n_bufs; b++) {
        const bufdesc *bd = &it->bufs[b];
        if (b == 0) { bufdata[0] = &dummy; bufelems[0] = 0; }     /* the body never reads its own output */
        else {
            buffer *bf = find_buf(o, bd->id);
            if (!bf) { snprintf(o->err, sizeof o->err, "oracle: input buffer %u has no data", bd->id); return 1; }
            bufdata[b] = bf->data; bufelems[b] = bf->elems;
        }
        int64_t st = 1;
        for (int d = bd->rank - 1; d >= 0; d--) { strides[b][d] = st; st *= (bd->shape[d] ? bd->shape[d] : 1); }
    }
    int out_dt = it->bufs[0].dtype;
    int nthreads = threads > 0 ? threads : 1;
    if (n < 8) nthreads = 1;
#pragma omp parallel num_threads(nthreads)
    {
#ifdef _OPENMP
        int tid = omp_get_thread_num(), nt = omp_get_num_threads();
#else
        int tid = 0, nt = 1;
#endif
        ectx c = proto;
        c.bufdata = bufdata; c.bufelems = bufelems; c.strides = strides;
        c.rval = calloc(it->n_ranges ? it->n_ranges : 1, sizeof(int32_t));
        c.rver = calloc(it->n_ranges ? it->n_ranges : 1, sizeof(uint64_t));
        c.cache = calloc(it->n_nodes, sizeof(val));
        c.cver = calloc(it->n_nodes, sizeof(uint64_t));
        c.nvar = noise_sigma ? calloc(it->n_nodes, sizeof(double)) : NULL;
        c.qvar = noise_sigma ? calloc(it->n_nodes, sizeof(double)) : NULL;
        for (int l = 0; l < nl; l++) { c.rval[lslots[l]] = -1; c.rver[lslots[l]] = 1; }
        const node *bn = &it->nodes[body];
        int body_is_float = (bn->cls == C_F32 || bn->cls == C_F16);
        int64_t lo = n * tid / nt, hi = n * (tid + 1) / nt;
        for (int64_t k = lo; k < hi; k++) {
            int64_t rem = flat[k];
            for (int l = nl - 1; l >= 0; l--) {
                int32_t v = (int32_t)(rem % lsize[l]); rem /= lsize[l];
                if (c.rval[lslots[l]] != v) { c.rval[lslots[l]] = v; c.rver[lslots[l]]++; }
            }
            val v = eval(&c, body);
            const int tracked = c.nvar && body_is_float && bn->op != OP_CONST && bn->op != OP_RANGE;
            double var = tracked ? c.nvar[body] : 0.0, qvr = tracked ? c.qvar[body] : 0.0;
            if (out_dt == DT_F16 || out_dt == DT_BF16 || (out_dt == DT_F32 && !body_is_float)) {
                float fv = as_f(bn, v);
                if (out_dt == DT_F16) { fv = f16_round_f(fv); if (var > 0.0) { qvr += f16_tip_var(var, (double)fv); var = 0.0; } }
                else if (out_dt == DT_BF16) fv = bf16_trunc(fv);
                out[k] = fv;
            } else memcpy(&out[k], &v, 4);
            if (noise_sigma) noise_sigma[k] = sqrt(var + qvr);
        }
        free(c.rval); free(c.rver); free(c.cache); free(c.cver); free(c.nvar); free(c.qvar);
    }
    return 0;
}
int64_t orc_buffer_elems(orc *o, uint32_t id) { buffer *b = find_buf(o, id); return b ? b->elems : -1; }
int orc_get_buffer(orc *o, uint32_t id, float *out, int64_t n) {
    buffer *b = find_buf(o, id);
    if (!b || n > b->elems) return 1;
    memcpy(out, b->data, (size_t)n * 4);
    return 0;
}
void orc_free(orc *o) {
    if (!o) return;
    for (int i = 0; i < o->n_items; i++) {
        item *it = &o->items[i];
        for (int k = 0; k < it->n_nodes; k++) free(it->nodes[k].dep);
        for (int s = 0; s < it->n_sym; s++) free(it->sym[s]);
        free(it->nodes); free(it->bufs); free(it->sym); free(it->range_node); free(it->srcpool);
    }
    for (int i = 0; i < o->n_buf; i++) free(o->bufs[i].data);
    free(o->items); free(o->bufs); free(o);
}
/* host-side conversions exposed for the dtype known-answer tests */
uint16_t orc_f32_to_f16_bits(float f) {
    val v; v.f = f; uint32_t s = (v.u >> 31) << 15;
    if (f != f) {                                  /* NaN stays NaN: shifted payload, never zero (uop/dtype.go:404-412) */
        uint32_t m = (v.u & 0x7FFFFF) >> 13;
        return (uint16_t)(s | 0x7C00 | (m ? m : 1));
    }
    float r = f16_round_f(f);
    if (isinf(r)) return (uint16_t)(s | 0x7C00);
    if (r == 0) return (uint16_t)s;
    int e; double m = frexp(fabs((double)r), &e);  /* |r| = m*2^e, m in [0.5,1) */
    int lead = e - 1;
    if (lead < -14) return (uint16_t)(s | (uint32_t)ldexp(fabs((double)r), 24));
    return (uint16_t)(s | ((uint32_t)(lead + 15) << 10) | ((uint32_t)ldexp(m, 11) & 0x3FF));
}
float orc_f16_round(float f) { return f16_round_f(f); }
