// Lowers one scheduled kernel (SINK → END → STORE(INDEX(PARAM0, ranges), body)) to CUDA C
// for sm_100a.  What the reference does in codegen/lower.go + codegen/wgsl.go for WGSL, redone
// for a machine with 32-wide warps, shared memory and 128-bit global accesses:
//
//  * index arithmetic is canonicalised first.  The scheduler emits reshape/permute/pad as
//    unsimplified i32 div/mod chains (schedule/index.go:231-293); here every integer node is
//    folded into an affine form over the loop variables using their bounds, so that
//    ((r0*I + r1) / I) % B becomes r0.  Strides recovered this way drive the choice between
//    vector and scalar accesses and the thread layout of reductions;
//  * a kernel without REDUCE becomes one thread per V consecutive outputs with 128-bit loads and
//    stores when alignment is provable, scalar otherwise;
//  * REDUCE nodes (several per kernel are allowed, codegen/lower.go:654-719) are evaluated by
//    groups of L threads: lanes stride the flattened reduce space, partial accumulators are
//    combined by warp shuffles and, across warps, shared memory.  L = 1 reproduces the reference's
//    serial ascending loop exactly;
//  * a single long REDUCE feeding few outputs is split over many blocks: a partials kernel writes
//    f32 partials to scratch memory, a finish kernel combines them in ascending order and applies
//    the epilogue, so results do not depend on scheduling;
//  * loads whose index cannot be proven inside the buffer (the guarded load of a PAD,
//    schedule/index.go:101-134) are clamped: WGSL defines out-of-range reads, CUDA does not;
//  * guards that compare a SMALL static range with constants are decided while generating: a
//    convolution reaches the device as a sum of K padded slices, each live for exactly one value of
//    the patch index k (tensor/nn/nn.go:256-276), i.e. K selects per multiply.  A reduce loop over
//    such a range is emitted once per value of the range, an output range of that kind becomes a
//    switch over its values, and in every copy the guards fold to true or false — what is left is the
//    one live slice, a direct convolution with the bounds checks of its padding and no im2col buffer.
//
// Arithmetic follows codegen/wgsl.go:240-447: f16 values use native half add/sub/mul outside
// reductions and are widened to f32 inside an f16 reduction with a single narrowing at the end
// (codegen/lower.go:158-171, 698-716); bf16 lives in 32-bit slots and is truncated at the store;
// reduce identities are 0, 1 and -FLT_MAX; infinite literals clamp to +-FLT_MAX.
#include "codegen.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>

namespace anl {

uint64_t structure_hash(const Item& item) {
    uint64_t h = 1469598103934665603ull;
    for (const Node& n : item.nodes) {
        int64_t rec[5] = {n.op, n.dtype, n.flags, (int64_t)n.aux, n.arg};
        h = fnv1a(rec, sizeof rec, h);
        for (int s : n.src) h = fnv1a(&s, sizeof s, h);
    }
    for (const BufDesc& b : item.bufs) {
        int64_t rec[2] = {b.dtype, (int64_t)b.shape.size()};
        h = fnv1a(rec, sizeof rec, h);
        for (int64_t s : b.shape) h = fnv1a(&s, sizeof s, h);
    }
    for (const std::string& s : item.sym_vars) h = fnv1a(s.data(), s.size(), h);
    return h;
}

namespace {

enum Cls { CF32, CF16, CINT, CUINT, CBOOL };

Cls dtype_cls(int dt) {
    switch (dt) {
        case DT_F16: return CF16;
        case DT_BOOL: return CBOOL;
        case DT_F32: case DT_BF16: case DT_F64: case DT_VOID: return CF32;
        case DT_U8: case DT_U16: case DT_U32: case DT_U64: return CUINT;
        default: return CINT;
    }
}
const char* cls_ctype(Cls c) {
    switch (c) { case CF32: return "float"; case CF16: return "__half"; case CINT: return "int"; case CUINT: return "unsigned"; default: return "bool"; }
}
const char* buf_ctype(int dt) {
    switch (dtype_cls(dt)) { case CF16: return "__half"; case CF32: return "float"; case CINT: return "int"; default: return "unsigned"; }
}

// ── affine forms over loop variables ────────────────────────────────────────────────────────────
struct Lin {
    int64_t c = 0;
    std::vector<std::pair<int, int64_t>> t;   // (atom, coefficient), sorted by atom
    bool is_const() const { return t.empty(); }
};

struct Atom {
    enum Kind { RANGE, DIV, MOD, OPAQUE } kind = RANGE;
    int node = -1;        // RANGE / OPAQUE: node index
    Lin inner;            // DIV / MOD
    int64_t d = 1;
    int64_t lo = 0, hi = 0;
};

const int64_t UNBOUNDED = (int64_t)1 << 40;

struct Gen {
    const Item& it;
    const CodegenOpts& opts;
    std::string err;

    int n;                                 // nodes
    int sink, end, store, body, dst;
    std::vector<int> loop_ranges;          // node indices, END order, loop axis
    std::vector<int> all_ranges;           // every RANGE node
    std::vector<int> range_slot;           // node → slot or -1
    std::vector<std::vector<bool>> dep;    // node × range slot
    std::vector<bool> widen;
    std::vector<int> reduces;              // REDUCE nodes in node order
    bool has_sym = false;

    // ranges that hold one known value while the code around them is being rendered (enumeration)
    std::map<int, int64_t> fixed_range;
    void fix_range(int r, int64_t v) { fixed_range[r] = v; lin_memo.clear(); }
    void unfix_range(int r) { fixed_range.erase(r); lin_memo.clear(); }

    std::vector<Atom> atoms;
    std::map<std::string, int> atom_key;
    std::vector<int> range_atom;           // node → atom
    std::map<int, Lin> lin_memo;

    explicit Gen(const Item& i, const CodegenOpts& o) : it(i), opts(o) {}

    const Node& N(int i) const { return it.nodes[i]; }
    Cls cls(int i) const { Cls c = dtype_cls(N(i).dtype); return (c == CF16 && widen[i]) ? CF32 : c; }

    bool fail(const std::string& m) { if (err.empty()) err = m; return false; }

    // ── structure ──────────────────────────────────────────────────────────────────────────────
    bool analyse() {
        n = (int)it.nodes.size();
        if (n == 0) return fail("codegen: item has no AST");
        sink = n - 1;
        if (N(sink).op != OP_SINK || N(sink).src.empty()) return fail("codegen: last node is not a SINK");
        end = N(sink).src[0];
        if (N(end).op != OP_END || N(end).src.empty()) return fail("codegen: SINK source is not END");
        store = N(end).src[0];
        if (N(store).op != OP_STORE || N(store).src.size() != 2) return fail("codegen: END source is not STORE");
        dst = N(store).src[0];
        body = N(store).src[1];
        range_slot.assign(n, -1);
        for (int i = 0; i < n; i++)
            if (N(i).op == OP_RANGE) { range_slot[i] = (int)all_ranges.size(); all_ranges.push_back(i); if (N(i).symbolic()) has_sym = true; }
        for (size_t s = 1; s < N(end).src.size(); s++) {
            int r = N(end).src[s];
            if (N(r).op == OP_RANGE && N(r).axis() != 1) loop_ranges.push_back(r);
        }
        int nr = (int)all_ranges.size();
        dep.assign(n, std::vector<bool>(nr, false));
        widen.assign(n, false);
        for (int i = 0; i < n; i++) {
            const Node& nd = N(i);
            if (nd.op == OP_RANGE) dep[i][range_slot[i]] = true;
            for (int s : nd.src) for (int r = 0; r < nr; r++) if (dep[s][r]) dep[i][r] = true;
            if (nd.op == OP_REDUCE) {
                reduces.push_back(i);
                for (size_t s = 1; s < nd.src.size(); s++) if (N(nd.src[s]).op == OP_RANGE) dep[i][range_slot[nd.src[s]]] = false;
            }
        }
        // only nodes reachable from the body matter
        std::vector<bool> live(n, false);
        std::function<void(int)> mark = [&](int i) { if (live[i]) return; live[i] = true; for (int s : N(i).src) mark(s); };
        mark(body);
        std::vector<int> lr;
        for (int r : reduces) if (live[r]) lr.push_back(r);
        reduces = lr;
        std::function<void(int)> mw = [&](int i) {
            if (widen[i]) return;
            widen[i] = true;
            if (N(i).op == OP_INDEX) return;
            for (int s : N(i).src) mw(s);
        };
        for (int r : reduces) if (N(r).dtype == DT_F16) mw(N(r).src[0]);
        // atoms for ranges
        range_atom.assign(n, -1);
        for (int r : all_ranges) {
            Atom a; a.kind = Atom::RANGE; a.node = r; a.lo = 0;
            a.hi = N(r).symbolic() ? UNBOUNDED : std::max<int64_t>(N(r).arg - 1, 0);
            range_atom[r] = (int)atoms.size();
            atoms.push_back(a);
        }
        return true;
    }

    // ── guards decided at generation time ─────────────────────────────────────────────────────
    std::set<int> enum_reduce;              // REDUCE nodes whose single small range is emitted value by value
    std::vector<int> enum_out;              // small output ranges turned into a switch over their values

    // Which ranges an integer comparison reads once its operands are in canonical affine form (the
    // scheduler's reshape chains mention every range of the kernel; (n*7056 + hw*9 + k) % 9 is k).
    // False when something other than ranges decides it.
    bool guard_ranges(int i, std::vector<bool>& reads) {
        const Node& nd = N(i);
        if ((nd.op != OP_CMPLT && nd.op != OP_CMPEQ && nd.op != OP_CMPNE) || !is_live(i)) return false;
        if (!is_intlike(nd.src[0]) || !is_intlike(nd.src[1])) return false;
        Lin d = ladd(lin(nd.src[0]), lin(nd.src[1]), -1);
        std::function<bool(const Lin&)> only_ranges = [&](const Lin& l) {
            for (auto& t : l.t) { const Atom& a = atoms[t.first]; if (a.kind == Atom::OPAQUE) return false; if (a.kind != Atom::RANGE && !only_ranges(a.inner)) return false; }
            return true;
        };
        if (!only_ranges(d)) return false;
        reads.assign(all_ranges.size(), false);
        bool any = false;
        for (size_t r = 0; r < all_ranges.size(); r++) if (lin_reads(d, all_ranges[r])) { reads[r] = true; any = true; }
        return any;
    }
    // Fraction of the value combinations of `ranges` for which guard `g` holds (1 where it does not fold).
    double guard_truth(int g, const std::vector<int>& ranges) {
        int64_t combos = 1;
        for (int r : ranges) combos *= N(r).arg;
        int64_t yes = 0;
        const Node& nd = N(g);
        for (int64_t cs = 0; cs < combos; cs++) {
            int64_t rem = cs;
            for (int e = (int)ranges.size() - 1; e >= 0; e--) { fixed_range[ranges[e]] = rem % N(ranges[e]).arg; rem /= N(ranges[e]).arg; }
            lin_memo.clear();
            Lin d = ladd(lin(nd.src[0]), lin(nd.src[1]), -1);
            bool t = true;
            if (d.is_const()) t = nd.op == OP_CMPLT ? d.c < 0 : nd.op == OP_CMPEQ ? d.c == 0 : d.c != 0;
            if (t) yes++;
        }
        for (int r : ranges) fixed_range.erase(r);
        lin_memo.clear();
        return (double)yes / (double)combos;
    }

    // Decides which small ranges are enumerated.  A set of ranges qualifies when at least four guards
    // read exactly that set and, averaged over the set's value combinations, those guards hold less
    // than three times out of four: they select slices (a patch index equal to a constant) instead of
    // merely trimming a border (a padded row, true almost everywhere).
    void plan_enumeration() {
        enum_reduce.clear(); enum_out.clear();
        if (has_sym || opts.debug_bounds) return;
        const size_t nr = all_ranges.size();
        std::map<std::vector<int>, std::vector<int>> by_set;       // ranges read (node indices, sorted) -> guards
        std::vector<bool> reads;
        for (int i = 0; i < n; i++) {
            if (!guard_ranges(i, reads)) continue;
            std::vector<int> key; int64_t prod = 1; bool ok = true;
            for (size_t r = 0; r < nr; r++) if (reads[r]) {
                const Node& rn = N(all_ranges[r]);
                if (rn.symbolic() || rn.arg < 2 || rn.arg > 128) { ok = false; break; }
                key.push_back(all_ranges[r]); prod *= rn.arg;
            }
            if (ok && !key.empty() && prod <= 128) by_set[key].push_back(i);
        }
        struct Cand { std::vector<int> ranges; double score; };
        std::vector<Cand> outs;
        for (auto& kv : by_set) {
            if (kv.second.size() < 4) continue;
            double frac = 0;
            for (int g : kv.second) frac += guard_truth(g, kv.first);
            frac /= (double)kv.second.size();
            if (frac > 0.75) continue;
            // a single reduce range: value-by-value loop of the REDUCE that owns it
            if (kv.first.size() == 1 && N(kv.first[0]).axis() == 1) {
                for (int red : reduces) {
                    std::vector<int> rr;
                    for (size_t s2 = 1; s2 < N(red).src.size(); s2++) if (N(N(red).src[s2]).op == OP_RANGE) rr.push_back(N(red).src[s2]);
                    if (rr.size() == 1 && rr[0] == kv.first[0]) enum_reduce.insert(red);
                }
                continue;
            }
            bool all_out = true;
            for (int r : kv.first) if (std::find(loop_ranges.begin(), loop_ranges.end(), r) == loop_ranges.end()) all_out = false;
            if (all_out) outs.push_back(Cand{kv.first, (double)kv.second.size() * (1.0 - frac)});
        }
        std::sort(outs.begin(), outs.end(), [](const Cand& x, const Cand& y) { return x.score > y.score; });
        std::set<int> chosen; int64_t prod = 1;
        for (auto& c : outs) {
            int64_t p2 = prod;
            for (int r : c.ranges) if (!chosen.count(r)) p2 *= N(r).arg;
            if (p2 > 128) continue;
            for (int r : c.ranges) chosen.insert(r);
            prod = p2;
        }
        for (int r : loop_ranges) if (chosen.count(r)) enum_out.push_back(r);
    }

    // forget what was rendered inside reduce loop `red` (ctx == red), so that it can be rendered again
    void forget_loop(int red) {
        for (auto it = memo.begin(); it != memo.end();) { if (it->first.second == red) it = memo.erase(it); else ++it; }
        loop[red] = Block();
    }

    bool depends_on_reduce(int node, int red) const {
        const Node& r = N(red);
        for (size_t s = 1; s < r.src.size(); s++) {
            int rn = r.src[s];
            if (N(rn).op == OP_RANGE && dep[node][range_slot[rn]]) return true;
        }
        return false;
    }

    // ── Lin algebra ────────────────────────────────────────────────────────────────────────────
    static Lin lconst(int64_t c) { Lin l; l.c = c; return l; }
    Lin latom(int a) const { Lin l; l.t.push_back({a, 1}); return l; }
    static Lin ladd(const Lin& a, const Lin& b, int64_t sb = 1) {
        Lin r; r.c = a.c + sb * b.c;
        size_t i = 0, j = 0;
        while (i < a.t.size() || j < b.t.size()) {
            if (j == b.t.size() || (i < a.t.size() && a.t[i].first < b.t[j].first)) r.t.push_back(a.t[i++]);
            else if (i == a.t.size() || b.t[j].first < a.t[i].first) { r.t.push_back({b.t[j].first, sb * b.t[j].second}); j++; }
            else { int64_t c = a.t[i].second + sb * b.t[j].second; if (c) r.t.push_back({a.t[i].first, c}); i++; j++; }
        }
        return r;
    }
    static Lin lscale(const Lin& a, int64_t k) {
        Lin r; if (k == 0) return r;
        r.c = a.c * k; for (auto& p : a.t) r.t.push_back({p.first, p.second * k});
        return r;
    }
    int64_t llo(const Lin& l) const {
        int64_t v = l.c;
        for (auto& p : l.t) { int64_t b = p.second > 0 ? atoms[p.first].lo : atoms[p.first].hi; if (std::llabs(b) >= UNBOUNDED) return p.second > 0 ? (b < 0 ? -UNBOUNDED : v) : -UNBOUNDED; v += p.second * b; }
        return v;
    }
    int64_t lhi(const Lin& l) const {
        int64_t v = l.c;
        for (auto& p : l.t) { int64_t b = p.second > 0 ? atoms[p.first].hi : atoms[p.first].lo; if (std::llabs(b) >= UNBOUNDED) return UNBOUNDED; v += p.second * b; }
        return v;
    }
    std::string lkey(const Lin& l) const {
        std::ostringstream o; o << l.c;
        for (auto& p : l.t) o << "+" << p.second << "*a" << p.first;
        return o.str();
    }
    int make_atom(Atom::Kind k, const Lin& inner, int64_t d, int64_t lo, int64_t hi, int node = -1) {
        std::ostringstream key;
        key << (int)k << ":" << node << ":" << d << ":" << lkey(inner);
        auto f = atom_key.find(key.str());
        if (f != atom_key.end()) return f->second;
        Atom a; a.kind = k; a.inner = inner; a.d = d; a.lo = lo; a.hi = hi; a.node = node;
        atoms.push_back(a);
        atom_key[key.str()] = (int)atoms.size() - 1;
        return (int)atoms.size() - 1;
    }
    // split e = d*q + r with every coefficient of q*d a multiple of d and 0 <= const(r) < d
    void split(const Lin& e, int64_t d, Lin& q, Lin& r) const {
        q = Lin(); r = Lin();
        int64_t cq = e.c / d, cr = e.c % d;
        if (cr < 0) { cr += d; cq -= 1; }
        q.c = cq; r.c = cr;
        for (auto& p : e.t) {
            if (p.second % d == 0) q.t.push_back({p.first, p.second / d});
            else r.t.push_back(p);
        }
    }
    Lin ldiv(const Lin& e, int64_t d) {
        if (d == 1) return e;
        if (e.is_const()) return lconst(e.c / d);
        int64_t lo = llo(e), hi = lhi(e);
        if (d <= 0 || lo < 0) return latom(make_atom(Atom::DIV, e, d, -UNBOUNDED, UNBOUNDED));
        Lin q, r; split(e, d, q, r);
        if (r.is_const()) return q;                       // r.c in [0,d)
        int64_t rlo = llo(r), rhi = lhi(r);
        if (rlo >= 0 && rhi < d) return q;
        if (rlo >= 0) return ladd(q, latom(make_atom(Atom::DIV, r, d, rlo / d, rhi >= UNBOUNDED ? UNBOUNDED : rhi / d)));
        return latom(make_atom(Atom::DIV, e, d, lo / d, hi >= UNBOUNDED ? UNBOUNDED : hi / d));
    }
    Lin lmod(const Lin& e, int64_t m) {
        if (m == 1) return lconst(0);
        if (e.is_const() && m > 0) return lconst(e.c % m);
        int64_t lo = llo(e), hi = lhi(e);
        if (m <= 0 || lo < 0) return latom(make_atom(Atom::MOD, e, m, -UNBOUNDED, UNBOUNDED));
        if (hi < m) return e;
        Lin q, r; split(e, m, q, r);
        if (r.is_const()) return lconst(r.c);
        int64_t rlo = llo(r), rhi = lhi(r);
        if (rlo >= 0 && rhi < m) return r;
        if (rlo >= 0) return latom(make_atom(Atom::MOD, r, m, 0, std::min(m - 1, rhi)));
        return latom(make_atom(Atom::MOD, e, m, 0, m - 1));
    }

    bool is_intlike(int i) const { Cls c = dtype_cls(N(i).dtype); return c == CINT || c == CUINT; }

    Lin lin(int i) {
        auto f = lin_memo.find(i);
        if (f != lin_memo.end()) return f->second;
        const Node& nd = N(i);
        Lin r;
        switch (nd.op) {
            case OP_CONST: r = lconst(nd.arg); break;
            case OP_RANGE: { auto fx = fixed_range.find(i); r = fx != fixed_range.end() ? lconst(fx->second) : latom(range_atom[i]); break; }
            case OP_ADD: r = ladd(lin(nd.src[0]), lin(nd.src[1])); break;
            case OP_SUB: r = ladd(lin(nd.src[0]), lin(nd.src[1]), -1); break;
            case OP_NEG: r = lscale(lin(nd.src[0]), -1); break;
            case OP_MUL: {
                Lin a = lin(nd.src[0]), b = lin(nd.src[1]);
                if (b.is_const()) r = lscale(a, b.c);
                else if (a.is_const()) r = lscale(b, a.c);
                else r = latom(make_atom(Atom::OPAQUE, Lin(), 1, -UNBOUNDED, UNBOUNDED, i));
                break;
            }
            case OP_IDIV: {
                Lin b = lin(nd.src[1]);
                if (b.is_const() && b.c > 0) r = ldiv(lin(nd.src[0]), b.c);
                else r = latom(make_atom(Atom::OPAQUE, Lin(), 1, -UNBOUNDED, UNBOUNDED, i));
                break;
            }
            case OP_MOD: {
                Lin b = lin(nd.src[1]);
                if (b.is_const() && b.c > 0) r = lmod(lin(nd.src[0]), b.c);
                else r = latom(make_atom(Atom::OPAQUE, Lin(), 1, -UNBOUNDED, UNBOUNDED, i));
                break;
            }
            default: r = latom(make_atom(Atom::OPAQUE, Lin(), 1, -UNBOUNDED, UNBOUNDED, i)); break;
        }
        lin_memo[i] = r;
        return r;
    }

    // does the affine form read loop variable `range_node`, directly or through an atom?
    bool lin_reads(const Lin& l, int range_node) const {
        for (auto& p : l.t) {
            const Atom& a = atoms[p.first];
            if (a.kind == Atom::RANGE) { if (a.node == range_node) return true; }
            else if (a.kind == Atom::OPAQUE) { if (dep[a.node][range_slot[range_node]]) return true; }
            else if (lin_reads(a.inner, range_node)) return true;
        }
        return false;
    }
    // coefficient of a loop variable when it appears only as a direct term; ok=false otherwise
    int64_t lin_coef(const Lin& l, int range_node, bool& ok) const {
        int64_t c = 0; ok = true;
        for (auto& p : l.t) {
            const Atom& a = atoms[p.first];
            if (a.kind == Atom::RANGE && a.node == range_node) c = p.second;
            else if (a.kind != Atom::RANGE) {
                Lin one; one.t.push_back({p.first, 1});
                if (lin_reads(one, range_node)) ok = false;
            }
        }
        return c;
    }

    // ── flat load index ────────────────────────────────────────────────────────────────────────
    Lin flat_index(int index_node) {
        const Node& nd = N(index_node);
        int p = (int)N(nd.src[0]).arg;
        int ndim = (int)nd.src.size() - 1;
        if (ndim == 0) return lconst(0);
        if (ndim == 1) return lin(nd.src[1]);
        const std::vector<int64_t>& sh = it.bufs[p].shape;
        std::vector<int64_t> st(ndim, 1);
        for (int d = ndim - 2; d >= 0; d--) st[d] = (d + 1 < (int)sh.size()) ? st[d + 1] * (sh[d + 1] ? sh[d + 1] : 1) : 1;
        Lin r;
        for (int d = 0; d < ndim; d++) r = ladd(r, lscale(lin(nd.src[1 + d]), st[d]));
        return r;
    }
    bool in_bounds(const Lin& f, int param) const {
        const BufDesc& b = it.bufs[param];
        int64_t lo = llo(f), hi = lhi(f);
        if (!b.symbolic()) return lo >= 0 && hi < b.elems(0);
        // symbolic outermost dim: need coef(sym range) == trailing and the rest inside one row
        int64_t tr = b.trailing();
        Lin rest; rest.c = f.c; bool found = false;
        for (auto& p : f.t) {
            const Atom& a = atoms[p.first];
            if (a.kind == Atom::RANGE && N(a.node).symbolic()) { if (p.second != tr) return false; found = true; }
            else rest.t.push_back(p);
        }
        return found && llo(rest) >= 0 && lhi(rest) < tr;
    }

    // ── emission ───────────────────────────────────────────────────────────────────────────────
    struct Block { std::string code; int indent = 1; };
    Block top;                              // statements outside reduce loops
    std::map<int, Block> loop;              // REDUCE node → statements inside its loop
    std::map<std::pair<int, int>, std::string> memo;   // (node, ctx) → expression
    int vec_range = -1;                     // loop variable unrolled by the vector path, or -1
    std::map<int, std::string> vec_load;    // INDEX node → array name holding V preloaded values
    int finish_reduce = -1;                 // finish kernel: this REDUCE reads partials instead
    std::string reduce_combine_mode;        // set by the kernel builder
    int lanes = 1, touts = 1, threads = 256; bool rc_layout = true;

    Block prelude;                          // vector path: statements that must precede the unrolled loop
    Block* cur_top = nullptr;
    std::map<int, std::vector<bool>> atom_dep_memo;

    Block& T() { return cur_top ? *cur_top : top; }

    void stmt(int ctx, const std::string& s) {
        Block& b = ctx < 0 ? (cur_top ? *cur_top : top) : loop[ctx];
        b.code += std::string((ctx < 0 ? 1 : 2) * 2, ' ') + s + "\n";
    }

    // loop variables an atom reads, as a bitset over range slots
    const std::vector<bool>& atom_dep(int ai) {
        auto f = atom_dep_memo.find(ai);
        if (f != atom_dep_memo.end()) return f->second;
        std::vector<bool> d(all_ranges.size(), false);
        const Atom& a = atoms[ai];
        if (a.kind == Atom::RANGE) d[range_slot[a.node]] = true;
        else if (a.kind == Atom::OPAQUE) d = dep[a.node];
        else for (auto& p : a.inner.t) { const std::vector<bool>& s = atom_dep(p.first); for (size_t r = 0; r < d.size(); r++) if (s[r]) d[r] = true; }
        return atom_dep_memo[ai] = d;
    }
    bool atom_in_reduce(int ai, int red) {
        const std::vector<bool>& d = atom_dep(ai);
        const Node& r = N(red);
        for (size_t s = 1; s < r.src.size(); s++) if (N(r.src[s]).op == OP_RANGE && d[range_slot[r.src[s]]]) return true;
        return false;
    }
    // DIV / MOD atoms get a named temporary in the outermost context that can hold them
    std::string atom_name(int ai, int ctx) {
        if (ctx >= 0 && !atom_in_reduce(ai, ctx)) ctx = -1;
        auto key = std::make_pair(-(ai + 1), ctx);
        auto f = memo.find(key);
        if (f != memo.end()) return f->second;
        const Atom& a = atoms[ai];
        std::string name = "a" + std::to_string(ai);
        stmt(ctx, "const int " + name + " = " + render(a.inner, ctx) + (a.kind == Atom::DIV ? " / " : " % ") + std::to_string(a.d) + ";");
        memo[key] = name;
        return name;
    }

    std::string range_name(int r) const {
        auto fx = fixed_range.find(r);
        if (fx != fixed_range.end()) return std::to_string(fx->second);
        std::string s = "r" + std::to_string(N(r).aux);
        return r == vec_range ? "(" + s + " + u)" : s;
    }

    std::string render(const Lin& l, int ctx) {
        if (l.is_const()) return l.c < 0 ? "(" + std::to_string(l.c) + ")" : std::to_string(l.c);
        std::string s = "(";
        bool first = true;
        for (auto& p : l.t) {
            const Atom& a = atoms[p.first];
            std::string v;
            switch (a.kind) {
                case Atom::RANGE: v = range_name(a.node); break;
                case Atom::DIV: case Atom::MOD: v = atom_name(p.first, ctx); break;
                case Atom::OPAQUE: v = opaque_int(a.node, ctx); break;
            }
            int64_t c = p.second;
            if (!first) s += c < 0 ? " - " : " + ";
            else if (c < 0) s += "-";
            int64_t ac = std::llabs(c);
            s += ac == 1 ? v : v + " * " + std::to_string(ac);
            first = false;
        }
        if (l.c > 0) s += " + " + std::to_string(l.c);
        else if (l.c < 0) s += " - " + std::to_string(-l.c);
        return s + ")";
    }

    static std::string flit(double d) {
        float f = (float)d;
        if (std::isnan(f)) return "__int_as_float(0x7fc00000)";
        if (std::isinf(f)) return f < 0 ? "__int_as_float(0xff7fffff)" : "__int_as_float(0x7f7fffff)";
        char b[64]; std::snprintf(b, sizeof b, "%af", (double)f);
        return std::string(b);
    }
    static bool is_zero_lit(const std::string& e) { return e == "0x0p+0f" || e == "__float2half_rn(0x0p+0f)"; }
    // x * 1.0 is x bit for bit in IEEE arithmetic (the gradient of a sum multiplies by ones)
    bool is_float_one(int i) const {
        const Node& nd = N(i);
        if (nd.op != OP_CONST || !dt_is_float(nd.dtype)) return false;
        double d; std::memcpy(&d, &nd.arg, 8);
        return d == 1.0;
    }

    std::string const_lit(int i) {
        const Node& nd = N(i);
        if (dt_is_float(nd.dtype)) {
            double d; std::memcpy(&d, &nd.arg, 8);
            bool f16 = nd.dtype == DT_F16;
            if (f16 && std::isinf(d)) d = d < 0 ? -65504.0 : 65504.0;
            std::string f = flit(d);
            return (f16 && !widen[i]) ? "__float2half_rn(" + f + ")" : f;
        }
        if (nd.dtype == DT_BOOL) return nd.arg ? "true" : "false";
        if (nd.arg == INT32_MIN) return "(-2147483647 - 1)";
        return nd.arg < 0 ? "(" + std::to_string(nd.arg) + ")" : std::to_string(nd.arg);
    }

    // integer node that the affine engine could not absorb: plain C on its operands
    std::string opaque_int(int i, int ctx) {
        if (ctx >= 0 && !depends_on_reduce(i, ctx)) ctx = -1;
        auto key = std::make_pair(i, ctx);
        auto f = memo.find(key);
        if (f != memo.end()) return f->second;
        const Node& nd = N(i);
        std::string e;
        auto a = [&](int k) { return val(nd.src[k], ctx); };
        switch (nd.op) {
            case OP_MUL: e = "(" + a(0) + " * " + a(1) + ")"; break;
            case OP_IDIV: e = "idiv_(" + a(0) + ", " + a(1) + ")"; break;
            case OP_MOD: e = "imod_(" + a(0) + ", " + a(1) + ")"; break;
            case OP_MAX: e = "max(" + a(0) + ", " + a(1) + ")"; break;
            case OP_SHL: e = "(" + a(0) + " << (" + a(1) + " & 31))"; break;
            case OP_SHR: e = "(" + a(0) + " >> (" + a(1) + " & 31))"; break;
            case OP_AND: e = "(" + a(0) + " & " + a(1) + ")"; break;
            case OP_OR: e = "(" + a(0) + " | " + a(1) + ")"; break;
            case OP_XOR: e = "(" + a(0) + " ^ " + a(1) + ")"; break;
            case OP_WHERE: e = "(" + a(0) + " ? " + a(1) + " : " + a(2) + ")"; break;
            case OP_MULACC: e = "(" + a(0) + " + (" + a(1) + " * " + a(2) + "))"; break;
            case OP_CAST: case OP_BITCAST: e = cast_expr(i, ctx); break;
            case OP_INDEX: e = load_expr(i, ctx); break;
            case OP_REDUCE: e = reduce_expr(i); break;
            default: fail("codegen: unhandled integer op " + std::to_string(nd.op)); e = "0"; break;
        }
        std::string name = "t" + std::to_string(i);
        stmt(ctx, std::string("const ") + cls_ctype(cls(i)) + " " + name + " = " + e + ";");
        memo[key] = name;
        return name;
    }

    std::string to_float(int src, const std::string& e) {
        switch (cls(src)) { case CF32: return e; case CF16: return "__half2float(" + e + ")"; case CBOOL: return "(" + e + " ? 1.0f : 0.0f)"; default: return "(float)(" + e + ")"; }
    }
    std::string cast_expr(int i, int ctx) {
        const Node& nd = N(i);
        int s = nd.src[0];
        std::string e = val(s, ctx);
        Cls to = cls(i), from = cls(s);
        if (nd.op == OP_BITCAST) {
            if (to == from) return e;
            if (to == CF32 && (from == CINT || from == CUINT)) return "__int_as_float((int)" + e + ")";
            if ((to == CINT || to == CUINT) && from == CF32) return std::string("(") + cls_ctype(to) + ")__float_as_int(" + e + ")";
            fail("codegen: unsupported bitcast"); return "0";
        }
        if (to == from) return e;
        switch (to) {
            case CF32: return to_float(s, e);
            case CF16: return "__float2half_rn(" + to_float(s, e) + ")";
            case CBOOL: return from == CF16 ? "(__half2float(" + e + ") != 0.0f)" : from == CF32 ? "(" + e + " != 0.0f)" : "(" + e + " != 0)";
            case CINT: return from == CF16 ? "(int)__half2float(" + e + ")" : "(int)(" + e + ")";
            default: return from == CF16 ? "(unsigned)__half2float(" + e + ")" : "(unsigned)(" + e + ")";
        }
    }

    bool unroll_short_loops = false;
    int chain_vec = 1;
    std::string dp = "data";                         // name prefix of the buffer pointers
    std::map<int, std::string> chain_subst;          // row chain: parameter → register holding this row's value

    // Row-chain stages with chain_vec > 1: INDEX nodes below `root` (nested reductions excluded) that
    // sweep `sweep` with unit stride and whose address is provably a multiple of chain_vec elements
    // when the sweep variable is (16-byte aligned bases, every other term a multiple of chain_vec).
    // Each gets one wide load per chunk into a small array; load_expr then hands out array[u].
    // Returns the declarations + loads, written for a scope in which the sweep variable holds the
    // chunk's first index.
    std::string chain_wide_loads(int root, int sweep, int ctx) {
        std::string code;
        if (chain_vec <= 1 || opts.debug_bounds) return code;
        std::vector<int> stack{root}, seen_nodes;
        std::set<int> seen;
        while (!stack.empty()) {
            int j = stack.back(); stack.pop_back();
            if (!seen.insert(j).second) continue;
            const Node& nd = N(j);
            if (nd.op == OP_REDUCE && j != root) continue;
            if (nd.op == OP_INDEX) { seen_nodes.push_back(j); continue; }
            for (int c : nd.src) stack.push_back(c);
        }
        std::sort(seen_nodes.begin(), seen_nodes.end());
        const std::string V = std::to_string(chain_vec);
        for (int j : seen_nodes) {
            const Node& nd = N(j);
            if (N(nd.src[0]).op != OP_PARAM || !dep[j][range_slot[sweep]]) continue;
            int p = (int)N(nd.src[0]).arg;
            if (p <= 0 || p >= (int)it.bufs.size() || chain_subst.count(p)) continue;
            Cls bc = dtype_cls(it.bufs[p].dtype);
            if (bc != cls(j) || (bc != CF32 && bc != CF16) || dtype_cls(nd.dtype) == CBOOL) continue;
            Lin f = flat_index(j);
            if (!in_bounds(f, p) || f.c % chain_vec != 0) continue;
            bool ok = true;
            for (auto& t : f.t) {
                const Atom& a = atoms[t.first];
                if (a.kind != Atom::RANGE) { ok = false; break; }
                if (a.node == sweep ? t.second != 1 : t.second % chain_vec != 0) { ok = false; break; }
            }
            bool cok; if (!ok || lin_coef(f, sweep, cok) != 1 || !cok) continue;
            const std::string arr = "vl" + std::to_string(j) + "_" + std::to_string(ctx < 0 ? 0 : ctx), bt = buf_ctype(it.bufs[p].dtype);
            code += "    " + bt + " " + arr + "[" + V + "];\n";
            code += "    ldv_<" + bt + ", " + V + ">(" + dp + std::to_string(p) + " + " + render(f, ctx) + ", " + arr + ");\n";
            vec_load[j] = arr;
        }
        return code;
    }

    std::string load_expr(int i, int ctx) {
        if (vec_load.count(i)) return vec_load[i] + "[u]";
        const Node& nd = N(i);
        if (N(nd.src[0]).op != OP_PARAM) { fail("codegen: INDEX of a non-parameter"); return "0"; }
        int p = (int)N(nd.src[0]).arg;
        if (p < 0 || p >= (int)it.bufs.size()) { fail("codegen: PARAM number out of range"); return "0"; }
        Lin f = flat_index(i);
        auto cs = chain_subst.find(p);
        if (cs != chain_subst.end()) {
            // produced by an earlier stage of the same row chain: only this row's element is available
            bool row_only = f.c == 0 && f.t.size() == 1 && f.t[0].second == 1 && atoms[f.t[0].first].kind == Atom::RANGE &&
                            !loop_ranges.empty() && atoms[f.t[0].first].node == loop_ranges[0];
            if (!row_only) { fail("chain: a stage reads another row of an earlier stage's output"); return "0"; }
            std::string e = cs->second;
            Cls bc = dtype_cls(it.bufs[p].dtype), want = cls(i);
            if (dtype_cls(nd.dtype) == CBOOL) return "(" + e + " != 0u)";
            if (bc == CF16 && want == CF32) return "__half2float(" + e + ")";
            if (bc == CF32 && want == CF16) return "__float2half_rn(" + e + ")";
            if (bc != want && (want == CINT || want == CUINT)) return std::string("(") + cls_ctype(want) + ")" + e;
            if (bc != want && want == CF32) return "(float)" + e;
            return e;
        }
        std::string idx = render(f, ctx);
        if (opts.debug_bounds || !in_bounds(f, p)) {
            const BufDesc& b = it.bufs[p];
            std::string hi = b.symbolic() ? "(n0 * " + std::to_string(b.trailing()) + " - 1)" : std::to_string(std::max<int64_t>(b.elems(0) - 1, 0));
            idx = "clampi_(" + idx + ", " + hi + ")";
        }
        std::string e = dp + std::to_string(p) + "[" + idx + "]";
        Cls bc = dtype_cls(it.bufs[p].dtype);
        Cls want = cls(i);
        if (dtype_cls(nd.dtype) == CBOOL) return "(" + e + " != 0u)";
        if (bc == CF16 && want == CF32) return "__half2float(" + e + ")";
        if (bc == CF32 && want == CF16) return "__float2half_rn(" + e + ")";
        if (bc != want && (want == CINT || want == CUINT)) return std::string("(") + cls_ctype(want) + ")" + e;
        if (bc != want && want == CF32) return "(float)" + e;
        return e;
    }

    std::string identity(int rop, Cls c) {
        if (c == CF32 || c == CF16) return rop == OP_MUL ? "1.0f" : rop == OP_MAX ? "__int_as_float(0xff7fffff)" : "0.0f";
        if (c == CUINT) return rop == OP_MUL ? "1u" : "0u";
        return rop == OP_MUL ? "1" : rop == OP_MAX ? "(-2147483647 - 1)" : "0";
    }
    std::string combine(int rop, Cls c, const std::string& a, const std::string& b) {
        bool f = (c == CF32 || c == CF16);
        switch (rop) {
            case OP_MUL: return "(" + a + " * " + b + ")";
            case OP_MAX: return f ? "fmaxf(" + a + ", " + b + ")" : "max(" + a + ", " + b + ")";
            default: return "(" + a + " + " + b + ")";
        }
    }
    const char* rop_tag(int rop) { return rop == OP_MUL ? "mul" : rop == OP_MAX ? "max" : "add"; }

    // bound of a reduce range as a C expression
    std::string range_bound(int r) { return N(r).symbolic() ? "n0" : std::to_string(N(r).arg); }

    std::string reduce_expr(int i) {
        const Node& nd = N(i);
        int rop = (int)nd.aux;
        Cls c = dtype_cls(nd.dtype);
        bool isf = (c == CF32 || c == CF16);
        Cls acc_c = isf ? CF32 : c;
        const char* at = isf ? "float" : cls_ctype(acc_c);
        std::string acc = "acc" + std::to_string(i);
        std::vector<int> rr;
        for (size_t s = 1; s < nd.src.size(); s++) if (N(nd.src[s]).op == OP_RANGE) rr.push_back(nd.src[s]);
        stmt(-1, std::string(at) + " " + acc + " = " + identity(rop, acc_c) + ";");
        if (i == finish_reduce) {
            // finish kernel of a split reduce: partials in ascending part order
            std::string pe = "scratch[(long long)g * SPLIT + p]";
            if (!isf) pe = std::string("(") + at + ")__float_as_int(" + pe + ")";
            stmt(-1, "for (int p = 0; p < SPLIT; p++) " + acc + " = " + combine(rop, acc_c, acc, pe) + ";");
        } else {
            if (enum_reduce.count(i) && lanes == 1 && rr.size() == 1) {
                // one copy of the loop body per value of the range: the guards that read it fold away, and
                // so does every term of the body that they switch off
                const int R = rr[0];
                for (int64_t kk = 0; kk < N(R).arg; kk++) {
                    fix_range(R, kk);
                    forget_loop(i);
                    std::string e = val(nd.src[0], i);
                    std::string ef = (isf && cls(nd.src[0]) == CF16) ? "__half2float(" + e + ")" : e;
                    if (rop == OP_ADD && is_zero_lit(e) && loop[i].code.empty()) continue;       // nothing live for this value
                    T().code += "  {   // r" + std::to_string(N(R).aux) + " = " + std::to_string(kk) + "\n" + loop[i].code;
                    T().code += "    " + acc + " = " + combine(rop, acc_c, acc, ef) + ";\n  }\n";
                }
                unfix_range(R);
                forget_loop(i);
                if (nd.dtype == DT_F16) return "__float2half_rn(" + acc + ")";
                return acc;
            }
            // row-chain stage sweeping the row in chunks: the wide loads must be known before the body is rendered
            bool chunked = false;
            std::string wide;
            std::vector<int> wide_nodes;
            if (rr.size() == 1 && unroll_short_loops && chain_vec > 1 && !N(rr[0]).symbolic() &&
                N(rr[0]).arg <= (int64_t)lanes * 32 && N(rr[0]).arg % ((int64_t)lanes * chain_vec) == 0) {
                chunked = true;
                std::map<int, std::string> before = vec_load;
                wide = chain_wide_loads(nd.src[0], rr[0], i);
                for (auto& kv : vec_load) if (!before.count(kv.first)) wide_nodes.push_back(kv.first);
            }
            std::string e = val(nd.src[0], i);
            for (int j : wide_nodes) vec_load.erase(j);
            std::string ef = (isf && cls(nd.src[0]) == CF16) ? "__half2float(" + e + ")" : e;
            // emit: loop header, hoisted code is already in `top`, then the loop body
            std::string hdr;
            if (rr.empty()) {
                hdr = "if (lane == 0) {";
            } else if (rr.size() == 1) {
                std::string rn = "r" + std::to_string(N(rr[0]).aux);
                hdr = "for (int " + rn + " = RED_BEGIN(" + range_bound(rr[0]) + "); " + rn + " < RED_END(" + range_bound(rr[0]) + "); " + rn + " += RED_STEP) {";
                // short trip counts are unrolled: the loads of one stage of a row chain can then stay in
                // registers for the next stage instead of being fetched from L1 again
                if (unroll_short_loops && !N(rr[0]).symbolic() && N(rr[0]).arg <= (int64_t)lanes * 32) {
                    if (chunked) {
                        // each lane takes chain_vec consecutive elements per trip; unit-stride operands
                        // arrive by one explicit 128-bit load per chunk (the inner declaration of the
                        // sweep variable shadows the chunk's first index the loads are written with)
                        std::string V = std::to_string(chain_vec), nb = range_bound(rr[0]);
                        hdr = "_Pragma(\"unroll\") for (int " + rn + "b = lane * " + V + "; " + rn + "b < " + nb + "; " + rn + "b += LANES * " + V + ") {\n"
                              "    const int " + rn + " = " + rn + "b; (void)" + rn + ";\n" + wide +
                              "  _Pragma(\"unroll\") for (int u = 0; u < " + V + "; u++) { const int " + rn + " = " + rn + "b + u;";
                    } else hdr = "_Pragma(\"unroll\") " + hdr;
                }
            } else {
                std::string tot = "(";
                for (size_t k = 0; k < rr.size(); k++) tot += (k ? " * " : "") + range_bound(rr[k]);
                tot += ")";
                hdr = "for (int q = RED_BEGIN" + tot + "; q < RED_END" + tot + "; q += RED_STEP) {";
            }
            T().code += "  " + hdr + "\n";
            if (rr.size() > 1) {
                // decompose q, last range fastest
                std::string stride = "1";
                for (int k = (int)rr.size() - 1; k >= 0; k--) {
                    std::string rn = "r" + std::to_string(N(rr[k]).aux);
                    std::string b = range_bound(rr[k]);
                    T().code += "    const int " + rn + " = " + (k == 0 ? "q / (" + stride + ")" : "(q / (" + stride + ")) % " + b) + ";\n";
                    stride = stride + " * " + b;
                }
            }
            T().code += loop[i].code;
            T().code += "    " + acc + " = " + combine(rop, acc_c, acc, ef) + ";\n";
            T().code += chunked ? "  } }\n" : "  }\n";
            if (reduce_combine_mode == "group")
                stmt(-1, acc + " = group_" + rop_tag(rop) + "_" + (isf ? "f" : "i") + "(" + acc + ", lane, grp, red_smem);");
            else if (reduce_combine_mode == "partial")
                stmt(-1, acc + " = group_" + rop_tag(rop) + "_" + (isf ? "f" : "i") + "(" + acc + ", lane, grp, red_smem);");
        }
        if (nd.dtype == DT_F16) return "__float2half_rn(" + acc + ")";
        return acc;
    }

    // value of node i as a C expression usable in context ctx (-1 = outside reduce loops)
    std::string val(int i, int ctx) {
        const Node& nd = N(i);
        if (nd.op == OP_CONST) return const_lit(i);
        if (nd.op == OP_RANGE) return range_name(i);
        if (ctx >= 0 && !depends_on_reduce(i, ctx)) ctx = -1;
        Cls c = cls(i);
        if ((c == CINT || c == CUINT) && nd.op != OP_INDEX && nd.op != OP_REDUCE && nd.op != OP_CAST && nd.op != OP_BITCAST && nd.op != OP_WHERE)
            return render(lin(i), ctx);
        if (c == CINT || c == CUINT) return opaque_int(i, ctx);
        auto key = std::make_pair(i, ctx);
        auto f = memo.find(key);
        if (f != memo.end()) return f->second;
        std::string e;
        auto a = [&](int k) { return val(nd.src[k], ctx); };
        auto af = [&](int k) { return to_float(nd.src[k], val(nd.src[k], ctx)); };
        // operand k in this node's own compute class: a node shared between an f16 reduction (where it
        // is evaluated widened) and f16 code outside it is narrowed at the point of use
        auto ac = [&](int k) {
            std::string v = val(nd.src[k], ctx);
            Cls sc = cls(nd.src[k]);
            if (sc == c) return v;
            if (c == CF16 && sc == CF32) return "__float2half_rn(" + v + ")";
            if (c == CF32 && sc == CF16) return "__half2float(" + v + ")";
            return v;
        };
        bool h = (c == CF16);
        auto wrap = [&](const std::string& fexpr) { return h ? "__float2half_rn(" + fexpr + ")" : fexpr; };
        if (c == CBOOL) {
            switch (nd.op) {
                case OP_CMPLT: case OP_CMPNE: case OP_CMPEQ: {
                    int s0 = nd.src[0], s1 = nd.src[1];
                    const char* o = nd.op == OP_CMPLT ? " < " : nd.op == OP_CMPNE ? " != " : " == ";
                    if (is_intlike(s0) && is_intlike(s1)) {
                        Lin d = ladd(lin(s0), lin(s1), -1);     // s0 - s1
                        int64_t lo = llo(d), hi = lhi(d);
                        if (nd.op == OP_CMPLT) { if (hi < 0) return "true"; if (lo >= 0) return "false"; }
                        if (nd.op == OP_CMPNE) { if (hi < 0 || lo > 0) return "true"; if (lo == 0 && hi == 0) return "false"; }
                        if (nd.op == OP_CMPEQ) { if (hi < 0 || lo > 0) return "false"; if (lo == 0 && hi == 0) return "true"; }
                        e = "(" + render(lin(s0), ctx) + o + render(lin(s1), ctx) + ")";
                    } else if (cls(s0) == CF16 || cls(s1) == CF16) e = "(" + af(0) + o + af(1) + ")";
                    else e = "(" + a(0) + o + a(1) + ")";
                    break;
                }
                case OP_AND: { std::string x = a(0), y = a(1); if (x == "false" || y == "false") return "false"; if (x == "true") return y; if (y == "true") return x; e = "(" + x + " && " + y + ")"; break; }
                case OP_OR: { std::string x = a(0), y = a(1); if (x == "true" || y == "true") return "true"; if (x == "false") return y; if (y == "false") return x; e = "(" + x + " || " + y + ")"; break; }
                case OP_XOR: e = "(" + a(0) + " != " + a(1) + ")"; break;
                case OP_WHERE: e = "(" + a(0) + " ? " + a(1) + " : " + a(2) + ")"; break;
                case OP_CAST: case OP_BITCAST: e = cast_expr(i, ctx); break;
                case OP_INDEX: e = load_expr(i, ctx); break;
                default: fail("codegen: unhandled bool op " + std::to_string(nd.op)); return "false";
            }
        } else {
            switch (nd.op) {
                case OP_INDEX: e = load_expr(i, ctx); break;
                case OP_REDUCE: if (ctx >= 0) { fail("codegen: nested REDUCE"); return "0.0f"; } e = reduce_expr(i); break;
                case OP_CAST: case OP_BITCAST: e = cast_expr(i, ctx); break;
                case OP_WHERE: { std::string cnd = a(0); if (cnd == "true") return ac(1); if (cnd == "false") return ac(2); e = "(" + cnd + " ? " + ac(1) + " : " + ac(2) + ")"; break; }
                // one MUFU: results below 2^-126 flush to zero instead of going through exp2f's rescaling
                // for subnormals (absolute difference < 1.2e-38)
                case OP_EXP2: e = h ? "__float2half_rn(ex2_h_(" + af(0) + "))" : "ex2_h_(" + af(0) + ")"; break;
                case OP_LOG2: e = wrap("log2f(" + af(0) + ")"); break;
                case OP_SIN: e = wrap("sinf(" + af(0) + ")"); break;
                case OP_SQRT: e = wrap("sqrtf(" + af(0) + ")"); break;
                case OP_RECIP: e = h ? "__float2half_rn(rcp_h_(" + af(0) + "))" : "__frcp_rn(" + af(0) + ")"; break;
                case OP_TRUNC: e = wrap("truncf(" + af(0) + ")"); break;
                case OP_NEG: e = h ? "__hneg(" + ac(0) + ")" : "(-" + ac(0) + ")"; break;
                case OP_ADD: {
                    // x + 0 where the zero is what a guard folded to (a padded slice that is not live):
                    // the value of x, at worst with the sign of a zero changed
                    std::string x0 = ac(0), x1 = ac(1);
                    if (is_zero_lit(x0)) return x1;
                    if (is_zero_lit(x1)) return x0;
                    e = h ? "__hadd(" + x0 + ", " + x1 + ")" : "(" + x0 + " + " + x1 + ")"; break;
                }
                case OP_SUB: e = h ? "__hsub(" + ac(0) + ", " + ac(1) + ")" : "(" + ac(0) + " - " + ac(1) + ")"; break;
                case OP_MUL:
                    if (is_float_one(nd.src[0]) && cls(nd.src[1]) == c) return ac(1);
                    if (is_float_one(nd.src[1]) && cls(nd.src[0]) == c) return ac(0);
                    e = h ? "__hmul(" + ac(0) + ", " + ac(1) + ")" : "(" + ac(0) + " * " + ac(1) + ")"; break;
                case OP_FDIV: e = wrap("(" + af(0) + " / " + af(1) + ")"); break;
                case OP_MAX: e = h ? "__hmax(" + ac(0) + ", " + ac(1) + ")" : "fmaxf(" + ac(0) + ", " + ac(1) + ")"; break;
                case OP_POW: e = wrap("powf(" + af(0) + ", " + af(1) + ")"); break;
                case OP_MOD: e = wrap("fmodf(" + af(0) + ", " + af(1) + ")"); break;
                case OP_MULACC: e = h ? "__hadd(" + ac(0) + ", __hmul(" + ac(1) + ", " + ac(2) + "))" : "(" + ac(0) + " + (" + ac(1) + " * " + ac(2) + "))"; break;
                default: fail("codegen: unhandled op " + std::to_string(nd.op)); return "0.0f";
            }
        }
        std::string name = "t" + std::to_string(i);
        stmt(ctx, std::string("const ") + cls_ctype(c) + " " + name + " = " + e + ";");
        memo[key] = name;
        return name;
    }

    // ── paired f16 evaluation ────────────────────────────────────────────────────────────────
    // An elementwise kernel whose values are all f16 (or comparisons of f16 values) is evaluated two
    // elements at a time in __half2: every arithmetic instruction then serves two outputs, which is
    // what an instruction-bound GELU needs to get back under the memory roofline.  Each lane
    // computes exactly what the one-element form computes (the *2 intrinsics round per lane, exp2 and
    // the reciprocal go through the same f32 approximations), so the two forms agree bit for bit.
    bool h2 = false;

    bool h2_node_ok(int i, std::vector<char>& seen) {
        if (seen[i]) return seen[i] == 1;
        seen[i] = 1;
        const Node& nd = N(i);
        Cls c = cls(i);
        auto fail_ = [&]() { seen[i] = 2; return false; };
        if (nd.op == OP_CONST) return (nd.dtype == DT_F16 && c == CF16) ? true : fail_();
        if (nd.op == OP_INDEX) {
            if (c != CF16 || N(nd.src[0]).op != OP_PARAM) return fail_();
            int p = (int)N(nd.src[0]).arg;
            if (p < 0 || p >= (int)it.bufs.size() || it.bufs[p].dtype != DT_F16) return fail_();
            return true;                                   // the index subtree is integer code, rendered as usual
        }
        if (c == CF16) {
            switch (nd.op) {
                case OP_NEG: case OP_ADD: case OP_SUB: case OP_MUL: case OP_MAX: case OP_MULACC:
                case OP_EXP2: case OP_LOG2: case OP_SQRT: case OP_RECIP: case OP_SIN: break;
                case OP_WHERE: if (cls(nd.src[0]) != CBOOL) return fail_(); break;
                default: return fail_();
            }
        } else if (c == CBOOL) {
            switch (nd.op) {
                case OP_CMPLT: case OP_CMPNE: case OP_CMPEQ:
                    if (cls(nd.src[0]) != CF16 || cls(nd.src[1]) != CF16) return fail_();
                    break;
                case OP_AND: case OP_OR: case OP_XOR: case OP_WHERE: break;
                default: return fail_();
            }
        } else return fail_();
        for (int sidx : nd.src) if (!h2_node_ok(sidx, seen)) return fail_();
        return true;
    }
    bool h2_eligible(int V) {
        if (V < 2 || (V & 1) || it.bufs[0].dtype != DT_F16 || cls(body) != CF16) return false;
        std::vector<char> seen(n, 0);
        return h2_node_ok(body, seen);
    }

    std::string val_h2(int i) {
        const Node& nd = N(i);
        auto key = std::make_pair(i, -1);
        auto f = memo.find(key);
        if (f != memo.end()) return f->second;
        if (nd.op == OP_CONST) {
            double d; std::memcpy(&d, &nd.arg, 8);
            if (std::isinf(d)) d = d < 0 ? -65504.0 : 65504.0;
            return "__float2half2_rn(" + flit(d) + ")";
        }
        Cls c = cls(i);
        auto a = [&](int k) { return val_h2(nd.src[k]); };
        std::string e;
        switch (nd.op) {
            case OP_INDEX: e = vec_load.count(i) ? vec_load[i] + "[u]" : "__half2half2(" + load_expr(i, -1) + ")"; break;
            case OP_NEG: e = "__hneg2(" + a(0) + ")"; break;
            case OP_ADD: e = "__hadd2(" + a(0) + ", " + a(1) + ")"; break;
            case OP_SUB: e = "__hsub2(" + a(0) + ", " + a(1) + ")"; break;
            case OP_MUL:
                if (is_float_one(nd.src[0])) return a(1);
                if (is_float_one(nd.src[1])) return a(0);
                e = "__hmul2(" + a(0) + ", " + a(1) + ")"; break;
            case OP_MAX: e = "__hmax2(" + a(0) + ", " + a(1) + ")"; break;
            case OP_MULACC: e = "__hadd2(" + a(0) + ", __hmul2(" + a(1) + ", " + a(2) + "))"; break;
            case OP_EXP2: e = "h2_ex2_(" + a(0) + ")"; break;
            case OP_RECIP: e = "h2_rcp_(" + a(0) + ")"; break;
            case OP_LOG2: e = "h2_log2_(" + a(0) + ")"; break;
            case OP_SQRT: e = "h2_sqrt_(" + a(0) + ")"; break;
            case OP_SIN: e = "h2_sin_(" + a(0) + ")"; break;
            case OP_CMPLT: e = "__hlt2_mask(" + a(0) + ", " + a(1) + ")"; break;
            case OP_CMPEQ: e = "__heq2_mask(" + a(0) + ", " + a(1) + ")"; break;
            case OP_CMPNE: e = "__hneu2_mask(" + a(0) + ", " + a(1) + ")"; break;
            case OP_AND: e = "(" + a(0) + " & " + a(1) + ")"; break;
            case OP_OR: e = "(" + a(0) + " | " + a(1) + ")"; break;
            case OP_XOR: e = "(" + a(0) + " ^ " + a(1) + ")"; break;
            case OP_WHERE:
                e = c == CBOOL ? "((" + a(0) + " & " + a(1) + ") | (~" + a(0) + " & " + a(2) + "))" : "h2_sel_(" + a(0) + ", " + a(1) + ", " + a(2) + ")";
                break;
            default: fail("codegen: paired f16 form met op " + std::to_string(nd.op)); return "__float2half2_rn(0.0f)";
        }
        std::string name = "t" + std::to_string(i);
        stmt(-1, std::string("const ") + (c == CBOOL ? "unsigned" : "__half2") + " " + name + " = " + e + ";");
        memo[key] = name;
        return name;
    }

    std::string store_value(const std::string& v, int node) {
        int odt = it.bufs[0].dtype;
        Cls vc = cls(node);
        switch (dtype_cls(odt)) {
            case CF16: return vc == CF16 ? v : "__float2half_rn(" + to_float(node, v) + ")";
            case CF32: {
                std::string f = to_float(node, v);
                return odt == DT_BF16 ? "__int_as_float(__float_as_int(" + f + ") & 0xFFFF0000)" : f;
            }
            case CINT: return vc == CBOOL ? "(" + v + " ? 1 : 0)" : "(int)(" + v + ")";
            default: return vc == CBOOL ? "(" + v + " ? 1u : 0u)" : "(unsigned)(" + v + ")";
        }
    }

    // ── kernel assembly ────────────────────────────────────────────────────────────────────────
    static const char* preamble() {
        return
            "#include <cuda_fp16.h>\n"
            "__device__ __forceinline__ int clampi_(int i, int hi) { return i < 0 ? 0 : (i > hi ? hi : i); }\n"
            "__device__ __forceinline__ int idiv_(int a, int b) { return b == 0 ? 0 : a / b; }\n"
            "__device__ __forceinline__ int imod_(int a, int b) { return b == 0 ? 0 : a % b; }\n"
            "template <int BYTES> struct vec_t_;\n"
            "template <> struct vec_t_<16> { typedef uint4 type; };\n"
            "template <> struct vec_t_<8> { typedef uint2 type; };\n"
            "template <> struct vec_t_<4> { typedef unsigned type; };\n"
            "template <> struct vec_t_<2> { typedef unsigned short type; };\n"
            "template <class T, int V> __device__ __forceinline__ void ldv_(const T* p, T* out) {\n"
            "  typedef typename vec_t_<sizeof(T) * V>::type W;\n"
            "  W w = __ldg(reinterpret_cast<const W*>(p));\n"
            "  *reinterpret_cast<W*>(out) = w;\n"
            "}\n"
            "template <class T, int V> __device__ __forceinline__ void stv_(T* p, const T* in) {\n"
            "  typedef typename vec_t_<sizeof(T) * V>::type W;\n"
            "  *reinterpret_cast<W*>(p) = *reinterpret_cast<const W*>(in);\n"
            "}\n"
            // f16-class exp2 and reciprocal: one MUFU on the widened value, rounded back to f16.  The
            // f32 approximation is within 2 ulp (f32), far below the f16 rounding that follows.
            "__device__ __forceinline__ float ex2_h_(float x) { float r; asm(\"ex2.approx.ftz.f32 %0, %1;\" : \"=f\"(r) : \"f\"(x)); return r; }\n"
            "__device__ __forceinline__ float rcp_h_(float x) { float r; asm(\"rcp.approx.ftz.f32 %0, %1;\" : \"=f\"(r) : \"f\"(x)); return r; }\n"
            "#define DEF_H2MAP_(NAME, F) __device__ __forceinline__ __half2 NAME(__half2 x) { return __floats2half2_rn(F(__low2float(x)), F(__high2float(x))); }\n"
            "DEF_H2MAP_(h2_ex2_, ex2_h_)\n"
            "DEF_H2MAP_(h2_rcp_, rcp_h_)\n"
            "DEF_H2MAP_(h2_log2_, log2f)\n"
            "DEF_H2MAP_(h2_sqrt_, sqrtf)\n"
            "DEF_H2MAP_(h2_sin_, sinf)\n"
            "__device__ __forceinline__ __half2 h2_sel_(unsigned m, __half2 a, __half2 b) {\n"
            "  unsigned x = *reinterpret_cast<unsigned*>(&a), y = *reinterpret_cast<unsigned*>(&b), r = (x & m) | (y & ~m);\n"
            "  return *reinterpret_cast<__half2*>(&r);\n"
            "}\n"
            "__device__ __forceinline__ float op_add_f(float a, float b) { return a + b; }\n"
            "__device__ __forceinline__ float op_mul_f(float a, float b) { return a * b; }\n"
            "__device__ __forceinline__ float op_max_f(float a, float b) { return fmaxf(a, b); }\n"
            "__device__ __forceinline__ int op_add_i(int a, int b) { return a + b; }\n"
            "__device__ __forceinline__ int op_mul_i(int a, int b) { return a * b; }\n"
            "__device__ __forceinline__ int op_max_i(int a, int b) { return a > b ? a : b; }\n"
            // Combine the partial accumulators of the LANES threads that share one output.  RC layout:
            // the lanes of a group are consecutive threads; OC layout: they are TOUTS threads apart.
            // The combine order is fixed, so a kernel gives the same bits on every run.
            "#define DEF_GROUP_(NAME, T, OP) \\\n"
            "__device__ __forceinline__ T NAME(T v, int lane, int grp, float* sm) { \\\n"
            "  if (LANES == 1) return v; \\\n"
            "  if (RC_LAYOUT) { \\\n"
            "    _Pragma(\"unroll\") for (int o = (LANES < 32 ? LANES : 32) / 2; o > 0; o >>= 1) v = OP(v, __shfl_xor_sync(0xffffffffu, v, o)); \\\n"
            "    if (LANES > 32) { \\\n"
            "      T* s = reinterpret_cast<T*>(sm); \\\n"
            "      __syncthreads(); \\\n"
            "      if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v; \\\n"
            "      __syncthreads(); \\\n"
            "      const int w0 = grp * (LANES / 32); \\\n"
            "      v = s[w0]; \\\n"
            "      for (int w = 1; w < LANES / 32; w++) v = OP(v, s[w0 + w]); \\\n"
            "    } \\\n"
            "    return v; \\\n"
            "  } else { \\\n"
            "    T* s = reinterpret_cast<T*>(sm); \\\n"
            "    __syncthreads(); \\\n"
            "    s[lane * TOUTS + grp] = v; \\\n"
            "    __syncthreads(); \\\n"
            "    v = s[grp]; \\\n"
            "    for (int l = 1; l < LANES; l++) v = OP(v, s[l * TOUTS + grp]); \\\n"
            "    return v; \\\n"
            "  } \\\n"
            "}\n"
            "DEF_GROUP_(group_add_f, float, op_add_f)\n"
            "DEF_GROUP_(group_mul_f, float, op_mul_f)\n"
            "DEF_GROUP_(group_max_f, float, op_max_f)\n"
            "DEF_GROUP_(group_add_i, int, op_add_i)\n"
            "DEF_GROUP_(group_mul_i, int, op_mul_i)\n"
            "DEF_GROUP_(group_max_i, int, op_max_i)\n";
    }

    std::string signature(const std::string& name, bool with_scratch, int nthreads) {
        std::string s = "extern \"C\" __global__ void __launch_bounds__(" + std::to_string(nthreads) + ") " + name + "(";
        for (size_t b = 0; b < it.bufs.size(); b++) {
            s += (b ? ", " : "");
            s += (b ? "const " : "");
            s += buf_ctype(it.bufs[b].dtype);
            s += "* __restrict__ data" + std::to_string(b);
        }
        if (with_scratch) s += ", float* __restrict__ scratch";
        if (has_sym) s += ", const int n0";
        return s + ")";
    }

    int64_t static_total() const {
        int64_t t = 1;
        for (int r : loop_ranges) if (!N(r).symbolic()) t *= N(r).arg;
        return t;
    }
    bool sym_output() const { for (int r : loop_ranges) if (N(r).symbolic()) return true; return false; }
    std::string total_expr() const {
        return sym_output() ? "((long long)n0 * " + std::to_string(static_total()) + ")" : std::to_string(static_total()) + "LL";
    }

    // r_i = (g / stride_i) % size_i for loop ranges [first, last), innermost last
    std::string decompose(const std::string& g, size_t first = 0, size_t last = (size_t)-1, const std::string& indent = "  ") {
        if (last == (size_t)-1) last = loop_ranges.size();
        std::string s;
        int64_t stride = 1;
        for (int k = (int)last - 1; k >= (int)first; k--) {
            int r = loop_ranges[k];
            std::string rn = "r" + std::to_string(N(r).aux);
            std::string e = stride == 1 ? g : "(" + g + " / " + std::to_string(stride) + ")";
            if (k == (int)first || N(r).symbolic()) s += indent + "const int " + rn + " = (int)" + e + ";\n";
            else s += indent + "const int " + rn + " = (int)(" + e + " % " + std::to_string(N(r).arg) + ");\n";
            if (!N(r).symbolic()) stride *= N(r).arg;
        }
        return s;
    }

    void reset_emit() { top = Block(); prelude = Block(); cur_top = nullptr; loop.clear(); memo.clear(); vec_load.clear(); vec_range = -1; finish_reduce = -1; }

    // vector width the elementwise path may use, and the loads it can preload as vectors
    int pick_vector(std::vector<int>& vloads) {
        if (opts.vector_width == 1 || loop_ranges.empty() || opts.debug_bounds) return 1;
        int rv = loop_ranges.back();
        if (N(rv).symbolic()) return 1;
        bool all16 = dt_storage_bytes(it.bufs[0].dtype) == 2;
        std::vector<int> idx_nodes;
        for (int i = 0; i < n; i++) if (N(i).op == OP_INDEX && i != dst && is_live(i)) idx_nodes.push_back(i);
        for (int i : idx_nodes) if (dt_storage_bytes(it.bufs[(int)N(N(i).src[0]).arg].dtype) != 2) { all16 = false; }
        int V = opts.vector_width > 1 ? opts.vector_width : (all16 ? 8 : 4);
        if (!all16 && V > 4) V = 4;            // one access is at most 128 bits
        if (V != 4 && V != 8 && V != 2) V = all16 ? 8 : 4;
        if (N(rv).arg % V != 0) return 1;
        vloads.clear();
        for (int i : idx_nodes) {
            int p = (int)N(N(i).src[0]).arg;
            Lin f = flat_index(i);
            bool ok; int64_t c = lin_coef(f, rv, ok);
            if (!ok) return 1;                 // the unrolled variable is buried in a div/mod
            if (c == 0) continue;              // broadcast along the vector
            if (c != 1) return 1;
            if (!in_bounds(f, p)) return 1;
            if (f.c % V != 0) return 1;
            for (auto& t : f.t) {
                const Atom& a = atoms[t.first];
                if (a.kind == Atom::RANGE && a.node == rv) continue;
                if (t.second % V != 0) return 1;
            }
            vloads.push_back(i);
        }
        return V;
    }
    std::vector<bool> live_;
    bool is_live(int i) {
        if (live_.empty()) {
            live_.assign(n, false);
            std::function<void(int)> mark = [&](int k) { if (live_[k]) return; live_[k] = true; for (int s : N(k).src) mark(s); };
            mark(body);
        }
        return live_[i];
    }

    bool build_elementwise(Rendered& out) {
        std::vector<int> vloads;
        int V = pick_vector(vloads);
        int T = opts.block_threads > 0 ? opts.block_threads : 256;
        reset_emit();
        std::ostringstream k;
        k << "#define LANES 1\n#define TOUTS 1\n#define RC_LAYOUT 1\n";
        k << preamble();
        std::string name = "ew_fused";
        k << signature(name, false, T) << " {\n";
        k << "  const long long g = (long long)blockIdx.x * " << T << " + threadIdx.x;\n";
        if (V == 1) {
            k << "  if (g >= " << total_expr() << ") return;\n";
            k << decompose("g");
            std::string v = val(body, -1);
            if (!err.empty()) return false;
            k << top.code;
            k << "  data0[g] = " << store_value(v, body) << ";\n";
        } else {
            int rv = loop_ranges.back();
            h2 = opts.vector_width >= 0 && h2_eligible(V);
            const int U = h2 ? V / 2 : V;                  // iterations of the unrolled loop
            k << "  const long long base = g * " << V << ";\n";
            k << "  if (base >= " << total_expr() << ") return;\n";
            k << decompose("base");
            // preload the unit-stride operands with one wide access each
            vec_range = -1;
            int vi = 0;
            cur_top = &prelude;
            for (int i : vloads) {
                int p = (int)N(N(i).src[0]).arg;
                Lin f = flat_index(i);
                std::string arr = "v" + std::to_string(vi++);
                std::string bt = buf_ctype(it.bufs[p].dtype), VS = std::to_string(V);
                std::string idx = render(f, -1);
                if (h2) {
                    stmt(-1, "__half2 " + arr + "_raw[" + std::to_string(U) + "];");
                    stmt(-1, "ldv_<__half2, " + std::to_string(U) + ">(reinterpret_cast<const __half2*>(data" + std::to_string(p) + " + " + idx + "), " + arr + "_raw);");
                    vec_load[i] = arr + "_raw";
                    continue;
                }
                stmt(-1, bt + " " + arr + "_raw[" + VS + "];");
                stmt(-1, "ldv_<" + bt + ", " + VS + ">(data" + std::to_string(p) + " + " + idx + ", " + arr + "_raw);");
                // convert to the compute class of the INDEX node
                Cls bc = dtype_cls(it.bufs[p].dtype), want = cls(i);
                if (dtype_cls(N(i).dtype) == CBOOL) {
                    stmt(-1, "bool " + arr + "[" + VS + "];");
                    stmt(-1, "_Pragma(\"unroll\") for (int u = 0; u < " + VS + "; u++) " + arr + "[u] = " + arr + "_raw[u] != 0u;");
                    vec_load[i] = arr;
                } else if (bc == CF16 && want == CF32) {
                    stmt(-1, "float " + arr + "[" + VS + "];");
                    stmt(-1, "_Pragma(\"unroll\") for (int u = 0; u < " + VS + "; u++) " + arr + "[u] = __half2float(" + arr + "_raw[u]);");
                    vec_load[i] = arr;
                } else {
                    vec_load[i] = arr + "_raw";
                }
            }
            cur_top = nullptr;
            vec_range = rv;
            std::string v = h2 ? val_h2(body) : val(body, -1);
            if (!err.empty()) return false;
            k << prelude.code;
            const std::string ot = h2 ? "__half2" : buf_ctype(it.bufs[0].dtype);
            k << "  " << ot << " outv[" << U << "];\n";
            k << "  _Pragma(\"unroll\") for (int u = 0; u < " << U << "; u++) {\n";
            k << top.code;
            k << "    outv[u] = " << (h2 ? v : store_value(v, body)) << ";\n";
            k << "  }\n";
            if (h2) k << "  stv_<__half2, " << U << ">(reinterpret_cast<__half2*>(data0 + base), outv);\n";
            else k << "  stv_<" << ot << ", " << V << ">(data0 + base, outv);\n";
        }
        k << "}\n";
        out.klass = KC_ELEMENTWISE;
        out.source = k.str();
        out.vector_width = V;
        out.main.entry = name;
        out.main.block = T;
        out.main.outputs_per_block = (int64_t)T * V;
        out.main.static_outputs = static_total();
        out.main.sym_trailing = sym_output() ? static_total() : 0;
        out.uses_sym = has_sym;
        out.note = "elementwise V=" + std::to_string(V) + (h2 ? " paired f16" : "");
        return true;
    }

    // flattened size of a REDUCE's ranges; 0 if symbolic
    int64_t reduce_total(int r) const {
        int64_t t = 1;
        for (size_t s = 1; s < N(r).src.size(); s++) {
            int rn = N(r).src[s];
            if (N(rn).op != OP_RANGE) continue;
            if (N(rn).symbolic()) return 0;
            t *= N(rn).arg;
        }
        return t;
    }

    void choose_layout(int64_t total, int64_t rtot_max) {
        // votes: bytes of loads that are unit-stride along the innermost reduce range (RC) against
        // loads unit-stride along the innermost output range (OC)
        int64_t rc = 0, oc = 0;
        int oc_min_bytes = 4;
        int out_inner = loop_ranges.empty() ? -1 : loop_ranges.back();
        for (int r : reduces) {
            int red_inner = -1;
            for (size_t s = 1; s < N(r).src.size(); s++) if (N(N(r).src[s]).op == OP_RANGE) red_inner = N(r).src[s];
            if (red_inner < 0) continue;
            for (int i = 0; i < n; i++) {
                if (N(i).op != OP_INDEX || i == dst || !is_live(i) || !dep[i][range_slot[red_inner]]) continue;
                Lin f = flat_index(i);
                bool ok1, ok2 = false;
                int64_t c1 = lin_coef(f, red_inner, ok1);
                int64_t c2 = out_inner >= 0 ? lin_coef(f, out_inner, ok2) : 0;
                int bytes = dt_storage_bytes(it.bufs[(int)N(N(i).src[0]).arg].dtype);
                if (ok1 && std::llabs(c1) == 1) rc += bytes;
                else if (ok2 && std::llabs(c2) == 1) { oc += bytes; oc_min_bytes = std::min(oc_min_bytes, bytes); }
            }
        }
        threads = opts.block_threads > 0 ? opts.block_threads : 256;
        const int64_t want_threads = 148LL * 1024;     // enough to fill the machine
        if (oc > 0) {
            rc_layout = false;
            int L = 1;
            if (opts.reduce_lanes > 0) L = opts.reduce_lanes;
            else {
                while (L < 32 && total * L < want_threads && rtot_max / (L * 2) >= 16) L *= 2;
                // the threads that share a row cover TOUTS adjacent outputs: keep that run at least one
                // 32-byte sector wide, or every sector fetched is only partly used (f16: 16 outputs)
                const int min_touts = std::max(1, 32 / std::max(1, oc_min_bytes));
                while (L > 1 && threads / L < min_touts) L /= 2;
            }
            lanes = L;
        } else {
            rc_layout = true;
            int L;
            if (opts.reduce_lanes > 0) L = opts.reduce_lanes;
            else if (rtot_max == 0) L = 32;          // symbolic bound
            else if (rtot_max <= 16) L = 1;
            else if (rtot_max < 1024) { L = 32; while (L > rtot_max) L /= 2; }
            else L = threads;
            if (opts.reduce_lanes == 0 && L < threads && total * L < want_threads / 4 && rtot_max >= 64) {
                while (L < threads && total * L < want_threads / 4 && rtot_max / (L * 2) >= 4) L *= 2;
            }
            lanes = L;
        }
        if (!enum_reduce.empty() && opts.reduce_lanes == 0) lanes = 1;      // value-by-value loops are per thread
        if (lanes > threads) lanes = threads;
        touts = threads / lanes;
    }

    std::string reduce_macros(bool partial) {
        std::ostringstream m;
        m << "#define LANES " << lanes << "\n#define TOUTS " << touts << "\n#define RC_LAYOUT " << (rc_layout ? 1 : 0) << "\n";
        if (partial) {
            // each block owns a contiguous chunk of the flattened reduce space
            m << "#define RED_BEGIN(n) (part_begin((n)) + lane)\n#define RED_END(n) part_end((n))\n#define RED_STEP LANES\n";
        } else {
            m << "#define RED_BEGIN(n) lane\n#define RED_END(n) (n)\n#define RED_STEP LANES\n";
        }
        return m.str();
    }

    // One stage of a row chain.  Requirements: static ranges, the first loop range is the row, every
    // REDUCE is invariant along the other loop ranges (they are swept after the reductions).  Emits
    //   <decl>  : declaration of the stage's per-row result (when the stage has no inner ranges)
    //   <code>  : a braced block computing it for row `row`
    bool build_chain_stage(int k, int threads_, std::string& decl, std::string& code, std::string& result_var, int64_t& rows, bool& has_inner) {
        if (!analyse()) return false;
        if (has_sym || loop_ranges.empty()) return fail("chain: symbolic or scalar kernel");
        rows = N(loop_ranges[0]).arg;
        for (size_t r = 1; r < loop_ranges.size(); r++)
            for (int red : reduces) if (dep[red][range_slot[loop_ranges[r]]]) return fail("chain: a reduction depends on an inner output range");
        // every load must be unit-stride (or constant) along the innermost range it sweeps inside the row,
        // otherwise one block per row would stride through memory (a column sum is not a row chain)
        for (int i = 0; i < n; i++) {
            if (N(i).op != OP_INDEX || i == dst || !is_live(i)) continue;
            int innermost = -1;
            for (int r : all_ranges) if (r != loop_ranges[0] && dep[i][range_slot[r]]) innermost = std::max(innermost, r);
            if (innermost < 0) continue;
            bool ok; int64_t c = lin_coef(flat_index(i), innermost, ok);
            if (!ok || std::llabs(c) > 1) return fail("chain: strided access inside the row");
        }
        has_inner = loop_ranges.size() > 1;
        int64_t inner = 1;
        for (size_t r = 1; r < loop_ranges.size(); r++) inner *= N(loop_ranges[r]).arg;
        threads = threads_; lanes = threads; touts = 1; rc_layout = true;
        reset_emit();
        reduce_combine_mode = "group";
        unroll_short_loops = true;
        // 4-element chunks per lane with explicit 128-bit loads and stores where a row allows it
        chain_vec = 4;
        dp = "s" + std::to_string(k) + "_data";
        std::ostringstream c;
        std::string bt = buf_ctype(it.bufs[0].dtype);
        result_var = "stage" + std::to_string(k);
        if (!has_inner) decl = "  " + bt + " " + result_var + ";\n";
        c << "  {   // stage " << k << "\n";
        c << "  const int r" << N(loop_ranges[0]).aux << " = row;\n";
        cur_top = &prelude;
        for (int r : reduces) { val(r, -1); if (!err.empty()) return false; }
        cur_top = nullptr;
        // the last stage writes the row in chunks of chain_vec outputs per lane: wide loads of its
        // unit-stride operands, one wide store
        const Cls oc = dtype_cls(it.bufs[0].dtype);
        const bool chunk_sweep = has_inner && chain_vec > 1 && inner <= (int64_t)threads * 32 && inner % ((int64_t)threads * chain_vec) == 0 &&
                                 N(loop_ranges.back()).arg % chain_vec == 0 && (oc == CF32 || oc == CF16) && it.bufs[0].dtype != DT_BF16;
        std::string wide;
        if (chunk_sweep) wide = chain_wide_loads(body, loop_ranges.back(), -1);
        std::string v = val(body, -1);
        if (!err.empty()) return false;
        c << prelude.code;
        if (has_inner) {
            if (chunk_sweep) {
                c << "  _Pragma(\"unroll\") for (int gb = threadIdx.x * " << chain_vec << "; gb < " << inner << "; gb += " << threads * chain_vec << ") {\n";
                c << "    " << bt << " outv[" << chain_vec << "];\n";
                // the loads are written with the chunk's first index; the per-element scope below shadows it
                c << "    const int gi = gb; (void)gi;\n" << decompose("gi", 1, loop_ranges.size(), "    ") << wide;
                c << "  _Pragma(\"unroll\") for (int u = 0; u < " << chain_vec << "; u++) { const int gi = gb + u;\n";
            } else {
                c << (inner <= (int64_t)threads * 32 ? "  _Pragma(\"unroll\")\n" : "");
                c << "  for (int gi = threadIdx.x; gi < " << inner << "; gi += " << threads << ") {\n";
            }
            c << decompose("gi", 1, loop_ranges.size(), "    ");
            c << top.code;
            if (chunk_sweep) {
                c << "    outv[u] = " << store_value(v, body) << ";\n  }\n";
                c << "    stv_<" << bt << ", " << chain_vec << ">(" << dp << "0 + ((long long)row * " << inner << "LL + gb), outv);\n";
            } else c << "    " << dp << "0[(long long)row * " << inner << "LL + gi] = " << store_value(v, body) << ";\n";
            c << "  }\n";
        } else {
            c << top.code;
            c << "  " << result_var << " = " << store_value(v, body) << ";\n";
            c << "  if (threadIdx.x == 0) " << dp << "0[row] = " << result_var << ";\n";
        }
        c << "  }\n";
        code = c.str();
        return true;
    }

    // Every REDUCE is invariant along the trailing `ninv` output ranges (a row statistic consumed by
    // an elementwise expression over the row, the shape epilogue fusion produces for softmax-like
    // graphs, schedule/schedule.go:197-233).  The reference re-runs the reduction for every output
    // element; here one block owns one outer index, all threads cooperate on each reduction once,
    // then sweep the invariant ranges.
    bool build_rowbcast(Rendered& out, size_t ninv, int64_t inner) {
        threads = opts.block_threads > 0 ? opts.block_threads : 256;
        lanes = threads; touts = 1; rc_layout = true;
        size_t nouter = loop_ranges.size() - ninv;
        int64_t outer = 1; bool osym = false;
        for (size_t k = 0; k < nouter; k++) { if (N(loop_ranges[k]).symbolic()) osym = true; else outer *= N(loop_ranges[k]).arg; }
        reset_emit();
        reduce_combine_mode = "group";
        std::ostringstream k;
        k << reduce_macros(false) << preamble();
        std::string name = "reduce_rowbcast";
        k << signature(name, false, threads) << " {\n";
        k << "  __shared__ float red_smem[" << std::max(threads / 32, 1) << "];\n";
        k << "  const int lane = threadIdx.x, grp = 0;\n";
        k << "  const long long go = blockIdx.x;\n";
        k << decompose("go", 0, nouter);
        cur_top = &prelude;
        for (int r : reduces) { val(r, -1); if (!err.empty()) return false; }
        cur_top = nullptr;
        std::string v = val(body, -1);
        if (!err.empty()) return false;
        k << prelude.code;
        k << "  for (int gi = threadIdx.x; gi < " << inner << "; gi += " << threads << ") {\n";
        k << decompose("gi", nouter, loop_ranges.size(), "    ");
        k << top.code;
        k << "    data0[go * " << inner << "LL + gi] = " << store_value(v, body) << ";\n";
        k << "  }\n}\n";
        out.klass = KC_REDUCE;
        out.source = k.str();
        out.main.entry = name;
        out.main.block = threads;
        out.main.outputs_per_block = 1;
        out.main.static_outputs = outer;
        out.main.sym_trailing = osym ? outer : 0;
        out.uses_sym = has_sym;
        out.note = "reduce row-broadcast inner=" + std::to_string(inner) + " lanes=" + std::to_string(lanes);
        return true;
    }

    bool build_reduce(Rendered& out) {
        if (opts.reduce_lanes == 0 && opts.split <= 1 && enum_out.empty() && enum_reduce.empty()) {
            size_t ninv = 0; int64_t inner = 1;
            for (int k = (int)loop_ranges.size() - 1; k >= 0; k--) {
                int r = loop_ranges[k];
                if (N(r).symbolic()) break;
                bool used = false;
                for (int red : reduces) if (dep[red][range_slot[r]]) used = true;
                if (used) break;
                ninv++; inner *= N(r).arg;
            }
            if (ninv > 0 && inner >= 64) return build_rowbcast(out, ninv, inner);
        }
        int64_t total = static_total();
        int64_t rmax = 0; bool rsym = false;
        for (int r : reduces) { int64_t t = reduce_total(r); if (t == 0) rsym = true; rmax = std::max(rmax, t); }
        if (rsym) rmax = 0;
        int64_t est_total = sym_output() ? total * (opts.sym_hint > 0 ? opts.sym_hint : 1024) : total;
        choose_layout(est_total, rmax);

        // split one long reduction over several blocks?
        int split = 1;
        if (reduces.size() == 1 && !rsym && !sym_output() && opts.split != 1) {
            if (opts.split > 1) split = opts.split;
            else if (total <= 64 && rmax >= (1 << 16)) {
                int64_t s = std::max<int64_t>(2, (148 * 4) / std::max<int64_t>(total, 1));
                s = std::min<int64_t>(s, rmax / 4096);
                split = (int)std::max<int64_t>(1, std::min<int64_t>(s, 1024));
            }
        }
        if (split > 1 && enum_out.empty()) return build_split(out, split, total, rmax);
        // a switch over output ranges is only safe where the threads that synchronise share the case:
        // no cooperation at all (one lane per output) or one output per block
        if (!enum_out.empty() && !(lanes == 1 || touts == 1)) enum_out.clear();

        reset_emit();
        reduce_combine_mode = "group";
        std::ostringstream k;
        k << reduce_macros(false) << preamble();
        std::string name = "reduce_fused";
        k << signature(name, false, threads) << " {\n";
        k << "  __shared__ float red_smem[" << (rc_layout ? std::max(threads / 32, 1) : threads) << "];\n";
        if (rc_layout) k << "  const int lane = threadIdx.x % LANES, grp = threadIdx.x / LANES;\n";
        else k << "  const int grp = threadIdx.x % TOUTS, lane = threadIdx.x / TOUTS;\n";
        k << "  long long g = (long long)blockIdx.x * TOUTS + grp;\n";
        k << "  const bool valid = g < " << total_expr() << ";\n";
        k << "  if (!valid) g = " << total_expr() << " - 1;\n";
        k << decompose("g");
        if (enum_out.empty()) {
            std::string v = val(body, -1);
            if (!err.empty()) return false;
            k << top.code;
            k << "  if (valid && lane == 0) data0[g] = " << store_value(v, body) << ";\n";
        } else {
            // one case per combination of the enumerated output ranges; inside a case they are constants
            std::string sel = "0";
            int64_t cases = 1;
            for (int r : enum_out) { sel = "(" + sel + " * " + std::to_string(N(r).arg) + " + r" + std::to_string(N(r).aux) + ")"; cases *= N(r).arg; }
            k << "  switch (" << sel << ") {\n";
            for (int64_t cs = 0; cs < cases; cs++) {
                int64_t rem = cs;
                for (int e = (int)enum_out.size() - 1; e >= 0; e--) { fix_range(enum_out[e], rem % N(enum_out[e]).arg); rem /= N(enum_out[e]).arg; }
                top = Block(); loop.clear(); memo.clear();
                std::string v = val(body, -1);
                if (!err.empty()) return false;
                k << "  case " << cs << ": {\n" << top.code;
                k << "  if (valid && lane == 0) data0[g] = " << store_value(v, body) << ";\n  } break;\n";
            }
            for (int r : enum_out) unfix_range(r);
            k << "  }\n";
        }
        k << "}\n";
        out.klass = KC_REDUCE;
        out.source = k.str();
        out.main.entry = name;
        out.main.block = threads;
        out.main.outputs_per_block = touts;
        out.main.static_outputs = total;
        out.main.sym_trailing = sym_output() ? total : 0;
        out.uses_sym = has_sym;
        out.note = std::string("reduce ") + (rc_layout ? "RC" : "OC") + " lanes=" + std::to_string(lanes) + " touts=" + std::to_string(touts);
        if (!enum_reduce.empty()) out.note += " value-by-value reduce";
        if (!enum_out.empty()) out.note += " switch over " + std::to_string(enum_out.size()) + " output ranges";
        return true;
    }

    bool build_split(Rendered& out, int split, int64_t total, int64_t rtot) {
        // partials kernel: block b reduces chunk (b % SPLIT) of output (b / SPLIT)
        threads = opts.block_threads > 0 ? opts.block_threads : 256;
        lanes = threads; touts = 1; rc_layout = true;
        int red = reduces[0];
        Cls rc = dtype_cls(N(red).dtype);
        bool isf = (rc == CF32 || rc == CF16);
        reset_emit();
        reduce_combine_mode = "partial";
        std::ostringstream k;
        k << "#define SPLIT " << split << "\n";
        k << reduce_macros(true) << preamble();
        k << "__device__ __forceinline__ int part_begin(int n);\n__device__ __forceinline__ int part_end(int n);\n";
        std::string pname = "reduce_partials", fname = "reduce_finish";
        k << signature(pname, true, threads) << " {\n";
        k << "  __shared__ float red_smem[" << std::max(threads / 32, 1) << "];\n";
        k << "  const int lane = threadIdx.x, grp = 0;\n";
        k << "  const long long g = blockIdx.x / SPLIT;\n";
        k << decompose("g");
        // evaluate only the REDUCE; its hoisted operands land in `top`
        std::string accv = val(red, -1);
        (void)accv;
        if (!err.empty()) return false;
        k << top.code;
        std::string acc = "acc" + std::to_string(red);
        k << "  if (lane == 0) scratch[blockIdx.x] = " << (isf ? acc : "__int_as_float((int)" + acc + ")") << ";\n";
        k << "}\n";
        int64_t chunk = (rtot + split - 1) / split;
        k << "__device__ __forceinline__ int part_begin(int n) { return (int)((blockIdx.x % SPLIT) * " << chunk << "LL); }\n";
        k << "__device__ __forceinline__ int part_end(int n) { long long e = ((blockIdx.x % SPLIT) + 1) * " << chunk << "LL; return (int)(e < n ? e : n); }\n";
        // finish kernel
        reset_emit();
        finish_reduce = red;
        reduce_combine_mode = "";
        k << "#undef RED_BEGIN\n#undef RED_END\n#undef RED_STEP\n";
        k << "#define RED_BEGIN(n) 0\n#define RED_END(n) (n)\n#define RED_STEP 1\n";
        k << signature(fname, true, 128) << " {\n";
        k << "  const int lane = 0;\n  (void)lane;\n";
        k << "  const long long g = (long long)blockIdx.x * 128 + threadIdx.x;\n";
        k << "  if (g >= " << total_expr() << ") return;\n";
        k << decompose("g");
        std::string v = val(body, -1);
        if (!err.empty()) return false;
        k << top.code;
        k << "  data0[g] = " << store_value(v, body) << ";\n";
        k << "}\n";
        out.klass = KC_REDUCE_SPLIT;
        out.source = k.str();
        out.split = split;
        out.scratch_elems = total * split;
        out.main.entry = pname;
        out.main.block = threads;
        out.main.outputs_per_block = 1;
        out.main.static_outputs = total * split;
        out.finish.entry = fname;
        out.finish.block = 128;
        out.finish.outputs_per_block = 128;
        out.finish.static_outputs = total;
        out.uses_sym = has_sym;
        out.note = "split reduce parts=" + std::to_string(split);
        return true;
    }

    // The elementwise kernel `it` as a device function for the contraction kernel's epilogue: eight
    // consecutive outputs of one row at a time, paired f16 arithmetic, the value of parameter
    // `acc_param` at the output position taken from registers instead of memory.  Only kernels the
    // paired-f16 vector path covers qualify; everything else stays a launch of its own.
    bool build_epilogue(int acc_param, int64_t M, int64_t Ncols, EpilogueRendered& out) {
        if (!analyse()) return false;
        if (!reduces.empty() || has_sym) return fail("epilogue: not a static elementwise kernel");
        if (loop_ranges.size() != 2 || N(loop_ranges[0]).arg != M || N(loop_ranges[1]).arg != Ncols) return fail("epilogue: iteration space differs from the contraction's output");
        if (it.bufs[0].dtype != DT_F16 || (int)it.bufs.size() > 8) return fail("epilogue: output is not f16 or too many operands");
        std::vector<int> vloads;
        const int V = pick_vector(vloads);
        if (V != 8 || !h2_eligible(V)) return fail("epilogue: not a paired-f16 vector kernel");
        reset_emit();
        h2 = true;
        const int r0 = loop_ranges[0], r1 = loop_ranges[1];
        bool saw_acc = false;
        cur_top = &prelude;
        int vi = 0;
        std::ostringstream loads;
        for (int i = 0; i < n; i++) {
            if (N(i).op != OP_INDEX || i == dst || !is_live(i)) continue;
            const int p = (int)N(N(i).src[0]).arg;
            if (p != acc_param) continue;
            // must be exactly the contraction's own output position
            Lin f = flat_index(i);
            bool ok0, ok1;
            if (f.c != 0 || f.t.size() != 2 || lin_coef(f, r0, ok0) != Ncols || !ok0 || lin_coef(f, r1, ok1) != 1 || !ok1) return fail("epilogue: the consumer reads the contraction at another position");
            vec_load[i] = "acc";
            saw_acc = true;
        }
        if (!saw_acc) return fail("epilogue: the consumer does not read the contraction");
        for (int i : vloads) {
            if (vec_load.count(i)) continue;
            const int p = (int)N(N(i).src[0]).arg;
            Lin f = flat_index(i);
            // the loads live in a function of their own (epi8_load_), so that the contraction kernel can
            // issue them a chunk ahead of the arithmetic that needs them
            const std::string arr = "v" + std::to_string(vi);
            loads << "  ldv_<__half2, 4>(reinterpret_cast<const __half2*>(data" << p << " + " << render(f, -1) << "), raw[" << vi << "]);\n";
            stmt(-1, "const __half2* " + arr + "_raw = raw[" + std::to_string(vi) + "];");
            vi++;
            vec_load[i] = arr + "_raw";
        }
        cur_top = nullptr;
        vec_range = r1;
        const std::string v = val_h2(body);
        if (!err.empty()) return false;
        std::ostringstream k;
        k << "#define LANES 1\n#define TOUTS 1\n#define RC_LAYOUT 1\n" << preamble();
        std::ostringstream head;
        head << "  const int r" << N(r0).aux << " = row; (void)r" << N(r0).aux << ";\n";
        head << "  const int r" << N(r1).aux << " = col; (void)r" << N(r1).aux << ";\n";
        out.params.clear();
        for (int b = 1; b < (int)it.bufs.size(); b++) {
            if (b == acc_param) continue;
            if (it.bufs[b].dtype != DT_F16) return fail("epilogue: an operand is not f16");
            head << "  const __half* __restrict__ data" << b << " = reinterpret_cast<const __half*>(ep[" << out.params.size() << "]); (void)data" << b << ";\n";
            out.params.push_back(b);
        }
        if (out.params.size() > 6) return fail("epilogue: more than six operands");
        // EPI_NRAW groups of 8 consecutive f16 are loaded per call; raw[k] holds group k as four pairs
        k << "#define EPI_NRAW " << vi << "\n";
        k << "__device__ __forceinline__ void epi8_load_(const int row, const int col, const void* const* ep, __half2 (*raw)[4]) {\n";
        k << head.str() << loads.str() << "}\n";
        k << "__device__ __forceinline__ void epi8_(const int row, const int col, const __half2* __restrict__ acc, __half2* __restrict__ out, const void* const* ep, const __half2 (*raw)[4]) {\n";
        k << head.str();
        k << prelude.code;
        k << "  _Pragma(\"unroll\") for (int u = 0; u < 4; u++) {\n" << top.code << "    out[u] = " << v << ";\n  }\n}\n";
        out.source = k.str();
        out.note = "epilogue of " + std::to_string(out.params.size()) + " operands";
        return true;
    }

    bool opts_untuned() const { return !opts.reduce_lanes && !opts.split; }

    bool run(Rendered& out) {
        if (!analyse()) return false;
        if (it.bufs.empty()) return fail("codegen: kernel has no output buffer");
        if (static_total() >= ((int64_t)1 << 31)) return fail("codegen: more than 2^31 outputs");
        if (!reduces.empty() && opts_untuned()) plan_enumeration();
        bool ok = reduces.empty() ? build_elementwise(out) : build_reduce(out);
        return ok && err.empty();
    }
};

}  // namespace

bool match_contraction(const Item& item, Contraction& c) {
    CodegenOpts o;
    Gen g(item, o);
    if (!g.analyse()) return false;
    if (g.reduces.size() != 1 || g.reduces[0] != g.body) return false;
    const Node& red = g.N(g.body);
    if ((int)red.aux != OP_ADD) return false;
    std::vector<int> rr;
    for (size_t s = 1; s < red.src.size(); s++) if (g.N(red.src[s]).op == OP_RANGE) rr.push_back(red.src[s]);
    if (rr.size() != 1) return false;
    int k = rr[0];
    const Node& mul = g.N(red.src[0]);
    if (mul.op != OP_MUL || mul.src.size() != 2) return false;
    int ia = mul.src[0], ib = mul.src[1];
    if (g.N(ia).op != OP_INDEX || g.N(ib).op != OP_INDEX) return false;
    if (g.loop_ranges.empty() || g.loop_ranges.size() > 3) return false;
    // output = [..m ranges.., n]: n is the innermost loop range read by exactly one operand
    int pa = (int)g.N(g.N(ia).src[0]).arg, pb = (int)g.N(g.N(ib).src[0]).arg;
    if (g.N(g.N(ia).src[0]).op != OP_PARAM || g.N(g.N(ib).src[0]).op != OP_PARAM) return false;
    Lin fa = g.flat_index(ia), fb = g.flat_index(ib);
    if (!g.in_bounds(fa, pa) || !g.in_bounds(fb, pb)) return false;
    auto only_ranges = [&](const Lin& l) { for (auto& t : l.t) if (g.atoms[t.first].kind != Atom::RANGE) return false; return true; };
    if (!only_ranges(fa) || !only_ranges(fb)) return false;
    auto coef = [&](const Lin& l, int r) { bool ok; return g.lin_coef(l, r, ok); };
    // decide which operand carries n (the innermost output range)
    int n_range = g.loop_ranges.back();
    if (coef(fa, n_range) != 0 && coef(fb, n_range) == 0) { std::swap(ia, ib); std::swap(pa, pb); std::swap(fa, fb); }
    if (coef(fa, n_range) != 0 || coef(fb, n_range) == 0) return false;
    // remaining output ranges form M; they must index only A, with nested strides
    // a symbolic extent (the bound batch) may be all of M or all of K; its value arrives at launch
    if (g.N(n_range).symbolic()) return false;
    int64_t M = 1, a_sm = 0;
    c.m_sym = false; c.k_sym = g.N(k).symbolic();
    for (int i = (int)g.loop_ranges.size() - 2; i >= 0; i--) {
        int r = g.loop_ranges[i];
        if (coef(fb, r) != 0) return false;
        int64_t ca = coef(fa, r);
        if (g.N(r).symbolic()) {
            if (g.loop_ranges.size() != 2) return false;
            c.m_sym = true; a_sm = ca; M = 0;
            break;
        }
        if (M == 1) a_sm = ca;
        else if (ca != a_sm * M) return false;
        M *= g.N(r).arg;
    }
    if (g.loop_ranges.size() == 1) { M = 1; a_sm = 0; }
    c.a_param = pa; c.b_param = pb;
    c.M = M; c.N = g.N(n_range).arg; c.K = c.k_sym ? 0 : g.N(k).arg;
    c.a_sm = a_sm; c.a_sk = coef(fa, k); c.a_off = fa.c;
    c.b_sn = coef(fb, n_range); c.b_sk = coef(fb, k); c.b_off = fb.c;
    if (c.a_sk == 0 || c.b_sk == 0 || c.b_sn == 0 || ((M > 1 || c.m_sym) && a_sm == 0)) return false;
    c.in_dtype = item.bufs[pa].dtype;
    if (item.bufs[pb].dtype != c.in_dtype) return false;
    c.out_dtype = item.bufs[0].dtype;
    return true;
}

bool render_gemm_epilogue(const Item& consumer, int acc_param, int64_t M, int64_t N, EpilogueRendered& out, std::string& err) {
    CodegenOpts o;
    Gen g(consumer, o);
    bool ok = g.build_epilogue(acc_param, M, N, out);
    if (!ok) err = g.err.empty() ? "epilogue: rejected" : g.err;
    return ok && g.err.empty();
}

bool match_column_sum(const Item& item, int& src_param, int64_t& rows, int64_t& cols) {
    CodegenOpts o;
    Gen g(item, o);
    if (!g.analyse() || g.has_sym) return false;
    if (g.reduces.size() != 1 || g.reduces[0] != g.body || g.loop_ranges.size() != 1) return false;
    const Node& red = g.N(g.body);
    if ((int)red.aux != OP_ADD || red.dtype != DT_F16 || item.bufs[0].dtype != DT_F16) return false;
    std::vector<int> rr;
    for (size_t s = 1; s < red.src.size(); s++) if (g.N(red.src[s]).op == OP_RANGE) rr.push_back(red.src[s]);
    if (rr.size() != 1) return false;
    const int src = red.src[0];
    if (g.N(src).op != OP_INDEX || g.N(g.N(src).src[0]).op != OP_PARAM) return false;
    const int p = (int)g.N(g.N(src).src[0]).arg;
    if (p < 1 || p >= (int)item.bufs.size() || item.bufs[p].dtype != DT_F16) return false;
    const int64_t n = g.N(g.loop_ranges[0]).arg, m = g.N(rr[0]).arg;
    Lin f = g.flat_index(src);
    bool ok0, ok1;
    if (f.c != 0 || f.t.size() != 2 || g.lin_coef(f, rr[0], ok0) != n || !ok0 || g.lin_coef(f, g.loop_ranges[0], ok1) != 1 || !ok1) return false;
    if (item.bufs[p].elems(0) != m * n) return false;
    src_param = p; rows = m; cols = n;
    return true;
}

bool render_row_chain(const std::vector<const Item*>& items, const std::vector<std::vector<std::pair<int, int>>>& chain_reads,
                      const CodegenOpts& opts, ChainRendered& out, std::string& err) {
    if (items.size() < 2 || chain_reads.size() != items.size()) { err = "chain: needs at least two stages"; return false; }
    const int threads = opts.block_threads > 0 ? opts.block_threads : 512;
    std::ostringstream k, sig, body, aligned;
    std::vector<std::string> result(items.size());
    std::vector<bool> inner(items.size(), false);
    int64_t rows = -1;
    // ask for full occupancy (2048 threads per SM): without the second bound the run-time compiler took 36
    // registers for the 8192-wide softmax chain and one of four resident blocks was lost (0.1665 ms
    // against 0.1604 with the bound)
    sig << "extern \"C\" __global__ void __launch_bounds__(" << threads;
    if (threads <= 1024 && 2048 % threads == 0) sig << ", " << 2048 / threads;
    sig << ") row_chain(";
    bool first_arg = true;
    std::string decls;
    for (size_t s = 0; s < items.size(); s++) {
        Gen g(*items[s], opts);
        for (auto& pr : chain_reads[s]) {
            if (pr.second < 0 || pr.second >= (int)s || inner[pr.second]) { err = "chain: stage input is not a per-row result of an earlier stage"; return false; }
            g.chain_subst[pr.first] = result[pr.second];
        }
        std::string decl, code; int64_t r = 0; bool has_inner = false;
        if (!g.build_chain_stage((int)s, threads, decl, code, result[s], r, has_inner)) { err = g.err.empty() ? "chain: stage rejected" : g.err; return false; }
        if (rows >= 0 && r != rows) { err = "chain: stages iterate different row counts"; return false; }
        rows = r;
        inner[s] = has_inner;
        if (has_inner && s + 1 != items.size()) { err = "chain: only the last stage may produce a full row"; return false; }
        decls += decl;
        body << code;
        for (size_t b = 0; b < items[s]->bufs.size(); b++) {
            bool is_chain_out = b == 0;      // written by this kernel: never const/restrict
            std::string ty = std::string(is_chain_out ? "" : "const ") + buf_ctype(items[s]->bufs[b].dtype) + "*";
            sig << (first_arg ? "" : ", ") << ty << " __restrict__ s" << s << "_data" << b << "_";
            // device blocks are 256-byte aligned (pool granularity, 128-element view offsets)
            const std::string local = "s" + std::to_string(s) + "_data" + std::to_string(b);
            aligned << "  " << ty << " __restrict__ " << local << " = (" << ty << ")__builtin_assume_aligned(" << local << "_, 16);\n";
            first_arg = false;
        }
    }
    sig << ")";
    k << "#define LANES " << threads << "\n#define TOUTS 1\n#define RC_LAYOUT 1\n";
    k << "#define RED_BEGIN(n) lane\n#define RED_END(n) (n)\n#define RED_STEP LANES\n";
    k << Gen::preamble();
    k << sig.str() << " {\n";
    k << "  __shared__ float red_smem[" << std::max(threads / 32, 1) << "];\n";
    k << "  const int lane = threadIdx.x, grp = 0;\n  (void)grp;\n";
    k << "  const int row = blockIdx.x;\n";
    k << aligned.str();
    k << decls << body.str() << "}\n";
    out.source = k.str();
    out.block = (unsigned)threads;
    out.rows = rows;
    out.note = "row chain of " + std::to_string(items.size()) + " stages, " + std::to_string(rows) + " rows";
    return true;
}

bool render_cuda(const Item& item, const CodegenOpts& opts, Rendered& out, std::string& err) {
    Gen g(item, opts);
    bool ok = g.run(out);
    if (!ok) err = g.err.empty() ? "codegen: failed" : g.err;
    return ok;
}

}  // namespace anl
