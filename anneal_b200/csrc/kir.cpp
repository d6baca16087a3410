#include "kir.hpp"

#include <cstring>

namespace anl {

uint64_t fnv1a(const void* p, size_t n, uint64_t h) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}

namespace {
struct Reader {
    const uint8_t* p; const uint8_t* end; bool ok = true;
    template <class T> T get() {
        T v{};
        if (p + sizeof(T) > end) { ok = false; return v; }
        std::memcpy(&v, p, sizeof(T)); p += sizeof(T);
        return v;
    }
    bool skip(size_t n) { if (p + n > end) { ok = false; return false; } p += n; return true; }
};

// Structural checks on one parsed item, so that the code generator and the runtime can index
// `bufs`, `src` and shapes without re-checking: known opcodes with at least the sources they
// need, PARAM numbers inside the buffer table, INDEX rooted at a PARAM, extents and shapes that are
// non-negative and small enough that no product of them overflows 63 bits.
bool validate_item(const Item& it, std::string& err) {
    const int64_t kMaxExtent = (int64_t)1 << 40;
    for (const BufDesc& b : it.bufs) {
        if (b.dtype < DT_BOOL || b.dtype > DT_INDEX) { err = "kir: unknown buffer dtype"; return false; }
        if (b.size < 0 || b.size > kMaxExtent) { err = "kir: buffer size out of range"; return false; }
        int64_t prod = 1; int zeros = 0;
        for (int64_t d : b.shape) {
            if (d < 0 || d > kMaxExtent) { err = "kir: buffer shape out of range"; return false; }
            if (d == 0) { zeros++; continue; }
            if (prod > kMaxExtent / d) { err = "kir: buffer has more than 2^40 elements"; return false; }
            prod *= d;
        }
        if (zeros > 1) { err = "kir: more than one symbolic dimension in a buffer"; return false; }
    }
    for (size_t i = 0; i < it.nodes.size(); i++) {
        const Node& nd = it.nodes[i];
        size_t need = 0;
        switch (nd.op) {
            case OP_PARAM:
                if (nd.arg < 0 || nd.arg >= (int64_t)it.bufs.size()) { err = "kir: PARAM number outside the buffer table"; return false; }
                break;
            case OP_CONST: break;
            case OP_RANGE:
                if (nd.arg < 0 || nd.arg > kMaxExtent) { err = "kir: RANGE extent out of range"; return false; }
                if (!nd.symbolic() && nd.arg == 0) { err = "kir: empty RANGE"; return false; }
                break;
            case OP_INDEX:
                need = 1;
                if (!nd.src.empty() && it.nodes[nd.src[0]].op != OP_PARAM) { err = "kir: INDEX of a non-parameter"; return false; }
                if (nd.src.size() > 9) { err = "kir: INDEX with more than 8 coordinates"; return false; }
                break;
            case OP_CAST: case OP_BITCAST: case OP_EXP2: case OP_LOG2: case OP_SIN: case OP_SQRT: case OP_RECIP:
            case OP_NEG: case OP_TRUNC: case OP_SINK: case OP_END: case OP_REDUCE:
                need = 1; break;
            case OP_ADD: case OP_MUL: case OP_SHL: case OP_SHR: case OP_IDIV: case OP_MAX: case OP_MOD: case OP_CMPLT:
            case OP_CMPNE: case OP_CMPEQ: case OP_XOR: case OP_OR: case OP_AND: case OP_SUB: case OP_FDIV: case OP_POW:
            case OP_STORE:
                need = 2; break;
            case OP_WHERE: case OP_MULACC:
                need = 3; break;
            default:
                err = "kir: unknown opcode " + std::to_string(nd.op); return false;
        }
        if (nd.src.size() < need) { err = "kir: node with too few sources"; return false; }
        if (nd.dtype < DT_VOID || nd.dtype > DT_INDEX) { err = "kir: unknown node dtype"; return false; }
    }
    if (!it.nodes.empty() && it.nodes.back().op != OP_SINK) { err = "kir: last node is not the SINK"; return false; }
    return true;
}
}  // namespace

bool parse_kir(const uint8_t* blob, size_t len, std::vector<Item>& out, std::string& err) {
    out.clear();
    if (!blob || len < 8 || std::memcmp(blob, "KIR1", 4) != 0) { err = "kir: bad magic"; return false; }
    Reader r{blob + 4, blob + len};
    uint32_t n_items = r.get<uint32_t>();
    for (uint32_t k = 0; k < n_items && r.ok; k++) {
        const uint8_t* item_begin = r.p;
        Item it;
        uint32_t n_nodes = r.get<uint32_t>(), n_srcs = r.get<uint32_t>(), n_bufs = r.get<uint32_t>();
        uint32_t n_sym = r.get<uint32_t>(), src_len = r.get<uint32_t>();
        for (int i = 0; i < 3; i++) it.local[i] = r.get<uint32_t>();
        for (int i = 0; i < 3; i++) it.grid[i] = r.get<uint32_t>();
        if (!r.ok) break;
        if ((size_t)(r.end - r.p) < (size_t)n_nodes * 24 + (size_t)n_srcs * 4) { r.ok = false; break; }
        const uint8_t* nodes_p = r.p;
        r.skip((size_t)n_nodes * 24);
        const uint8_t* srcs_p = r.p;
        r.skip((size_t)n_srcs * 4);
        it.nodes.resize(n_nodes);
        for (uint32_t i = 0; i < n_nodes; i++) {
            const uint8_t* q = nodes_p + (size_t)i * 24;
            uint16_t op; uint32_t nsrc, off, aux; int64_t arg;
            std::memcpy(&op, q, 2); std::memcpy(&nsrc, q + 4, 4); std::memcpy(&off, q + 8, 4);
            std::memcpy(&aux, q + 12, 4); std::memcpy(&arg, q + 16, 8);
            Node& nd = it.nodes[i];
            nd.op = op; nd.dtype = q[2]; nd.flags = q[3]; nd.aux = aux; nd.arg = arg;
            if ((uint64_t)off + nsrc > n_srcs) { err = "kir: source list out of range"; return false; }
            nd.src.resize(nsrc);
            for (uint32_t s = 0; s < nsrc; s++) {
                uint32_t v; std::memcpy(&v, srcs_p + ((size_t)off + s) * 4, 4);
                if (v >= i) { err = "kir: nodes are not in sources-before-users order"; return false; }
                nd.src[s] = (int)v;
            }
        }
        // every buffer record takes at least 20 bytes, every name at least 2
        if ((size_t)(r.end - r.p) / 20 < n_bufs || (size_t)(r.end - r.p) / 2 < n_sym) { r.ok = false; break; }
        it.bufs.resize(n_bufs);
        for (uint32_t b = 0; b < n_bufs && r.ok; b++) {
            BufDesc& bd = it.bufs[b];
            bd.id = r.get<uint32_t>(); bd.slot = r.get<int32_t>();
            bd.dtype = r.get<uint8_t>(); int rank = r.get<uint8_t>(); r.get<uint16_t>();
            bd.size = r.get<int64_t>();
            if (rank > 8) { err = "kir: buffer rank above 8"; return false; }
            bd.shape.resize(rank);
            for (int d = 0; d < rank; d++) bd.shape[d] = r.get<int64_t>();
        }
        for (uint32_t s = 0; s < n_sym && r.ok; s++) {
            uint16_t l = r.get<uint16_t>();
            if (!r.ok || (size_t)(r.end - r.p) < l) { r.ok = false; break; }
            it.sym_vars.emplace_back(reinterpret_cast<const char*>(r.p), l);
            r.skip(l);
        }
        if (r.ok && (size_t)(r.end - r.p) >= src_len) {
            it.source.assign(reinterpret_cast<const char*>(r.p), src_len);
            r.skip(src_len);
        } else {
            r.ok = false;
        }
        if (!r.ok) break;
        if (!validate_item(it, err)) { out.clear(); return false; }
        it.hash = fnv1a(item_begin, (size_t)(r.p - item_begin));
        out.push_back(std::move(it));
    }
    if (!r.ok) { err = "kir: truncated blob"; out.clear(); return false; }
    return true;
}

}  // namespace anl
