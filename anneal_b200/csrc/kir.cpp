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
        it.hash = fnv1a(item_begin, (size_t)(r.p - item_begin));
        out.push_back(std::move(it));
    }
    if (!r.ok) { err = "kir: truncated blob"; out.clear(); return false; }
    return true;
}

}  // namespace anl
