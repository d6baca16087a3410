// Kernel-IR: the in-memory form of one schedule.ExecItem (schedule/exec.go:6-32)
// as it arrives over the C ABI.  The byte layout is documented beside the
// serialiser (anneal_b200/kir.py); opcodes are anneal's uop.Op values
// (uop/ops.go:12-157).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace anl {

enum Op : int {
    OP_PARAM = 7, OP_SINK = 13, OP_INDEX = 18, OP_STORE = 20, OP_CAST = 22, OP_BITCAST = 23,
    OP_EXP2 = 24, OP_LOG2 = 25, OP_SIN = 26, OP_SQRT = 27, OP_RECIP = 28, OP_NEG = 29, OP_TRUNC = 30,
    OP_ADD = 31, OP_MUL = 32, OP_SHL = 33, OP_SHR = 34, OP_IDIV = 35, OP_MAX = 36, OP_MOD = 37,
    OP_CMPLT = 38, OP_CMPNE = 39, OP_CMPEQ = 40, OP_XOR = 41, OP_OR = 42, OP_AND = 43, OP_SUB = 45,
    OP_FDIV = 46, OP_POW = 47, OP_WHERE = 48, OP_MULACC = 49, OP_RANGE = 51, OP_END = 53, OP_CONST = 56,
    OP_REDUCE = 82
};

enum DT : int {
    DT_VOID = 0, DT_BOOL = 1, DT_I8 = 2, DT_U8 = 3, DT_I16 = 4, DT_U16 = 5, DT_I32 = 6, DT_U32 = 7,
    DT_I64 = 8, DT_U64 = 9, DT_F16 = 10, DT_BF16 = 11, DT_F32 = 12, DT_F64 = 13, DT_INDEX = 14
};

inline bool dt_is_float(int d) { return d == DT_F16 || d == DT_BF16 || d == DT_F32 || d == DT_F64; }
// bytes one element occupies in device memory: f16 is 2, every other dtype sits in a
// 32-bit slot, bf16 included (backend/webgpu/executor.go:473-478, codegen/wgsl.go:433-447)
inline int dt_storage_bytes(int d) { return d == DT_F16 ? 2 : 4; }

struct Node {
    int op = 0, dtype = 0, flags = 0;
    std::vector<int> src;
    uint32_t aux = 0;
    int64_t arg = 0;
    // RANGE helpers
    int axis() const { return flags & 7; }
    bool symbolic() const { return (flags >> 3) & 1; }
    int sym_param() const { return (flags >> 4) & 15; }
};

struct BufDesc {
    uint32_t id = 0;
    int slot = -1, dtype = DT_F32;
    int64_t size = 0;
    std::vector<int64_t> shape;   // 0 marks the symbolic dimension
    bool symbolic() const { for (auto s : shape) if (s == 0) return true; return false; }
    int64_t trailing() const { int64_t p = 1; for (auto s : shape) if (s) p *= s; return p; }
    int64_t elems(int64_t sym_value) const {
        if (shape.empty()) return size > 0 ? size : 1;
        return symbolic() ? trailing() * sym_value : trailing();
    }
};

struct Item {
    std::vector<Node> nodes;      // sources before users; last is the SINK
    std::vector<BufDesc> bufs;    // bufs[0] is the output (PARAM 0)
    std::vector<std::string> sym_vars;
    std::string source;           // optional pre-rendered source
    uint32_t local[3] = {1, 1, 1}, grid[3] = {1, 1, 1};
    uint64_t hash = 0;            // FNV-1a of the item's bytes: the compile / graph cache key
};

// Parses a blob; returns false and fills err on malformed input.
bool parse_kir(const uint8_t* blob, size_t len, std::vector<Item>& out, std::string& err);

uint64_t fnv1a(const void* p, size_t n, uint64_t h = 1469598103934665603ull);

}  // namespace anl
