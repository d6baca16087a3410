// CUDA C renderer for scheduled kernels: the sm_100a counterpart of the
// reference's Lower + RenderWGSL pair (codegen/lower.go:98-105, codegen/wgsl.go:36-39).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "kir.hpp"

namespace anl {

enum KernelClass : int {
    KC_ELEMENTWISE = 0,   // no REDUCE node: one thread per V outputs, 128-bit accesses when provable
    KC_REDUCE = 1,        // REDUCE nodes evaluated cooperatively by groups of threads
    KC_REDUCE_SPLIT = 2,  // one REDUCE split over several blocks: partials kernel + finish kernel
    KC_GEMM = 3,          // routed to the hand-written contraction kernels
    KC_RAW = 4            // caller-supplied source
};

// Transform requests, the retargeted form of the reference's four opts
// (codegen/opt.go:50-72): Local → threads per block, Tile → outputs per block,
// Upcast → lanes cooperating on one reduction, Vectorize → elements per access.
struct CodegenOpts {
    int block_threads = 0;     // 0 = heuristic
    int reduce_lanes = 0;      // threads cooperating per output (power of two); 0 = heuristic
    int vector_width = 0;      // 0 = heuristic, 1 disables 128-bit accesses
    int split = 0;             // blocks per output for KC_REDUCE_SPLIT; 0 = heuristic, 1 = never split
    bool debug_bounds = false; // clamp every load and record violations in a status word
};

struct Launch {
    std::string entry;
    unsigned block = 1;
    // grid.x = ceil(outputs / outputs_per_block) where outputs = static_outputs, or
    // sym_value * sym_trailing for a kernel with a symbolic output range
    int64_t static_outputs = 1;
    int64_t sym_trailing = 0;      // >0 when the output count depends on the bound variable
    int64_t outputs_per_block = 1;
    unsigned smem_bytes = 0;
};

struct Rendered {
    int klass = KC_ELEMENTWISE;
    std::string source;            // one translation unit, may define two entry points
    Launch main;                   // the kernel (or the partials kernel of a split reduce)
    Launch finish;                 // KC_REDUCE_SPLIT only
    int split = 1;                 // partials per output
    int64_t scratch_elems = 0;     // f32 partials the split kernels exchange through global memory
    bool uses_sym = false;         // kernel takes the bound variable as its last int argument
    int vector_width = 1;
    std::string note;              // human-readable summary of the decisions taken
};

bool render_cuda(const Item& item, const CodegenOpts& opts, Rendered& out, std::string& err);

// Hash of everything that determines the rendered source (node table, buffer dtypes and
// shapes) and nothing that does not (buffer ids, slots).
uint64_t structure_hash(const Item& item);

}  // namespace anl
