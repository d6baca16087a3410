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
    int sym_hint = 0;          // value the bound batch is expected to have when a kernel is laid out for it; 0 = 1024
    // contraction kernels (0 = heuristic): tile width, ring depth, raster group (-1: none), streaming
    // stores, one-CTA kernel forced, last wave kept in whole tiles
    int gemm_tile_n = 0, gemm_stages = 0, gemm_group_m = 0, gemm_stream_stores = 0, gemm_single_cta = 0, gemm_whole_tail = 0;
};

struct Launch {
    std::string entry;
    unsigned block = 1, block_y = 1, block_z = 1;   // y and z only for caller-supplied source
    unsigned grid_y = 1, grid_z = 1;
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

// A kernel whose body is exactly SUM_k a[..] * b[..] over two buffers with affine indices:
//   out[m, n] = sum_k A[a_off + m*a_sm + k*a_sk] * B[b_off + n*b_sn + k*b_sk],  out row-major [M, N].
// This is the pattern Tensor.Matmul, nn.Linear and their gradients schedule to
// (tensor/reduce.go:105-166, tensor/nn/nn.go:154-162, tensor/gradient_ruleset.go:137-140, 207-233).
struct Contraction {
    int a_param = 0, b_param = 0;
    int64_t M = 0, N = 0, K = 0;
    int64_t a_sm = 0, a_sk = 0, a_off = 0;
    int64_t b_sn = 0, b_sk = 0, b_off = 0;
    int in_dtype = DT_F32, out_dtype = DT_F32;
    bool m_sym = false, k_sym = false;   // M (or K) is the symbolic batch: 0 here, bound at launch
};
// Contraction selection (the schedule/kernels.go hook the CUDA device adds): true when `item`
// is such a kernel.  Leading output ranges are folded into M when they are contiguous with it.
bool match_contraction(const Item& item, Contraction& out);

// An elementwise kernel that reads a contraction's output at the output's own position, rendered as
// a device function for the contraction kernel's epilogue (the reference splices such a consumer
// into the reduce kernel, schedule/schedule.go:197-233; here the splice happens at launch time, on
// the accumulator's registers, so the scheduled kernels stay what the reference would schedule):
//   __device__ void epi8_(int row, int col, const __half2* acc, __half2* out, const void* const* ep)
// maps the 8 narrowed accumulator values at (row, col .. col+7) to the consumer's 8 outputs, with
// the arithmetic of the stand-alone kernel (paired f16, bit for bit).  `params` lists the consumer's
// other parameter numbers in the order ep[] expects them.
struct EpilogueRendered {
    std::string source, note;
    std::vector<int> params;
};
bool render_gemm_epilogue(const Item& consumer, int acc_param, int64_t M, int64_t N, EpilogueRendered& out, std::string& err);

// True when `item` is out[n] = SUM_m src[m * cols + n] over one f16 buffer with an f16 result: the
// bias gradient of a linear layer (tensor/gradient_ruleset.go:207-233 applied to nn.go:154-162).
bool match_column_sum(const Item& item, int& src_param, int64_t& rows, int64_t& cols);

// Row chain: consecutive kernels that all iterate the same outer ("row") range, reduce only over
// ranges inside the row, and hand each other one value per row (a softmax forward+backward is five
// such kernels).  Rendered as ONE kernel with one block per row: the stages run back to back, each
// stage's per-row result stays in a register for the later stages (and is still written to its
// buffer), and the row's operands are read from DRAM once and from L1/L2 afterwards.  The reference
// launches each stage separately and re-reads every operand from memory each time.
struct ChainRendered {
    std::string source, entry = "row_chain", note;
    unsigned block = 256;
    int64_t rows = 0;
};
// True when `items` (in schedule order, at least two) form such a chain.  `ext_reads[k]` must list,
// for stage k, which of its input parameters are outputs of EARLIER stages of the chain, as
// (parameter number, producing stage).  Kernel arguments: every stage's buffers in order.
bool render_row_chain(const std::vector<const Item*>& items, const std::vector<std::vector<std::pair<int, int>>>& chain_reads,
                      const CodegenOpts& opts, ChainRendered& out, std::string& err);

// Hash of everything that determines the rendered source (node table, buffer dtypes and
// shapes) and nothing that does not (buffer ids, slots).
uint64_t structure_hash(const Item& item);

}  // namespace anl
