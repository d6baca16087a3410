// Device runtime behind the C ABI: context, stream, buffer pool, NVRTC module cache, schedule
// execution.  Replaces backend/webgpu/{open,executor,benchmark}.go of the reference.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/anneal_cuda.h"
#include "codegen.hpp"
#include "kir.hpp"

namespace anl {

struct DriverApi {
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    bool loaded = false;
};

struct Module {
    CUmodule mod = nullptr;
    std::unordered_map<std::string, CUfunction> fn;
};

// One item ready to launch: rendered source, compiled entry points, or a GEMM route.
struct GemmPlan;

// Tunables of the tcgen05 contraction kernels, the retargeted form of the reference's Tile / Upcast
// choices for matmul (codegen/opt.go:206-307, 318-556).  Zero means "let the heuristic decide".
struct GemmTuning {
    int tile_n = 0;         // 256 or 128 columns per tile
    int stages = 0;         // depth of the shared-memory ring
    int group_m = 0;        // raster group in tile rows; -1: down whole columns
    int stream_stores = 0;  // 1: streaming hint on the output stores
    int single_cta = 0;     // 1: the one-CTA kernel even where a CTA pair applies
    int no_split_tail = 0;  // 1: the tiles of a partly filled last wave stay whole
};
constexpr int kDefaultGroupM = 2;     // measured best or within 1% of best on every wide-MLP shape (sweep over -1, 2, 4, 8, 16)

// What the epilogue of one contraction launch does besides (or instead of) storing the contraction.
struct GemmFusion {
    const std::string* epilogue = nullptr;   // generated epi8_() of the elementwise consumer, or null
    void* d_out = nullptr;                   // the consumer's output buffer
    const void* ep[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // its other operands
    bool store_raw = true;                   // false when nothing but the consumer reads the contraction
    float* colsum = nullptr;                 // [ceil(M/32), N] partial column sums of the last value stored
};
// Several consecutive items rendered as one row-chain kernel (codegen.hpp ChainRendered).
struct ChainPlan {
    ChainRendered r;
    CUfunction fn = nullptr;
};

// A contraction and the elementwise kernel behind it, prepared to run as one launch.
struct FusedEpilogue {
    bool on = false;
    EpilogueRendered epi;
    int acc_param = 0;
};

struct Plan {
    Rendered r;
    CUfunction main = nullptr, finish = nullptr;
    // A kernel whose output count follows the bound batch is laid out twice when that changes the
    // layout: for a large batch (threads spread over the outputs) and for a handful of rows (threads
    // cooperate on each output); both are compiled on first use, the launch picks by the bound value.
    Rendered r_small;
    CUfunction main_small = nullptr;
    int64_t small_below = 0;     // bound values below this take the small-batch layout
    std::shared_ptr<GemmPlan> gemm;
    bool gemm_dynamic = false;   // a symbolic extent decides per launch between `gemm` and the rendered kernel
};

}  // namespace anl

struct anl_buffer {
    anl_device* dev = nullptr;
    int dtype = ANL_F32;
    int64_t elems = 0;
    void* ptr = nullptr;
    size_t bytes = 0;
    bool view = false;      // a window of another buffer: the memory is not ours to release
    // pipelined upload: an f32 block the copy stream fills while the compute stream still works on
    // the buffer's current contents
    void* stage = nullptr;
    int64_t staged_elems = 0;
    bool staged_stored = false;   // the staged bytes are already in the buffer's storage format
    cudaEvent_t stage_ready = nullptr, stage_free = nullptr;
    bool stage_free_recorded = false;
    // asynchronous read-back: widening block for f16 buffers, event behind the last copy begun
    void* dl_stage = nullptr;
    int64_t dl_stage_elems = 0;
    cudaEvent_t dl_done = nullptr;
    bool dl_pending = false;
};

struct anl_device {
    int ordinal = 0;
    unsigned flags = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaStream_t copy_stream = nullptr;   // host-to-device staging of the next batch, created on first use
    cudaEvent_t comm_event = nullptr, comm_done = nullptr;
    std::string err;
    cudaDeviceProp prop{};
    anl::DriverApi drv;
    std::unordered_map<uint64_t, std::shared_ptr<anl::Plan>> plans;   // structure hash ^ opts → plan
    std::unordered_map<uint64_t, std::shared_ptr<anl::Module>> modules;  // source hash → module
    std::unordered_map<uint64_t, std::shared_ptr<anl::FusedEpilogue>> fused;   // (contraction, consumer) -> generated epilogue, or a record that they do not fuse
    std::unordered_map<uint64_t, std::shared_ptr<anl::ChainPlan>> chains; // hash of member items → fused kernel, or null if they do not fuse
    std::multimap<size_t, void*> pool;                                // free device blocks by size
    std::unordered_map<void*, size_t> live;                           // blocks handed out
    anl_stats stats{};
    cudaEvent_t timer0 = nullptr, timer1 = nullptr;
    bool profiling = false;
    struct ProfRec { cudaEvent_t e0, e1; int klass; double flops; };
    std::vector<ProfRec> prof;
    struct BeamEntry { uint64_t src_hash = 0; int opts[4] = {0, 0, 0, 0}; double us = 0; };
    std::unordered_map<uint64_t, BeamEntry> beam_cache;
    std::string beam_cache_path;
    bool beam_loaded = false;
    static constexpr int kGemmCounterSlots = 16;
    int* gemm_tile_counter = nullptr;     // device words the persistent GEMMs draw tile numbers from, 256 bytes per stream
    std::vector<cudaStream_t> gemm_counter_streams;   // slot k belongs to this stream
    int* gemm_status_host = nullptr;      // mapped, host-visible: code of a barrier wait that ran out
    int* gemm_status_dev = nullptr;
    bool gemm_attr_set = false;
    std::unordered_map<std::string, void*> pair_kernels;   // configuration (tunables + fused consumer's text) -> loaded two-CTA kernel
    anl::GemmTuning gemm_defaults;        // device-wide tunables of the contraction kernels; a plan's own non-zero fields win
    void* nccl_comm = nullptr;
    int rank = 0, nranks = 1;
    bool comm_pending = false;
    bool comm_aborted = false;            // set by the watchdog: collectives refuse until a new anl_comm_init
    int comm_timeout_ms = 0;              // 0: wait without limit
    int comm_reserved_sms = 0;            // SMs the persistent GEMM leaves to collectives when nranks > 1

    int fail(int code, const std::string& m) { err = m; return code; }
    int alloc(size_t bytes, void** out);
    void release(void* p);
    void trim();
};

namespace anl {

int ensure_driver(anl_device* dev);
int compile_source(anl_device* dev, const std::string& src, std::shared_ptr<Module>& out);
int get_plan(anl_device* dev, const Item& item, const CodegenOpts& opts, std::shared_ptr<Plan>& out);
// keep_scratch: when not null, scratch blocks a launch needs are appended there (the caller releases
// them) instead of going back to the pool at once
int launch_plan(anl_device* dev, const Plan& plan, const Item& item, void* const* bufs, int64_t sym_value, cudaStream_t stream,
                std::vector<void*>* keep_scratch);

// dtype conversion at the boundary (backend/webgpu/executor.go:161-179, 457-519)
int upload_f32(anl_device* dev, void* dst, int dtype, const float* host, int64_t elems, cudaStream_t s);
int download_f32(anl_device* dev, float* host, const void* src, int dtype, int64_t elems, cudaStream_t s);

// hand-written contraction kernels (gemm.cu); returns ANL_OK and fills plan.gemm if the item is a
// dense SUM-of-products over buffers that they cover, ANL_ERR_UNSUPPORTED otherwise
int plan_gemm(const Item& item, const GemmTuning& tune, Plan& plan);
int launch_gemm(anl_device* dev, const Plan& plan, void* const* bufs, int64_t sym_value, cudaStream_t stream,
                int64_t m_begin = 0, int64_t m_end = -1, const GemmFusion* fusion = nullptr, std::vector<void*>* keep_scratch = nullptr);
// true when the plan runs on the two-CTA kernel, the one that can carry a fused consumer
void launch_hold_stream(cudaStream_t stream, unsigned long long ns);
bool gemm_pair_eligible(const Plan& plan);
bool gemm_tf32_eligible(const Plan& plan);
int gemm_tf32_source(const Plan& plan, std::string& out, std::string& note);
void gemm_shape(const Plan& plan, int64_t* M, int64_t* N, int64_t* K);
// compiles the kernel variant a launch of this plan (with this epilogue text) will use
int gemm_prepare(anl_device* dev, const Plan& plan, const std::string& epilogue);
// the source that would be compiled, for inspection
int gemm_pair_source(anl_device* dev, const Plan& plan, const std::string& epilogue, std::string& out);
int launch_colsum_finish(anl_device* dev, const float* partials, int64_t parts, int64_t n, void* out, cudaStream_t stream);
// reports (once) a barrier wait that ran out in an earlier contraction launch and resets the state
int gemm_check_status(anl_device* dev);
int gemm_inject_status(anl_device* dev, int code, int counter_value);
// rows of a static f16 contraction's output, or 0 when the plan is not one (no row windows then)
int64_t gemm_window_rows(const Plan& plan, int64_t* row_elems);
double gemm_flops(const Plan& plan, int64_t sym_value);
// true when this launch (with the symbolic extent bound to sym_value) goes to the contraction kernel
bool gemm_taken(const Plan& plan, int64_t sym_value);
bool gemm_f32_worth(int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk);
bool gemm_tf32_shape_ok(int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk);
int launch_gemm_f32(anl_device* dev, const float* a, const float* b, float* d, int64_t M, int64_t N, int64_t K,
                    int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk, cudaStream_t stream);

// data parallel (comm.cpp): queue an all-reduce of [ptr, ptr+elems) on the communication stream after
// everything queued so far on `stream`; comm_join makes `stream` wait for all of them
int comm_fork(anl_device* dev, cudaStream_t stream);     // side stream waits for everything queued on `stream`
int comm_allreduce_async(anl_device* dev, void* ptr, int64_t elems, int dtype, cudaStream_t stream);
bool comm_can_shard(anl_device* dev);
int comm_reduce_scatter_async(anl_device* dev, void* ptr, int64_t elems, int dtype, cudaStream_t stream);
int comm_allgather_async(anl_device* dev, void* ptr, int64_t elems, int dtype);
int launch_sgd(anl_device* dev, anl_buffer* master, anl_buffer* param, anl_buffer* grad, float lr, float scale, cudaStream_t stream);
int comm_join(anl_device* dev, cudaStream_t stream);
// cudaStreamSynchronize under the collective watchdog: with a communicator and a timeout set the
// wait is a bounded poll that aborts the communicator at the deadline (ANL_ERR_COMM)
int wait_stream_watched(anl_device* dev, cudaStream_t stream, const char* what);

// autotuning (beam.cpp)
int beam_search(anl_device* dev, const Item& it, int width, int depth, anl_beam_result* out);
// the contraction kernel's tunables as a search result packs them: {tile_n, stages, group_m, flags}
CodegenOpts gemm_beam_opts(const int* o, bool debug);
void beam_cache_load(anl_device* dev, const std::string& path);
bool beam_cache_lookup(anl_device* dev, uint64_t key, uint64_t src_hash, int* opts);   // 2*M*N*K of a routed contraction

}  // namespace anl
