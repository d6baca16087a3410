/*
 * anneal_cuda.h — C ABI of the B200 device backend for anneal.
 *
 * This is what a Go `backend/cuda` package binds (through cgo or a dlopen-style FFI) to provide
 * anneal's device interfaces, backend/device.go:10-37:
 *
 *     Executor.Run / Close, SymbolicExecutor.RunSymbolic, Benchmarker.Benchmark
 *
 * plus the optional residency, optimiser and data-parallel calls that a CUDA device needs to keep
 * parameters on the GPU between steps.  Every function returns 0 on success and a non-zero
 * anl_status otherwise; none throws, aborts or allocates on behalf of the caller except where
 * stated.  After a failure anl_last_error(dev) describes it.  A schedule crosses the boundary as one
 * kernel-IR blob: the serialised []schedule.ExecItem (schedule/exec.go:6-32); its byte layout is
 * documented in anneal_b200/kir.py.
 *
 * Threading: calls on one anl_device must not overlap (the reference funnels every device call
 * through one owner goroutine, backend/webgpu/open.go:63-82); different devices are independent.
 */
#ifndef ANNEAL_CUDA_H
#define ANNEAL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct anl_device anl_device;
typedef struct anl_buffer anl_buffer;
typedef struct anl_graph anl_graph;

typedef enum {
    ANL_OK = 0,
    ANL_ERR_INVALID = 1,      /* malformed blob or argument */
    ANL_ERR_CUDA = 2,         /* a CUDA runtime / driver call failed */
    ANL_ERR_COMPILE = 3,      /* NVRTC rejected generated or supplied source */
    ANL_ERR_UNSUPPORTED = 4,  /* valid request this backend cannot serve */
    ANL_ERR_NO_DEVICE = 5,    /* no usable GPU, or the GPU lacks a required feature */
    ANL_ERR_COMM = 6,         /* NCCL failure or timeout */
    ANL_ERR_LIMIT = 7         /* a stated size limit was exceeded */
} anl_status;

/* storage dtypes, numbered as the kernel-IR numbers them */
enum { ANL_BOOL = 1, ANL_I32 = 6, ANL_U32 = 7, ANL_F16 = 10, ANL_BF16 = 11, ANL_F32 = 12 };

typedef struct {
    char name[128];
    int sm_major, sm_minor, sm_count;
    size_t total_mem;
    int has_f16, has_bf16, has_tcgen05;
} anl_info;

/* A leaf input of a schedule.  Values travel as float32 whatever the storage dtype and are
 * quantised on upload (backend/webgpu/executor.go:161-179); `resident`, when not NULL, names a
 * device buffer that already holds the data and `data` is ignored. */
typedef struct {
    uint32_t uop_idx;
    const float* data;
    int64_t elems;
    anl_buffer* resident;
} anl_input;

typedef struct { const char* name; int64_t value; } anl_binding;

/* A final output.  In `outs` (filled by the library): `data` is a float32 array of `elems` values
 * that the library allocated, released with anl_outputs_free, unless the output was placed.  In
 * `placed` (filled by the caller): where one output should go instead: `resident` keeps it on the
 * device in that buffer (nothing is copied back), `data` names a caller-owned host array with room
 * for `elems` values (for instance pinned memory). */
typedef struct {
    uint32_t uop_idx;
    float* data;
    int64_t elems;
    anl_buffer* resident;
    int allreduce;   /* placed + resident only: 1 = sum this output over all ranks as soon as its kernel
                        has been queued, on the communication stream, overlapping the rest of the
                        schedule; the run (or graph replay) completes after the reduction.
                        2 = with an update attached (sgd_master) and a length that divides by the rank
                        count: reduce-scatter instead, each rank updates only its own 1/nranks of
                        the parameter and the new parameter values are all-gathered — same bytes on
                        the wire, 1/nranks of the update's memory traffic per GPU.  The f32 masters
                        are then current only in each rank's shard (anl_allgather assembles them) and
                        the gradient buffer holds the reduced sum only there.  Falls back to 1 when
                        the length does not divide. */
    /* placed + resident only, optional: treat this output as the gradient of a parameter and apply
     * anl_sgd_step(sgd_master, sgd_param, this output, sgd_lr, sgd_scale) right behind it (after the
     * all-reduce when one is requested) on the same side stream, so the update of early-finished
     * gradients overlaps the rest of the backward pass.  NULL sgd_master = no update. */
    anl_buffer* sgd_master;
    anl_buffer* sgd_param;
    float sgd_lr, sgd_scale;
} anl_output;

/* Benchmarker result: backend/device.go:30-37 BenchmarkResult, microseconds. */
typedef struct { double min_us, median_us, max_us, mean_us, stddev_us, cv; } anl_bench_result;

/* counters since open: the CUDA-side extension of schedule.CompilerStats (schedule/stats.go:3-18) */
typedef struct {
    uint64_t kernels_launched, gemm_launched, nvrtc_compiles, nvrtc_cache_hits, lower_cache_hits;
    uint64_t h2d_bytes, d2h_bytes, graph_replays, graph_captures, device_allocs;
    uint64_t epilogues_fused;   /* elementwise kernels run inside the epilogue of the contraction before them */
    uint64_t colsums_fused;     /* row-sum kernels finished from partial sums a contraction's epilogue left */
    uint64_t side_launches;     /* small kernels with no later reader that a captured graph runs beside the main stream */
} anl_stats;

/* ── lifecycle: webgpu.Open / Device.Close / AdapterName / HasShaderF16 (backend/webgpu/open.go:89-175) ── */
int anl_open(int ordinal, unsigned flags, anl_device** out);
void anl_close(anl_device* dev);
int anl_device_info(anl_device* dev, anl_info* info);
const char* anl_last_error(anl_device* dev);
int anl_get_stats(anl_device* dev, anl_stats* out);
/* flags for anl_open */
#define ANL_OPEN_DEBUG_BOUNDS 1u   /* clamp and check every generated load */
#define ANL_OPEN_NO_GEMM 2u        /* never route contractions to the tensor-core kernels */
#define ANL_OPEN_NO_ROW_CHAIN 8u    /* launch every item on its own instead of fusing per-row kernel chains */
#define ANL_OPEN_BEAM 4u           /* apply / search autotuned transforms (the reference's ANNEAL_BEAM=1) */
#define ANL_OPEN_NO_EPILOGUE_FUSION 32u /* launch a contraction, its elementwise consumer and a bias gradient separately */
#define ANL_OPEN_NO_TF32X3 64u          /* keep f32 contractions of more than 32 rows off the tensor cores' 3 x TF32 form: fused
                                         multiply-add in ascending k on the FP32 pipes instead */
#define ANL_OPEN_TAIL_SPLIT 16u    /* split the last all-reduced contraction into two row windows even on one rank
                                      (done by itself when ranks > 1; the flag exists to test the path on one GPU) */

/* ── Executor.Run / SymbolicExecutor.RunSymbolic (backend/device.go:10-28; backend/webgpu/executor.go:26-240, 576-810) ──
 * Runs the items of `blob` in order.  `outs` has room for `*n_outs` entries on entry; on return
 * `*n_outs` is the number of final outputs (buffers no later item reads, plus written buffers the
 * planner left with slot -1 although a later item reads them) and the first entries of `outs`
 * describe them.  Inputs with unknown ids are ignored; an empty schedule returns 0 outputs.
 * `binds` gives the value of each symbolic variable; pass n_binds = 0 for a static schedule.
 * `placed` (may be NULL) redirects chosen outputs, see anl_output. */
int anl_run(anl_device* dev, const uint8_t* blob, size_t blob_len,
            const anl_input* inputs, int n_inputs,
            const anl_binding* binds, int n_binds,
            const anl_output* placed, int n_placed,
            anl_output* outs, int* n_outs);
void anl_outputs_free(anl_output* outs, int n_outs);

/* ── codegen.Lower + RenderWGSL (codegen/lower.go:98-105, codegen/wgsl.go:36-39), CUDA flavour ──
 * Renders item `index` of the blob to CUDA C without touching the GPU.  `opts` (NULL, or
 * ANL_NUM_OPTS ints, in every call that takes them) is {block_threads, reduce_lanes, vector_width,
 * split, debug_bounds} for generated kernels followed by {tile_n, stages, group_m, stream_stores,
 * single_cta, whole_tail} for the tcgen05 contraction kernels — the reference's Local / Upcast / Vectorize /
 * Tile choices (codegen/opt.go:57-72) retargeted; 0 means "choose", group_m -1 "no grouping".  The
 * source is copied to `src` (capacity src_cap, always NUL-terminated) and its full length is
 * returned in *src_len; `klass`, `block`, `outputs_per_block` describe the launch. */
#define ANL_NUM_OPTS 11
int anl_lower(anl_device* dev_or_null, const uint8_t* blob, size_t blob_len, int index, const int* opts,
              char* src, size_t src_cap, size_t* src_len, int* klass, int* block, int64_t* outputs_per_block,
              char* note, size_t note_cap);

/* Renders items [first, first+count) of the blob as one row-chain kernel (one block per row, the
 * stages back to back, per-row results in registers) if they qualify; ANL_ERR_UNSUPPORTED with the
 * reason in `note` otherwise.  anl_run does this by itself; the call exists for inspection. */
int anl_lower_chain(const uint8_t* blob, size_t blob_len, int first, int count,
                    char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap);

/* The source of the two-CTA tcgen05 contraction kernel as it would be compiled for item `index`
 * (a dense f16 sum of products with at least 256 output rows), with the elementwise kernel of item
 * index+1 in its epilogue when `fuse_next` is not 0; ANL_ERR_UNSUPPORTED with the reason in `note`
 * when the item does not take that kernel or the next item does not fuse.  anl_run makes this choice
 * by itself; the call exists for inspection (the reference prints its kernels the same way,
 * cmd_kernels.go:59-96) and needs no GPU. */
int anl_lower_gemm(anl_device* dev_or_null, const uint8_t* blob, size_t blob_len, int index, int fuse_next, const int* opts,
                   char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap);

/* NVRTC-compiles CUDA C for sm_100a; needs no GPU.  Returns ANL_ERR_COMPILE with the log in `log`. */
int anl_compile_check(const char* src, char* log, size_t log_cap);

/* ── Benchmarker.Benchmark (backend/webgpu/benchmark.go:18-208): CUDA-event timing of one item ── */
int anl_benchmark(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, const int* opts,
                  int warmup, int iterations, anl_bench_result* out);

/* ── codegen.BeamSearch / BeamApplyToItems (codegen/beam.go:271-406, 470-541) ──
 * Searches the transform space of one generated kernel {threads per block, lanes per reduction,
 * vector width, split}: beam of `width` (default 4), at most `depth` levels (default 4), one knob
 * changed per level, candidates timed with CUDA events (min of 5 after 2 warm-ups) on the
 * reference's deterministic test inputs, rejected unless the output matches the default kernel's
 * (bit-identical without a REDUCE, 1e-4 relative with one).  The winner is stored in a disk cache
 * (`cache_path`, or $ANNEAL_BEAM_CACHE, or ~/.cache/anneal/beam_cache_cuda.json) keyed by the
 * kernel's structure hash and guarded by its default source hash.  A device opened with
 * ANL_OPEN_BEAM applies cached winners in anl_run and searches on a miss.
 * A dense f16 contraction (routed to the tcgen05 kernels) is searched over that kernel's tunables
 * instead: `opts` is then {tile_n, stages, group_m, flags} with flags bit 0 = streaming stores,
 * bit 1 = one-CTA kernel, and the guard is bit-identity (none of them reorders a sum). */
typedef struct { int opts[4]; double base_us, best_us; int candidates_tried, candidates_rejected, from_cache; } anl_beam_result;
int anl_beam_search(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, int width, int depth,
                    const char* cache_path, anl_beam_result* out);

/* ── JIT replay (tensor/jit.go:179-246): a schedule frozen into a CUDA graph ──
 * anl_graph_create runs nothing; the first anl_graph_replay instantiates buffers, compiles the
 * kernels and captures them on the device stream; later replays with the same bindings relaunch
 * the captured graph.  Inputs and outputs follow anl_run, with one difference: a replay of a built
 * graph whose inputs and outputs are all resident buffers returns as soon as the graph is queued,
 * without waiting for the GPU (the next download, anl_synchronize or host-bound output waits). */
int anl_graph_create(anl_device* dev, const uint8_t* blob, size_t blob_len, anl_graph** out);
int anl_graph_replay(anl_graph* g, const anl_input* inputs, int n_inputs,
                     const anl_binding* binds, int n_binds,
                     const anl_output* placed, int n_placed, anl_output* outs, int* n_outs);
void anl_graph_release(anl_graph* g);

/* ── resident buffers: Parameter.Load / Value without the per-step round trip (tensor/nn/nn.go:56-61) ── */
int anl_buffer_create(anl_device* dev, int dtype, int64_t elems, anl_buffer** out);
int anl_buffer_upload(anl_buffer* buf, const float* data, int64_t elems);
int anl_buffer_download(anl_buffer* buf, float* data, int64_t elems);
/* Read-back that does not stall the host: `begin` queues the copy of the first `elems` values (as
 * float32) into `host` (pinned memory) behind the work already queued and returns; `wait` blocks
 * until the last copy begun on this buffer has landed.  Lets a loop read step i's loss while step
 * i+1 runs (the reference reads every output back before Run returns, executor.go:205-240). */
int anl_buffer_download_begin(anl_buffer* buf, float* host, int64_t elems);
int anl_buffer_download_wait(anl_buffer* buf);
/* Pipelined upload of the next batch (the data-loader side of examples/mlp.go:111-142, where the
 * reference re-uploads x and y inside Run every step).  `upload_begin` queues the host-to-device
 * copy on a copy stream into a staging block and returns; the buffer still holds the previous
 * contents and kernels already queued keep reading them.  `upload_commit` makes the compute stream
 * wait for that copy and convert it into the buffer, in order with the launches around it.  `data`
 * should be pinned (anl_host_alloc) and must stay unchanged until the commit has executed. */
int anl_buffer_upload_begin(anl_buffer* buf, const float* data, int64_t elems);
int anl_buffer_upload_commit(anl_buffer* buf);
/* The same first half for host data that is already in the buffer's storage format: IEEE half
 * bit patterns (2 bytes each) for an f16 buffer, 4-byte slots otherwise (a bf16 slot with its low
 * 16 bits clear).  The reference quantises a leaf on the host when it is set (tensor/tensor.go:58-68)
 * and again on upload (backend/webgpu/executor.go:166-175); a loader that keeps its batches in the
 * stored format moves half the bytes for f16 and needs no conversion pass on the device. */
int anl_buffer_upload_begin_stored(anl_buffer* buf, const void* data, int64_t elems);
void anl_buffer_release(anl_buffer* buf);
/* A window [offset, offset+elems) of `parent` as a buffer of its own (same dtype, no copy).  Used
 * to lay all parameters, or all gradients, out in one contiguous bucket so that one all-reduce and
 * one optimiser launch cover them.  `offset` must be a multiple of 128 elements.  Release the view
 * before the parent. */
int anl_buffer_view(anl_buffer* parent, int64_t offset, int64_t elems, anl_buffer** out);
void* anl_buffer_device_ptr(anl_buffer* buf);
int64_t anl_buffer_elems(anl_buffer* buf);

/* ── Parameter.SGDStep / SGD.Step on the device (tensor/nn/nn.go:69-76, 98-106) ──
 * master[i] -= lr * grad[i] * grad_scale in f32 (master is an F32 buffer), then param[i] =
 * quantise(master[i]) into `param` (F16/BF16/F32 storage; may equal master). */
int anl_sgd_step(anl_device* dev, anl_buffer* master, anl_buffer* param, anl_buffer* grad, float lr, float grad_scale);

/* ── data parallelism (no counterpart in the reference, which is single-device: README.md:109-111) ──
 * One process per GPU.  Rank 0 obtains an id, every rank passes the same 128 bytes to init. */
int anl_comm_unique_id(uint8_t id[128]);
int anl_comm_init(anl_device* dev, int rank, int nranks, const uint8_t id[128]);
int anl_allreduce_sum(anl_device* dev, anl_buffer* buf);     /* in place, on the comm stream, ordered after prior work */
int anl_allgather(anl_device* dev, anl_buffer* buf);         /* in place: rank r contributes elements [r*n/R, (r+1)*n/R) */
int anl_comm_destroy(anl_device* dev);
/* Watchdog.  With a timeout set (milliseconds, 0 = none), anl_comm_wait — and anl_synchronize,
 * which calls it first — polls the communication stream instead of blocking on it, asks NCCL for
 * asynchronous errors, and on an error or when the time is up aborts the communicator
 * (ncclCommAbort), returns ANL_ERR_COMM and makes every later collective fail until anl_comm_init
 * is called again.  anl_comm_abort does the same on request (another rank was reported dead by the
 * launcher).  anl_comm_inject_delay is host-side failure injection for tests: a host callback
 * holds the communication stream back; nothing on the GPU faults or spins. */
int anl_comm_set_timeout(anl_device* dev, int milliseconds);
int anl_comm_wait(anl_device* dev);
int anl_comm_abort(anl_device* dev);
int anl_comm_inject_delay(anl_device* dev, int milliseconds);

/* host staging memory that the GPU can copy from directly */
int anl_host_alloc(size_t bytes, void** out);
void anl_host_free(void* p);

/* ── timing (Benchmarker's clock, for whole steps): CUDA events on the compute stream ── */
int anl_timer_start(anl_device* dev);
int anl_timer_stop(anl_device* dev, float* elapsed_ms);   /* waits for the stop event */

/* Per-kernel-class breakdown.  While enabled every launch is bracketed by an event pair (this
 * perturbs back-to-back launches slightly, so do not take whole-step times with it on).
 * anl_profile_read waits for the device, then returns one entry per kernel class seen since the
 * last anl_profile_enable(dev, 1). */
typedef struct { int klass; int launches; double total_ms; double flops; } anl_profile_entry;
int anl_profile_enable(anl_device* dev, int on);
int anl_profile_read(anl_device* dev, anl_profile_entry* out, int cap, int* n);

/* ── sum of an f32 device array without touching the allocator (no counterpart in the reference) ──
 * For callers that cannot allocate: a host whose own pool already owns all device memory, or a loop
 * that cannot take cudaMalloc's device-wide synchronisation.  `x` (n values) and `out` (1 value) are
 * device pointers the caller owns; the work is queued on `stream` (a cudaStream_t, NULL for the
 * default stream) and is not waited for.  The two-stage reduction keeps its partials in a 4 KiB
 * array that is part of the library image on every GPU, so n is limited to [1, 2^30]; other sizes
 * return ANL_ERR_LIMIT with the reason in `err`.  The first call on each device also looks up that
 * array's address, so make it before starting any stream capture.  All calls on a device share the
 * array: two calls whose kernels can overlap (different streams) race; calls on one stream do not. */
int anl_sum_f32_static(const float* x, int64_t n, float* out, void* stream, char* err, size_t err_cap);

/* blocks until all work queued on the device has finished */
int anl_synchronize(anl_device* dev);

/* Device-wide tunables of the tcgen05 contraction kernel, for a deployment that has searched them
 * offline (anl_beam_search) and wants them applied to every contraction without opening the device
 * in search mode: `opts` as everywhere (ANL_NUM_OPTS ints; only the contraction fields are read,
 * NULL resets to the built-in heuristics).  A plan's own tunables, when a search set them, win. */
int anl_gemm_set_defaults(anl_device* dev, const int* opts);

/* Diagnostic: leaves the device as a contraction launch does whose bounded barrier wait ran out — a
 * non-zero code in the host-visible status word and tile counters holding `counter_value` — without
 * any kernel waiting or failing.  The next call that waits for the device (anl_run, a replay,
 * anl_synchronize) must then return ANL_ERR_CUDA once, and the calls after it must run correctly
 * again.  No counterpart in the reference. */
int anl_gemm_inject_status(anl_device* dev, int code, int counter_value);

/* The cudaStream_t this device queues its kernels and copies on (non-blocking: it is not ordered
 * with the default stream).  A caller that launches work of its own on device buffers — through
 * anl_sum_f32_static, say — passes this handle to stay in order with uploads, runs and downloads;
 * anl_synchronize then covers that work too.  No counterpart in the reference, whose queue is
 * private to its owner goroutine (backend/webgpu/open.go:63-82). */
void* anl_stream(anl_device* dev);

#ifdef __cplusplus
}
#endif
#endif
