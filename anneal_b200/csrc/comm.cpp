// Data-parallel gradient exchange: NCCL all-reduce over NVLink, one process per GPU.
// The reference has no multi-device support at all (README.md:109-111; uop/ops.go:129 lists
// OpAllReduce without any lowering), so this is new surface.  NCCL is bound at run time with
// dlopen so that the library loads on machines without it and shares the copy a host process
// (for example PyTorch) may already have loaded.
#include <dlfcn.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <string>
#include <thread>

#include "runtime.hpp"

namespace {
typedef struct { char internal[128]; } nccl_uid;
struct Nccl {
    void* h = nullptr;
    int (*GetUniqueId)(nccl_uid*) = nullptr;
    int (*CommInitRank)(void**, int, nccl_uid, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*CommAbort)(void*) = nullptr;
    int (*CommGetAsyncError)(void*, int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};
Nccl& nccl() {
    static Nccl n;
    if (n.h) return n;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* nm : names) { n.h = dlopen(nm, RTLD_NOW | RTLD_GLOBAL); if (n.h) break; }
    if (!n.h) return n;
    n.GetUniqueId = (int (*)(nccl_uid*))dlsym(n.h, "ncclGetUniqueId");
    n.CommInitRank = (int (*)(void**, int, nccl_uid, int))dlsym(n.h, "ncclCommInitRank");
    n.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(n.h, "ncclAllReduce");
    n.ReduceScatter = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(n.h, "ncclReduceScatter");
    n.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(n.h, "ncclAllGather");
    n.CommDestroy = (int (*)(void*))dlsym(n.h, "ncclCommDestroy");
    n.CommAbort = (int (*)(void*))dlsym(n.h, "ncclCommAbort");
    n.CommGetAsyncError = (int (*)(void*, int*))dlsym(n.h, "ncclCommGetAsyncError");
    n.GetErrorString = (const char* (*)(int))dlsym(n.h, "ncclGetErrorString");
    n.ok = n.GetUniqueId && n.CommInitRank && n.AllReduce && n.CommDestroy;
    return n;
}
// ncclDataType_t / ncclRedOp_t values from nccl.h
enum { NCCL_FLOAT16 = 6, NCCL_FLOAT32 = 7, NCCL_SUM = 0 };
}  // namespace

extern "C" {

int anl_comm_unique_id(uint8_t id[128]) {
    Nccl& n = nccl();
    if (!n.ok) return ANL_ERR_COMM;
    nccl_uid u;
    if (n.GetUniqueId(&u) != 0) return ANL_ERR_COMM;
    std::memcpy(id, u.internal, 128);
    return ANL_OK;
}

int anl_comm_init(anl_device* dev, int rank, int nranks, const uint8_t id[128]) {
    if (!dev || rank < 0 || rank >= nranks) return ANL_ERR_INVALID;
    Nccl& n = nccl();
    if (!n.ok) return dev->fail(ANL_ERR_COMM, "nccl: library not found");
    cudaSetDevice(dev->ordinal);
    nccl_uid u;
    std::memcpy(u.internal, id, 128);
    int r = n.CommInitRank(&dev->nccl_comm, nranks, u, rank);
    if (r != 0) return dev->fail(ANL_ERR_COMM, std::string("nccl: ncclCommInitRank: ") + (n.GetErrorString ? n.GetErrorString(r) : "?"));
    dev->rank = rank; dev->nranks = nranks; dev->comm_aborted = false;
    return ANL_OK;
}

// Sum `buf` over all ranks in place.  The collective runs on the device's communication stream,
// ordered after everything queued so far on the compute stream; the compute stream then waits for
// it, so later kernels see the reduced values while kernels queued before the call overlap with it.
int anl_allreduce_sum(anl_device* dev, anl_buffer* buf) {
    if (!dev || !buf) return ANL_ERR_INVALID;
    if (dev->comm_aborted) return dev->fail(ANL_ERR_COMM, "nccl: the communicator was aborted; create a new one with anl_comm_init");
    if (dev->nranks == 1 || !dev->nccl_comm) return ANL_OK;
    Nccl& n = nccl();
    int dt = buf->dtype == ANL_F16 ? NCCL_FLOAT16 : NCCL_FLOAT32;
    cudaSetDevice(dev->ordinal);
    cudaEventRecord(dev->comm_event, dev->stream);
    cudaStreamWaitEvent(dev->comm_stream, dev->comm_event, 0);
    int r = n.AllReduce(buf->ptr, buf->ptr, (size_t)buf->elems, dt, NCCL_SUM, dev->nccl_comm, dev->comm_stream);
    if (r != 0) return dev->fail(ANL_ERR_COMM, std::string("nccl: ncclAllReduce: ") + (n.GetErrorString ? n.GetErrorString(r) : "?"));
    cudaEventRecord(dev->comm_done, dev->comm_stream);
    cudaStreamWaitEvent(dev->stream, dev->comm_done, 0);
    return ANL_OK;
}

}  // extern "C"

namespace anl {
int comm_fork(anl_device* dev, cudaStream_t stream) {
    cudaEventRecord(dev->comm_event, stream);
    cudaStreamWaitEvent(dev->comm_stream, dev->comm_event, 0);
    dev->comm_pending = true;
    return ANL_OK;
}
int comm_allreduce_async(anl_device* dev, void* ptr, int64_t elems, int dtype, cudaStream_t stream) {
    if (dev->comm_aborted) return dev->fail(ANL_ERR_COMM, "nccl: the communicator was aborted; create a new one with anl_comm_init");
    if (dev->nranks == 1 || !dev->nccl_comm) return ANL_OK;
    Nccl& n = nccl();
    comm_fork(dev, stream);
    int r = n.AllReduce(ptr, ptr, (size_t)elems, dtype == ANL_F16 ? NCCL_FLOAT16 : NCCL_FLOAT32, NCCL_SUM, dev->nccl_comm, dev->comm_stream);
    if (r != 0) return dev->fail(ANL_ERR_COMM, std::string("nccl: ncclAllReduce: ") + (n.GetErrorString ? n.GetErrorString(r) : "?"));
    dev->comm_pending = true;
    return ANL_OK;
}
static size_t nccl_elem_bytes(int dtype) { return dtype == ANL_F16 ? 2 : 4; }
bool comm_can_shard(anl_device* dev) { Nccl& n = nccl(); return dev->nranks > 1 && dev->nccl_comm && n.ReduceScatter && n.AllGather; }
// In-place reduce-scatter: afterwards rank r holds the sum of elements [r*elems/nranks, (r+1)*elems/nranks)
// at their own position; the other positions hold partial garbage.  elems must divide by nranks.
int comm_reduce_scatter_async(anl_device* dev, void* ptr, int64_t elems, int dtype, cudaStream_t stream) {
    if (dev->comm_aborted) return dev->fail(ANL_ERR_COMM, "nccl: the communicator was aborted; create a new one with anl_comm_init");
    Nccl& n = nccl();
    const int64_t cnt = elems / dev->nranks;
    comm_fork(dev, stream);
    char* base = (char*)ptr;
    int r = n.ReduceScatter(base, base + (size_t)dev->rank * cnt * nccl_elem_bytes(dtype), (size_t)cnt,
                            dtype == ANL_F16 ? NCCL_FLOAT16 : NCCL_FLOAT32, NCCL_SUM, dev->nccl_comm, dev->comm_stream);
    if (r != 0) return dev->fail(ANL_ERR_COMM, std::string("nccl: ncclReduceScatter: ") + (n.GetErrorString ? n.GetErrorString(r) : "?"));
    dev->comm_pending = true;
    return ANL_OK;
}
// In-place all-gather on the communication stream (behind whatever was queued there): every rank
// contributes its own shard of `ptr` and receives the others'.
int comm_allgather_async(anl_device* dev, void* ptr, int64_t elems, int dtype) {
    if (dev->comm_aborted) return dev->fail(ANL_ERR_COMM, "nccl: the communicator was aborted; create a new one with anl_comm_init");
    Nccl& n = nccl();
    const int64_t cnt = elems / dev->nranks;
    char* base = (char*)ptr;
    int r = n.AllGather(base + (size_t)dev->rank * cnt * nccl_elem_bytes(dtype), base, (size_t)cnt,
                        dtype == ANL_F16 ? NCCL_FLOAT16 : NCCL_FLOAT32, dev->nccl_comm, dev->comm_stream);
    if (r != 0) return dev->fail(ANL_ERR_COMM, std::string("nccl: ncclAllGather: ") + (n.GetErrorString ? n.GetErrorString(r) : "?"));
    dev->comm_pending = true;
    return ANL_OK;
}
int comm_join(anl_device* dev, cudaStream_t stream) {
    if (!dev->comm_pending) return ANL_OK;
    cudaEventRecord(dev->comm_done, dev->comm_stream);
    cudaStreamWaitEvent(stream, dev->comm_done, 0);
    dev->comm_pending = false;
    return ANL_OK;
}
}  // namespace anl

extern "C" {

int anl_comm_destroy(anl_device* dev) {
    if (!dev) return ANL_OK;
    dev->comm_aborted = false;
    if (!dev->nccl_comm) return ANL_OK;
    Nccl& n = nccl();
    if (n.ok) n.CommDestroy(dev->nccl_comm);
    dev->nccl_comm = nullptr; dev->nranks = 1; dev->rank = 0;
    return ANL_OK;
}

// Every rank's shard of `buf` (elems / nranks each, in rank order) gathered into all ranks' copies,
// in place; ordered after prior work on the compute stream, which then waits for it.  Used to
// assemble the f32 master weights when the update is sharded across ranks.
int anl_allgather(anl_device* dev, anl_buffer* buf) {
    if (!dev || !buf) return ANL_ERR_INVALID;
    if (dev->comm_aborted) return dev->fail(ANL_ERR_COMM, "nccl: the communicator was aborted; create a new one with anl_comm_init");
    if (dev->nranks == 1 || !dev->nccl_comm) return ANL_OK;
    if (!anl::comm_can_shard(dev)) return dev->fail(ANL_ERR_COMM, "nccl: ncclAllGather not available");
    if (buf->elems % dev->nranks) return dev->fail(ANL_ERR_INVALID, "allgather: buffer length is not a multiple of the rank count");
    cudaSetDevice(dev->ordinal);
    anl::comm_fork(dev, dev->stream);
    if (int rc = anl::comm_allgather_async(dev, buf->ptr, buf->elems, buf->dtype)) return rc;
    return anl::comm_join(dev, dev->stream);
}

// ── watchdog ────────────────────────────────────────────────────────────────────────────────
// A rank that has died or never joined leaves the others inside a collective for ever.  The host
// side therefore never blocks on the communication stream without a limit once a timeout is set:
// it polls the stream, asks NCCL for asynchronous errors, and on either an error or the deadline
// aborts the communicator (ncclCommAbort ends the kernels that are waiting for the missing peer),
// reports ANL_ERR_COMM and refuses further collectives until anl_comm_init is called again.
static void abort_comm(anl_device* dev) {
    Nccl& n = nccl();
    if (dev->nccl_comm && n.CommAbort) n.CommAbort(dev->nccl_comm);
    dev->nccl_comm = nullptr;
    dev->comm_aborted = true;
}

int anl_comm_set_timeout(anl_device* dev, int milliseconds) {
    if (!dev || milliseconds < 0) return ANL_ERR_INVALID;
    dev->comm_timeout_ms = milliseconds;
    return ANL_OK;
}

int anl_comm_abort(anl_device* dev) {
    if (!dev) return ANL_ERR_INVALID;
    abort_comm(dev);
    return ANL_OK;
}

}  // extern "C"

namespace anl {
// Waits for `stream` under the watchdog.  A collective may sit on the communication stream (eager
// launches) or inside a captured graph that was launched on the compute stream (replays): in both
// cases the host must not block without a limit while a communicator with a timeout exists.
int wait_stream_watched(anl_device* dev, cudaStream_t stream, const char* what) {
    if (!stream) return ANL_OK;
    if (!(dev->nccl_comm && dev->comm_timeout_ms > 0)) {
        cudaError_t e = cudaStreamSynchronize(stream);
        return e == cudaSuccess ? ANL_OK : dev->fail(ANL_ERR_CUDA, std::string("cuda: ") + what + ": " + cudaGetErrorString(e));
    }
    Nccl& n = nccl();
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t q = cudaStreamQuery(stream);
        if (q == cudaSuccess) return ANL_OK;
        if (q != cudaErrorNotReady) return dev->fail(ANL_ERR_CUDA, std::string("cuda: ") + what + ": " + cudaGetErrorString(q));
        if (dev->nccl_comm && n.CommGetAsyncError) {
            int ae = 0;
            if (n.CommGetAsyncError(dev->nccl_comm, &ae) == 0 && ae != 0) {
                abort_comm(dev);
                cudaStreamSynchronize(stream);      // the aborted collective's kernels leave; the rest of the queue drains
                return dev->fail(ANL_ERR_COMM, std::string("nccl: asynchronous error: ") + (n.GetErrorString ? n.GetErrorString(ae) : "?") + "; communicator aborted");
            }
        }
        auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= dev->comm_timeout_ms) {
            abort_comm(dev);
            cudaStreamSynchronize(stream);
            return dev->fail(ANL_ERR_COMM, "nccl: collective did not finish within " + std::to_string(dev->comm_timeout_ms) + " ms (a peer is missing or stalled); communicator aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}
}  // namespace anl

extern "C" {

int anl_comm_wait(anl_device* dev) {
    if (!dev) return ANL_ERR_INVALID;
    if (!dev->comm_stream) return ANL_OK;
    cudaSetDevice(dev->ordinal);
    Nccl& n = nccl();
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t q = cudaStreamQuery(dev->comm_stream);
        if (q == cudaSuccess) return ANL_OK;
        if (q != cudaErrorNotReady) return dev->fail(ANL_ERR_CUDA, std::string("cuda: communication stream: ") + cudaGetErrorString(q));
        if (dev->nccl_comm && n.CommGetAsyncError) {
            int ae = 0;
            if (n.CommGetAsyncError(dev->nccl_comm, &ae) == 0 && ae != 0) {
                abort_comm(dev);
                return dev->fail(ANL_ERR_COMM, std::string("nccl: asynchronous error: ") + (n.GetErrorString ? n.GetErrorString(ae) : "?") + "; communicator aborted");
            }
        }
        if (dev->comm_timeout_ms > 0) {
            auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            if (ms >= dev->comm_timeout_ms) {
                abort_comm(dev);
                return dev->fail(ANL_ERR_COMM, "nccl: collective did not finish within " + std::to_string(dev->comm_timeout_ms) + " ms (a peer is missing or stalled); communicator aborted");
            }
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

// Host-side failure injection for tests: holds the communication stream back by `milliseconds`
// with a host callback (the GPU is idle meanwhile; nothing on the device faults or spins).
static void CUDART_CB comm_host_sleep(void* p) { usleep((useconds_t)(intptr_t)p * 1000); }
int anl_comm_inject_delay(anl_device* dev, int milliseconds) {
    if (!dev || !dev->comm_stream || milliseconds < 0) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    if (cudaLaunchHostFunc(dev->comm_stream, comm_host_sleep, (void*)(intptr_t)milliseconds) != cudaSuccess)
        return dev->fail(ANL_ERR_CUDA, "cuda: cannot queue the host callback");
    return ANL_OK;
}

}  // extern "C"
