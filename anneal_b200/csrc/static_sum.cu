// anl_sum_f32_static: the split scalar reduction (partials kernel + finish kernel) with its scratch
// in a fixed device array instead of pool memory, for callers that must not reach the CUDA
// allocator.  For n >= 65536 it mirrors, launch for launch, what the code generator emits for SUM
// over one f32 buffer (the generator splits a reduction over several blocks from that length on;
// shorter sums it runs in one block, so there the order of the additions differs from this file's
// and the two agree to rounding, not bit for bit): every block reduces one contiguous chunk with 256
// lanes striding it, lanes are combined by an xor-shuffle butterfly and then across the eight warps
// in ascending order, and one thread adds the partials in ascending order.  Nothing here allocates:
// no cudaMalloc/cudaFree, no pool, no NVRTC.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "../../include/anneal_cuda.h"

namespace {

constexpr int kMaxParts = 1024;                  // 4 KiB of scratch per GPU that loads the library
constexpr long long kMaxElems = 1ll << 30;       // int-indexed chunks; also keeps one call under a few ms
constexpr int kThreads = 256;

// Partials of the call in flight.  One array per device, shared by every call on that device and
// holding the previous call's partials until overwritten; calls that overlap on the GPU race on it.
static __device__ __align__(256) float g_sum_scratch[kMaxParts];

__global__ void __launch_bounds__(kThreads) static_sum_partials(const float* __restrict__ x, long long n, long long chunk,
                                                                float* __restrict__ scratch) {
    __shared__ float warp_part[kThreads / 32];
    const long long begin = (long long)blockIdx.x * chunk;
    long long end = begin + chunk;
    if (end > n) end = n;
    float acc = 0.0f;
    for (long long i = begin + threadIdx.x; i < end; i += kThreads) acc = acc + x[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc = acc + __shfl_xor_sync(0xffffffffu, acc, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    float v = warp_part[0];
    for (int w = 1; w < kThreads / 32; w++) v = v + warp_part[w];
    if (threadIdx.x == 0) scratch[blockIdx.x] = v;      // every slot in [0, parts) is rewritten: nothing to clear
}

__global__ void static_sum_finish(const float* __restrict__ scratch, int parts, float* __restrict__ out) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float acc = 0.0f;
        for (int p = 0; p < parts; p++) acc = acc + scratch[p];
        *out = acc;
    }
}

// device address of g_sum_scratch per device ordinal; the symbol's name is only a host-side handle.
// Two host threads that make the first call on one device together both resolve the same address
// and store the same value; the atomic makes that store and the later loads well defined.
std::atomic<float*> g_scratch_addr[64] = {};

void set_err(char* err, size_t cap, const char* msg) { if (err && cap) std::snprintf(err, cap, "%s", msg); }

}  // namespace

extern "C" int anl_sum_f32_static(const float* x, int64_t n, float* out, void* stream, char* err, size_t err_cap) {
    if (!x || !out) { set_err(err, err_cap, "static sum: null device pointer"); return ANL_ERR_INVALID; }
    if (n < 1 || n > kMaxElems) {
        char m[160];
        std::snprintf(m, sizeof m, "static sum: %lld elements is outside [1, %lld], the range the fixed scratch array is sized for", (long long)n, kMaxElems);
        set_err(err, err_cap, m);
        return ANL_ERR_LIMIT;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { set_err(err, err_cap, "static sum: no current CUDA device"); return ANL_ERR_NO_DEVICE; }
    float* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        // first call on this device: resolve the array's device address (the current device is `dev`)
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_sum_scratch);
        if (e != cudaSuccess || !p) { set_err(err, err_cap, cudaGetErrorString(e)); return ANL_ERR_CUDA; }
        scratch = static_cast<float*>(p);
        g_scratch_addr[dev].store(scratch, std::memory_order_release);
    }
    // same split the code generator picks for one output: about four blocks per SM, chunks of >= 4096
    long long parts = n / 4096;
    if (parts > 592) parts = 592;
    if (parts < 1) parts = 1;
    const long long chunk = (n + parts - 1) / parts;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    static_sum_partials<<<(unsigned)parts, kThreads, 0, s>>>(x, n, chunk, scratch);
    static_sum_finish<<<1, 32, 0, s>>>(scratch, (int)parts, out);
    e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, err_cap, cudaGetErrorString(e)); return ANL_ERR_CUDA; }
    return ANL_OK;
}
