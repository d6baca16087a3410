// Device runtime: everything backend/webgpu/executor.go does per Run call (allocate, upload with
// dtype conversion, compile, dispatch, read back, release) redone for CUDA so that the per-call
// costs the reference pays every time are paid once: rendered sources and compiled modules are
// cached by content, device blocks come from a size-keyed pool, conversion runs on the GPU.
#include "runtime.hpp"

#include <cuda_fp16.h>
#include <nvrtc.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <set>
#include <unordered_set>

using namespace anl;

#define CK(dev, call)                                                                            \
    do {                                                                                         \
        cudaError_t e_ = (call);                                                                 \
        if (e_ != cudaSuccess)                                                                   \
            return (dev)->fail(ANL_ERR_CUDA, std::string("cuda: ") + #call + ": " + cudaGetErrorString(e_)); \
    } while (0)

// ── boundary conversions ─────────────────────────────────────────────────────────────────────
// f32 → f16 is round-to-nearest-even, f32 → bf16 clears the low 16 bits and keeps a 32-bit slot
// (uop/dtype.go:392-487, backend/webgpu/executor.go:480-519).
__global__ void cvt_f32_to_f16(const float* __restrict__ in, __half* __restrict__ out, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __float2half_rn(in[i]);
}
__global__ void cvt_f32_to_bf16slot(const float* __restrict__ in, float* __restrict__ out, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __int_as_float(__float_as_int(in[i]) & 0xFFFF0000);
}
__global__ void cvt_f16_to_f32(const __half* __restrict__ in, float* __restrict__ out, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __half2float(in[i]);
}

// Parameter.SGDStep (tensor/nn/nn.go:69-76) with the re-quantisation of Parameter.Load
// (tensor/nn/nn.go:56-61) fused: one pass over master, grad and param.
// Streaming accesses (evict-first): the 12 bytes per parameter this pass moves are not needed again
// before the next step, while the contractions running beside it live on the operand tiles they
// keep in L2.  Two groups of four parameters per thread and trip when the views are 16-byte aligned.
template <class T> __device__ __forceinline__ float sgd_ld(const T* p) { return (float)__ldcs(p); }
template <> __device__ __forceinline__ float sgd_ld<__half>(const __half* p) { return __half2float(__ldcs(p)); }

// four gradients as f32 from one 8- or 16-byte streaming load
template <class G> __device__ __forceinline__ void sgd_ld4(const G* grad, long long q, float g[4]);
template <> __device__ __forceinline__ void sgd_ld4<__half>(const __half* grad, long long q, float g[4]) {
    uint2 raw = __ldcs(reinterpret_cast<const uint2*>(grad) + q);
    const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x), hi = *reinterpret_cast<const __half2*>(&raw.y);
    g[0] = __low2float(lo); g[1] = __high2float(lo); g[2] = __low2float(hi); g[3] = __high2float(hi);
}
template <> __device__ __forceinline__ void sgd_ld4<float>(const float* grad, long long q, float g[4]) {
    float4 raw = __ldcs(reinterpret_cast<const float4*>(grad) + q);
    g[0] = raw.x; g[1] = raw.y; g[2] = raw.z; g[3] = raw.w;
}

template <class P>
__device__ __forceinline__ void sgd_apply4(float* master, P* param, long long q, float4 m, const float g[4],
                                           float lr, float scale, bool separate, int bf16) {
    float r[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float gs = g[j] * scale;
        r[j] = r[j] - lr * gs;
    }
    __stcs(reinterpret_cast<float4*>(master) + q, make_float4(r[0], r[1], r[2], r[3]));
    if (separate) {
        if (sizeof(P) == 2) {
            const __half2 lo = __floats2half2_rn(r[0], r[1]), hi = __floats2half2_rn(r[2], r[3]);
            uint2 o; o.x = *reinterpret_cast<const unsigned*>(&lo); o.y = *reinterpret_cast<const unsigned*>(&hi);
            __stcs(reinterpret_cast<uint2*>(param) + q, o);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) if (bf16) r[j] = __int_as_float(__float_as_int(r[j]) & 0xFFFF0000);
            __stcs(reinterpret_cast<float4*>(param) + q, make_float4(r[0], r[1], r[2], r[3]));
        }
    }
}

// Two 4-element groups per thread and iteration, both groups' loads issued before either is used:
// 48 bytes in flight per thread keep enough of HBM's latency covered at 2048 threads per SM.
template <class G, class P>
__global__ void __launch_bounds__(256, 6) sgd_kernel(float* __restrict__ master, P* __restrict__ param, const G* __restrict__ grad,
                           float lr, float scale, long long n, int bf16, int vec) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const bool separate = (void*)param != (void*)master;
    long long done = 0;
    if (vec) {
        const long long n4 = n >> 2;
#pragma unroll 1
        for (long long q = tid; q < n4; q += 2 * stride) {
            const long long q1 = q + stride;
            const bool two = q1 < n4;
            float g0[4], g1[4];
            float4 m0 = __ldcs(reinterpret_cast<const float4*>(master) + q), m1 = m0;
            if (two) m1 = __ldcs(reinterpret_cast<const float4*>(master) + q1);
            sgd_ld4<G>(grad, q, g0);
            if (two) sgd_ld4<G>(grad, q1, g1);
            sgd_apply4<P>(master, param, q, m0, g0, lr, scale, separate, bf16);
            if (two) sgd_apply4<P>(master, param, q1, m1, g1, lr, scale, separate, bf16);
        }
        done = n4 << 2;
    }
    for (long long i = done + tid; i < n; i += stride) {
        float g = sgd_ld(grad + i) * scale;
        float m = master[i] - lr * g;
        master[i] = m;
        if (bf16) m = __int_as_float(__float_as_int(m) & 0xFFFF0000);
        if (separate) param[i] = (P)m;
    }
}

// Holds the stream for about `ns` nanoseconds (bounded: at most 4096 sleeps of 1 us), so that the launch
// to be timed is already queued behind the first event when the GPU reaches it; without it the host's
// time to prepare the launch is measured as part of the kernel.
__global__ void hold_stream(unsigned long long ns) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (int i = 0; i < 4096; i++) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 >= ns) break;
        __nanosleep(1000);
    }
}

// Benchmark operands: finite values of magnitude 0.5 .. 1 with random signs and mantissas (f16 pairs or
// f32 words), so that a timed contraction switches as many bits as one fed with real activations; a
// zero-filled operand lets the tensor cores idle and flatters the clock.
__global__ void fill_benchmark_pattern(unsigned* __restrict__ p, long long words, int f16, unsigned seed) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < words; i += stride) {
        unsigned x = (unsigned)i * 2654435761u + seed;
        x ^= x >> 15; x *= 2246822519u; x ^= x >> 13; x *= 3266489917u; x ^= x >> 16;
        p[i] = f16 ? ((x & 0x83FF83FFu) | 0x38003800u) : ((x & 0x807FFFFFu) | 0x3F000000u);
    }
}

static unsigned grid_for(long long n, int block, int sms) {
    long long g = (n + block - 1) / block;
    long long cap = (long long)sms * 16;
    return (unsigned)std::max<long long>(1, std::min(g, cap));
}

// ── device memory pool ───────────────────────────────────────────────────────────────────────
int anl_device::alloc(size_t bytes, void** out) {
    if (bytes == 0) bytes = 4;
    bytes = (bytes + 255) & ~(size_t)255;
    auto it = pool.find(bytes);
    if (it != pool.end()) {
        *out = it->second;
        pool.erase(it);
    } else {
        cudaError_t e = cudaMalloc(out, bytes);
        if (e != cudaSuccess) {
            trim();
            e = cudaMalloc(out, bytes);
        }
        if (e != cudaSuccess) return fail(ANL_ERR_CUDA, std::string("cuda: cudaMalloc(") + std::to_string(bytes) + "): " + cudaGetErrorString(e));
        stats.device_allocs++;
    }
    live[*out] = bytes;
    return ANL_OK;
}
void anl_device::release(void* p) {
    if (!p) return;
    auto it = live.find(p);
    if (it == live.end()) return;
    pool.insert({it->second, p});
    live.erase(it);
}
void anl_device::trim() {
    for (auto& kv : pool) cudaFree(kv.second);
    pool.clear();
}

namespace anl {

void launch_hold_stream(cudaStream_t stream, unsigned long long ns) { hold_stream<<<1, 1, 0, stream>>>(ns); }

int ensure_driver(anl_device* dev) {
    if (dev->drv.loaded) return ANL_OK;
    auto get = [&](const char* name, void** fn) -> bool {
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPointByVersion(name, fn, 12000, cudaEnableDefault, &q);
        return e == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn;
    };
    bool ok = get("cuModuleLoadData", (void**)&dev->drv.ModuleLoadData) && get("cuModuleUnload", (void**)&dev->drv.ModuleUnload) &&
              get("cuModuleGetFunction", (void**)&dev->drv.ModuleGetFunction) && get("cuLaunchKernel", (void**)&dev->drv.LaunchKernel) &&
              get("cuGetErrorString", (void**)&dev->drv.GetErrorString) && get("cuTensorMapEncodeTiled", (void**)&dev->drv.TensorMapEncodeTiled) &&
              get("cuLaunchKernelEx", (void**)&dev->drv.LaunchKernelEx) && get("cuFuncSetAttribute", (void**)&dev->drv.FuncSetAttribute);
    if (!ok) return dev->fail(ANL_ERR_CUDA, "cuda: driver entry points unavailable");
    dev->drv.loaded = true;
    return ANL_OK;
}

static std::string cuda_include_dir() {
    const char* h = std::getenv("CUDA_HOME");
    if (!h) h = std::getenv("CUDA_PATH");
    return std::string("-I") + (h ? h : "/usr/local/cuda") + "/include";
}

// NVRTC → cubin for sm_100a.  No fast-math and no fused multiply-add contraction: generated
// kernels keep the rounding of the expression tree they were given.
static int nvrtc_compile(const std::string& src, std::vector<char>& cubin, std::string& log) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, src.c_str(), "anneal_kernel.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS) { log = "nvrtcCreateProgram failed"; return ANL_ERR_COMPILE; }
    std::string inc = cuda_include_dir();
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", inc.c_str(), "-default-device"};
    nvrtcResult r = nvrtcCompileProgram(prog, 5, opts);
    size_t ls = 0;
    nvrtcGetProgramLogSize(prog, &ls);
    if (ls > 1) { log.resize(ls); nvrtcGetProgramLog(prog, &log[0]); }
    if (r != NVRTC_SUCCESS) { nvrtcDestroyProgram(&prog); if (log.empty()) log = nvrtcGetErrorString(r); return ANL_ERR_COMPILE; }
    size_t cs = 0;
    nvrtcGetCUBINSize(prog, &cs);
    cubin.resize(cs);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    return ANL_OK;
}

int compile_source(anl_device* dev, const std::string& src, std::shared_ptr<Module>& out) {
    uint64_t h = fnv1a(src.data(), src.size());
    auto it = dev->modules.find(h);
    if (it != dev->modules.end()) { dev->stats.nvrtc_cache_hits++; out = it->second; return ANL_OK; }
    if (int rc = ensure_driver(dev)) return rc;
    std::vector<char> cubin; std::string log;
    if (int rc = nvrtc_compile(src, cubin, log)) return dev->fail(rc, "cuda: compile failed: " + log + "\n--- source ---\n" + src);
    dev->stats.nvrtc_compiles++;
    auto m = std::make_shared<Module>();
    CUresult cr = dev->drv.ModuleLoadData(&m->mod, cubin.data());
    if (cr != CUDA_SUCCESS) { const char* s = nullptr; dev->drv.GetErrorString(cr, &s); return dev->fail(ANL_ERR_CUDA, std::string("cuda: cuModuleLoadData: ") + (s ? s : "?")); }
    dev->modules[h] = m;
    out = m;
    return ANL_OK;
}

static int get_function(anl_device* dev, Module& m, const std::string& name, CUfunction* fn) {
    auto it = m.fn.find(name);
    if (it != m.fn.end()) { *fn = it->second; return ANL_OK; }
    CUresult cr = dev->drv.ModuleGetFunction(fn, m.mod, name.c_str());
    if (cr != CUDA_SUCCESS) return dev->fail(ANL_ERR_CUDA, "cuda: entry point " + name + " not found in compiled module");
    m.fn[name] = *fn;
    return ANL_OK;
}

static bool opts_default(const CodegenOpts& o) { return !o.block_threads && !o.reduce_lanes && !o.vector_width && !o.split; }
static GemmTuning tuning_of(const CodegenOpts& o) {
    GemmTuning t;
    t.tile_n = o.gemm_tile_n; t.stages = o.gemm_stages; t.group_m = o.gemm_group_m; t.stream_stores = o.gemm_stream_stores; t.single_cta = o.gemm_single_cta; t.no_split_tail = o.gemm_whole_tail;
    return t;
}

int get_plan(anl_device* dev, const Item& item, const CodegenOpts& opts, std::shared_ptr<Plan>& out) {
    int64_t ok[11] = {opts.block_threads, opts.reduce_lanes, opts.vector_width, opts.split, opts.debug_bounds,
                      opts.gemm_tile_n, opts.gemm_stages, opts.gemm_group_m, opts.gemm_stream_stores, opts.gemm_single_cta, opts.gemm_whole_tail};
    uint64_t key = fnv1a(ok, sizeof ok, structure_hash(item));
    if (!item.source.empty()) key = fnv1a(item.source.data(), item.source.size(), key);
    auto it = dev->plans.find(key);
    if (it != dev->plans.end()) { dev->stats.lower_cache_hits++; out = it->second; return ANL_OK; }
    auto p = std::make_shared<Plan>();
    if (!item.source.empty()) {
        // pre-rendered source with its launch shape (the reference's ExecItem.WGSL route,
        // schedule/cache.go:80-88, backend/webgpu/executor.go:53-64): entry point "main_kernel"
        p->r.klass = KC_RAW;
        p->r.source = item.source;
        p->r.main.entry = "main_kernel";
        p->r.main.block = item.local[0]; p->r.main.block_y = item.local[1]; p->r.main.block_z = item.local[2];
        p->r.main.static_outputs = (int64_t)item.grid[0];
        p->r.main.grid_y = item.grid[1]; p->r.main.grid_z = item.grid[2];
        p->r.main.outputs_per_block = 1;
    } else {
        bool routed = false;
        if (opts_default(opts) && !(dev->flags & ANL_OPEN_NO_GEMM)) routed = plan_gemm(item, tuning_of(opts), *p) == ANL_OK;
        if (!routed || p->gemm_dynamic) {
            std::string err;
            if (!render_cuda(item, opts, p->r, err)) return dev->fail(ANL_ERR_UNSUPPORTED, err);
        }
    }
    if (p->r.klass != KC_GEMM) {
        std::shared_ptr<Module> m;
        if (int rc = compile_source(dev, p->r.source, m)) return rc;
        if (int rc = get_function(dev, *m, p->r.main.entry, &p->main)) return rc;
        if (p->r.klass == KC_REDUCE_SPLIT)
            if (int rc = get_function(dev, *m, p->r.finish.entry, &p->finish)) return rc;
        if (p->r.klass == KC_REDUCE && p->r.uses_sym && p->r.main.sym_trailing > 0 && item.source.empty() && opts.sym_hint == 0) {
            CodegenOpts few = opts; few.sym_hint = 1;
            std::string err;
            if (render_cuda(item, few, p->r_small, err) && p->r_small.klass == KC_REDUCE && p->r_small.source != p->r.source) {
                std::shared_ptr<Module> ms;
                if (int rc = compile_source(dev, p->r_small.source, ms)) return rc;
                if (int rc = get_function(dev, *ms, p->r_small.main.entry, &p->main_small)) return rc;
                p->small_below = 64;
            }
        }
    }
    dev->plans[key] = p;
    out = p;
    return ANL_OK;
}

static int launch_one(anl_device* dev, CUfunction fn, const Launch& l, int64_t sym, std::vector<void*>& args, cudaStream_t stream) {
    int64_t work = l.sym_trailing > 0 ? sym * l.sym_trailing : l.static_outputs;
    if (work <= 0) return ANL_OK;
    int64_t grid = (work + l.outputs_per_block - 1) / l.outputs_per_block;
    if (grid > 0x7fffffffLL) return dev->fail(ANL_ERR_LIMIT, "cuda: grid too large");
    CUresult cr = dev->drv.LaunchKernel(fn, (unsigned)grid, l.grid_y, l.grid_z, l.block, l.block_y, l.block_z, l.smem_bytes, (CUstream)stream, args.data(), nullptr);
    if (cr != CUDA_SUCCESS) { const char* s = nullptr; dev->drv.GetErrorString(cr, &s); return dev->fail(ANL_ERR_CUDA, std::string("cuda: cuLaunchKernel(") + l.entry + "): " + (s ? s : "?")); }
    dev->stats.kernels_launched++;
    return ANL_OK;
}

static int launch_plan_inner(anl_device* dev, const Plan& plan, const Item& item, void* const* bufs, int64_t sym_value, cudaStream_t stream,
                             std::vector<void*>* keep_scratch);

int launch_plan(anl_device* dev, const Plan& plan, const Item& item, void* const* bufs, int64_t sym_value, cudaStream_t stream,
                std::vector<void*>* keep_scratch) {
    if (!dev->profiling) return launch_plan_inner(dev, plan, item, bufs, sym_value, stream, keep_scratch);
    anl_device::ProfRec r{};
    cudaEventCreate(&r.e0); cudaEventCreate(&r.e1);
    const bool gemm = gemm_taken(plan, sym_value);
    r.klass = gemm ? KC_GEMM : plan.r.klass; r.flops = gemm ? gemm_flops(plan, sym_value) : 0.0;
    cudaEventRecord(r.e0, stream);
    int rc = launch_plan_inner(dev, plan, item, bufs, sym_value, stream, keep_scratch);
    cudaEventRecord(r.e1, stream);
    dev->prof.push_back(r);
    return rc;
}

static int launch_plan_inner(anl_device* dev, const Plan& plan, const Item& item, void* const* bufs, int64_t sym_value, cudaStream_t stream,
                             std::vector<void*>* keep_scratch) {
    if (gemm_taken(plan, sym_value)) return launch_gemm(dev, plan, bufs, sym_value, stream, 0, -1, nullptr, keep_scratch);
    int nb = (int)item.bufs.size();
    std::vector<void*> ptrs(bufs, bufs + nb);
    int n0 = (int)sym_value;
    void* scratch = nullptr;
    std::vector<void*> args;
    for (int b = 0; b < nb; b++) args.push_back(&ptrs[b]);
    if (plan.r.klass == KC_REDUCE_SPLIT) {
        // partials travel through global scratch memory owned by the pool for the duration of the
        // two launches; stream order makes re-use by a later kernel safe
        if (int rc = dev->alloc((size_t)plan.r.scratch_elems * 4, &scratch)) return rc;
        args.push_back(&scratch);
    }
    if (plan.r.uses_sym) args.push_back(&n0);
    if (plan.main_small && sym_value < plan.small_below) return launch_one(dev, plan.main_small, plan.r_small.main, sym_value, args, stream);
    int rc = launch_one(dev, plan.main, plan.r.main, sym_value, args, stream);
    if (rc == ANL_OK && plan.r.klass == KC_REDUCE_SPLIT) rc = launch_one(dev, plan.finish, plan.r.finish, sym_value, args, stream);
    if (scratch) { if (keep_scratch) keep_scratch->push_back(scratch); else dev->release(scratch); }
    return rc;
}

int launch_sgd(anl_device* dev, anl_buffer* master, anl_buffer* param, anl_buffer* grad, float lr, float scale, cudaStream_t stream) {
    if (master->dtype != ANL_F32) return dev->fail(ANL_ERR_INVALID, "sgd: master weights must be f32");
    if (grad->elems < master->elems || param->elems < master->elems) return dev->fail(ANL_ERR_INVALID, "sgd: gradient length != parameter length");
    long long n = master->elems;
    if (n == 0) return ANL_OK;
    auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const int vec = n >= 4 && al16(master->ptr) && al16(param->ptr) && al16(grad->ptr);
    const int sms = dev->prop.multiProcessorCount;
    unsigned g = grid_for(vec ? (n + 3) / 4 : n, 256, sms);
    float* m = (float*)master->ptr;
    bool gh = grad->dtype == ANL_F16, ph = param->dtype == ANL_F16;
    int bf = param->dtype == ANL_BF16;
    if (gh && ph) sgd_kernel<__half, __half><<<g, 256, 0, stream>>>(m, (__half*)param->ptr, (const __half*)grad->ptr, lr, scale, n, 0, vec);
    else if (gh) sgd_kernel<__half, float><<<g, 256, 0, stream>>>(m, (float*)param->ptr, (const __half*)grad->ptr, lr, scale, n, bf, vec);
    else if (ph) sgd_kernel<float, __half><<<g, 256, 0, stream>>>(m, (__half*)param->ptr, (const float*)grad->ptr, lr, scale, n, 0, vec);
    else sgd_kernel<float, float><<<g, 256, 0, stream>>>(m, (float*)param->ptr, (const float*)grad->ptr, lr, scale, n, bf, vec);
    dev->stats.kernels_launched++;
    CK(dev, cudaGetLastError());
    return ANL_OK;
}

int upload_f32(anl_device* dev, void* dst, int dtype, const float* host, int64_t elems, cudaStream_t s) {
    if (elems <= 0) return ANL_OK;
    dev->stats.h2d_bytes += (uint64_t)elems * 4;
    if (dtype != DT_F16 && dtype != DT_BF16) {
        CK(dev, cudaMemcpyAsync(dst, host, (size_t)elems * 4, cudaMemcpyHostToDevice, s));
        return ANL_OK;
    }
    void* stage = nullptr;
    if (int rc = dev->alloc((size_t)elems * 4, &stage)) return rc;
    cudaError_t e = cudaMemcpyAsync(stage, host, (size_t)elems * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        unsigned g = grid_for(elems, 256, dev->prop.multiProcessorCount);
        if (dtype == DT_F16) cvt_f32_to_f16<<<g, 256, 0, s>>>((const float*)stage, (__half*)dst, elems);
        else cvt_f32_to_bf16slot<<<g, 256, 0, s>>>((const float*)stage, (float*)dst, elems);
        e = cudaGetLastError();
        dev->stats.kernels_launched++;
    }
    dev->release(stage);   // stream-ordered: later users of the block run after the conversion
    if (e != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("cuda: upload: ") + cudaGetErrorString(e));
    return ANL_OK;
}

int download_f32(anl_device* dev, float* host, const void* src, int dtype, int64_t elems, cudaStream_t s) {
    if (elems <= 0) return ANL_OK;
    dev->stats.d2h_bytes += (uint64_t)elems * 4;
    if (dtype != DT_F16) {
        CK(dev, cudaMemcpyAsync(host, src, (size_t)elems * 4, cudaMemcpyDeviceToHost, s));
        return ANL_OK;
    }
    void* stage = nullptr;
    if (int rc = dev->alloc((size_t)elems * 4, &stage)) return rc;
    cvt_f16_to_f32<<<grid_for(elems, 256, dev->prop.multiProcessorCount), 256, 0, s>>>((const __half*)src, (float*)stage, elems);
    dev->stats.kernels_launched++;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, stage, (size_t)elems * 4, cudaMemcpyDeviceToHost, s);
    dev->release(stage);
    if (e != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("cuda: download: ") + cudaGetErrorString(e));
    return ANL_OK;
}

}  // namespace anl

// ── schedule execution ───────────────────────────────────────────────────────────────────────
namespace {

// host arrays handed out through anl_output.data; anl_outputs_free releases only these, never a
// caller-placed array
std::mutex g_owned_mu;
std::unordered_set<float*> g_owned_outputs;

struct DevBuf { void* ptr = nullptr; size_t bytes = 0; int dtype = DT_F32; int64_t elems = 0; bool owned = false; };

struct Bindings {
    std::vector<std::pair<std::string, int64_t>> v;
    int64_t get(const std::string& name, int64_t dflt) const { for (auto& p : v) if (p.first == name) return p.second; return dflt; }
    int64_t any() const { return v.empty() ? -1 : v[0].second; }
};

int64_t item_sym(const Item& it, const Bindings& b) {
    if (!it.sym_vars.empty()) return b.get(it.sym_vars[0], b.any());
    return b.any();
}

// Buffer table of one schedule: slot-shared intermediates, dedicated outputs, leaves
// (backend/webgpu/executor.go:66-151).
struct Table {
    std::unordered_map<uint32_t, DevBuf> bufs;
    std::vector<void*> owned;
    std::set<uint32_t> written, read;
    std::vector<uint32_t> finals;      // in schedule order
    std::unordered_map<uint32_t, anl_output> after;   // output id → placed entry asking for an all-reduce and/or an SGD update
};

int build_table(anl_device* dev, const std::vector<Item>& items, const Bindings& binds,
                const anl_input* inputs, int n_inputs, const anl_output* placed, int n_placed, Table& t) {
    for (auto& it : items) { t.written.insert(it.bufs[0].id); for (size_t b = 1; b < it.bufs.size(); b++) t.read.insert(it.bufs[b].id); }
    std::map<int, size_t> slot_bytes;
    for (auto& it : items) {
        const BufDesc& o = it.bufs[0];
        if (o.slot >= 0) { size_t by = (size_t)o.elems(item_sym(it, binds)) * dt_storage_bytes(o.dtype); slot_bytes[o.slot] = std::max(slot_bytes[o.slot], by); }
    }
    std::map<int, void*> slot_ptr;
    for (auto& kv : slot_bytes) { void* p; if (int rc = dev->alloc(kv.second, &p)) return rc; slot_ptr[kv.first] = p; t.owned.push_back(p); }
    for (auto& it : items) {
        const BufDesc& o = it.bufs[0];
        int64_t sym = item_sym(it, binds);
        DevBuf d; d.dtype = o.dtype; d.elems = o.elems(sym); d.bytes = (size_t)d.elems * dt_storage_bytes(o.dtype);
        if (o.slot >= 0) d.ptr = slot_ptr[o.slot];
        else {
            bool is_final = true;
            const anl_output* pl = nullptr;
            for (int k = 0; k < n_placed; k++) if (placed[k].uop_idx == o.id && placed[k].resident) pl = &placed[k];
            if (is_final && pl) {
                if (pl->resident->elems < d.elems || pl->resident->dtype != o.dtype) return dev->fail(ANL_ERR_INVALID, "run: resident output buffer has the wrong size or dtype");
                d.ptr = pl->resident->ptr;
                if (pl->allreduce || pl->sgd_master) t.after[o.id] = *pl;
            } else if (!t.bufs.count(o.id)) {
                if (int rc = dev->alloc(d.bytes, &d.ptr)) return rc;
                t.owned.push_back(d.ptr); d.owned = true;
            } else d.ptr = t.bufs[o.id].ptr;
        }
        t.bufs[o.id] = d;
    }
    for (auto& it : items) {
        int64_t sym = item_sym(it, binds);
        for (size_t b = 1; b < it.bufs.size(); b++) {
            const BufDesc& bd = it.bufs[b];
            if (t.written.count(bd.id) || t.bufs.count(bd.id)) continue;
            DevBuf d; d.dtype = bd.dtype; d.elems = bd.elems(sym); d.bytes = (size_t)d.elems * dt_storage_bytes(bd.dtype);
            const anl_input* in = nullptr;
            for (int k = 0; k < n_inputs; k++) if (inputs[k].uop_idx == bd.id) in = &inputs[k];
            if (in && in->resident) {
                if (in->resident->elems < d.elems) return dev->fail(ANL_ERR_INVALID, "run: resident input " + std::to_string(bd.id) + " is smaller than the schedule expects");
                d.ptr = in->resident->ptr;
            } else {
                if (int rc = dev->alloc(d.bytes, &d.ptr)) return rc;
                t.owned.push_back(d.ptr); d.owned = true;
                if (in && in->data) {
                    if (in->elems < d.elems) return dev->fail(ANL_ERR_INVALID, "run: input " + std::to_string(bd.id) + " has " + std::to_string(in->elems) + " values, schedule expects " + std::to_string(d.elems));
                    if (int rc = upload_f32(dev, d.ptr, bd.dtype, in->data, d.elems, dev->stream)) return rc;
                } else {
                    CK(dev, cudaMemsetAsync(d.ptr, 0, d.bytes ? d.bytes : 4, dev->stream));
                }
            }
            t.bufs[bd.id] = d;
        }
    }
    // final outputs: never read again, or read again but deliberately left un-aliased by the planner
    for (auto& it : items) if (!t.read.count(it.bufs[0].id) || it.bufs[0].slot < 0) t.finals.push_back(it.bufs[0].id);
    return ANL_OK;
}

// Row chains: greedily take the longest run of items starting at `first` that iterate the same row
// count, produce one value per row (the last may produce a whole row) and are not wanted by an
// all-reduce / update hook; render them as one kernel (cached, negative results included).
int try_row_chain(anl_device* dev, const std::vector<Item>& items, size_t first, Table& t, cudaStream_t stream, size_t* used) {
    *used = 0;
    auto rows_of = [&](const Item& it, bool& full_row) -> int64_t {
        const BufDesc& o = it.bufs[0];
        if (!it.source.empty() || !it.sym_vars.empty() || o.shape.empty() || o.symbolic()) return -1;
        for (auto& b : it.bufs) if (b.symbolic()) return -1;
        full_row = o.shape.size() > 1;
        return o.shape[0];
    };
    bool full = false;
    int64_t rows = rows_of(items[first], full);
    if (rows < 128 || full) return ANL_OK;
    std::vector<const Item*> members;
    std::vector<std::vector<std::pair<int, int>>> reads;
    uint64_t key = 0x9E3779B97F4A7C15ull;
    for (size_t j = first; j < items.size(); j++) {
        const Item& it = items[j];
        bool f = false;
        if (rows_of(it, f) != rows || t.after.count(it.bufs[0].id)) break;
        Contraction c;
        if (match_contraction(it, c) && c.in_dtype == DT_F16 && !(dev->flags & ANL_OPEN_NO_GEMM)) break;
        std::vector<std::pair<int, int>> rd;
        for (size_t b = 1; b < it.bufs.size(); b++)
            for (size_t m = 0; m < members.size(); m++)
                if (members[m]->bufs[0].id == it.bufs[b].id) rd.push_back({(int)b, (int)m});
        members.push_back(&it);
        reads.push_back(rd);
        uint64_t h = structure_hash(it);
        key = fnv1a(&h, sizeof h, key);
        for (auto& pr : rd) key = fnv1a(&pr, sizeof pr, key);
        if (f) break;               // a full-row producer ends the chain
    }
    // try the longest run first, then shorter prefixes
    while (members.size() >= 2) {
        uint64_t k2 = fnv1a(&key, sizeof key, members.size());
        for (auto* m : members) { uint64_t h = structure_hash(*m); k2 = fnv1a(&h, sizeof h, k2); }
        auto f = dev->chains.find(k2);
        std::shared_ptr<ChainPlan> cp;
        if (f != dev->chains.end()) cp = f->second;
        else {
            cp = std::make_shared<ChainPlan>();
            CodegenOpts o; std::string err;
            if (!render_row_chain(members, reads, o, cp->r, err)) cp.reset();
            else {
                std::shared_ptr<Module> mod;
                if (int rc = compile_source(dev, cp->r.source, mod)) return rc;
                CUresult cr = dev->drv.ModuleGetFunction(&cp->fn, mod->mod, cp->r.entry.c_str());
                if (cr != CUDA_SUCCESS) return dev->fail(ANL_ERR_CUDA, "cuda: row_chain entry point missing");
            }
            dev->chains[k2] = cp;
        }
        if (cp) {
            std::vector<void*> ptrs;
            for (auto* m : members) for (auto& b : m->bufs) ptrs.push_back(t.bufs[b.id].ptr);
            std::vector<void*> args;
            for (auto& p : ptrs) args.push_back(&p);
            cudaEvent_t e0 = nullptr, e1 = nullptr;
            if (dev->profiling) { cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventRecord(e0, stream); }
            CUresult cr = dev->drv.LaunchKernel(cp->fn, (unsigned)cp->r.rows, 1, 1, cp->r.block, 1, 1, 0, (CUstream)stream, args.data(), nullptr);
            if (dev->profiling) { cudaEventRecord(e1, stream); dev->prof.push_back({e0, e1, KC_REDUCE, 0.0}); }
            if (cr != CUDA_SUCCESS) { const char* s = nullptr; dev->drv.GetErrorString(cr, &s); return dev->fail(ANL_ERR_CUDA, std::string("cuda: cuLaunchKernel(row_chain): ") + (s ? s : "?")); }
            dev->stats.kernels_launched++;
            *used = members.size();
            return ANL_OK;
        }
        members.pop_back();
        reads.pop_back();
    }
    return ANL_OK;
}


// ── a contraction and the elementwise kernel behind it as one launch ────────────────────────────
// The schedule keeps what the reference would schedule: item i a dense contraction, item i+1 an
// elementwise kernel that reads it at the output's own position (bias add, activation, the product
// with an activation's derivative), possibly a later item that sums item i+1's output over the rows
// (a bias gradient).  At launch the three run as one contraction kernel: the consumer's generated
// code sits in the epilogue on the narrowed accumulator registers, the contraction's own output is
// still written when anything else reads it, and per-32-row column sums go to scratch memory for a
// small finish kernel.  Values are those of the separate kernels (the consumer bit for bit; the
// bias gradient sums the same f16 values in f32 in another order).
static std::shared_ptr<FusedEpilogue> fused_epilogue_for(anl_device* dev, const Item& gemm, const Item& consumer, int64_t M, int64_t N) {
    uint64_t hk[2] = {structure_hash(gemm), structure_hash(consumer)};
    int acc = 0, hits = 0;
    for (size_t b = 1; b < consumer.bufs.size(); b++) if (consumer.bufs[b].id == gemm.bufs[0].id) { acc = (int)b; hits++; }
    uint64_t key = fnv1a(hk, sizeof hk, (uint64_t)acc * 1315423911ull + 7);
    auto f = dev->fused.find(key);
    if (f != dev->fused.end()) return f->second;
    auto fe = std::make_shared<FusedEpilogue>();
    std::string err;
    if (hits == 1 && consumer.source.empty() && consumer.sym_vars.empty() && render_gemm_epilogue(consumer, acc, M, N, fe->epi, err)) { fe->on = true; fe->acc_param = acc; }
    dev->fused[key] = fe;
    return fe;
}

int run_items(anl_device* dev, const std::vector<Item>& items, const Bindings& binds, Table& t, cudaStream_t stream, bool keep_scratch = false) {
    CodegenOpts opts; opts.debug_bounds = (dev->flags & ANL_OPEN_DEBUG_BOUNDS) != 0;
    // A parameter may only be updated once every kernel of this schedule that reads it has been
    // queued: the update of output X waits for max(producer of X, last reader of its parameter).
    std::unordered_map<size_t, std::vector<uint32_t>> sgd_at;
    for (auto& kv : t.after) {
        if (!kv.second.sgd_master) continue;
        const void* pp = (kv.second.sgd_param ? kv.second.sgd_param : kv.second.sgd_master)->ptr;
        const void* mp = kv.second.sgd_master->ptr;
        size_t at = 0;
        for (size_t i = 0; i < items.size(); i++) {
            if (items[i].bufs[0].id == kv.first) at = std::max(at, i);
            for (size_t b = 1; b < items[i].bufs.size(); b++) {
                const void* q = t.bufs[items[i].bufs[b].id].ptr;
                if (q == pp || q == mp) at = std::max(at, i);
            }
        }
        sgd_at[at].push_back(kv.first);
    }
    const bool chains_on = !(dev->flags & ANL_OPEN_NO_ROW_CHAIN) && !(dev->flags & ANL_OPEN_BEAM);
    // the last all-reduced output of the schedule, when it is a large contraction whose update is
    // not deferred past it: candidate for the split described at its launch below
    size_t tail_split = (size_t)-1;
    if ((dev->nranks > 1 || (dev->flags & ANL_OPEN_TAIL_SPLIT)) && !dev->profiling && !(dev->flags & ANL_OPEN_BEAM)) {
        for (size_t i = items.size(); i-- > 0;) {
            auto ra = t.after.find(items[i].bufs[0].id);
            if (ra == t.after.end() || !ra->second.allreduce) continue;
            const anl_output& a = ra->second;
            auto sg = sgd_at.find(i);
            bool own_update = a.sgd_master && a.resident && sg != sgd_at.end() && sg->second.size() == 1 && sg->second[0] == items[i].bufs[0].id;
            std::shared_ptr<Plan> p;
            if (own_update && items[i].source.empty() && get_plan(dev, items[i], opts, p) == ANL_OK) {
                int64_t row_elems = 0, rows = gemm_window_rows(*p, &row_elems);
                if (rows >= 1024 && rows * row_elems >= (4ll << 20) && a.resident->elems == rows * row_elems) tail_split = i;
            }
            break;      // only the very last collective is exposed
        }
    }
    // A gradient flagged `allreduce == 2` with an update attached is handled the sharded way when its
    // length divides by the rank count: reduce-scatter, every rank updates only its own 1/nranks of
    // the parameter (the update is pure memory traffic, 12 bytes per parameter, and costs as much
    // step time beside the backward pass as after it), then the new parameter values are
    // all-gathered.  The bytes on the wire equal an all-reduce's.  Otherwise: plain all-reduce and a
    // full update on every rank.
    bool allow_shard = true;      // cleared around the tail split: its halves would shard at other boundaries
    auto sharded = [&](const anl_output& a, int64_t cnt) {
        return allow_shard && a.allreduce == 2 && a.sgd_master && a.resident && comm_can_shard(dev) && cnt > 0 && cnt % dev->nranks == 0;
    };
    auto reduce_part = [&](const anl_output& a, int64_t off, int64_t cnt) -> int {
        char* g = (char*)a.resident->ptr + off * dt_storage_bytes(a.resident->dtype);
        if (sharded(a, cnt)) return comm_reduce_scatter_async(dev, g, cnt, a.resident->dtype, stream);
        return comm_allreduce_async(dev, g, cnt, a.resident->dtype, stream);
    };
    auto update_part = [&](const anl_output& a, int64_t off, int64_t cnt) -> int {
        const bool sh = sharded(a, cnt);
        const int64_t sc = sh ? cnt / dev->nranks : cnt, so = sh ? off + dev->rank * sc : off;
        anl_buffer gv = *a.resident, mv = *a.sgd_master, pv = a.sgd_param ? *a.sgd_param : *a.sgd_master;
        gv.ptr = (char*)gv.ptr + so * dt_storage_bytes(gv.dtype); gv.elems = sc;
        mv.ptr = (char*)mv.ptr + so * dt_storage_bytes(mv.dtype); mv.elems = sc;
        pv.ptr = (char*)pv.ptr + so * dt_storage_bytes(pv.dtype); pv.elems = sc;
        comm_fork(dev, stream);
        if (int rc = launch_sgd(dev, &mv, &pv, &gv, a.sgd_lr, a.sgd_scale, dev->comm_stream)) return rc;
        if (sh) {
            const anl_buffer* pb = a.sgd_param ? a.sgd_param : a.sgd_master;
            if (int rc = comm_allgather_async(dev, (char*)pb->ptr + off * dt_storage_bytes(pb->dtype), cnt, pb->dtype)) return rc;
        }
        return ANL_OK;
    };
    struct Absorbed { void* partials; int64_t parts, cols; };
    std::unordered_map<size_t, Absorbed> absorbed;      // item index -> column sums a contraction's epilogue computes for it
    const bool fusion_on = !(dev->flags & (ANL_OPEN_NO_EPILOGUE_FUSION | ANL_OPEN_NO_GEMM));
    // [update the parameter] hooks that fall due once item `at` has been queued
    auto updates_due = [&](size_t at) -> int {
        auto sg = sgd_at.find(at);
        if (sg == sgd_at.end()) return ANL_OK;
        for (uint32_t id : sg->second) {
            const anl_output& a = t.after[id];
            if (int rc = update_part(a, 0, a.sgd_master->elems)) return rc;
        }
        return ANL_OK;
    };
    // A small kernel whose output nothing later in the schedule reads (the scalar loss, a bias gradient)
    // need not hold up the contractions behind it: inside a captured graph it goes to the side stream,
    // behind what has been queued so far, and joins at the end like the updates.  Only where that is
    // plainly safe: scratch stays with the graph (keep_scratch), and no later kernel writes memory this
    // one reads or writes (slots share allocations, so memory is compared, not buffer ids).
    auto side_ok = [&](size_t i, const std::vector<void*>& ptrs) -> bool {
        if (!keep_scratch || dev->profiling || !dev->comm_stream || (dev->flags & ANL_OPEN_BEAM)) return false;
        for (size_t r = i + 1; r < items.size(); r++) {
            for (size_t b = 1; b < items[r].bufs.size(); b++)
                if (items[r].bufs[b].id == items[i].bufs[0].id || t.bufs[items[r].bufs[b].id].ptr == ptrs[0]) return false;
            void* w = t.bufs[items[r].bufs[0].id].ptr;
            for (void* q : ptrs) if (q == w) return false;
        }
        return true;
    };
    for (size_t i = 0; i < items.size(); i++) {
        const Item& it = items[i];
        if (chains_on && !absorbed.count(i)) {
            size_t used = 0;
            int rc = try_row_chain(dev, items, i, t, stream, &used);
            if (rc != ANL_OK) return rc;
            if (used > 0) {
                // a member of the chain may be the last reader of a parameter: its update falls due now
                for (size_t j = i; j < i + used; j++) if (int rc2 = updates_due(j)) return rc2;
                i += used - 1;
                continue;
            }
        }
        std::shared_ptr<Plan> plan;
        CodegenOpts use = opts;
        if ((dev->flags & ANL_OPEN_BEAM) && it.source.empty()) {
            // BeamApplyToItems (codegen/beam.go:470-541): cached winner, else search now
            bool sym = false; for (auto& b : it.bufs) if (b.symbolic()) sym = true;
            Contraction c;
            bool gemm = !(dev->flags & ANL_OPEN_NO_GEMM) && match_contraction(it, c) && c.in_dtype == DT_F16 && c.out_dtype == DT_F16 && !c.m_sym && !c.k_sym;
            if (!sym) {
                if (!dev->beam_loaded) { beam_cache_load(dev, ""); dev->beam_loaded = true; }
                anl_beam_result br;
                cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
                cudaStreamIsCapturing(stream, &cs);
                if (cs == cudaStreamCaptureStatusNone && beam_search(dev, it, 0, 0, &br) == ANL_OK) {
                    if (gemm) use = gemm_beam_opts(br.opts, use.debug_bounds);     // the tensor-core kernel's own tunables
                    else { use.block_threads = br.opts[0]; use.reduce_lanes = br.opts[1]; use.vector_width = br.opts[2]; use.split = br.opts[3]; }
                }
            }
        }
        if (int rc = get_plan(dev, it, use, plan)) { dev->err = "kernel " + std::to_string(i) + ": " + dev->err; return rc; }
        std::vector<void*> ptrs;
        for (auto& b : it.bufs) ptrs.push_back(t.bufs[b.id].ptr);
        auto ra = t.after.find(it.bufs[0].id);
        {
            auto ab = absorbed.find(i);
            if (ab != absorbed.end()) {
                // a bias gradient whose partial column sums an earlier contraction's epilogue produced
                cudaStream_t on = stream;
                if (side_ok(i, ptrs)) { comm_fork(dev, stream); on = dev->comm_stream; dev->stats.side_launches++; }
                if (int rc = launch_colsum_finish(dev, (const float*)ab->second.partials, ab->second.parts, ab->second.cols, ptrs[0], on)) return rc;
                if (keep_scratch) t.owned.push_back(ab->second.partials); else dev->release(ab->second.partials);
                dev->stats.colsums_fused++;
                if (ra != t.after.end() && ra->second.allreduce)
                    if (int rc = reduce_part(ra->second, 0, ra->second.resident->elems)) return rc;
                if (int rc = updates_due(i)) return rc;
                continue;
            }
        }
        if (fusion_on && ra == t.after.end() && i != tail_split && gemm_pair_eligible(*plan)) {
            int64_t M = 0, N = 0, K = 0;
            gemm_shape(*plan, &M, &N, &K);
            const uint32_t out_id = it.bufs[0].id;
            // the elementwise consumer, if it is the very next item
            std::shared_ptr<FusedEpilogue> fe;
            if (i + 1 < items.size() && N % 8 == 0 && !absorbed.count(i + 1)) {
                fe = fused_epilogue_for(dev, it, items[i + 1], M, N);
                if (fe->on) {
                    // the consumer's output must not live in memory this contraction still reads
                    void* o1 = t.bufs[items[i + 1].bufs[0].id].ptr;
                    for (void* q : ptrs) if (q == o1) fe.reset();
                }
                if (fe && !fe->on) fe.reset();
            }
            const Item* last = fe ? &items[i + 1] : &it;          // the kernel whose output the epilogue stores last
            // a later item that sums that output over the rows
            size_t cs_item = 0; bool have_cs = false;
            if (N % 8 == 0) {
                for (size_t r = i + 1 + (fe ? 1 : 0); r < items.size() && !have_cs; r++) {
                    if (absorbed.count(r) || items[r].bufs.size() != 2 || items[r].bufs[1].id != last->bufs[0].id || items[r].bufs[0].slot >= 0) continue;
                    int sp = 0; int64_t rows = 0, cols = 0;
                    if (match_column_sum(items[r], sp, rows, cols) && rows == M && cols == N) { cs_item = r; have_cs = true; }
                }
            }
            if (fe || have_cs) {
                GemmFusion fz;
                if (fe) {
                    fz.epilogue = &fe->epi.source;
                    fz.d_out = t.bufs[items[i + 1].bufs[0].id].ptr;
                    for (size_t k = 0; k < fe->epi.params.size(); k++) fz.ep[k] = t.bufs[items[i + 1].bufs[fe->epi.params[k]].id].ptr;
                    // the contraction itself is stored only when something besides the consumer wants it
                    bool wanted = false;
                    for (uint32_t fid : t.finals) if (fid == out_id) wanted = true;
                    for (size_t r = i + 2; r < items.size() && !wanted; r++)
                        for (size_t b = 1; b < items[r].bufs.size(); b++) if (items[r].bufs[b].id == out_id) wanted = true;
                    fz.store_raw = wanted;
                }
                void* partials = nullptr;
                const int64_t parts = (M + 31) / 32;
                if (have_cs) {
                    if (int rc = dev->alloc((size_t)parts * (size_t)N * 4, &partials)) return rc;
                    fz.colsum = (float*)partials;
                    absorbed[cs_item] = Absorbed{partials, parts, N};
                }
                cudaEvent_t e0 = nullptr, e1 = nullptr;
                if (dev->profiling) { cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventRecord(e0, stream); }
                int rc = launch_gemm(dev, *plan, ptrs.data(), item_sym(it, binds), stream, 0, -1, &fz);
                if (dev->profiling) { cudaEventRecord(e1, stream); dev->prof.push_back({e0, e1, KC_GEMM, gemm_flops(*plan, 0)}); }
                if (rc) { dev->err = "kernel " + std::to_string(i) + ": " + dev->err; return rc; }
                if (int rc2 = updates_due(i)) return rc2;
                if (fe) {
                    dev->stats.epilogues_fused++;
                    // hooks of the consumer, which this launch has just run
                    auto rb = t.after.find(items[i + 1].bufs[0].id);
                    if (rb != t.after.end() && rb->second.allreduce)
                        if (int rc3 = reduce_part(rb->second, 0, rb->second.resident->elems)) return rc3;
                    if (int rc3 = updates_due(i + 1)) return rc3;
                    i += 1;
                }
                continue;
            }
        }
        if (i == tail_split && ra != t.after.end()) {
            // The last all-reduced gradient has nothing left to hide behind.  Its contraction is
            // launched as two row windows; the first half is reduced across ranks and applied while
            // the second half is still being computed, so only half of it stays exposed.
            const anl_output& a = ra->second;
            int64_t row_elems = 0, rows = gemm_window_rows(*plan, &row_elems);
            const int64_t cut = (rows / 2 + 255) / 256 * 256;
                        // both halves are all-reduced and updated in full on every rank: sharding each half would put
            // a rank's shards at other offsets than anl_allgather assumes for the whole parameter
            allow_shard = false;
            for (int h = 0; h < 2; h++) {
                const int64_t m0 = h ? cut : 0, m1 = h ? rows : cut;
                if (int rc = launch_gemm(dev, *plan, ptrs.data(), item_sym(it, binds), stream, m0, m1)) { dev->err = "kernel " + std::to_string(i) + ": " + dev->err; return rc; }
                const int64_t off = m0 * row_elems, cnt = (m1 - m0) * row_elems;
                if (int rc = reduce_part(a, off, cnt)) return rc;
                if (int rc = update_part(a, off, cnt)) return rc;
            }
            allow_shard = true;
            continue;
        }
        cudaStream_t on = stream;
        if (!gemm_taken(*plan, item_sym(it, binds)) && side_ok(i, ptrs)) { comm_fork(dev, stream); on = dev->comm_stream; dev->stats.side_launches++; }
        if (int rc = launch_plan(dev, *plan, it, ptrs.data(), item_sym(it, binds), on, keep_scratch ? &t.owned : nullptr)) { dev->err = "kernel " + std::to_string(i) + ": " + dev->err; return rc; }
        // side stream: [all-reduce this gradient] behind the producing kernel ...
        if (ra != t.after.end() && ra->second.allreduce)
            if (int rc = reduce_part(ra->second, 0, ra->second.resident->elems)) return rc;
        // ... [update the parameter] once its last reader has been queued as well
        if (int rc = updates_due(i)) return rc;
    }
    return comm_join(dev, stream);
}

// `may_return_early`: when no output goes to host memory the call returns with the work still
// queued (stream order keeps later calls correct; an asynchronous fault surfaces at the next call
// that waits).  Otherwise the stream is drained so that the host arrays are complete on return.
int collect_outputs(anl_device* dev, Table& t, const anl_output* placed, int n_placed, anl_output* outs, int* n_outs, cudaStream_t stream,
                    bool may_return_early = false) {
    int cap = *n_outs, n = 0;
    bool to_host = false;
    std::vector<float*> mine;
    int rc = ANL_OK;
    for (uint32_t id : t.finals) {
        if (n >= cap) { rc = dev->fail(ANL_ERR_LIMIT, "run: more final outputs than the caller made room for"); break; }
        DevBuf& d = t.bufs[id];
        anl_output o{}; o.uop_idx = id; o.elems = d.elems;
        const anl_output* pl = nullptr;
        for (int k = 0; k < n_placed; k++) if (placed[k].uop_idx == id) pl = &placed[k];
        if (pl && pl->resident) { o.resident = pl->resident; }
        else {
            if (pl && pl->data) {
                if (pl->elems < d.elems) { rc = dev->fail(ANL_ERR_INVALID, "run: placed output array is too small"); break; }
                o.data = pl->data;
            } else {
                o.data = (float*)std::malloc((size_t)std::max<int64_t>(d.elems, 1) * 4);
                if (!o.data) { rc = dev->fail(ANL_ERR_LIMIT, "run: out of host memory"); break; }
                mine.push_back(o.data);
                { std::lock_guard<std::mutex> lk(g_owned_mu); g_owned_outputs.insert(o.data); }
            }
            to_host = true;
            if ((rc = download_f32(dev, o.data, d.ptr, d.dtype, d.elems, stream))) break;
        }
        outs[n++] = o;
    }
    const bool waited = !(may_return_early && !to_host && rc == ANL_OK);
    if (waited) {
        // a captured step carries its collectives on this stream: wait under the watchdog
        int wrc = wait_stream_watched(dev, stream, "run");
        if (rc == ANL_OK) rc = wrc;
    }
    if (rc == ANL_OK && waited) rc = gemm_check_status(dev);
    if (rc != ANL_OK) {
        std::lock_guard<std::mutex> lk(g_owned_mu);
        for (float* p : mine) { g_owned_outputs.erase(p); std::free(p); }
        n = 0;
    }
    *n_outs = n;
    return rc;
}

Bindings make_bindings(const anl_binding* binds, int n) {
    Bindings b;
    for (int i = 0; i < n; i++) b.v.push_back({binds[i].name ? binds[i].name : "", binds[i].value});
    return b;
}

CodegenOpts opts_from(const int* o, unsigned flags) {
    CodegenOpts c;
    if (o) {
        c.block_threads = o[0]; c.reduce_lanes = o[1]; c.vector_width = o[2]; c.split = o[3]; c.debug_bounds = o[4] != 0;
        c.gemm_tile_n = o[5]; c.gemm_stages = o[6]; c.gemm_group_m = o[7]; c.gemm_stream_stores = o[8]; c.gemm_single_cta = o[9]; c.gemm_whole_tail = o[10];
    }
    if (flags & ANL_OPEN_DEBUG_BOUNDS) c.debug_bounds = true;
    return c;
}

}  // namespace

struct anl_graph {
    anl_device* dev = nullptr;
    std::vector<Item> items;
    Table table;
    bool built = false;
    uint64_t kernels_per_replay = 0, gemms_per_replay = 0;
    int64_t built_sym = -2;
    cudaGraphExec_t exec = nullptr;
    std::vector<std::pair<uint32_t, anl_buffer*>> resident_in, resident_out;
    uint64_t placed_key = 0;     // hash of what the capture baked in besides pointers: update targets, rate, scale, reduce mode
    // Captures for other bindings of the same schedule (a symbolic batch cycling through a few
    // values, tensor/jit.go:86-118 replaySym): parked with their buffers instead of being rebuilt
    // every time the bound value changes.
    struct Parked {
        Table table; cudaGraphExec_t exec; int64_t sym; uint64_t placed_key, kernels, gemms;
        std::vector<std::pair<uint32_t, anl_buffer*>> rin, rout;
    };
    std::vector<Parked> parked;
    static constexpr size_t kMaxParked = 7;
};

// ── exception fence ──────────────────────────────────────────────────────────────────────────
// The entry points that parse, generate code or build tables use the C++ library freely; nothing it
// throws (bad_alloc above all) may cross the C boundary, where the caller is Go or ctypes.
namespace {
template <class F> int fenced(anl_device* dev, const char* what, F&& f) noexcept {
    try { return f(); }
    catch (const std::bad_alloc&) { std::string m = std::string("cuda: ") + what + ": out of host memory"; return dev ? dev->fail(ANL_ERR_LIMIT, m) : ANL_ERR_LIMIT; }
    catch (const std::exception& e) { std::string m = std::string("cuda: ") + what + ": " + e.what(); return dev ? dev->fail(ANL_ERR_INVALID, m) : ANL_ERR_INVALID; }
    catch (...) { return dev ? dev->fail(ANL_ERR_INVALID, std::string("cuda: ") + what + ": unknown failure") : ANL_ERR_INVALID; }
}
}  // namespace


extern "C" {

int anl_open(int ordinal, unsigned flags, anl_device** out) {
    if (!out) return ANL_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || ordinal < 0 || ordinal >= count) return ANL_ERR_NO_DEVICE;
    auto* d = new anl_device();
    d->ordinal = ordinal; d->flags = flags;
    if (cudaSetDevice(ordinal) != cudaSuccess || cudaFree(0) != cudaSuccess || cudaGetDeviceProperties(&d->prop, ordinal) != cudaSuccess) { delete d; return ANL_ERR_NO_DEVICE; }
    if (d->prop.major < 10) { delete d; return ANL_ERR_NO_DEVICE; }   // kernels are built for sm_100a only
    if (cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking) != cudaSuccess) { delete d; return ANL_ERR_CUDA; }
    {   // collectives get the highest priority so their blocks are placed as soon as an SM frees up
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        cudaStreamCreateWithPriority(&d->comm_stream, cudaStreamNonBlocking, hi);
    }
    cudaEventCreateWithFlags(&d->comm_event, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&d->comm_done, cudaEventDisableTiming);
    if (ensure_driver(d) != ANL_OK) { delete d; return ANL_ERR_CUDA; }
    *out = d;
    return ANL_OK;
}

void anl_close(anl_device* dev) {
    if (!dev) return;
    cudaSetDevice(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    anl_comm_destroy(dev);
    for (auto& kv : dev->modules) if (kv.second->mod && dev->drv.ModuleUnload) dev->drv.ModuleUnload(kv.second->mod);
    dev->trim();
    for (auto& kv : dev->live) cudaFree(kv.first);
    if (dev->gemm_tile_counter) cudaFree(dev->gemm_tile_counter);
    if (dev->gemm_status_host) cudaFreeHost(dev->gemm_status_host);
    for (auto& r : dev->prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
    if (dev->timer0) { cudaEventDestroy(dev->timer0); cudaEventDestroy(dev->timer1); }
    if (dev->comm_event) cudaEventDestroy(dev->comm_event);
    if (dev->comm_done) cudaEventDestroy(dev->comm_done);
    if (dev->comm_stream) cudaStreamDestroy(dev->comm_stream);
    if (dev->copy_stream) cudaStreamDestroy(dev->copy_stream);
    if (dev->stream) cudaStreamDestroy(dev->stream);
    delete dev;
}

int anl_device_info(anl_device* dev, anl_info* info) {
    if (!dev || !info) return ANL_ERR_INVALID;
    std::memset(info, 0, sizeof *info);
    std::snprintf(info->name, sizeof info->name, "%s", dev->prop.name);
    info->sm_major = dev->prop.major; info->sm_minor = dev->prop.minor; info->sm_count = dev->prop.multiProcessorCount;
    info->total_mem = dev->prop.totalGlobalMem;
    info->has_f16 = 1; info->has_bf16 = 1; info->has_tcgen05 = dev->prop.major == 10;
    return ANL_OK;
}

const char* anl_last_error(anl_device* dev) { return dev ? dev->err.c_str() : "no device"; }

int anl_get_stats(anl_device* dev, anl_stats* out) { if (!dev || !out) return ANL_ERR_INVALID; *out = dev->stats; return ANL_OK; }

int anl_gemm_set_defaults(anl_device* dev, const int* o) {
    if (!dev) return ANL_ERR_INVALID;
    GemmTuning t;
    if (o) { t.tile_n = o[5]; t.stages = o[6]; t.group_m = o[7]; t.stream_stores = o[8]; t.single_cta = o[9]; t.no_split_tail = o[10]; }
    if (t.tile_n != 0 && t.tile_n != 128 && t.tile_n != 256) return dev->fail(ANL_ERR_INVALID, "gemm defaults: tile_n must be 0, 128 or 256");
    dev->gemm_defaults = t;
    return ANL_OK;
}

int anl_gemm_inject_status(anl_device* dev, int code, int counter_value) {
    if (!dev) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    return gemm_inject_status(dev, code, counter_value);
}

void* anl_stream(anl_device* dev) { return dev ? (void*)dev->stream : nullptr; }

int anl_synchronize(anl_device* dev) {
    if (!dev) return ANL_ERR_INVALID;
    // with a communication timeout set, the collective stream is waited for under the watchdog first:
    // the compute stream may itself be waiting for a collective that will never finish
    if (dev->comm_stream && dev->comm_timeout_ms > 0) if (int rc = anl_comm_wait(dev)) return rc;
    if (int rc = wait_stream_watched(dev, dev->stream, "synchronize")) return rc;      // replays carry their collectives here
    if (dev->comm_stream) CK(dev, cudaStreamSynchronize(dev->comm_stream));
    if (dev->copy_stream) CK(dev, cudaStreamSynchronize(dev->copy_stream));
    return gemm_check_status(dev);
}

static int run_impl(anl_device* dev, const uint8_t* blob, size_t blob_len, const anl_input* inputs, int n_inputs,
            const anl_binding* binds, int n_binds, const anl_output* placed, int n_placed, anl_output* outs, int* n_outs) {
    if (!dev || !n_outs) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    std::vector<Item> items; std::string perr;
    if (!parse_kir(blob, blob_len, items, perr)) return dev->fail(ANL_ERR_INVALID, perr);
    if (items.empty()) { *n_outs = 0; return ANL_OK; }     // empty schedule → (nil, nil), backend/webgpu/executor.go:27-29
    for (auto& it : items) if (it.bufs.empty()) return dev->fail(ANL_ERR_INVALID, "run: item without buffers");
    Bindings b = make_bindings(binds, n_binds);
    Table t;
    int rc = build_table(dev, items, b, inputs, n_inputs, placed, n_placed, t);
    if (rc == ANL_OK) rc = run_items(dev, items, b, t, dev->stream);
    if (rc == ANL_OK) rc = collect_outputs(dev, t, placed, n_placed, outs, n_outs, dev->stream);
    else { cudaStreamSynchronize(dev->stream); *n_outs = 0; }
    for (void* p : t.owned) dev->release(p);
    return rc;
}

void anl_outputs_free(anl_output* outs, int n_outs) {
    if (!outs) return;
    std::lock_guard<std::mutex> lk(g_owned_mu);
    for (int i = 0; i < n_outs; i++) {
        auto it = outs[i].data ? g_owned_outputs.find(outs[i].data) : g_owned_outputs.end();
        if (it != g_owned_outputs.end()) { std::free(outs[i].data); g_owned_outputs.erase(it); }
        outs[i].data = nullptr;
    }
}

static int lower_impl(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, const int* o,
              char* src, size_t src_cap, size_t* src_len, int* klass, int* block, int64_t* opb, char* note, size_t note_cap) {
    std::vector<Item> items; std::string err;
    if (!parse_kir(blob, blob_len, items, err)) { if (dev) dev->err = err; return ANL_ERR_INVALID; }
    if (index < 0 || index >= (int)items.size()) return ANL_ERR_INVALID;
    Rendered r;
    if (!render_cuda(items[index], opts_from(o, dev ? dev->flags : 0), r, err)) {
        if (dev) dev->err = err;
        if (note && note_cap) std::snprintf(note, note_cap, "%s", err.c_str());
        return ANL_ERR_UNSUPPORTED;
    }
    if (src && src_cap) { size_t n = std::min(src_cap - 1, r.source.size()); std::memcpy(src, r.source.data(), n); src[n] = 0; }
    if (src_len) *src_len = r.source.size();
    if (klass) *klass = r.klass;
    if (block) *block = (int)r.main.block;
    if (opb) *opb = r.main.outputs_per_block;
    {   // say when the device would route this item to a contraction kernel instead of this source
        Contraction c;
        if (match_contraction(items[index], c)) {
            auto ext = [](int64_t v, bool sym) { return sym ? std::string("n") : std::to_string(v); };
            r.note += (r.note.empty() ? "" : "; ") + std::string("contraction ") + (c.in_dtype == DT_F16 ? "f16" : c.in_dtype == DT_F32 ? "f32" : "other") +
                      " M=" + ext(c.M, c.m_sym) + " N=" + std::to_string(c.N) + " K=" + ext(c.K, c.k_sym);
        }
    }
    if (note && note_cap) std::snprintf(note, note_cap, "%s", r.note.c_str());
    return ANL_OK;
}

static int lower_chain_impl(const uint8_t* blob, size_t blob_len, int first, int count, char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap) {
    std::vector<Item> items; std::string err;
    if (!parse_kir(blob, blob_len, items, err) || first < 0 || count < 2 || first + count > (int)items.size()) {
        if (note && note_cap) std::snprintf(note, note_cap, "%s", err.empty() ? "chain: bad item range" : err.c_str());
        return ANL_ERR_INVALID;
    }
    std::vector<const Item*> members;
    std::vector<std::vector<std::pair<int, int>>> reads;
    for (int j = first; j < first + count; j++) {
        std::vector<std::pair<int, int>> rd;
        for (size_t b = 1; b < items[j].bufs.size(); b++)
            for (size_t m = 0; m < members.size(); m++)
                if (members[m]->bufs[0].id == items[j].bufs[b].id) rd.push_back({(int)b, (int)m});
        members.push_back(&items[j]);
        reads.push_back(rd);
    }
    ChainRendered r; CodegenOpts o;
    if (!render_row_chain(members, reads, o, r, err)) { if (note && note_cap) std::snprintf(note, note_cap, "%s", err.c_str()); return ANL_ERR_UNSUPPORTED; }
    if (src && src_cap) { size_t n = std::min(src_cap - 1, r.source.size()); std::memcpy(src, r.source.data(), n); src[n] = 0; }
    if (src_len) *src_len = r.source.size();
    if (note && note_cap) std::snprintf(note, note_cap, "%s", r.note.c_str());
    return ANL_OK;
}

static int lower_gemm_impl(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, int fuse_next, const int* o,
                           char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap) {
    std::vector<Item> items; std::string err;
    auto say = [&](const std::string& m) { if (dev) dev->err = m; if (note && note_cap) std::snprintf(note, note_cap, "%s", m.c_str()); };
    if (!parse_kir(blob, blob_len, items, err)) { say(err); return ANL_ERR_INVALID; }
    if (index < 0 || index >= (int)items.size()) { say("lower_gemm: item index out of range"); return ANL_ERR_INVALID; }
    Plan p;
    if (plan_gemm(items[index], tuning_of(opts_from(o, 0)), p) != ANL_OK || !(gemm_pair_eligible(p) || gemm_tf32_eligible(p))) { say("lower_gemm: the item does not run on the two-CTA contraction kernel"); return ANL_ERR_UNSUPPORTED; }
    std::string epilogue, what = p.r.note;
    if (gemm_tf32_eligible(p)) {
        if (fuse_next) { say("lower_gemm: the f32 form of the kernel takes no fused consumer"); return ANL_ERR_UNSUPPORTED; }
        std::string out;
        if (int rc = gemm_tf32_source(p, out, what)) return rc;
        if (src && src_cap) { size_t n = std::min(src_cap - 1, out.size()); std::memcpy(src, out.data(), n); src[n] = 0; }
        if (src_len) *src_len = out.size();
        if (note && note_cap) std::snprintf(note, note_cap, "%s", what.c_str());
        return ANL_OK;
    }
    if (fuse_next) {
        if (index + 1 >= (int)items.size()) { say("lower_gemm: no next item to fuse"); return ANL_ERR_UNSUPPORTED; }
        int64_t M, N, K; gemm_shape(p, &M, &N, &K);
        int acc = 0, hits = 0;
        for (size_t b = 1; b < items[index + 1].bufs.size(); b++) if (items[index + 1].bufs[b].id == items[index].bufs[0].id) { acc = (int)b; hits++; }
        EpilogueRendered er;
        if (hits != 1 || N % 8 != 0 || !render_gemm_epilogue(items[index + 1], acc, M, N, er, err)) { say(err.empty() ? "lower_gemm: the next item does not read this contraction once" : err); return ANL_ERR_UNSUPPORTED; }
        epilogue = er.source;
        what += "; " + er.note;
    }
    std::string out;
    if (int rc = gemm_pair_source(dev, p, epilogue, out)) return rc;
    if (src && src_cap) { size_t n = std::min(src_cap - 1, out.size()); std::memcpy(src, out.data(), n); src[n] = 0; }
    if (src_len) *src_len = out.size();
    if (note && note_cap) std::snprintf(note, note_cap, "%s", what.c_str());
    return ANL_OK;
}

int anl_compile_check(const char* src, char* log, size_t log_cap) {
    std::vector<char> cubin; std::string l;
    int rc = nvrtc_compile(src ? src : "", cubin, l);
    if (log && log_cap) std::snprintf(log, log_cap, "%s", l.c_str());
    return rc;
}

// Benchmarker.Benchmark (backend/webgpu/benchmark.go:18-208): the reference times submit+wait with
// the host clock and reports min/median/max/mean/stddev/CV; here each iteration is bracketed by CUDA
// events on the launching stream.  The reference's inputs are zero-filled buffers; here float
// operands get finite pseudo-random values, because a tensor-core kernel fed with zeros draws less
// power and clocks higher than it ever does on data.
static int benchmark_impl(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, const int* o, int warmup, int iterations, anl_bench_result* out) {
    if (!dev || !out || iterations <= 0) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    std::vector<Item> items; std::string perr;
    if (!parse_kir(blob, blob_len, items, perr)) return dev->fail(ANL_ERR_INVALID, perr);
    if (index < 0 || index >= (int)items.size()) return dev->fail(ANL_ERR_INVALID, "benchmark: item index out of range");
    const Item& it = items[index];
    for (auto& b : it.bufs) if (b.symbolic()) return dev->fail(ANL_ERR_UNSUPPORTED, "benchmark: symbolic kernels are not timed");
    std::shared_ptr<Plan> plan;
    if (int rc = get_plan(dev, it, opts_from(o, dev->flags), plan)) return rc;
    std::vector<void*> ptrs;
    int rc = ANL_OK;
    for (auto& b : it.bufs) {
        void* p = nullptr; size_t by = (size_t)b.elems(0) * dt_storage_bytes(b.dtype);
        if ((rc = dev->alloc(by, &p))) break;
        if (dt_is_float(b.dtype) && b.dtype != DT_BF16 && by >= 4)
            fill_benchmark_pattern<<<grid_for((long long)(by / 4), 256, dev->prop.multiProcessorCount), 256, 0, dev->stream>>>((unsigned*)p, (long long)(by / 4), b.dtype == DT_F16, 0x9E3779B9u * (unsigned)(ptrs.size() + 1));
        else cudaMemsetAsync(p, 0, by ? by : 4, dev->stream);
        ptrs.push_back(p);
    }
    std::vector<double> us;
    if (rc == ANL_OK) {
        cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
        for (int i = 0; i < warmup + iterations && rc == ANL_OK; i++) {
            launch_hold_stream(dev->stream, 200000);
            cudaEventRecord(e0, dev->stream);
            rc = launch_plan(dev, *plan, it, ptrs.data(), 0, dev->stream, nullptr);
            cudaEventRecord(e1, dev->stream);
            if (cudaEventSynchronize(e1) != cudaSuccess) rc = dev->fail(ANL_ERR_CUDA, "benchmark: kernel failed");
            float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
            if (i >= warmup) us.push_back(ms * 1000.0);
        }
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    for (void* p : ptrs) dev->release(p);
    if (rc != ANL_OK) return rc;
    std::sort(us.begin(), us.end());
    double sum = 0; for (double v : us) sum += v;
    double mean = sum / us.size(), var = 0;
    for (double v : us) var += (v - mean) * (v - mean);
    out->min_us = us.front(); out->max_us = us.back(); out->median_us = us[us.size() / 2];
    out->mean_us = mean; out->stddev_us = std::sqrt(var / us.size()); out->cv = mean > 0 ? out->stddev_us / mean : 0;
    return ANL_OK;
}

int anl_buffer_create(anl_device* dev, int dtype, int64_t elems, anl_buffer** out) {
    if (!dev || !out || elems < 0) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    auto* b = new anl_buffer();
    b->dev = dev; b->dtype = dtype; b->elems = elems; b->bytes = (size_t)elems * dt_storage_bytes(dtype);
    if (int rc = dev->alloc(b->bytes, &b->ptr)) { delete b; return rc; }
    cudaMemsetAsync(b->ptr, 0, b->bytes ? b->bytes : 4, dev->stream);
    *out = b;
    return ANL_OK;
}
int anl_buffer_upload(anl_buffer* buf, const float* data, int64_t elems) {
    if (!buf || !data || elems > buf->elems) return ANL_ERR_INVALID;
    cudaSetDevice(buf->dev->ordinal);
    if (int rc = upload_f32(buf->dev, buf->ptr, buf->dtype, data, elems, buf->dev->stream)) return rc;
    CK(buf->dev, cudaStreamSynchronize(buf->dev->stream));
    return ANL_OK;
}
int anl_buffer_download(anl_buffer* buf, float* data, int64_t elems) {
    if (!buf || !data || elems > buf->elems) return ANL_ERR_INVALID;
    cudaSetDevice(buf->dev->ordinal);
    if (int rc = download_f32(buf->dev, data, buf->ptr, buf->dtype, elems, buf->dev->stream)) return rc;
    return wait_stream_watched(buf->dev, buf->dev->stream, "download");
}
// Pipelined upload, first half: the copy stream moves `elems` floats from (pinned) host memory
// into the buffer's staging block and returns at once.  The buffer's contents are untouched, so
// kernels already queued on the compute stream keep reading the previous batch meanwhile.
static int upload_begin_impl(anl_buffer* buf, const void* data, int64_t elems, bool stored) {
    if (!buf || !data || elems <= 0 || elems > buf->elems) return ANL_ERR_INVALID;
    anl_device* dev = buf->dev;
    cudaSetDevice(dev->ordinal);
    if (!dev->copy_stream) CK(dev, cudaStreamCreateWithFlags(&dev->copy_stream, cudaStreamNonBlocking));
    if (!buf->stage) {
        if (int rc = dev->alloc((size_t)buf->elems * 4, &buf->stage)) return rc;
        CK(dev, cudaEventCreateWithFlags(&buf->stage_ready, cudaEventDisableTiming));
        CK(dev, cudaEventCreateWithFlags(&buf->stage_free, cudaEventDisableTiming));
        // the pool orders its blocks along the compute stream: let whatever used this block finish
        CK(dev, cudaEventRecord(buf->stage_free, dev->stream));
        buf->stage_free_recorded = true;
    }
    // host elements are f32, or already in the buffer's storage format (2 bytes for f16, else 4)
    const size_t esz = (stored && buf->dtype == DT_F16) ? 2 : 4;
    if (buf->stage_free_recorded) CK(dev, cudaStreamWaitEvent(dev->copy_stream, buf->stage_free, 0));
    CK(dev, cudaMemcpyAsync(buf->stage, data, (size_t)elems * esz, cudaMemcpyHostToDevice, dev->copy_stream));
    CK(dev, cudaEventRecord(buf->stage_ready, dev->copy_stream));
    buf->staged_elems = elems;
    buf->staged_stored = stored;
    dev->stats.h2d_bytes += (uint64_t)elems * esz;
    return ANL_OK;
}
int anl_buffer_upload_begin(anl_buffer* buf, const float* data, int64_t elems) { return upload_begin_impl(buf, data, elems, false); }
int anl_buffer_upload_begin_stored(anl_buffer* buf, const void* data, int64_t elems) { return upload_begin_impl(buf, data, elems, true); }
// Second half: the compute stream waits for the staged copy and converts it into the buffer's
// storage dtype, in stream order with the kernels around it.
int anl_buffer_upload_commit(anl_buffer* buf) {
    if (!buf) return ANL_ERR_INVALID;
    anl_device* dev = buf->dev;
    if (buf->staged_elems <= 0) return dev->fail(ANL_ERR_INVALID, "buffer: upload_commit without upload_begin");
    cudaSetDevice(dev->ordinal);
    const int64_t n = buf->staged_elems;
    CK(dev, cudaStreamWaitEvent(dev->stream, buf->stage_ready, 0));
    if (buf->staged_stored) {
        // already in storage format: bytes move as they are (a bf16 slot must arrive with its low half clear)
        CK(dev, cudaMemcpyAsync(buf->ptr, buf->stage, (size_t)n * (buf->dtype == DT_F16 ? 2 : 4), cudaMemcpyDeviceToDevice, dev->stream));
    } else if (buf->dtype == DT_F16 || buf->dtype == DT_BF16) {
        unsigned g = grid_for(n, 256, dev->prop.multiProcessorCount);
        if (buf->dtype == DT_F16) cvt_f32_to_f16<<<g, 256, 0, dev->stream>>>((const float*)buf->stage, (__half*)buf->ptr, n);
        else cvt_f32_to_bf16slot<<<g, 256, 0, dev->stream>>>((const float*)buf->stage, (float*)buf->ptr, n);
        CK(dev, cudaGetLastError());
        dev->stats.kernels_launched++;
    } else {
        CK(dev, cudaMemcpyAsync(buf->ptr, buf->stage, (size_t)n * 4, cudaMemcpyDeviceToDevice, dev->stream));
    }
    CK(dev, cudaEventRecord(buf->stage_free, dev->stream));
    buf->stage_free_recorded = true;
    buf->staged_elems = 0;
    return ANL_OK;
}
// Read-back without stalling the host.  `begin` queues, behind everything already queued on the compute
// stream, a copy of the buffer's first `elems` values (widened to f32) into `host` — pinned memory,
// or the copy is not asynchronous — and returns at once; `wait` blocks until the last copy begun on
// this buffer has landed.  A training loop reads step i's loss this way while step i+1 runs.
int anl_buffer_download_begin(anl_buffer* buf, float* host, int64_t elems) {
    if (!buf || !host || elems <= 0 || elems > buf->elems) return ANL_ERR_INVALID;
    anl_device* dev = buf->dev;
    cudaSetDevice(dev->ordinal);
    if (!buf->dl_done) CK(dev, cudaEventCreateWithFlags(&buf->dl_done, cudaEventDisableTiming));
    const void* src = buf->ptr;
    if (buf->dtype == DT_F16) {
        if (!buf->dl_stage || buf->dl_stage_elems < elems) {
            if (buf->dl_stage) dev->release(buf->dl_stage);
            if (int rc = dev->alloc((size_t)elems * 4, &buf->dl_stage)) return rc;
            buf->dl_stage_elems = elems;
        }
        cvt_f16_to_f32<<<grid_for(elems, 256, dev->prop.multiProcessorCount), 256, 0, dev->stream>>>((const __half*)buf->ptr, (float*)buf->dl_stage, elems);
        CK(dev, cudaGetLastError());
        dev->stats.kernels_launched++;
        src = buf->dl_stage;
    }
    CK(dev, cudaMemcpyAsync(host, src, (size_t)elems * 4, cudaMemcpyDeviceToHost, dev->stream));
    CK(dev, cudaEventRecord(buf->dl_done, dev->stream));
    buf->dl_pending = true;
    dev->stats.d2h_bytes += (uint64_t)elems * 4;
    return ANL_OK;
}
int anl_buffer_download_wait(anl_buffer* buf) {
    if (!buf) return ANL_ERR_INVALID;
    if (!buf->dl_pending) return buf->dev->fail(ANL_ERR_INVALID, "buffer: download_wait without download_begin");
    cudaSetDevice(buf->dev->ordinal);
    CK(buf->dev, cudaEventSynchronize(buf->dl_done));
    buf->dl_pending = false;
    return ANL_OK;
}
void anl_buffer_release(anl_buffer* buf) {
    if (!buf) return;
    cudaStreamSynchronize(buf->dev->stream);
    if (buf->dl_stage) buf->dev->release(buf->dl_stage);
    if (buf->dl_done) cudaEventDestroy(buf->dl_done);
    if (buf->stage) {
        if (buf->dev->copy_stream) cudaStreamSynchronize(buf->dev->copy_stream);
        buf->dev->release(buf->stage);
        cudaEventDestroy(buf->stage_ready); cudaEventDestroy(buf->stage_free);
    }
    if (!buf->view) buf->dev->release(buf->ptr);
    delete buf;
}
int anl_buffer_view(anl_buffer* parent, int64_t offset, int64_t elems, anl_buffer** out) {
    if (!parent || !out || offset < 0 || elems < 0 || offset + elems > parent->elems) return ANL_ERR_INVALID;
    if (offset % 128) return parent->dev->fail(ANL_ERR_INVALID, "buffer view: offset must be a multiple of 128 elements");
    auto* b = new anl_buffer();
    b->dev = parent->dev; b->dtype = parent->dtype; b->elems = elems; b->view = true;
    b->bytes = (size_t)elems * dt_storage_bytes(parent->dtype);
    b->ptr = (char*)parent->ptr + (size_t)offset * dt_storage_bytes(parent->dtype);
    *out = b;
    return ANL_OK;
}
void* anl_buffer_device_ptr(anl_buffer* buf) { return buf ? buf->ptr : nullptr; }
int64_t anl_buffer_elems(anl_buffer* buf) { return buf ? buf->elems : 0; }

int anl_sgd_step(anl_device* dev, anl_buffer* master, anl_buffer* param, anl_buffer* grad, float lr, float scale) {
    if (!dev || !master || !param || !grad) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    return anl::launch_sgd(dev, master, param, grad, lr, scale, dev->stream);
}

int anl_timer_start(anl_device* dev) {
    if (!dev) return ANL_ERR_INVALID;
    cudaSetDevice(dev->ordinal);
    if (!dev->timer0) { CK(dev, cudaEventCreate(&dev->timer0)); CK(dev, cudaEventCreate(&dev->timer1)); }
    CK(dev, cudaEventRecord(dev->timer0, dev->stream));
    return ANL_OK;
}
int anl_timer_stop(anl_device* dev, float* ms) {
    if (!dev || !ms || !dev->timer0) return ANL_ERR_INVALID;
    CK(dev, cudaEventRecord(dev->timer1, dev->stream));
    CK(dev, cudaEventSynchronize(dev->timer1));
    CK(dev, cudaEventElapsedTime(ms, dev->timer0, dev->timer1));
    return ANL_OK;
}
int anl_profile_enable(anl_device* dev, int on) {
    if (!dev) return ANL_ERR_INVALID;
    cudaStreamSynchronize(dev->stream);
    for (auto& r : dev->prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
    dev->prof.clear();
    dev->profiling = on != 0;
    return ANL_OK;
}
int anl_profile_read(anl_device* dev, anl_profile_entry* out, int cap, int* n) {
    if (!dev || !out || !n) return ANL_ERR_INVALID;
    CK(dev, cudaStreamSynchronize(dev->stream));
    std::map<int, anl_profile_entry> acc;
    for (auto& r : dev->prof) {
        float ms = 0; cudaEventElapsedTime(&ms, r.e0, r.e1);
        anl_profile_entry& e = acc[r.klass];
        e.klass = r.klass; e.launches++; e.total_ms += ms; e.flops += r.flops;
    }
    int k = 0;
    for (auto& kv : acc) { if (k >= cap) break; out[k++] = kv.second; }
    *n = k;
    return ANL_OK;
}

int anl_host_alloc(size_t bytes, void** out) { return cudaMallocHost(out, bytes ? bytes : 4) == cudaSuccess ? ANL_OK : ANL_ERR_CUDA; }
void anl_host_free(void* p) { if (p) cudaFreeHost(p); }

// ── JIT replay through a CUDA graph ──────────────────────────────────────────────────────────
static int graph_create_impl(anl_device* dev, const uint8_t* blob, size_t blob_len, anl_graph** out) {
    if (!dev || !out) return ANL_ERR_INVALID;
    auto* g = new anl_graph();
    g->dev = dev;
    std::string perr;
    if (!parse_kir(blob, blob_len, g->items, perr)) { delete g; return dev->fail(ANL_ERR_INVALID, perr); }
    for (auto& it : g->items) if (it.bufs.empty()) { delete g; return dev->fail(ANL_ERR_INVALID, "graph: item without buffers"); }
    *out = g;
    return ANL_OK;
}

static void graph_drop(anl_graph* g) {
    if (g->exec) { cudaGraphExecDestroy(g->exec); g->exec = nullptr; }
    for (void* p : g->table.owned) g->dev->release(p);
    g->table = Table();
    g->built = false;
}

// The current capture does not fit this call's binding or placements: park it, and bring back a
// parked one that does, if there is one.
static void graph_switch(anl_graph* g, int64_t sym, const std::vector<std::pair<uint32_t, anl_buffer*>>& rin,
                         const std::vector<std::pair<uint32_t, anl_buffer*>>& rout, uint64_t pkey) {
    if (g->built) {
        if (g->parked.size() >= anl_graph::kMaxParked) {
            // oldest out: wait for it, then free its graph and buffers
            cudaStreamSynchronize(g->dev->stream);
            anl_graph::Parked& old = g->parked.front();
            if (old.exec) cudaGraphExecDestroy(old.exec);
            for (void* p : old.table.owned) g->dev->release(p);
            g->parked.erase(g->parked.begin());
        }
        anl_graph::Parked pk;
        pk.table = std::move(g->table); pk.exec = g->exec; pk.sym = g->built_sym; pk.placed_key = g->placed_key;
        pk.kernels = g->kernels_per_replay; pk.gemms = g->gemms_per_replay; pk.rin = g->resident_in; pk.rout = g->resident_out;
        g->parked.push_back(std::move(pk));
        g->table = Table(); g->exec = nullptr; g->built = false;
    }
    for (size_t k = 0; k < g->parked.size(); k++) {
        anl_graph::Parked& pk = g->parked[k];
        if (pk.sym != sym || pk.placed_key != pkey || pk.rin != rin || pk.rout != rout) continue;
        g->table = std::move(pk.table); g->exec = pk.exec; g->built_sym = pk.sym; g->placed_key = pk.placed_key;
        g->kernels_per_replay = pk.kernels; g->gemms_per_replay = pk.gemms; g->resident_in = pk.rin; g->resident_out = pk.rout;
        g->built = true;
        g->parked.erase(g->parked.begin() + k);
        return;
    }
}

static int graph_replay_impl(anl_graph* g, const anl_input* inputs, int n_inputs, const anl_binding* binds, int n_binds,
                     const anl_output* placed, int n_placed, anl_output* outs, int* n_outs) {
    if (!g || !n_outs) return ANL_ERR_INVALID;
    anl_device* dev = g->dev;
    cudaSetDevice(dev->ordinal);
    if (g->items.empty()) { *n_outs = 0; return ANL_OK; }
    Bindings b = make_bindings(binds, n_binds);
    int64_t sym = b.any();
    // resident placements are baked into the captured pointers: any change rebuilds
    std::vector<std::pair<uint32_t, anl_buffer*>> rin, rout;
    for (int k = 0; k < n_inputs; k++) if (inputs[k].resident) rin.push_back({inputs[k].uop_idx, inputs[k].resident});
    for (int k = 0; k < n_placed; k++) if (placed[k].resident) rout.push_back({placed[k].uop_idx + (placed[k].allreduce ? 0x80000000u : 0u) + (placed[k].sgd_master ? 0x40000000u : 0u), placed[k].resident});
    // the learning rate, the gradient scale, the update's targets and the reduce mode are kernel
    // arguments inside the capture as well: a caller that changes one gets a new capture, not stale values
    uint64_t pkey = 1469598103934665603ull;
    for (int k = 0; k < n_placed; k++) {
        const anl_output& p = placed[k];
        struct { uint32_t id; int mode; const void* m; const void* q; float lr, scale; } rec;
        std::memset(&rec, 0, sizeof rec);
        rec.id = p.uop_idx; rec.mode = p.allreduce; rec.m = p.sgd_master; rec.q = p.sgd_param; rec.lr = p.sgd_lr; rec.scale = p.sgd_scale;
        pkey = fnv1a(&rec, sizeof rec, pkey);
    }
    if (g->built && (sym != g->built_sym || rin != g->resident_in || rout != g->resident_out || pkey != g->placed_key)) graph_switch(g, sym, rin, rout, pkey);
    int rc = ANL_OK;
    bool host_fed = !g->built;      // a replay whose leaves and outputs are all resident need not wait for the GPU
    if (!g->built) {
        // first call for this binding: allocate persistent buffers (uploading the inputs as a side
        // effect), compile every kernel eagerly, then capture the launches
        rc = build_table(dev, g->items, b, inputs, n_inputs, placed, n_placed, g->table);
        CodegenOpts opts; opts.debug_bounds = (dev->flags & ANL_OPEN_DEBUG_BOUNDS) != 0;
        for (size_t i = 0; i < g->items.size() && rc == ANL_OK; i++) { std::shared_ptr<Plan> p; rc = get_plan(dev, g->items[i], opts, p); }
        if (rc == ANL_OK) {
            cudaGraph_t graph = nullptr;
            cudaError_t e = cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeRelaxed);
            if (e != cudaSuccess) rc = dev->fail(ANL_ERR_CUDA, std::string("graph: begin capture: ") + cudaGetErrorString(e));
            if (rc == ANL_OK) {
                uint64_t k0 = dev->stats.kernels_launched, g0 = dev->stats.gemm_launched;
                int rrc = run_items(dev, g->items, b, g->table, dev->stream, true);   // scratch stays with the graph
                g->kernels_per_replay = dev->stats.kernels_launched - k0;
                g->gemms_per_replay = dev->stats.gemm_launched - g0;
                dev->stats.kernels_launched = k0; dev->stats.gemm_launched = g0;        // counted per replay below
                e = cudaStreamEndCapture(dev->stream, &graph);
                if (rrc != ANL_OK) rc = rrc;
                else if (e != cudaSuccess) rc = dev->fail(ANL_ERR_CUDA, std::string("graph: end capture: ") + cudaGetErrorString(e));
            }
            if (rc == ANL_OK) {
                e = cudaGraphInstantiate(&g->exec, graph, 0);
                if (e != cudaSuccess) rc = dev->fail(ANL_ERR_CUDA, std::string("graph: instantiate: ") + cudaGetErrorString(e));
            }
            if (graph) cudaGraphDestroy(graph);
        }
        if (rc != ANL_OK) { graph_drop(g); *n_outs = 0; return rc; }
        g->built = true; g->built_sym = sym; g->resident_in = rin; g->resident_out = rout; g->placed_key = pkey;
        dev->stats.graph_captures++;
    } else {
        // replay: refresh host-fed leaves in place
        for (int k = 0; k < n_inputs && rc == ANL_OK; k++) {
            if (inputs[k].resident || !inputs[k].data) continue;
            host_fed = true;
            auto f = g->table.bufs.find(inputs[k].uop_idx);
            if (f == g->table.bufs.end() || g->table.written.count(inputs[k].uop_idx)) continue;
            if (inputs[k].elems < f->second.elems) { rc = dev->fail(ANL_ERR_INVALID, "graph: input smaller than captured buffer"); break; }
            rc = upload_f32(dev, f->second.ptr, f->second.dtype, inputs[k].data, f->second.elems, dev->stream);
        }
        if (rc != ANL_OK) { *n_outs = 0; return rc; }
    }
    // a contraction of an earlier replay that gave up on a barrier left its code in the host-visible
    // status word: report it here instead of replaying on top of a tile counter it left dirty
    if (int src = gemm_check_status(dev)) { *n_outs = 0; return src; }
    cudaError_t e = cudaGraphLaunch(g->exec, dev->stream);
    if (e != cudaSuccess) { *n_outs = 0; return dev->fail(ANL_ERR_CUDA, std::string("graph: launch: ") + cudaGetErrorString(e)); }
    dev->stats.graph_replays++;
    dev->stats.kernels_launched += g->kernels_per_replay;
    dev->stats.gemm_launched += g->gemms_per_replay;
    return collect_outputs(dev, g->table, placed, n_placed, outs, n_outs, dev->stream, !host_fed);
}

void anl_graph_release(anl_graph* g) {
    if (!g) return;
    cudaStreamSynchronize(g->dev->stream);
    for (auto& pk : g->parked) {
        if (pk.exec) cudaGraphExecDestroy(pk.exec);
        for (void* p : pk.table.owned) g->dev->release(p);
    }
    g->parked.clear();
    graph_drop(g);
    delete g;
}

int anl_run(anl_device* dev, const uint8_t* blob, size_t blob_len, const anl_input* inputs, int n_inputs,
            const anl_binding* binds, int n_binds, const anl_output* placed, int n_placed, anl_output* outs, int* n_outs) {
    return fenced(dev, "run", [&] { return run_impl(dev, blob, blob_len, inputs, n_inputs, binds, n_binds, placed, n_placed, outs, n_outs); });
}
int anl_lower(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, const int* o,
              char* src, size_t src_cap, size_t* src_len, int* klass, int* block, int64_t* opb, char* note, size_t note_cap) {
    return fenced(dev, "lower", [&] { return lower_impl(dev, blob, blob_len, index, o, src, src_cap, src_len, klass, block, opb, note, note_cap); });
}
int anl_lower_chain(const uint8_t* blob, size_t blob_len, int first, int count, char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap) {
    return fenced(nullptr, "lower_chain", [&] { return lower_chain_impl(blob, blob_len, first, count, src, src_cap, src_len, note, note_cap); });
}
int anl_lower_gemm(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, int fuse_next, const int* o,
                   char* src, size_t src_cap, size_t* src_len, char* note, size_t note_cap) {
    return fenced(dev, "lower_gemm", [&] { return lower_gemm_impl(dev, blob, blob_len, index, fuse_next, o, src, src_cap, src_len, note, note_cap); });
}
int anl_benchmark(anl_device* dev, const uint8_t* blob, size_t blob_len, int index, const int* o, int warmup, int iterations, anl_bench_result* out) {
    return fenced(dev, "benchmark", [&] { return benchmark_impl(dev, blob, blob_len, index, o, warmup, iterations, out); });
}
int anl_graph_create(anl_device* dev, const uint8_t* blob, size_t blob_len, anl_graph** out) {
    return fenced(dev, "graph_create", [&] { return graph_create_impl(dev, blob, blob_len, out); });
}
int anl_graph_replay(anl_graph* g, const anl_input* inputs, int n_inputs, const anl_binding* binds, int n_binds,
                     const anl_output* placed, int n_placed, anl_output* outs, int* n_outs) {
    return fenced(nullptr, "graph_replay", [&] { return graph_replay_impl(g, inputs, n_inputs, binds, n_binds, placed, n_placed, outs, n_outs); });
}

}  // extern "C"
