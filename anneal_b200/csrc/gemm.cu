// Dense contractions on the 5th-generation tensor cores: D[M,N] = sum_k A[m,k] * B[n,k], f16
// operands, f32 accumulation in tensor memory, one rounding to f16 at the store — the arithmetic
// the reference specifies for an f16 REDUCE (f32 accumulator, operands widened, narrowed once:
// codegen/lower.go:654-719), reached through tcgen05.mma instead of its one-thread-per-output loop.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B k-blocks into a 4-stage
//               shared-memory ring (128-byte swizzle), completion on an mbarrier per stage;
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=256, K=16) four times per stage
//               and commits to the stage's "empty" barrier; owns the TMEM allocation;
//   warps 2-5   epilogue: tcgen05.ld the 128x256 f32 accumulator, convert, store.  Two accumulators
//               (2 x 256 TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
// Either operand may be K-major (k contiguous) or MN-major (m / n contiguous): the forward pass
// x·Wᵀ is K/K, the input gradient dY·W is K/MN, the weight gradient dYᵀ·X is MN/MN.  No operand
// is transposed in memory; the layout goes into the shared-memory and instruction descriptors.
// No multicast is used anywhere: every CTA issues its own loads.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in a host-visible
// status word and the CTA drains and frees its tensor memory instead of spinning.
//
// This file holds the one-CTA kernel (outputs with fewer than 256 rows) and the host side of both
// kernels.  The two-CTA kernel that the large contractions run on is gemm_pair_kernel.cuh: it is
// compiled at run time, once per configuration (operand major-ness, tile width, ring depth, raster,
// fused elementwise consumer), so that the consumer's generated code can sit in its epilogue and the
// tunables are compile-time constants a search can vary.  The same text serves f32 contractions in
// 3 x TF32 form; its host side (operand split pre-pass, K slices, their sum) is further down.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "gemm_pair_kernel.cuh"      // PairGemmArgs only: the device code is compiled at run time
#include "runtime.hpp"

namespace anl {

// text of gemm_pair_kernel.cuh, written beside the objects by the build step
static const char* const kPairKernelSource =
#include "gemm_pair_src.inc"
    ;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_TILE_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + alignment slack
constexpr int GEMM_THREADS = 192;
constexpr int PAIR_THREADS = 320;        // two-CTA kernel: producer, MMA issuer and eight epilogue warps
constexpr int TQ = 4;                               // depth of the per-CTA tile queue
constexpr unsigned WAIT_LIMIT = 1u << 20;

struct GemmPlan {
    Contraction c;
    bool a_mn = false, b_mn = false;     // MN-major operands
    int64_t lda = 0, ldb = 0;            // elements between consecutive rows of the 2-D global views
    bool f32 = false;                    // f32 operands: the FP32-pipe kernel instead of tcgen05
    GemmTuning tune;                     // zero fields: heuristics
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: false when the phase did not complete within WAIT_LIMIT polls, or when another
// role of this CTA has already given up (`failed`, in shared memory).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int* failed = nullptr) {
    for (unsigned i = 0; i < WAIT_LIMIT; i++) {
        if (failed && (i & 255u) == 255u && *failed) return false;
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
//   [46,48) descriptor version 1, [61,64) layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

// The tile counter must read zero when a launch starts.  Instead of a memset in front of every
// launch, the launch cleans up after itself: a CTA (or CTA pair) that has drawn its last number,
// one that is past the end, signs off on the second word, and the last to sign off zeroes both.
// Nobody draws after its own sign-off, so the reset cannot race with a draw.
__device__ __forceinline__ void retire_tile_counter(int* counter, int drawers) {
    __threadfence();
    if (atomicAdd(counter + 1, 1) == drawers - 1) {
        counter[0] = 0;
        counter[1] = 0;
        __threadfence();
    }
}

struct GemmArgs {
    __half* d;
    int M, N, K, ldd;
    int tiles_m, tiles_n;
    int* status;
    int* tile_counter;      // [0] next tile number, [1] drawers that have signed off; both zero between launches
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    // tile queue: the producer draws tile numbers from a global counter and hands them to the MMA
    // and epilogue roles, so a CTA that starts late (SMs busy with a collective) simply takes fewer
    __shared__ __align__(8) uint64_t tq_full[TQ], tq_empty[TQ];
    __shared__ int tile_ring[TQ];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int failed;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1 KiB alignment
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = g.tiles_m * g.tiles_n;
    const int kblocks = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 4); }
        for (int q = 0; q < TQ; q++) { mbar_init(smem_u32(&tq_full[q]), 1); mbar_init(smem_u32(&tq_empty[q]), 5); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // 512 columns: two 128x256 f32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ── producer ──
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int issued = 0;
            uint32_t qs = 0, qphase = 0;
            int next = atomicAdd(g.tile_counter, 1);
            while (ok) {
                if (!mbar_wait(smem_u32(&tq_empty[qs]), qphase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 5; break; }
                int t = next;
                if (t >= num_tiles) t = -1;
                tile_ring[qs] = t;
                mbar_arrive(smem_u32(&tq_full[qs]));
                if (++qs == TQ) { qs = 0; qphase ^= 1; }
                if (t < 0) { retire_tile_counter(g.tile_counter, (int)gridDim.x); break; }
                const int m0 = (t % g.tiles_m) * BM, n0 = (t / g.tiles_m) * BN;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 1; break; }
                    const uint32_t fb = smem_u32(&full_bar[stage]);
                    const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_TILE_BYTES;
                    mbar_expect_tx(fb, STAGE_BYTES);
                    const int k0 = kb * BK;
                    if (A_MN) { for (int j = 0; j < BM / 64; j++) tma_load_2d(sa + j * (BK * 128), &map_a, m0 + 64 * j, k0, fb); }
                    else tma_load_2d(sa, &map_a, k0, m0, fb);
                    if (B_MN) { for (int j = 0; j < BN / 64; j++) tma_load_2d(sb + j * (BK * 128), &map_b, n0 + 64 * j, k0, fb); }
                    else tma_load_2d(sb, &map_b, k0, n0, fb);
                    issued++;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                // drawn once this tile's loads are issued: no CTA holds a number it is not about to start, and
                // the ring of stages already loaded covers the atomic's latency
                if (ok) next = atomicAdd(g.tile_counter, 1);
            }
            if (!ok) {
                failed = 1;
                // let copies already in flight land before the CTA goes away
                int pending = issued < STAGES ? issued : STAGES;
                for (int i = 0; i < pending; i++) { stage = stage == 0 ? STAGES - 1 : stage - 1; mbar_wait(smem_u32(&full_bar[stage]), 0); mbar_wait(smem_u32(&full_bar[stage]), 1); }
            }
        }
    } else if (warp == 1) {
        // ── MMA issuer ──
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, f16 x f16, majors, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 4) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            uint32_t qs = 0, qphase = 0;
            while (ok) {
                if (!mbar_wait(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; *(volatile int*)g.status = 6; break; }
                const int t = tile_ring[qs];
                mbar_arrive(smem_u32(&tq_empty[qs]));
                if (++qs == TQ) { qs = 0; qphase ^= 1; }
                if (t < 0) break;
                if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 2; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &failed)) { ok = false; *(volatile int*)g.status = 3; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        // K-major: 16 k-elements = 32 bytes inside the 128-byte row, 8-row groups 1 KiB apart.
                        // MN-major: 16 k-rows = two 1 KiB atoms, 64-wide m/n groups one box (BK*128 B) apart.
                        const uint64_t ad = A_MN ? make_desc(sa + k * 2048, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_desc(sb + k * 2048, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
                        umma_f16(tmem_d, ad, bd, idesc, (kb | k) != 0);
                    }
                    umma_commit(smem_u32(&empty_bar[stage]));      // frees the stage when these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&acc_full[acc]));             // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
            if (!ok) failed = 1;
        }
    } else {
        // ── epilogue: warps 2..5, TMEM lane quadrant = warp % 4 ──
        const int quad = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        uint32_t qs = 0, qphase = 0;
        while (ok) {
            if (!mbar_wait(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 7; failed = 1; } break; }
            const int t = tile_ring[qs];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tq_empty[qs]));
            if (++qs == TQ) { qs = 0; qphase ^= 1; }
            if (t < 0) break;
            const int m0 = (t % g.tiles_m) * BM, n0 = (t / g.tiles_m) * BN;
            if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 4; failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quad * 32 + lane;
            __half* drow = g.d + (size_t)row * g.ldd + n0;
            const bool row_ok = row < g.M;
            const bool vec_ok = (g.ldd % 8 == 0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col = n0 + c * 32;
                if (!row_ok || col >= g.N) continue;
                if (vec_ok && col + 32 <= g.N) {
                    uint4* dst = reinterpret_cast<uint4*>(drow + c * 32);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        __half2 h0 = __floats2half2_rn(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                        __half2 h1 = __floats2half2_rn(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                        __half2 h2 = __floats2half2_rn(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                        __half2 h3 = __floats2half2_rn(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                        uint4 o;
                        o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                        o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                        dst[q] = o;
                    }
                } else {
                    // ragged right edge: constant indices keep v[] in registers
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (col + j < g.N) drow[c * 32 + j] = __float2half_rn(__uint_as_float(v[j]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}


static int encode_map(anl_device* dev, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer, bool f32 = false) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_elems * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = dev->drv.TensorMapEncodeTiled(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { const char* s = nullptr; dev->drv.GetErrorString(r, &s); return dev->fail(ANL_ERR_CUDA, std::string("gemm: cuTensorMapEncodeTiled: ") + (s ? s : "?")); }
    return ANL_OK;
}

// Host-visible status word and tile counters of this device.  A launch draws tile numbers from the
// counter that belongs to its stream, so contractions queued on different streams cannot disturb
// each other's draw; launches on one stream run one after the other and share one.
static int ensure_gemm_state(anl_device* dev) {
    if (!dev->gemm_status_host) {
        if (cudaHostAlloc((void**)&dev->gemm_status_host, 64, cudaHostAllocMapped) != cudaSuccess) return dev->fail(ANL_ERR_CUDA, "gemm: cannot allocate the status word");
        *dev->gemm_status_host = 0;
        if (cudaHostGetDevicePointer((void**)&dev->gemm_status_dev, dev->gemm_status_host, 0) != cudaSuccess) return dev->fail(ANL_ERR_CUDA, "gemm: cannot map the status word");
    }
    if (!dev->gemm_tile_counter) {
        const size_t bytes = (size_t)anl_device::kGemmCounterSlots * 256;
        if (cudaMalloc((void**)&dev->gemm_tile_counter, bytes) != cudaSuccess) return dev->fail(ANL_ERR_CUDA, "gemm: cannot allocate the tile counters");
        if (cudaMemset(dev->gemm_tile_counter, 0, bytes) != cudaSuccess) return dev->fail(ANL_ERR_CUDA, "gemm: cannot clear the tile counters");   // launches leave them zeroed again
    }
    if (!dev->gemm_attr_set) {
        cudaFuncSetAttribute(gemm_f16_tcgen05<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        dev->gemm_attr_set = true;
    }
    return ANL_OK;
}

static int* tile_counter_for(anl_device* dev, cudaStream_t stream) {
    int slot = -1;
    for (size_t k = 0; k < dev->gemm_counter_streams.size(); k++) if (dev->gemm_counter_streams[k] == stream) slot = (int)k;
    if (slot < 0) {
        if ((int)dev->gemm_counter_streams.size() < anl_device::kGemmCounterSlots) { dev->gemm_counter_streams.push_back(stream); slot = (int)dev->gemm_counter_streams.size() - 1; }
        else slot = 0;      // more streams than slots: those share the first one (never the case for this runtime's three)
    }
    return dev->gemm_tile_counter + slot * 64;
}

// A barrier wait that ran out leaves its code in the status word and the tile counters undefined (a
// CTA that gives up does not sign off).  Called where the host has just waited for the device: report
// once, clear the word and zero the counters so that later launches, replays included, start clean.
int gemm_check_status(anl_device* dev) {
    if (!dev->gemm_status_host || *dev->gemm_status_host == 0) return ANL_OK;
    const int code = *dev->gemm_status_host;
    cudaDeviceSynchronize();
    if (dev->gemm_tile_counter) cudaMemset(dev->gemm_tile_counter, 0, (size_t)anl_device::kGemmCounterSlots * 256);
    *dev->gemm_status_host = 0;
    return dev->fail(ANL_ERR_CUDA, "gemm: a launch timed out on a barrier (code " + std::to_string(code) + "); its output is incomplete");
}

// Test hook: puts the device in the state a timed-out barrier wait leaves behind (a code in the
// status word, a tile counter that was not signed off), without making any wait run out.
int gemm_inject_status(anl_device* dev, int code, int counter_value) {
    if (int rc = ensure_gemm_state(dev)) return rc;
    cudaStreamSynchronize(dev->stream);
    int words[2] = {counter_value, 0};
    for (int k = 0; k < anl_device::kGemmCounterSlots; k++)
        if (cudaMemcpy(dev->gemm_tile_counter + k * 64, words, sizeof words, cudaMemcpyHostToDevice) != cudaSuccess) return dev->fail(ANL_ERR_CUDA, "gemm: cannot write the tile counter");
    *dev->gemm_status_host = code;
    return ANL_OK;
}

int plan_gemm(const Item& item, const GemmTuning& tune, Plan& plan) {
    Contraction c;
    if (!match_contraction(item, c)) return ANL_ERR_UNSUPPORTED;
    const bool dynamic = c.m_sym || c.k_sym;
    if (c.in_dtype == DT_F32 && c.out_dtype == DT_F32) {
        if (c.a_sk != 1 && c.a_sm != 1) return ANL_ERR_UNSUPPORTED;
        if (c.b_sk != 1 && c.b_sn != 1) return ANL_ERR_UNSUPPORTED;
        if (!dynamic && !gemm_f32_worth(c.M, c.N, c.K, c.a_sm, c.a_sk, c.b_sn, c.b_sk)) return ANL_ERR_UNSUPPORTED;
        if (c.N < 64) return ANL_ERR_UNSUPPORTED;
        auto gp = std::make_shared<GemmPlan>();
        gp->c = c; gp->f32 = true;
        plan.gemm = gp;
        plan.gemm_dynamic = dynamic;
        if (!dynamic) {
            plan.r.klass = KC_GEMM;
            plan.r.note = "gemm f32 M=" + std::to_string(c.M) + " N=" + std::to_string(c.N) + " K=" + std::to_string(c.K);
        }
        return ANL_OK;
    }
    if (c.in_dtype != DT_F16 || c.out_dtype != DT_F16) return ANL_ERR_UNSUPPORTED;
    if (dynamic) return ANL_ERR_UNSUPPORTED;                                   // tcgen05 path: static extents only
    if (c.M < 64 || c.N < 64 || c.K < 32) return ANL_ERR_UNSUPPORTED;          // not worth a 128x256 tile
    auto gp = std::make_shared<GemmPlan>();
    gp->c = c;
    gp->tune = tune;
    // A: either k contiguous (K-major, row stride a_sm) or m contiguous (MN-major, row stride a_sk)
    if (c.a_sk == 1 && c.a_sm >= c.K) { gp->a_mn = false; gp->lda = c.a_sm; }
    else if (c.a_sm == 1 && c.a_sk >= c.M) { gp->a_mn = true; gp->lda = c.a_sk; }
    else return ANL_ERR_UNSUPPORTED;
    if (c.b_sk == 1 && c.b_sn >= c.K) { gp->b_mn = false; gp->ldb = c.b_sn; }
    else if (c.b_sn == 1 && c.b_sk >= c.N) { gp->b_mn = true; gp->ldb = c.b_sk; }
    else return ANL_ERR_UNSUPPORTED;
    // TMA: 16-byte aligned bases and row strides
    if (gp->lda % 8 || gp->ldb % 8 || c.a_off % 8 || c.b_off % 8) return ANL_ERR_UNSUPPORTED;
    if (c.M >= (1ll << 31) || c.N >= (1ll << 31) || c.K >= (1ll << 31)) return ANL_ERR_UNSUPPORTED;
    plan.gemm = gp;
    plan.r.klass = KC_GEMM;
    plan.r.note = std::string("gemm tcgen05 ") + (gp->a_mn ? "A:MN" : "A:K") + (gp->b_mn ? " B:MN" : " B:K") + " M=" + std::to_string(c.M) + " N=" + std::to_string(c.N) + " K=" + std::to_string(c.K);
    return ANL_OK;
}

// SMs the persistent GEMM may occupy.  When gradients are reduced while the backward pass is still
// running, a few SMs can be left free so that the collective's blocks (and the update kernels behind
// them) find a place at once instead of waiting for a persistent grid to drain.
static int gemm_sm_budget(anl_device* dev) {
    if (!dev) return 148;                                  // rendering without a device: a B200's count
    int sms = dev->prop.multiProcessorCount;
    int want = dev->nranks > 1 ? sms - dev->comm_reserved_sms : sms;
    want = std::max(2, std::min(want, sms));
    return want & ~1;
}

double gemm_flops(const Plan& plan, int64_t sym_value) {
    const Contraction& c = plan.gemm->c;
    return 2.0 * (double)(c.m_sym ? sym_value : c.M) * (double)c.N * (double)(c.k_sym ? sym_value : c.K);
}

int64_t gemm_window_rows(const Plan& plan, int64_t* row_elems) {
    if (!plan.gemm || plan.gemm_dynamic || plan.r.klass != KC_GEMM || plan.gemm->f32) return 0;
    if (row_elems) *row_elems = plan.gemm->c.N;
    return plan.gemm->c.M;
}

bool gemm_taken(const Plan& plan, int64_t sym_value) {
    if (!plan.gemm) return false;
    if (!plan.gemm_dynamic) return plan.r.klass == KC_GEMM;
    const Contraction& c = plan.gemm->c;
    return gemm_f32_worth(c.m_sym ? sym_value : c.M, c.N, c.k_sym ? sym_value : c.K, c.a_sm, c.a_sk, c.b_sn, c.b_sk);
}

bool gemm_pair_eligible(const Plan& plan) {
    if (!plan.gemm || plan.gemm_dynamic || plan.r.klass != KC_GEMM || plan.gemm->f32) return false;
    const Contraction& c = plan.gemm->c;
    return plan.gemm->tune.single_cta == 0 && c.M >= 2 * BM && c.N >= BN / 2;
}
void gemm_shape(const Plan& plan, int64_t* M, int64_t* N, int64_t* K) { *M = plan.gemm->c.M; *N = plan.gemm->c.N; *K = plan.gemm->c.K; }

// ── the run-time compiled two-CTA kernel ──────────────────────────────────────────────────────
namespace {

struct PairVariant { int bnt, stages, group_m, stream_stores; bool a_mn, b_mn; bool split_tail; bool tf32 = false; };
// k extent the 3 x TF32 form accumulates in tensor memory before adding to the output in f32.  Measured on
// 4096 x 2048 x 8192 (error against float64, of the largest output): 1024 -> 7.6e-6 at 226 TFLOP/s,
// 512 -> 3.5e-6 at 207, 256 -> 1.7e-6 at 146; the reference's serial f32 loop: 3.6e-6 (9.4e-6 at K = 65536).
constexpr int kTf32ChunkK = 1024;
constexpr int kDefaultStages = 7;      // the deepest ring that fits beside a 256-wide tile; 1% faster than 6 on every large shape measured

int pair_smem_bytes(int bnt, int stages, bool tf32 = false) { return stages * (tf32 ? 2 : 1) * (A_TILE_BYTES + (bnt / 2) * BK * 2) + 1024; }

// ring depth that fits beside the static barriers: 227 KiB per CTA
int max_stages(int bnt) { int s = 8; while (s > 2 && pair_smem_bytes(bnt, s) > 227 * 1024 - 512) s--; return s; }

std::string pair_source(const PairVariant& v, const std::string& epilogue) {
    std::string s;
    s += "#define ANL_PAIR_GEMM_DEVICE_CODE 1\n";
    s += "#define CFG_A_MN " + std::to_string(v.a_mn ? 1 : 0) + "\n#define CFG_B_MN " + std::to_string(v.b_mn ? 1 : 0) + "\n";
    s += "#define CFG_BNT " + std::to_string(v.bnt) + "\n#define CFG_STAGES " + std::to_string(v.stages) + "\n";
    s += "#define CFG_GROUP_M " + std::to_string(v.group_m) + "\n#define CFG_STREAM_STORES " + std::to_string(v.stream_stores) + "\n";
    s += "#define CFG_EPI " + std::string(epilogue.empty() ? "0" : "1") + "\n";
    s += "#define CFG_TF32 " + std::string(v.tf32 ? "1" : "0") + "\n";
    s += epilogue;
    s += kPairKernelSource;
    return s;
}

int get_pair_kernel(anl_device* dev, const PairVariant& v, const std::string& epilogue, CUfunction* fn) {
    // looked up by the configuration, so that a launch does not assemble and hash 40 KB of source
    char head[96];
    std::snprintf(head, sizeof head, "%d,%d,%d,%d,%d,%d,%d|", v.bnt, v.stages, v.group_m, v.stream_stores, (int)v.a_mn, (int)v.b_mn, (int)v.tf32);
    const std::string key = head + epilogue;
    auto hit = dev->pair_kernels.find(key);
    if (hit != dev->pair_kernels.end()) { *fn = (CUfunction)hit->second; return ANL_OK; }
    std::shared_ptr<Module> m;
    if (int rc = compile_source(dev, pair_source(v, epilogue), m)) return rc;
    auto f = m->fn.find("gemm_f16_tcgen05_pair");
    if (f != m->fn.end()) { *fn = f->second; dev->pair_kernels[key] = (void*)*fn; return ANL_OK; }
    CUresult cr = dev->drv.ModuleGetFunction(fn, m->mod, "gemm_f16_tcgen05_pair");
    if (cr != CUDA_SUCCESS) return dev->fail(ANL_ERR_CUDA, "gemm: pair kernel entry point missing");
    cr = dev->drv.FuncSetAttribute(*fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, pair_smem_bytes(v.bnt, v.stages, v.tf32));
    if (cr != CUDA_SUCCESS) { const char* e = nullptr; dev->drv.GetErrorString(cr, &e); return dev->fail(ANL_ERR_CUDA, std::string("gemm: cuFuncSetAttribute: ") + (e ? e : "?")); }
    m->fn["gemm_f16_tcgen05_pair"] = *fn;
    dev->pair_kernels[key] = (void*)*fn;
    return ANL_OK;
}

PairVariant choose_variant(anl_device* dev, const GemmPlan& gp_in, int64_t M) {
    // the plan's own tunables (a search result) first, then the device's defaults, then the heuristics
    GemmPlan gp = gp_in;
    if (dev) {
        const GemmTuning& d = dev->gemm_defaults;
        if (!gp.tune.tile_n) gp.tune.tile_n = d.tile_n;
        if (!gp.tune.stages) gp.tune.stages = d.stages;
        if (!gp.tune.group_m) gp.tune.group_m = d.group_m;
        if (!gp.tune.stream_stores) gp.tune.stream_stores = d.stream_stores;
        if (!gp.tune.no_split_tail) gp.tune.no_split_tail = d.no_split_tail;
    }
    const Contraction& c = gp.c;
    PairVariant v{};
    v.a_mn = gp.a_mn; v.b_mn = gp.b_mn;
    const int npairs = gemm_sm_budget(dev) / 2;
    const int tm2 = (int)((M + 2 * BM - 1) / (2 * BM));
    if (gp.tune.tile_n == 128 || gp.tune.tile_n == 256) v.bnt = gp.tune.tile_n;
    else {
        // The narrow tile fills the last wave of tiles better but stages 1.5x the bytes per flop and
        // measured 25% slower on 4096x4096x8192 (it becomes L2-bound), so it is only taken when the
        // wide tile would leave most pairs idle.
        auto fill = [&](int bnt) { long long t = (long long)tm2 * ((c.N + bnt - 1) / bnt); long long w = (t + npairs - 1) / npairs; return (double)t / (double)(w * npairs); };
        v.bnt = (fill(128) * 0.7 > fill(256)) ? 128 : 256;
    }
    v.stages = gp.tune.stages > 0 ? std::max(2, std::min(gp.tune.stages, max_stages(v.bnt))) : std::min(kDefaultStages, max_stages(v.bnt));
    v.group_m = gp.tune.group_m > 0 ? gp.tune.group_m : (gp.tune.group_m < 0 ? 0 : kDefaultGroupM);
    v.stream_stores = gp.tune.stream_stores > 0 ? 1 : 0;
    v.split_tail = gp.tune.no_split_tail == 0;
    return v;
}

}  // namespace

int gemm_pair_source(anl_device* dev, const Plan& plan, const std::string& epilogue, std::string& out) {
    if (!gemm_pair_eligible(plan)) return ANL_ERR_UNSUPPORTED;
    out = pair_source(choose_variant(dev, *plan.gemm, plan.gemm->c.M), epilogue);
    return ANL_OK;
}

int gemm_prepare(anl_device* dev, const Plan& plan, const std::string& epilogue) {
    if (!gemm_pair_eligible(plan)) return ANL_OK;
    CUfunction fn;
    return get_pair_kernel(dev, choose_variant(dev, *plan.gemm, plan.gemm->c.M), epilogue, &fn);
}

// ── f32 contractions on the tensor cores: 3 x TF32 ────────────────────────────────────────────
// hi = the operand rounded to TF32 (11 significant bits, round to nearest, ties away), lo = operand - hi
// (exact in f32), itself rounded to TF32.
__global__ void __launch_bounds__(256) split_tf32(const float* __restrict__ src, long long ld, long long rows, long long cols, long long ldo,
                                                  float* __restrict__ hi, float* __restrict__ lo) {
    const long long per_row = ldo >> 2;
    const long long total = rows * per_row;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const long long r = t / per_row, c = (t - r * per_row) << 2;
        float v[4], h[4], l[4];
        const float* p = src + r * ld + c;
        if (c + 3 < cols && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            const float4 q = *reinterpret_cast<const float4*>(p);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = (c + j < cols) ? p[j] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            unsigned u, w;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[j]));
            h[j] = __uint_as_float(u);
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v[j] - h[j]));     // the tensor core would cut it; rounding halves that error
            l[j] = __uint_as_float(w);
        }
        *reinterpret_cast<float4*>(hi + r * ldo + c) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(lo + r * ldo + c) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// The same split for an operand stored with its row index contiguous (element (r, k) at src[k * ld + r]):
// written out k-contiguous through a 32 x 32 shared-memory tile, so the tensor-core kernel sees one
// operand layout.  Block (32, 8); grid (ceil(k / 32), ceil(rows / 32)), rows folded into y then z.
__global__ void __launch_bounds__(256) split_tf32_transposed(const float* __restrict__ src, long long ld, long long rows, long long cols, long long ldo,
                                                             float* __restrict__ hi, float* __restrict__ lo) {
    __shared__ float tile[32][33];
    const long long k0 = (long long)blockIdx.x * 32;
    const long long r0 = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * 32;
    if (r0 >= rows) return;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const long long k = k0 + threadIdx.y + j, r = r0 + threadIdx.x;
        tile[threadIdx.y + j][threadIdx.x] = (k < cols && r < rows) ? src[k * ld + r] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const long long r = r0 + threadIdx.y + j, k = k0 + threadIdx.x;
        if (r < rows && k < ldo) {
            const float v = tile[threadIdx.x][threadIdx.y + j];
            unsigned u, w;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
            const float h = __uint_as_float(u);
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v - h));
            hi[r * ldo + k] = h;
            lo[r * ldo + k] = __uint_as_float(w);
        }
    }
}

// out[i] = copies[0][i] + copies[1][i] + ... in that order: finishes a contraction whose K was split
// between draws of the same tile.
__global__ void __launch_bounds__(256) sum_split_copies(const float* __restrict__ copies, long long stride, int n_copies, long long n, float* __restrict__ out) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    if (i + 3 < n && (stride & 3) == 0) {
        float4 v = *reinterpret_cast<const float4*>(copies + i);
        for (int c = 1; c < n_copies; c++) {
            const float4 w = *reinterpret_cast<const float4*>(copies + c * stride + i);
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        *reinterpret_cast<float4*>(out + i) = v;
    } else {
        for (long long j = i; j < n && j < i + 4; j++) {
            float v = copies[j];
            for (int c = 1; c < n_copies; c++) v += copies[c * stride + j];
            out[j] = v;
        }
    }
}

// f32 contractions of more than a few rows take the two-CTA tensor-core kernel in 3 x TF32 form unless
// the device was opened with ANL_OPEN_NO_TF32X3: operands contiguous along k or along their row index.
static bool tf32x3_shape_ok(const Contraction& c, int64_t M, int64_t K) { return gemm_tf32_shape_ok(M, c.N, K, c.a_sm, c.a_sk, c.b_sn, c.b_sk); }
static bool tf32x3_applies(anl_device* dev, const Contraction& c, int64_t M, int64_t K) {
    return !(dev->flags & ANL_OPEN_NO_TF32X3) && tf32x3_shape_ok(c, M, K);
}
static PairVariant tf32_variant() {
    PairVariant v{};
    v.a_mn = v.b_mn = false;        // the split pre-pass hands both operands over k-contiguous
    v.bnt = 256; v.tf32 = true; v.split_tail = false;
    v.stages = 3;                   // 64 KB each: hi and lo parts of both operands
    v.group_m = kDefaultGroupM;
    return v;
}
bool gemm_tf32_eligible(const Plan& plan) {
    if (!plan.gemm || plan.gemm_dynamic || plan.r.klass != KC_GEMM || !plan.gemm->f32) return false;
    return tf32x3_shape_ok(plan.gemm->c, plan.gemm->c.M, plan.gemm->c.K);
}
int gemm_tf32_source(const Plan& plan, std::string& out, std::string& note) {
    if (!gemm_tf32_eligible(plan)) return ANL_ERR_UNSUPPORTED;
    const PairVariant v = tf32_variant();
    out = pair_source(v, std::string());
    const Contraction& c = plan.gemm->c;
    note = std::string("gemm tcgen05 3xTF32 A:") + (c.a_sk == 1 ? "K" : "MN") + " B:" + (c.b_sk == 1 ? "K" : "MN") + " (both rewritten k-contiguous by the split pre-pass) M=" + std::to_string(c.M) + " N=" + std::to_string(c.N) + " K=" + std::to_string(c.K);
    return ANL_OK;
}

static int launch_gemm_tf32x3(anl_device* dev, const GemmPlan& gp, const float* a, const float* b, float* d, int64_t M, int64_t K,
                              cudaStream_t stream, std::vector<void*>* keep_scratch) {
    const Contraction& c = gp.c;
    const int64_t N = c.N;
    if (int rc = ensure_gemm_state(dev)) return rc;
    if (*dev->gemm_status_host != 0) return dev->fail(ANL_ERR_CUDA, "gemm: an earlier launch timed out on a barrier (code " + std::to_string(*dev->gemm_status_host) + ")");
    // both operands are rewritten as [rows, K] with k contiguous (rows = m or n), K padded to 4 floats
    const bool a_mn = !(c.a_sk == 1), b_mn = !(c.b_sk == 1);
    const int64_t ldo = (K + 3) & ~3ll;
    void* scratch[4] = {nullptr, nullptr, nullptr, nullptr};
    const size_t a_bytes = (size_t)M * ldo * 4, b_bytes = (size_t)N * ldo * 4;
    int rc = ANL_OK;
    for (int k = 0; k < 4 && rc == ANL_OK; k++) rc = dev->alloc(k < 2 ? a_bytes : b_bytes, &scratch[k]);
    auto done = [&](int code) {
        for (void* p : scratch) if (p) { if (keep_scratch) keep_scratch->push_back(p); else dev->release(p); }
        return code;
    };
    if (rc) return done(rc);
    float *a_hi = (float*)scratch[0], *a_lo = (float*)scratch[1], *b_hi = (float*)scratch[2], *b_lo = (float*)scratch[3];
    const int sms = dev->prop.multiProcessorCount;
    auto split = [&](const float* src, bool mn, int64_t rows, int64_t ld, float* hi, float* lo) {
        if (!mn) {
            const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((rows * (ldo / 4) + 255) / 256, (int64_t)sms * 16));
            split_tf32<<<grid, 256, 0, stream>>>(src, ld, rows, K, ldo, hi, lo);
        } else {
            const int64_t rt = (rows + 31) / 32;
            const unsigned gy = (unsigned)std::min<int64_t>(rt, 32768), gz = (unsigned)((rt + gy - 1) / gy);
            split_tf32_transposed<<<dim3((unsigned)((ldo + 31) / 32), gy, gz), dim3(32, 8), 0, stream>>>(src, ld, rows, K, ldo, hi, lo);
        }
    };
    split(a, a_mn, M, a_mn ? c.a_sk : c.a_sm, a_hi, a_lo);
    split(b, b_mn, N, b_mn ? c.b_sk : c.b_sn, b_hi, b_lo);
    if (cudaGetLastError() != cudaSuccess) return done(dev->fail(ANL_ERR_CUDA, "gemm: operand split launch failed"));
    dev->stats.kernels_launched += 2;

    const PairVariant v = tf32_variant();
    CUfunction fn;
    if ((rc = get_pair_kernel(dev, v, std::string(), &fn))) return done(rc);
    constexpr int BK32 = 32;
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    auto enc_a = [&](CUtensorMap* m, const float* base) { return encode_map(dev, m, base, (uint64_t)K, (uint64_t)M, (uint64_t)ldo, BK32, BM, true); };
    auto enc_b = [&](CUtensorMap* m, const float* base) { return encode_map(dev, m, base, (uint64_t)K, (uint64_t)N, (uint64_t)ldo, BK32, v.bnt / 2, true); };
    if ((rc = enc_a(&ma_hi, a_hi)) || (rc = enc_a(&ma_lo, a_lo)) || (rc = enc_b(&mb_hi, b_hi)) || (rc = enc_b(&mb_lo, b_lo))) return done(rc);
    PairGemmArgsF32 g{};
    g.d_raw = d;
    g.M = (int)M; g.N = (int)N; g.ldd = (int)N;
    g.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM)); g.tiles_n = (int)((N + v.bnt - 1) / v.bnt);
    g.full_tiles = g.tiles_m * g.tiles_n;
    g.status = dev->gemm_status_dev;
    g.tile_counter = tile_counter_for(dev, stream);
    const int npairs = gemm_sm_budget(dev) / 2;
    const int pairs = std::min(g.full_tiles, npairs);
    CUlaunchConfig cfg{};
    cfg.gridDimX = 2 * pairs; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = PAIR_THREADS; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = pair_smem_bytes(v.bnt, v.stages, v.tf32);
    cfg.hStream = (CUstream)stream;
    CUlaunchAttribute at[1];
    at[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    at[0].value.clusterDim.x = 2; at[0].value.clusterDim.y = 1; at[0].value.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    g.K = (int)K;
    g.chunk_kb = kTf32ChunkK / BK32;
    // few tiles and a long K: draw every tile several times, each draw a slice of K into its own copy
    // of the output (at least 8 k-blocks a slice), and add the copies afterwards in order
    const int kblocks = (int)((K + BK32 - 1) / BK32);
    int splits = std::min(npairs / std::max(1, g.full_tiles), kblocks / 8);
    void* copies = nullptr;
    if (splits > 1) {
        g.kb_per_split = (kblocks + splits - 1) / splits;
        splits = (kblocks + g.kb_per_split - 1) / g.kb_per_split;
    }
    if (splits > 1) {
        g.k_splits = splits;
        g.split_stride = (long long)(((M * N) + 3) & ~3ll);
        if ((rc = dev->alloc((size_t)splits * (size_t)g.split_stride * 4, &copies))) return done(rc);
        g.d_raw = copies;
        cfg.gridDimX = 2 * std::min(g.full_tiles * splits, npairs);
    }
    auto done2 = [&](int code) {
        if (copies) { if (keep_scratch) keep_scratch->push_back(copies); else dev->release(copies); }
        return done(code);
    };
    g.draw_late = g.full_tiles * std::max(1, g.k_splits) <= 2 * npairs;
    void* params[5] = {&ma_hi, &mb_hi, &ma_lo, &mb_lo, &g};
    CUresult cr = dev->drv.LaunchKernelEx(&cfg, fn, params, nullptr);
    if (cr != CUDA_SUCCESS) { const char* e = nullptr; dev->drv.GetErrorString(cr, &e); return done2(dev->fail(ANL_ERR_CUDA, std::string("gemm: tf32 pair launch: ") + (e ? e : "?"))); }
    dev->stats.kernels_launched++;
    if (splits > 1) {
        const long long n = (long long)M * N;
        sum_split_copies<<<(unsigned)((n + 1023) / 1024), 256, 0, stream>>>((const float*)copies, g.split_stride, splits, n, d);
        if (cudaGetLastError() != cudaSuccess) return done2(dev->fail(ANL_ERR_CUDA, "gemm: split sum launch failed"));
        dev->stats.kernels_launched++;
    }
    dev->stats.gemm_launched++;
    return done2(ANL_OK);
}

int launch_gemm(anl_device* dev, const Plan& plan, void* const* bufs, int64_t sym_value, cudaStream_t stream, int64_t m_begin, int64_t m_end,
                const GemmFusion* fusion, std::vector<void*>* keep_scratch) {
    const GemmPlan& gp = *plan.gemm;
    const Contraction& c = gp.c;
    // an optional row window [m_begin, m_end) of the output: the caller splits a contraction so that
    // a collective on the first rows can start while the remaining rows are still being computed
    const bool window = m_end >= 0;
    if (window && (gp.f32 || c.m_sym || m_begin < 0 || m_end > c.M || m_begin >= m_end || (m_begin % 8)))
        return dev->fail(ANL_ERR_INVALID, "gemm: bad row window");
    if (fusion && (window || gp.f32)) return dev->fail(ANL_ERR_INVALID, "gemm: a fused consumer needs the whole f16 contraction");
    const int64_t M = window ? m_end - m_begin : c.M;
    if (gp.f32) {
        const int64_t Mv = c.m_sym ? sym_value : c.M, Kv = c.k_sym ? sym_value : c.K;
        if (tf32x3_applies(dev, c, Mv, Kv))
            return launch_gemm_tf32x3(dev, gp, (const float*)bufs[c.a_param] + c.a_off, (const float*)bufs[c.b_param] + c.b_off, (float*)bufs[0], Mv, Kv, stream, keep_scratch);
        return launch_gemm_f32(dev, (const float*)bufs[c.a_param] + c.a_off, (const float*)bufs[c.b_param] + c.b_off, (float*)bufs[0],
                               Mv, c.N, Kv, c.a_sm, c.a_sk, c.b_sn, c.b_sk, stream);
    }
    if (int rc = ensure_gemm_state(dev)) return rc;
    if (*dev->gemm_status_host != 0) return dev->fail(ANL_ERR_CUDA, "gemm: an earlier launch timed out on a barrier (code " + std::to_string(*dev->gemm_status_host) + ")");
    const __half* a = (const __half*)bufs[c.a_param] + c.a_off + (window ? m_begin * c.a_sm : 0);
    const __half* b = (const __half*)bufs[c.b_param] + c.b_off;
    CUtensorMap ma, mb;
    int rc;
    if (gp.a_mn) rc = encode_map(dev, &ma, a, (uint64_t)M, (uint64_t)c.K, (uint64_t)gp.lda, 64, BK);
    else rc = encode_map(dev, &ma, a, (uint64_t)c.K, (uint64_t)M, (uint64_t)gp.lda, BK, BM);
    if (rc) return rc;
    int* const counter = tile_counter_for(dev, stream);
    if (gemm_pair_eligible(plan) && M >= 2 * BM) {
        const PairVariant v = choose_variant(dev, gp, M);
        // B is loaded in halves of bnt/2 columns, so its tensor map gets a box of that many rows; a
        // second map with half that box serves the half-width tiles of the last wave
        CUtensorMap mbh;
        if (gp.b_mn) rc = encode_map(dev, &mb, b, (uint64_t)c.N, (uint64_t)c.K, (uint64_t)gp.ldb, 64, BK);
        else rc = encode_map(dev, &mb, b, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)gp.ldb, BK, v.bnt / 2);
        if (rc) return rc;
        if (gp.b_mn) mbh = mb;
        else if ((rc = encode_map(dev, &mbh, b, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)gp.ldb, BK, v.bnt / 4))) return rc;
        CUfunction fn;
        if ((rc = get_pair_kernel(dev, v, fusion && fusion->epilogue ? *fusion->epilogue : std::string(), &fn))) return rc;
        PairGemmArgs g{};
        __half* out0 = (__half*)bufs[0] + (window ? m_begin * c.N : 0);
        g.d_raw = (!fusion || fusion->store_raw) ? out0 : nullptr;
        g.d_out = fusion ? fusion->d_out : nullptr;
        g.colsum = fusion ? fusion->colsum : nullptr;
        if (fusion) for (int k = 0; k < 6; k++) g.ep[k] = fusion->ep[k];
        g.M = (int)M; g.N = (int)c.N; g.K = (int)c.K; g.ldd = (int)c.N;
        g.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM)); g.tiles_n = (int)((c.N + v.bnt - 1) / v.bnt);
        g.status = dev->gemm_status_dev;
        g.tile_counter = counter;
        const int npairs = gemm_sm_budget(dev) / 2;
        // Last wave: when the tiles left over after the full waves would occupy at most half of the
        // pairs, they are drawn as half-width tiles and the wave costs half a tile instead of a whole one.
        const int whole = g.tiles_m * g.tiles_n;
        const int rest = whole % npairs;
        g.full_tiles = (v.split_tail && v.bnt == 256 && whole > npairs && rest > 0 && 2 * rest <= npairs) ? whole - rest : whole;
        const int pairs = std::min(whole + (whole - g.full_tiles), npairs);
        CUlaunchConfig cfg{};
        cfg.gridDimX = 2 * pairs; cfg.gridDimY = 1; cfg.gridDimZ = 1;
        cfg.blockDimX = PAIR_THREADS; cfg.blockDimY = 1; cfg.blockDimZ = 1;
        cfg.sharedMemBytes = pair_smem_bytes(v.bnt, v.stages, v.tf32);
        cfg.hStream = (CUstream)stream;
        CUlaunchAttribute at[1];
        at[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        at[0].value.clusterDim.x = 2; at[0].value.clusterDim.y = 1; at[0].value.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        g.draw_late = (whole + (whole - g.full_tiles)) <= 2 * pairs;
        void* params[4] = {&ma, &mb, &mbh, &g};
        CUresult cr = dev->drv.LaunchKernelEx(&cfg, fn, params, nullptr);
        if (cr != CUDA_SUCCESS) { const char* e = nullptr; dev->drv.GetErrorString(cr, &e); return dev->fail(ANL_ERR_CUDA, std::string("gemm: pair launch: ") + (e ? e : "?")); }
        dev->stats.kernels_launched++;
        dev->stats.gemm_launched++;
        return ANL_OK;
    }
    if (fusion) return dev->fail(ANL_ERR_INVALID, "gemm: a fused consumer needs the two-CTA kernel");
    if (gp.b_mn) rc = encode_map(dev, &mb, b, (uint64_t)c.N, (uint64_t)c.K, (uint64_t)gp.ldb, 64, BK);
    else rc = encode_map(dev, &mb, b, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)gp.ldb, BK, BN);
    if (rc) return rc;
    GemmArgs g;
    g.d = (__half*)bufs[0] + (window ? m_begin * c.N : 0);
    g.M = (int)M; g.N = (int)c.N; g.K = (int)c.K; g.ldd = (int)c.N;
    g.tiles_m = (int)((M + BM - 1) / BM); g.tiles_n = (int)((c.N + BN - 1) / BN);
    g.status = dev->gemm_status_dev;
    g.tile_counter = counter;
    int tiles = g.tiles_m * g.tiles_n;
    int grid = std::min(tiles, gemm_sm_budget(dev));
    if (gp.a_mn && gp.b_mn) gemm_f16_tcgen05<true, true><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
    else if (gp.a_mn) gemm_f16_tcgen05<true, false><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
    else if (gp.b_mn) gemm_f16_tcgen05<false, true><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
    else gemm_f16_tcgen05<false, false><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm: launch: ") + cudaGetErrorString(e));
    dev->stats.kernels_launched++;
    dev->stats.gemm_launched++;
    return ANL_OK;
}

// Finishes a bias gradient whose per-32-row partial column sums a contraction's epilogue left in
// `partials` [parts, N]: summed in f32 in a fixed order, one narrowing to f16 — the arithmetic of the REDUCE
// the schedule holds for it (f32 accumulator, narrowed once), with the rows grouped.
__global__ void __launch_bounds__(256) colsum_finish(const float* __restrict__ partials, int parts, int n, __half* __restrict__ out) {
    // a block owns 32 columns; its 8 warps take contiguous eighths of the parts (ascending inside each),
    // and the eight sums are added in warp order: a fixed order, wide enough to keep loads in flight
    __shared__ float part[8][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 32 + lane;
    const int per = (parts + 7) / 8, p0 = warp * per, p1 = (p0 + per) < parts ? (p0 + per) : parts;
    float acc = 0.0f;
    if (col < n) {
        int p = p0;
        for (; p + 4 <= p1; p += 4) {
            const float a = partials[(size_t)p * n + col], b = partials[(size_t)(p + 1) * n + col];
            const float c = partials[(size_t)(p + 2) * n + col], d = partials[(size_t)(p + 3) * n + col];
            acc = (((acc + a) + b) + c) + d;
        }
        for (; p < p1; p++) acc = acc + partials[(size_t)p * n + col];
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < n) {
        float v = part[0][lane];
#pragma unroll
        for (int w = 1; w < 8; w++) v = v + part[w][lane];
        out[col] = __float2half_rn(v);
    }
}

int launch_colsum_finish(anl_device* dev, const float* partials, int64_t parts, int64_t n, void* out, cudaStream_t stream) {
    colsum_finish<<<(unsigned)((n + 31) / 32), 256, 0, stream>>>(partials, (int)parts, (int)n, (__half*)out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm: column-sum finish: ") + cudaGetErrorString(e));
    dev->stats.kernels_launched++;
    return ANL_OK;
}

}  // namespace anl
