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
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "runtime.hpp"

namespace anl {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_TILE_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + alignment slack
constexpr int GEMM_THREADS = 192;
constexpr int TQ = 4;                               // depth of the per-CTA tile queue
constexpr unsigned WAIT_LIMIT = 1u << 20;

struct GemmPlan {
    Contraction c;
    bool a_mn = false, b_mn = false;     // MN-major operands
    int64_t lda = 0, ldb = 0;            // elements between consecutive rows of the 2-D global views
    bool f32 = false;                    // f32 operands: the FP32-pipe kernel instead of tcgen05
    int* status_host = nullptr;          // mapped, host-visible
    int* status_dev = nullptr;
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
                else next = atomicAdd(g.tile_counter, 1);      // drawn one tile ahead: its latency hides behind this tile's loads
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

// ── two-CTA variant ─────────────────────────────────────────────────────────────────────────────
// A pair of CTAs on neighbouring SMs (a cluster of 2) computes one 256x256 tile with
// tcgen05.mma.cta_group::2: each CTA holds 128 rows of A, HALF of B (128 of the 256 columns) and
// the 128x256 accumulator of its own rows; the tensor cores of both SMs read both halves of B.  Per
// k-block a CTA therefore moves 32 KiB through shared memory instead of 48 KiB for the same math,
// which is what the one-CTA kernel is short of (shared-memory bandwidth, not DRAM).  The even CTA
// leads: it owns the "full" barriers (both CTAs' loads complete on them) and issues the MMAs; its
// commits release the stage and publish the accumulator in both CTAs.  No load is multicast.
constexpr int STAGES2 = 6;
constexpr int B2_TILE_BYTES = (BN / 2) * BK * 2;               // 16 KiB: this CTA's half of B
constexpr int SMEM2_BYTES = STAGES2 * (A_TILE_BYTES + B2_TILE_BYTES) + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const volatile int* failed) {
    // like mbar_wait, but acquires at cluster scope: the data guarded by the barrier was written by the partner CTA
    for (unsigned i = 0; i < WAIT_LIMIT; i++) {
        if (failed && (i & 255u) == 255u && *failed) return false;
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// BNT = tile width in columns (256, or 128 when that fills the last wave of tiles better)
template <bool A_MN, bool B_MN, int BNT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_tcgen05_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES2], empty_bar[STAGES2], acc_full[2], acc_empty[2];
    // tile queue: the leader's producer draws tile numbers from the global counter and publishes each
    // one in both CTAs; a slot is recycled once all ten consumers of the pair have read it
    __shared__ __align__(8) uint64_t tq_full[TQ], tq_empty[TQ];
    __shared__ int tile_ring[TQ];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int failed;

    constexpr int BHALF_BYTES = (BNT / 2) * BK * 2;            // this CTA's half of the B tile
    constexpr int STAGE_B = A_TILE_BYTES + BHALF_BYTES;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 leads
    const int tiles_m = (g.M + 2 * BM - 1) / (2 * BM);
    const int num_tiles = tiles_m * g.tiles_n;
    const int kblocks = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; s++) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 8); }
        for (int q = 0; q < TQ; q++) { mbar_init(smem_u32(&tq_full[q]), 1); mbar_init(smem_u32(&tq_empty[q]), 10); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                  // both CTAs' barriers exist before any remote signal
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            uint32_t qs = 0, qphase = 0;
            int next = rank == 0 ? atomicAdd(g.tile_counter, 1) : 0;
            while (ok) {
                int t;
                if (rank == 0) {
                    if (!mbar_wait(smem_u32(&tq_empty[qs]), qphase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 15; break; }
                    t = next;
                    if (t >= num_tiles) t = -1;
                    else next = atomicAdd(g.tile_counter, 1);
                    tile_ring[qs] = t;
                    st_cluster_u32(map_to_cta(smem_u32(&tile_ring[qs]), 1), t);
                    mbar_arrive(smem_u32(&tq_full[qs]));
                    mbar_arrive_cluster(map_to_cta(smem_u32(&tq_full[qs]), 1));
                } else {
                    if (!mbar_wait_cluster(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; *(volatile int*)g.status = 16; break; }
                    t = *(volatile int*)&tile_ring[qs];
                    mbar_arrive_cluster(map_to_cta(smem_u32(&tq_empty[qs]), 0));
                }
                if (++qs == TQ) { qs = 0; qphase ^= 1; }
                if (t < 0) { if (rank == 0) retire_tile_counter(g.tile_counter, (int)gridDim.x / 2); break; }
                const int m0 = (t % tiles_m) * (2 * BM) + (int)rank * BM;          // this CTA's rows of A
                const int n0 = (t / tiles_m) * BNT + (int)rank * (BNT / 2);          // this CTA's half of B
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 11; break; }
                    const uint32_t own_fb = smem_u32(&full_bar[stage]);
                    const uint32_t fb = map_to_cta(own_fb, 0);                     // loads of both CTAs complete on the leader's barrier
                    const uint32_t sa = smem_base + stage * STAGE_B, sb = sa + A_TILE_BYTES;
                    if (rank == 0) mbar_expect_tx(own_fb, 2 * STAGE_B);
                    const int k0 = kb * BK;
                    if (A_MN) { for (int j = 0; j < BM / 64; j++) tma_load_2d_pair(sa + j * (BK * 128), &map_a, m0 + 64 * j, k0, fb); }
                    else tma_load_2d_pair(sa, &map_a, k0, m0, fb);
                    if (B_MN) { for (int j = 0; j < BNT / 128; j++) tma_load_2d_pair(sb + j * (BK * 128), &map_b, n0 + 64 * j, k0, fb); }
                    else tma_load_2d_pair(sb, &map_b, k0, n0, fb);
                    if (++stage == STAGES2) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) failed = 1;
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // M = 256 across the pair (M >> 4 = 16 at bit 24), N = 256
            const uint32_t idesc = (1u << 4) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            uint32_t qs = 0, qphase = 0;
            while (ok) {
                if (!mbar_wait(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; *(volatile int*)g.status = 17; break; }
                const int t = tile_ring[qs];
                mbar_arrive(smem_u32(&tq_empty[qs]));
                if (++qs == TQ) { qs = 0; qphase ^= 1; }
                if (t < 0) break;
                if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 12; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * BNT;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &failed)) { ok = false; *(volatile int*)g.status = 13; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_base + stage * STAGE_B, sb = sa + A_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        const uint64_t ad = A_MN ? make_desc(sa + k * 2048, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_desc(sb + k * 2048, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
                        umma_f16_pair(tmem_d, ad, bd, idesc, (kb | k) != 0);
                    }
                    const uint32_t eb = smem_u32(&empty_bar[stage]);
                    umma_commit_pair(map_to_cta(eb, 0));       // frees the stage here ...
                    umma_commit_pair(map_to_cta(eb, 1));       // ... and in the partner CTA
                    if (++stage == STAGES2) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                const uint32_t af = smem_u32(&acc_full[acc]);
                umma_commit_pair(map_to_cta(af, 0));
                umma_commit_pair(map_to_cta(af, 1));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
            if (!ok) failed = 1;
        }
    } else {
        const int quad = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        uint32_t qs = 0, qphase = 0;
        while (ok) {
            if (!mbar_wait_cluster(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 18; failed = 1; } break; }
            const int t = *(volatile int*)&tile_ring[qs];
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tq_empty[qs]), 0));
            if (++qs == TQ) { qs = 0; qphase ^= 1; }
            if (t < 0) break;
            const int m0 = (t % tiles_m) * (2 * BM) + (int)rank * BM, n0 = (t / tiles_m) * BNT;
            if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 14; failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quad * 32 + lane;
            __half* drow = g.d + (size_t)row * g.ldd + n0;
            const bool row_ok = row < g.M;
            const bool vec_ok = (g.ldd % 8 == 0);
#pragma unroll 1
            for (int c = 0; c < BNT / 32; c++) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BNT + c * 32, v);
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
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (col + j < g.N) drow[c * 32 + j] = __float2half_rn(__uint_as_float(v[j]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));   // the leader waits for both CTAs' epilogues
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                  // the leader's MMAs read the partner's shared memory: leave together
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

static int encode_map(anl_device* dev, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = dev->drv.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { const char* s = nullptr; dev->drv.GetErrorString(r, &s); return dev->fail(ANL_ERR_CUDA, std::string("gemm: cuTensorMapEncodeTiled: ") + (s ? s : "?")); }
    return ANL_OK;
}

int plan_gemm(anl_device* dev, const Item& item, Plan& plan) {
    Contraction c;
    if (!match_contraction(item, c)) return ANL_ERR_UNSUPPORTED;
    const bool dynamic = c.m_sym || c.k_sym;
    if (c.in_dtype == DT_F32 && c.out_dtype == DT_F32) {
        if (c.a_sk != 1 && c.a_sm != 1) return ANL_ERR_UNSUPPORTED;
        if (c.b_sk != 1 && c.b_sn != 1) return ANL_ERR_UNSUPPORTED;
        if (!dynamic && !gemm_f32_worth(c.M, c.N, c.K)) return ANL_ERR_UNSUPPORTED;
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
    static int* status_host = nullptr;
    static int* status_dev = nullptr;
    if (!status_host) {
        if (cudaHostAlloc((void**)&status_host, 64, cudaHostAllocMapped) != cudaSuccess) return ANL_ERR_UNSUPPORTED;
        *status_host = 0;
        if (cudaHostGetDevicePointer((void**)&status_dev, status_host, 0) != cudaSuccess) return ANL_ERR_UNSUPPORTED;
    }
    gp->status_host = status_host; gp->status_dev = status_dev;
    if (!dev->gemm_tile_counter) {
        if (cudaMalloc((void**)&dev->gemm_tile_counter, 256) != cudaSuccess) return ANL_ERR_UNSUPPORTED;
        if (cudaMemset(dev->gemm_tile_counter, 0, 256) != cudaSuccess) return ANL_ERR_UNSUPPORTED;   // launches leave it zeroed again
    }
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_f16_tcgen05<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_f16_tcgen05<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
#define ANL_PAIR_ATTR(AM, BM_) \
        cudaFuncSetAttribute(gemm_f16_tcgen05_pair<AM, BM_, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES); \
        cudaFuncSetAttribute(gemm_f16_tcgen05_pair<AM, BM_, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
        ANL_PAIR_ATTR(false, false) ANL_PAIR_ATTR(false, true) ANL_PAIR_ATTR(true, false) ANL_PAIR_ATTR(true, true)
#undef ANL_PAIR_ATTR
        attr_set = true;
    }
    plan.gemm = gp;
    plan.r.klass = KC_GEMM;
    plan.r.note = std::string("gemm tcgen05 ") + (gp->a_mn ? "A:MN" : "A:K") + (gp->b_mn ? " B:MN" : " B:K") + " M=" + std::to_string(c.M) + " N=" + std::to_string(c.N) + " K=" + std::to_string(c.K);
    return ANL_OK;
}

// SMs the persistent GEMM may occupy.  When gradients are reduced while the backward pass is still
// running, a few SMs are left free so that the collective's blocks (and the update kernels behind
// them) find a place at once instead of waiting for a 150-SM persistent grid to drain.
static int gemm_sm_budget(anl_device* dev) {
    static const int env = std::getenv("ANNEAL_GEMM_SMS") ? std::atoi(std::getenv("ANNEAL_GEMM_SMS")) : 0;
    int sms = dev->prop.multiProcessorCount;
    int want = env > 0 ? env : (dev->nranks > 1 ? sms - dev->comm_reserved_sms : sms);
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
    return gemm_f32_worth(c.m_sym ? sym_value : c.M, c.N, c.k_sym ? sym_value : c.K);
}

int launch_gemm(anl_device* dev, const Plan& plan, void* const* bufs, int64_t sym_value, cudaStream_t stream, int64_t m_begin, int64_t m_end) {
    const GemmPlan& gp = *plan.gemm;
    const Contraction& c = gp.c;
    // an optional row window [m_begin, m_end) of the output: the caller splits a contraction so that
    // a collective on the first rows can start while the remaining rows are still being computed
    const bool window = m_end >= 0;
    if (window && (gp.f32 || c.m_sym || m_begin < 0 || m_end > c.M || m_begin >= m_end || (m_begin % 8)))
        return dev->fail(ANL_ERR_INVALID, "gemm: bad row window");
    const int64_t M = window ? m_end - m_begin : c.M;
    if (gp.f32)
        return launch_gemm_f32(dev, (const float*)bufs[c.a_param] + c.a_off, (const float*)bufs[c.b_param] + c.b_off, (float*)bufs[0],
                               c.m_sym ? sym_value : c.M, c.N, c.k_sym ? sym_value : c.K, c.a_sm, c.a_sk, c.b_sn, c.b_sk, stream);
    if (*gp.status_host != 0) return dev->fail(ANL_ERR_CUDA, "gemm: an earlier launch timed out on a barrier (code " + std::to_string(*gp.status_host) + ")");
    const __half* a = (const __half*)bufs[c.a_param] + c.a_off + (window ? m_begin * c.a_sm : 0);
    const __half* b = (const __half*)bufs[c.b_param] + c.b_off;
    CUtensorMap ma, mb;
    int rc;
    if (gp.a_mn) rc = encode_map(dev, &ma, a, (uint64_t)M, (uint64_t)c.K, (uint64_t)gp.lda, 64, BK);
    else rc = encode_map(dev, &ma, a, (uint64_t)c.K, (uint64_t)M, (uint64_t)gp.lda, BK, BM);
    if (rc) return rc;
    if (gp.b_mn) rc = encode_map(dev, &mb, b, (uint64_t)c.N, (uint64_t)c.K, (uint64_t)gp.ldb, 64, BK);
    else rc = encode_map(dev, &mb, b, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)gp.ldb, BK, BN);
    if (rc) return rc;
    GemmArgs g;
    g.d = (__half*)bufs[0] + (window ? m_begin * c.N : 0);
    g.M = (int)M; g.N = (int)c.N; g.K = (int)c.K; g.ldd = (int)c.N;
    g.tiles_m = (int)((M + BM - 1) / BM); g.tiles_n = (int)((c.N + BN - 1) / BN);
    g.status = gp.status_dev;
    g.tile_counter = dev->gemm_tile_counter;
    static const bool pair_ok = std::getenv("ANNEAL_GEMM_PAIR") ? std::atoi(std::getenv("ANNEAL_GEMM_PAIR")) != 0 : true;
    if (pair_ok && M >= 2 * BM && c.N >= BN / 2) {
        // two-CTA tiles, 256 rows by 256 or 128 columns.  The narrow tile fills the last wave of tiles
        // better but stages 1.5x the bytes per flop and measured 25% slower on 4096x4096x8192 (it
        // becomes L2-bound), so it is only taken when the wide tile would leave most pairs idle.
        const int npairs = gemm_sm_budget(dev) / 2;
        const int tm2 = (int)((M + 2 * BM - 1) / (2 * BM));
        auto fill = [&](int bnt) { long long t = (long long)tm2 * ((c.N + bnt - 1) / bnt); long long w = (t + npairs - 1) / npairs; return (double)t / (double)(w * npairs); };
        const int bnt = (fill(128) * 0.7 > fill(256)) ? 128 : 256;
        // B is loaded in halves of bnt/2 columns, so its tensor map gets a box of that many rows
        if (gp.b_mn) rc = encode_map(dev, &mb, b, (uint64_t)c.N, (uint64_t)c.K, (uint64_t)gp.ldb, 64, BK);
        else rc = encode_map(dev, &mb, b, (uint64_t)c.K, (uint64_t)c.N, (uint64_t)gp.ldb, BK, bnt / 2);
        if (rc) return rc;
        g.tiles_n = (int)((c.N + bnt - 1) / bnt);
        int tiles2 = tm2 * g.tiles_n;
        int pairs = std::min(tiles2, npairs);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = SMEM2_BYTES; cfg.stream = stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaError_t le;
#define ANL_PAIR_LAUNCH(AM, BM_, W) cudaLaunchKernelEx(&cfg, gemm_f16_tcgen05_pair<AM, BM_, W>, ma, mb, g)
        if (bnt == 256) {
            if (gp.a_mn && gp.b_mn) le = ANL_PAIR_LAUNCH(true, true, 256);
            else if (gp.a_mn) le = ANL_PAIR_LAUNCH(true, false, 256);
            else if (gp.b_mn) le = ANL_PAIR_LAUNCH(false, true, 256);
            else le = ANL_PAIR_LAUNCH(false, false, 256);
        } else {
            if (gp.a_mn && gp.b_mn) le = ANL_PAIR_LAUNCH(true, true, 128);
            else if (gp.a_mn) le = ANL_PAIR_LAUNCH(true, false, 128);
            else if (gp.b_mn) le = ANL_PAIR_LAUNCH(false, true, 128);
            else le = ANL_PAIR_LAUNCH(false, false, 128);
        }
#undef ANL_PAIR_LAUNCH
        if (le != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm: pair launch: ") + cudaGetErrorString(le));
        dev->stats.kernels_launched++;
        dev->stats.gemm_launched++;
        return ANL_OK;
    }
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

}  // namespace anl
