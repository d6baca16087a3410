// Two-CTA tcgen05 contraction kernel, compiled at run time (NVRTC, sm_100a) once per configuration.
//
//   D[M,N] = sum_k A[m,k] * B[n,k]   f16 operands, f32 accumulation in tensor memory, ONE rounding
//   to f16 (the arithmetic of an f16 REDUCE in the reference: f32 accumulator, operands widened,
//   narrowed once, codegen/lower.go:654-719), then — optionally — the elementwise kernel that the
//   schedule runs next on that value (bias add, GELU, the GELU-backward product), evaluated on the
//   narrowed value in the accumulator's registers exactly as the separate kernel would evaluate it
//   after reading it back (the reference fuses such consumers into the reduce kernel itself,
//   schedule/schedule.go:197-233), and — optionally — per-32-row partial column sums of what was
//   stored (the bias gradient that the schedule computes from it with a REDUCE over the rows).
//
// A pair of CTAs on neighbouring SMs (a cluster of 2) computes one 256 x BNT tile with
// tcgen05.mma.cta_group::2: each CTA stages its 128 rows of A and HALF of the B tile and holds the
// 128 x BNT accumulator of its own rows; the tensor cores of both SMs read both halves of B.  The
// even CTA leads: it owns the "full" barriers (both CTAs' TMA loads complete on them) and issues the
// MMAs; its commits release the stage and publish the accumulator in both CTAs.  No load is
// multicast: every CTA issues its own.  Warp roles: 0 TMA producer, 1 MMA issuer (owns the tensor
// memory allocation), 2-9 epilogue (two per 32-lane quadrant of tensor memory, half of the columns
// each: with four, a fused consumer on a short K was bound by the epilogue).  Two accumulators
// let the epilogue of tile i run under the main loop of tile i+1.  Tile numbers are drawn from a
// global counter, so a pair that starts late (its SMs were busy with a collective) takes fewer.
//
// When the tile count does not fill the last wave of pairs, the tiles of that wave are drawn as two
// half-width tiles each (second tensor map for B with half the box, N = BNT/2 in the instruction
// descriptor, half the accumulator columns): the pairs that would have idled take the other halves.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in a host-visible status
// word, the roles of the CTA drain and the tensor memory is freed.
//
// f32 operands (CFG_TF32 = 1) take the same kernel in "3 x TF32" form: each operand arrives as two
// k-contiguous f32 arrays, hi = the value rounded to TF32's 11 significant bits and lo = value - hi (exact), and
// every k-block is loaded once as four parts (A_hi, A_lo, B_hi, B_lo: 64 KB a stage, three stages) and
// accumulated as three products — lo·hi, hi·lo, hi·hi — with
// tcgen05.mma.kind::tf32, whose products of 11-bit factors are exact in the f32 accumulator.  What is
// dropped is lo·lo (2^-22 of the product) and the bits of lo beyond TF32's reach (2^-22 of the
// operand); the sum carries f32 accumulation like the reference's loop, in another order.  The
// accumulator in tensor memory cuts each partial sum instead of rounding it, and that error grows with
// the number of additions, so K is taken in chunks of chunk_kb k-blocks: the two accumulators
// alternate between chunks instead of between tiles, and the epilogue adds each chunk's result to the
// output in f32 round-to-nearest (the tile stays in L2 meanwhile) under the next chunk's main loop.
// Where the tiles are too few to occupy the pairs and K is long, the host also splits K between
// draws of the same tile: each writes its own copy of the output and the host adds the copies in a
// fixed order.
//
// The host prepends the configuration:
//   CFG_A_MN, CFG_B_MN   1 when the operand's m / n index is the contiguous one (else k is)
//   CFG_BNT              tile width in columns: 256 or 128
//   CFG_STAGES           depth of the shared-memory ring of k-blocks
//   CFG_GROUP_M          raster: tiles are numbered down groups of this many tile rows, so the pairs
//                        working at the same time share few A row blocks AND few B column blocks
//                        (0: down whole columns of tiles)
//   CFG_TF32             1: f32 operands and output in 3 x TF32 form (no fused consumer, no column sums)
//   CFG_EPI              1 when a fused elementwise consumer epi8_() has been prepended
//   CFG_STREAM_STORES    1: outputs are written with the streaming hint (they are not read again by
//                        this kernel and should not push operand tiles out of L2)
// and, when CFG_EPI is 1, the text of
//   EPI_NRAW                                  how many groups of 8 consecutive f16 the consumer loads per call
//   __device__ void epi8_load_(int row, int col, const void* const* ep, __half2 (*raw)[4])
//   __device__ void epi8_(int row, int col, const __half2* acc, __half2* out, const void* const* ep, const __half2 (*raw)[4])
// the second of which maps 8 consecutive narrowed values acc[0..3] at (row, col..col+7) to the 8 outputs
// from the operand values the first one loaded (the kernel calls it a chunk of 32 columns ahead: the
// loads' latency would otherwise be paid once per chunk by each of a handful of epilogue warps).
#pragma once

// Arguments of the f16 form.  The layout is kept at 120 bytes on purpose: with 24 more bytes of
// fields that only the f32 form reads, the f16 kernel ran 6% slower on every large shape, whatever its
// code did with them; the f32 form therefore has a block of its own.
struct PairGemmArgs {
    void* d_raw;            // [M, ldd] f16: the contraction itself; null when nothing else reads it
    void* d_out;            // [M, ldd] f16: output of the fused consumer; null without one
    float* colsum;          // [ceil(M/32), N] f32 partial column sums of the last value stored; null when not wanted
    const void* ep[6];      // operands of the fused consumer, in its parameter order
    int M, N, K, ldd;
    int tiles_m, tiles_n;   // in 256-row pair tiles and BNT-column tiles
    int full_tiles;         // tile numbers below this are BNT wide; each tile from here on is drawn as two halves
                            // of BNT/2 columns, so that the last, partly filled wave of tiles costs half a tile
    int draw_late;          // 1: few tiles, draw the next tile number after this tile's loads; 0: draw one tile ahead
    int* status;
    int* tile_counter;      // [0] next tile number, [1] pairs that have signed off; both zero between launches
};

// Arguments of the f32 (3 x TF32) form.
struct PairGemmArgsF32 {
    void* d_raw;            // [M, ldd] f32 output, or the copies of it when K is split between draws
    int M, N, K, ldd;
    int tiles_m, tiles_n;
    int full_tiles;         // = tiles_m * tiles_n: this form draws no half-width tiles
    int draw_late;
    int chunk_kb;           // k-blocks accumulated in tensor memory before the partial result is added, in f32
                            // round-to-nearest, to what the output holds (0: all of K in one go)
    int k_splits;           // with few tiles and a long K, every tile is drawn k_splits times, each draw taking
    int kb_per_split;       // kb_per_split k-blocks and writing its sum to its own copy of the output, split_stride
    int reserved;
    long long split_stride; // elements after the one before; the host adds the copies in order afterwards (<= 1: off)
    int* status;
    int* tile_counter;
};

#ifdef ANL_PAIR_GEMM_DEVICE_CODE

#include <cuda_fp16.h>

struct alignas(64) TensorMap { unsigned long long opaque[16]; };
#ifndef CFG_TF32
#define CFG_TF32 0
#endif
#if CFG_TF32
typedef PairGemmArgsF32 Args;
#else
typedef PairGemmArgs Args;
#endif

#ifndef CFG_TF32
#define CFG_TF32 0
#endif
// a k-block is one 128-byte swizzle row of k: 64 f16 or 32 f32 elements
constexpr int ESZ = CFG_TF32 ? 4 : 2;
constexpr int BM = 128, BK = 128 / ESZ;
constexpr int MNBOX = 64;                   // f16 elements of m (or n) in one row of an MN-major box
constexpr int KSTEP_BYTES_MN = 16 * 128;    // one MMA's k-rows in an MN-major tile
static_assert(!(CFG_TF32 && (CFG_A_MN || CFG_B_MN)), "the f32 form takes k-contiguous operands only: the host's split pre-pass rewrites the others");
constexpr int BNT = CFG_BNT, NSTAGE = CFG_STAGES;
constexpr int A_TILE_BYTES = BM * BK * ESZ;
constexpr int BHALF_BYTES = (BNT / 2) * BK * ESZ;
// a stage holds this CTA's A rows and its half of B; in the f32 form both as hi and lo parts, so that one
// set of loads serves the three products (A_hi, A_lo, B_hi, B_lo: 64 KB)
constexpr int STAGE_B = (CFG_TF32 ? 2 : 1) * (A_TILE_BYTES + BHALF_BYTES);
constexpr int TQ = 4;
constexpr int EPI_WARPS = 8;         // two per 32-lane quadrant of tensor memory, each taking half of the tile's columns
constexpr unsigned WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded waits: false when the phase did not complete within WAIT_LIMIT polls, or when another
// role of this CTA has already given up (`failed`, in shared memory).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, const volatile int* failed) {
    for (unsigned i = 0; i < WAIT_LIMIT; i++) {
        if (failed && (i & 255u) == 255u && *failed) return false;
        unsigned done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait_cluster(unsigned bar, unsigned parity, const volatile int* failed) {
    // acquires at cluster scope: the data guarded by the barrier was written by the partner CTA
    for (unsigned i = 0; i < WAIT_LIMIT; i++) {
        if (failed && (i & 255u) == 255u && *failed) return false;
        unsigned done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ unsigned cluster_ctarank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned map_to_cta(unsigned saddr, unsigned rank) {
    unsigned r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(unsigned cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// both CTAs' loads complete on the leader's barrier; no multicast
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const TensorMap* map, int c0, int c1, unsigned leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(leader_bar) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle: bits [0,14) start address >> 4, [16,30) leading
// byte offset >> 4, [32,46) stride byte offset >> 4, [46,48) version 1, [61,64) layout type 2.
__device__ __forceinline__ unsigned long long make_desc(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((saddr >> 4) & 0x3FFF);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
#if CFG_TF32
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#else
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#endif
}
__device__ __forceinline__ void umma_commit_pair(unsigned cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned* v) {
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

// The tile counter must read zero when a launch starts.  The launch cleans up after itself: a pair
// that has drawn a number past the end signs off on the second word, and the last to sign off zeroes
// both.  Nobody draws after its own sign-off, so the reset cannot race with a draw.
__device__ __forceinline__ void retire_tile_counter(int* counter, int drawers) {
    __threadfence();
    if (atomicAdd(counter + 1, 1) == drawers - 1) {
        counter[0] = 0;
        counter[1] = 0;
        __threadfence();
    }
}

// tile number -> (tile row, tile column)
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    if (CFG_GROUP_M <= 0 || CFG_GROUP_M >= tiles_m) { tm = t % tiles_m; tn = t / tiles_m; return; }
    const int per_group = CFG_GROUP_M * tiles_n;
    const int grp = t / per_group, first = grp * CFG_GROUP_M;
    const int rows = (tiles_m - first) < CFG_GROUP_M ? (tiles_m - first) : CFG_GROUP_M;
    const int r = t - grp * per_group;
    tm = first + r % rows; tn = r / rows;
}

// drawn number -> (tile row, first column, width)
__device__ __forceinline__ void tile_of(int t, int tiles_m, int tiles_n, int full_tiles, int& tm, int& col0, int& width) {
    int tn;
    if (t < full_tiles) { tile_coords(t, tiles_m, tiles_n, tm, tn); col0 = tn * BNT; width = BNT; return; }
    const int h = t - full_tiles;
    tile_coords(full_tiles + (h >> 1), tiles_m, tiles_n, tm, tn);
    col0 = tn * BNT + (h & 1) * (BNT / 2); width = BNT / 2;
}

__device__ __forceinline__ void store16(void* p, uint4 v) {
#if CFG_STREAM_STORES
    __stcs(reinterpret_cast<uint4*>(p), v);
#else
    *reinterpret_cast<uint4*>(p) = v;
#endif
}

__device__ __forceinline__ uint4 shfl_xor_u4(uint4 v, int mask) {
    v.x = __shfl_xor_sync(0xffffffffu, v.x, mask); v.y = __shfl_xor_sync(0xffffffffu, v.y, mask);
    v.z = __shfl_xor_sync(0xffffffffu, v.z, mask); v.w = __shfl_xor_sync(0xffffffffu, v.w, mask);
    return v;
}
__device__ __forceinline__ uint4 sel_u4(bool c, uint4 a, uint4 b) { return c ? a : b; }

// drawn number -> tile number and the k-blocks it covers (all of them unless the f32 form splits K)
__device__ __forceinline__ void split_of(const Args& g, int t, int tile_numbers, int kblocks, int& tile, int& sp, int& kb_first, int& nkb_all) {
#if CFG_TF32
    if (g.k_splits > 1) {
        sp = t / tile_numbers; tile = t - sp * tile_numbers;
        kb_first = sp * g.kb_per_split;
        nkb_all = (kblocks - kb_first) < g.kb_per_split ? (kblocks - kb_first) : g.kb_per_split;
        return;
    }
#endif
    tile = t; sp = 0; kb_first = 0; nkb_all = kblocks;
}

extern "C" __global__ void __launch_bounds__(64 + 32 * EPI_WARPS, 1)
#if CFG_TF32
gemm_f16_tcgen05_pair(const __grid_constant__ TensorMap map_a, const __grid_constant__ TensorMap map_b,
                      const __grid_constant__ TensorMap map_a_lo, const __grid_constant__ TensorMap map_b_lo, const Args g) {
    const TensorMap& map_b_half = map_b;         // the f32 form draws no half-width tiles
#else
gemm_f16_tcgen05_pair(const __grid_constant__ TensorMap map_a, const __grid_constant__ TensorMap map_b, const __grid_constant__ TensorMap map_b_half,
                      const Args g) {
    const TensorMap& map_a_lo = map_a;           // read by the f32 form only
    const TensorMap& map_b_lo = map_b;
#endif
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[NSTAGE], empty_bar[NSTAGE], acc_full[2], acc_empty[2];
    // tile queue: the leader's producer draws tile numbers from the global counter and publishes each
    // one in both CTAs; a slot is recycled once all consumers of the pair have read it
    __shared__ __align__(8) unsigned long long tq_full[TQ], tq_empty[TQ];
    __shared__ int tile_ring[TQ];
    __shared__ unsigned tmem_base_slot;
    __shared__ volatile int failed;

    const unsigned smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1 KiB alignment
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();            // 0 leads
    const int tiles_m = g.tiles_m;
    const int whole_tiles = tiles_m * g.tiles_n;
    const int tile_numbers = whole_tiles + (whole_tiles - g.full_tiles);  // every tile past full_tiles counts twice
    const int kblocks = (g.K + BK - 1) / BK;
#if CFG_TF32
    const int num_tiles = tile_numbers * (g.k_splits > 1 ? g.k_splits : 1);
    const int chunk_kb = (g.chunk_kb > 0 && g.chunk_kb < kblocks) ? g.chunk_kb : (kblocks > 0 ? kblocks : 1);
#else
    const int num_tiles = tile_numbers;
    const int chunk_kb = kblocks > 0 ? kblocks : 1;
#endif

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 2 * EPI_WARPS); }
        for (int q = 0; q < TQ; q++) { mbar_init(smem_u32(&tq_full[q]), 1); mbar_init(smem_u32(&tq_empty[q]), 2 + 2 * EPI_WARPS); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // 512 columns: two 128 x BNT f32 accumulators (BNT <= 256)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                  // both CTAs' barriers exist before any remote signal
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ── producer ──
        if (lane == 0) {
            unsigned stage = 0, phase = 0;
            bool ok = true;
            unsigned qs = 0, qphase = 0;
            int next = rank == 0 ? atomicAdd(g.tile_counter, 1) : 0;
            while (ok) {
                int t;
                if (rank == 0) {
                    if (!mbar_wait(smem_u32(&tq_empty[qs]), qphase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 15; break; }
                    t = next;
                    if (t >= num_tiles) t = -1;
                    else if (!g.draw_late) next = atomicAdd(g.tile_counter, 1);    // one tile ahead: the latency hides behind this tile's loads
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
                int tt, sp, kb_first, nkb_all;
                split_of(g, t, tile_numbers, kblocks, tt, sp, kb_first, nkb_all);
                const int chunks = (nkb_all + chunk_kb - 1) / chunk_kb;
                int tm, col0, width;
                tile_of(tt, tiles_m, g.tiles_n, g.full_tiles, tm, col0, width);
                const bool narrow = width != BNT;
                const int m0 = tm * (2 * BM) + (int)rank * BM;           // this CTA's rows of A
                const int n0 = col0 + (int)rank * (width / 2);           // this CTA's half of B
                const unsigned stage_bytes = A_TILE_BYTES + (narrow ? BHALF_BYTES / 2 : BHALF_BYTES);
                const TensorMap* const mb = narrow ? &map_b_half : &map_b;
                for (int ch = 0; ch < chunks && ok; ch++) {
                    const int kb0 = kb_first + ch * chunk_kb, nkb = (nkb_all - ch * chunk_kb) < chunk_kb ? (nkb_all - ch * chunk_kb) : chunk_kb;
                    for (int it = 0; it < nkb && ok; it++) {
                        const int kb = kb0 + it;
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 11; break; }
                        const unsigned own_fb = smem_u32(&full_bar[stage]);
                        const unsigned fb = map_to_cta(own_fb, 0);
                        const int k0 = kb * BK;
#if CFG_TF32
                        // hi and lo parts of both operands: A_hi, A_lo, B_hi, B_lo
                        const unsigned sa = smem_base + stage * STAGE_B, sb = sa + 2 * A_TILE_BYTES;
                        if (rank == 0) mbar_expect_tx(own_fb, 2 * STAGE_B);
                        tma_load_2d_pair(sa, &map_a, k0, m0, fb);
                        tma_load_2d_pair(sa + A_TILE_BYTES, &map_a_lo, k0, m0, fb);
                        tma_load_2d_pair(sb, &map_b, k0, n0, fb);
                        tma_load_2d_pair(sb + BHALF_BYTES, &map_b_lo, k0, n0, fb);
                        (void)stage_bytes; (void)mb;
#else
                        const unsigned sa = smem_base + stage * STAGE_B, sb = sa + A_TILE_BYTES;
                        if (rank == 0) mbar_expect_tx(own_fb, 2 * stage_bytes);
                        if (CFG_A_MN) { for (int j = 0; j < BM / MNBOX; j++) tma_load_2d_pair(sa + j * (BK * 128), &map_a, m0 + MNBOX * j, k0, fb); }
                        else tma_load_2d_pair(sa, &map_a, k0, m0, fb);
                        if (CFG_B_MN) { for (int j = 0; j < (width / 2) / MNBOX; j++) tma_load_2d_pair(sb + j * (BK * 128), mb, n0 + MNBOX * j, k0, fb); }
                        else tma_load_2d_pair(sb, mb, k0, n0, fb);
#endif
                        if (++stage == NSTAGE) { stage = 0; phase ^= 1; }
                    }
                }
                // With few tiles (draw_late) the next number is drawn only once this tile's loads are issued, so
                // that every pair gets one tile before any pair gets two; that puts the atomic's latency on the
                // producer's path once per tile, which costs about 5% where the tiles are many, so there the
                // number is drawn a tile ahead instead.  Nothing is added to the loop above: one more
                // instruction in it cost a tenth of the kernel's throughput.
                if (rank == 0 && g.draw_late && ok) next = atomicAdd(g.tile_counter, 1);
            }
            if (!ok) failed = 1;
        }
    } else if (warp == 1) {
        // ── MMA issuer (leader CTA only) ──
        if (lane == 0 && rank == 0) {
            // instruction descriptor: f32 accumulate, f16 x f16, majors, N >> 3 at bit 17, M >> 4 at bit 24 (256 across the pair)
            // bits [4,6) accumulator f32; [7,10) and [10,13) operand formats (0 f16, 2 tf32); 15/16 majors
            const unsigned idesc_base = (1u << 4) | ((CFG_TF32 ? 2u : 0u) << 7) | ((CFG_TF32 ? 2u : 0u) << 10) |
                                        ((CFG_A_MN ? 1u : 0u) << 15) | ((CFG_B_MN ? 1u : 0u) << 16) | ((unsigned)((2 * BM) >> 4) << 24);
            unsigned stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            unsigned qs = 0, qphase = 0;
            while (ok) {
                if (!mbar_wait(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; *(volatile int*)g.status = 17; break; }
                const int t = tile_ring[qs];
                mbar_arrive(smem_u32(&tq_empty[qs]));
                if (++qs == TQ) { qs = 0; qphase ^= 1; }
                if (t < 0) break;
                int tt, sp, kb_first, nkb_all;
                split_of(g, t, tile_numbers, kblocks, tt, sp, kb_first, nkb_all);
                const int chunks = (nkb_all + chunk_kb - 1) / chunk_kb;
                const unsigned idesc = idesc_base | ((unsigned)((tt < g.full_tiles ? BNT : BNT / 2) >> 3) << 17);
                for (int ch = 0; ch < chunks && ok; ch++) {
                    const int nkb = (nkb_all - ch * chunk_kb) < chunk_kb ? (nkb_all - ch * chunk_kb) : chunk_kb;
                    if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1, &failed)) { ok = false; *(volatile int*)g.status = 12; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned tmem_d = tmem_base + acc * BNT;
                    for (int kb = 0; kb < nkb; kb++) {
                        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &failed)) { ok = false; *(volatile int*)g.status = 13; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#if CFG_TF32
                        // 3 x TF32 on one set of loads: A_lo · B_hi, A_hi · B_lo, A_hi · B_hi (k-contiguous operands)
                        const unsigned sa = smem_base + stage * STAGE_B, sb = sa + 2 * A_TILE_BYTES;
#pragma unroll
                        for (int pass = 0; pass < 3; pass++) {
                            const unsigned pa = pass == 0 ? sa + A_TILE_BYTES : sa, pb = pass == 1 ? sb + BHALF_BYTES : sb;
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                umma_f16_pair(tmem_d, make_desc(pa + k * 32, 16, 1024), make_desc(pb + k * 32, 16, 1024), idesc, (kb | pass | k) != 0);
                        }
#else
                        const unsigned sa = smem_base + stage * STAGE_B, sb = sa + A_TILE_BYTES;
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            // One MMA covers 32 bytes of k (16 f16 elements): four per k-block.
                            // K-major: 32 bytes inside the 128-byte row, 8-row groups 1 KiB apart.
                            // MN-major: the MMA's k-rows are whole 128-byte rows (KSTEP_BYTES_MN of them per
                            // step), m/n groups of one swizzle row's width one box (BK*128 B) apart.
                            const unsigned long long ad = CFG_A_MN ? make_desc(sa + k * KSTEP_BYTES_MN, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
                            const unsigned long long bd = CFG_B_MN ? make_desc(sb + k * KSTEP_BYTES_MN, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
                            umma_f16_pair(tmem_d, ad, bd, idesc, (kb | k) != 0);
                        }
#endif
                        const unsigned eb = smem_u32(&empty_bar[stage]);
                        umma_commit_pair(map_to_cta(eb, 0));       // frees the stage here ...
                        umma_commit_pair(map_to_cta(eb, 1));       // ... and in the partner CTA
                        if (++stage == NSTAGE) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    const unsigned af = smem_u32(&acc_full[acc]);
                    umma_commit_pair(map_to_cta(af, 0));
                    umma_commit_pair(map_to_cta(af, 1));
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
            }
            if (!ok) failed = 1;
        }
    } else {
        // ── epilogue: warps 2..9, tensor-memory lane quadrant = warp % 4, column half = (warp - 2) / 4 ──
        const int quad = warp & 3, col_half = (warp - 2) >> 2;
        unsigned acc = 0, acc_phase = 0;
        bool ok = true;
        unsigned qs = 0, qphase = 0;
        __half* const d_raw = (__half*)g.d_raw; (void)d_raw;
#if CFG_EPI
        __half* const d_out = (__half*)g.d_out;
        // the fused consumer's operands, loaded one 32-column chunk ahead of the arithmetic that needs
        // them: [group of 8 columns][operand][pair]
        constexpr int EPI_NR = EPI_NRAW > 0 ? EPI_NRAW : 1;
        __half2 raw_next[4][EPI_NR][4];
#endif
        while (ok) {
            if (!mbar_wait_cluster(smem_u32(&tq_full[qs]), qphase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 18; failed = 1; } break; }
            const int t = *(volatile int*)&tile_ring[qs];
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tq_empty[qs]), 0));
            if (++qs == TQ) { qs = 0; qphase ^= 1; }
            if (t < 0) break;
            int tt, sp, kb_first, nkb_all;
            split_of(g, t, tile_numbers, kblocks, tt, sp, kb_first, nkb_all);
            const int chunks = (nkb_all + chunk_kb - 1) / chunk_kb;
            int tm, n0, width;
            tile_of(tt, tiles_m, g.tiles_n, g.full_tiles, tm, n0, width);
            const int m0 = tm * (2 * BM) + (int)rank * BM;
            const int row = m0 + quad * 32 + lane;
            #if CFG_TF32
            const size_t row_off = (size_t)row * g.ldd + (size_t)sp * (size_t)g.split_stride;
#else
            const size_t row_off = (size_t)row * g.ldd;
#endif
            const bool row_ok = row < g.M;
            const bool vec_ok = (g.ldd % 8 == 0); (void)vec_ok;
            const int c_begin = col_half * (width / 64), c_end = c_begin + width / 64;      // this warp's 32-column chunks
            // After the narrowing, groups of four lanes exchange their rows' 8-column pieces, so that lane 4g+i
            // holds piece i (8 columns from ucol) of the rows urow0 .. urow0+3: a store or load instruction then
            // touches 8 rows x 64 contiguous bytes instead of 32 rows x 16.
            const int urow0 = m0 + quad * 32 + (lane & ~3), ucol = 8 * (lane & 3);
            (void)urow0; (void)ucol;
#if CFG_EPI
            // the first chunk's operands are asked for before the accumulator is even complete
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (urow0 + q < g.M && n0 + c_begin * 32 + ucol < g.N) epi8_load_(urow0 + q, n0 + c_begin * 32 + ucol, g.ep, raw_next[q]);
#endif
            for (int ch = 0; ch < chunks; ch++) {
            if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase, &failed)) { ok = false; if (lane == 0) { *(volatile int*)g.status = 14; failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = c_begin; c < c_end; c++) {
                unsigned v[32];
                tmem_ld32(tmem_base + ((unsigned)(quad * 32) << 16) + acc * BNT + c * 32, v);
#if CFG_EPI
                __half2 raw[4][EPI_NR][4];
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int k = 0; k < EPI_NR; k++)
#pragma unroll
                        for (int u = 0; u < 4; u++) raw[q][k][u] = raw_next[q][k][u];
                if (c + 1 < c_end) {
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        if (urow0 + q < g.M && n0 + (c + 1) * 32 + ucol < g.N) epi8_load_(urow0 + q, n0 + (c + 1) * 32 + ucol, g.ep, raw_next[q]);
                }
#endif
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col = n0 + c * 32;
                if (col >= g.N) continue;                  // warp-uniform
#if CFG_TF32
                // f32 result of this chunk of k: stored, or added to the sum of the chunks before it
                if (row_ok) {
                    float* out = reinterpret_cast<float*>(g.d_raw) + row_off + col;
                    if ((g.ldd & 3) == 0 && col + 32 <= g.N) {
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            float4 r = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                            if ((ch > 0)) { const float4 o = *reinterpret_cast<const float4*>(out + 4 * q); r.x = o.x + r.x; r.y = o.y + r.y; r.z = o.z + r.z; r.w = o.w + r.w; }
                            *reinterpret_cast<float4*>(out + 4 * q) = r;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col + j < g.N) out[j] = (ch > 0) ? out[j] + __uint_as_float(v[j]) : __uint_as_float(v[j]);
                    }
                }
#else
                // the single narrowing of the f32 accumulator
                __half2 h[16];
#pragma unroll
                for (int j = 0; j < 16; j++) h[j] = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                if (vec_ok) {
                    // 4 x 4 transpose of 16-byte pieces inside each group of four lanes: two exchange rounds
                    const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0;
                    const uint4* const Q = reinterpret_cast<const uint4*>(h);
                    uint4 A[2][2], T[4];
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const uint4 got = shfl_xor_u4(sel_u4(b0, Q[2 * k], Q[2 * k + 1]), 1), keep = sel_u4(b0, Q[2 * k + 1], Q[2 * k]);
                        A[k][0] = sel_u4(b0, got, keep);          // piece 2k + (lane & 1) of the even lane's row
                        A[k][1] = sel_u4(b0, keep, got);          // ... of the odd lane's row
                    }
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        const uint4 got = shfl_xor_u4(sel_u4(b1, A[0][j], A[1][j]), 2), keep = sel_u4(b1, A[1][j], A[0][j]);
                        T[j] = sel_u4(b1, got, keep);             // rows urow0 + 0, 1
                        T[2 + j] = sel_u4(b1, keep, got);         // rows urow0 + 2, 3
                    }
                    const int ucolc = col + ucol;
                    float x[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) x[j] = 0.0f;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const bool on = urow0 + q < g.M && ucolc < g.N;      // N is a multiple of 8 here: a piece is all in or all out
                        const size_t off = (size_t)(urow0 + q) * g.ldd + ucolc;
                        if (on && d_raw) store16(d_raw + off, T[q]);
#if CFG_EPI
                        uint4 O = make_uint4(0u, 0u, 0u, 0u);
                        if (on) {
                            epi8_(urow0 + q, ucolc, reinterpret_cast<const __half2*>(&T[q]), reinterpret_cast<__half2*>(&O), g.ep, raw[q]);
                            store16(d_out + off, O);
                        }
#else
                        const uint4 O = on ? T[q] : make_uint4(0u, 0u, 0u, 0u);
#endif
                        const __half2* const oh = reinterpret_cast<const __half2*>(&O);
#pragma unroll
                        for (int j = 0; j < 4; j++) { const float2 f = __half22float2(oh[j]); x[2 * j] += f.x; x[2 * j + 1] += f.y; }
                    }
                    if (g.colsum && m0 + quad * 32 < g.M) {      // warp-uniform: groups of 32 rows that start inside the matrix
                        // partial column sums over this warp's 32 rows of what was stored (rows and columns outside
                        // the matrix contribute zero): the four rows of a lane first, then across the eight groups
#pragma unroll
                        for (int off = 4; off <= 16; off <<= 1)
#pragma unroll
                            for (int j = 0; j < 8; j++) x[j] += __shfl_xor_sync(0xffffffffu, x[j], off);
                        if (lane < 4 && ucolc < g.N) {
                            float* const cs = g.colsum + (size_t)((m0 + quad * 32) >> 5) * g.N + ucolc;
#pragma unroll
                            for (int j = 0; j < 8; j++) cs[j] = x[j];
                        }
                    }
                } else if (row_ok) {
                    // row stride not a multiple of 16 bytes (no fused consumer on this route): scalar stores
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        if (col + 2 * j < g.N) d_raw[row_off + col + 2 * j] = __low2half(h[j]);
                        if (col + 2 * j + 1 < g.N) d_raw[row_off + col + 2 * j + 1] = __high2half(h[j]);
                    }
                }
#endif
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));   // the leader waits for both CTAs' epilogues
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
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

#endif  // ANL_PAIR_GEMM_DEVICE_CODE
