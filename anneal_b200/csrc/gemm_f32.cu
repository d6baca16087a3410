// f32 contraction kernel: D[m, n] = sum_k A[m, k] * B[n, k] with f32 operands, f32 accumulation in
// ascending k, f32 result.  The reference lowers such a kernel to one thread per output element
// that walks k serially (codegen/lower.go:158-171 and the REDUCE loop of codegen/wgsl.go); this is
// the same sum in the same order per output element (fused multiply-add instead of multiply then
// add, so results differ from the reference by rounding only), tiled through shared memory so that
// every operand element is read from HBM once per tile row/column instead of once per output.
//
// There is no single-precision tensor-core mode on sm_100 that keeps f32 products exact (TF32 drops
// 13 mantissa bits), so this path stays on the FP32 pipes: 128x128 output tile per CTA, 16-deep k
// slices double-buffered in shared memory, 8x8 outputs per thread.  Either operand may have k or
// its row index contiguous; both are staged k-major so the inner loop reads 128-bit vectors.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <string>

#include "runtime.hpp"
#include <cooperative_groups.h>

namespace anl {

// Unroll factor of the 16-step inner product and CTAs per SM.  Two CTAs of 128 registers per
// thread hide each other's barriers; unrolling by 2 keeps the register allocator under that cap
// without spills and measured fastest (45-50 TFLOP/s on 8192x4096x1024 against 40-47 unrolled
// fully, 34-44 with one 255-register CTA per SM).
#ifndef ANL_F32_UNROLL
#define ANL_F32_UNROLL 2
#endif
#ifndef ANL_F32_MINBLOCKS
#define ANL_F32_MINBLOCKS 2
#endif
constexpr int F_UNROLL = ANL_F32_UNROLL;
constexpr int F_BM = 128, F_BN = 128, F_BK = 16, F_THREADS = 256, F_LD = F_BM + 4;

struct GemmF32Args {
    const float* a; const float* b; float* d;
    int M, N, K;
    long long a_sm, a_sk, b_sn, b_sk;
    int ldd, tiles_m, tiles_n;
};

// Fetches this thread's 8 elements (two groups of 4) of each [128 rows x 16 k] operand slice.
// KC: the groups run along k (element (r, k) at base[r * s_r + k * s_k], s_k == 1 when VEC);
// otherwise along the row index (s_r == 1 when VEC).  The pointer walks down k by one slice per
// load, so the loop carries one pointer per operand instead of recomputing 64-bit products.
// VEC: 128-bit loads are legal (alignment and extents checked by the host), and a group is then
// either fully inside the operand or fully outside.
template <bool KC, bool VEC>
struct SliceFetch {
    const float* p;
    long long second, step, sg;    // offset of the second group, one slice along k, stride inside a group
    int kofs, fc0, fc1;            // k offset of the first group; valid elements along the fixed index

    __device__ __forceinline__ void init(const float* base, long long s_r, long long s_k, int r0, int R, int tid) {
        if (KC) {
            const int row = tid >> 2;
            kofs = (tid & 3) * 4;
            p = base + (long long)(r0 + row) * s_r + (long long)kofs * s_k;
            second = 64 * s_r; sg = s_k;
            fc0 = r0 + row < R ? 4 : 0; fc1 = r0 + row + 64 < R ? 4 : 0;
        } else {
            const int rq = (tid & 31) * 4;
            kofs = tid >> 5;
            p = base + (long long)kofs * s_k + (long long)(r0 + rq) * s_r;
            second = 8 * s_k; sg = s_r;
            fc0 = fc1 = max(0, min(4, R - (r0 + rq)));
        }
        step = F_BK * s_k;
    }

    __device__ __forceinline__ void load(int k0, int K, float (&v)[8]) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float* q = j ? p + second : p;
            const int kv = K - (k0 + kofs + (KC ? 0 : 8 * j));
            const int fc = j ? fc1 : fc0;
            const int cnt = KC ? min(fc, max(kv, 0)) : (kv > 0 ? fc : 0);
            if (VEC) {
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (cnt >= 4) x = *reinterpret_cast<const float4*>(q);
                v[j * 4 + 0] = x.x; v[j * 4 + 1] = x.y; v[j * 4 + 2] = x.z; v[j * 4 + 3] = x.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) v[j * 4 + i] = i < cnt ? q[i * sg] : 0.f;
            }
        }
        p += step;
    }
};

// Store the fetched elements k-major: slice[k][row].
template <bool KC>
__device__ __forceinline__ void stage_slice(float (*slice)[F_LD], int tid, const float (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int f = tid + j * F_THREADS;
        if (KC) {
            const int row = f >> 2, kq = (f & 3) * 4;
#pragma unroll
            for (int i = 0; i < 4; i++) slice[kq + i][row] = v[j * 4 + i];
        } else {
            const int kk = f >> 5, rq = (f & 31) * 4;
            *reinterpret_cast<float4*>(&slice[kk][rq]) = make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        }
    }
}

template <bool A_KC, bool B_KC, bool VEC>
__global__ void __launch_bounds__(F_THREADS, ANL_F32_MINBLOCKS) gemm_f32_simt(const GemmF32Args g) {
    __shared__ __align__(16) float As[2][F_BK][F_LD];
    __shared__ __align__(16) float Bs[2][F_BK][F_LD];
    const int tid = threadIdx.x;
    // tiles are numbered so that consecutive CTAs share one column panel of B and walk down M in
    // groups of 8 row tiles: the group's A panels and the B panel stay in L2 while they are reused
    const int group = 8;
    const int per_group = group * g.tiles_n;
    const int bid = blockIdx.x;
    const int g0 = (bid / per_group) * group;
    const int gsz = min(group, g.tiles_m - g0);
    const int tm = g0 + (bid % per_group) % gsz;
    const int tn = (bid % per_group) / gsz;
    const int m0 = tm * F_BM, n0 = tn * F_BN;
    const int tx = tid & 15, ty = tid >> 4;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    float ra[8], rb[8];
    const int nk = (g.K + F_BK - 1) / F_BK;
    SliceFetch<A_KC, VEC> fa;
    SliceFetch<B_KC, VEC> fb;
    fa.init(g.a, g.a_sm, g.a_sk, m0, g.M, tid);
    fb.init(g.b, g.b_sn, g.b_sk, n0, g.N, tid);
    fa.load(0, g.K, ra);
    fb.load(0, g.K, rb);
    stage_slice<A_KC>(As[0], tid, ra);
    stage_slice<B_KC>(Bs[0], tid, rb);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        if (kt + 1 < nk) {
            fa.load((kt + 1) * F_BK, g.K, ra);
            fb.load((kt + 1) * F_BK, g.K, rb);
        }
#pragma unroll F_UNROLL
        for (int k = 0; k < F_BK; k++) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            stage_slice<A_KC>(As[cur ^ 1], tid, ra);
            stage_slice<B_KC>(Bs[cur ^ 1], tid, rb);
        }
        __syncthreads();
    }
    const bool vec_out = VEC && (g.ldd & 3) == 0 && (g.N & 3) == 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= g.M) continue;
        float* drow = g.d + (long long)m * g.ldd;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int n = n0 + h * 64 + tx * 4;
            if (vec_out) {
                if (n < g.N) *reinterpret_cast<float4*>(drow + n) = make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) if (n + j < g.N) drow[n + j] = acc[i][h * 4 + j];
            }
        }
    }
}

// ── contractions with a handful of rows, or a handful of terms ─────────────────────────────────────
// The symbolic-batch MLP is replayed with batches of 1 and 17 as well as 65536.  With few rows a
// 128x128 tile is almost empty, and the generated one-block-per-output kernel reads the whole weight
// matrix once per ROW; these kernels read it once per group of up to 16 rows, which is what the
// bytes cost.  All accumulate in f32 with fused multiply-add; the order of the additions differs
// from the reference's serial loop where lanes or warps share one sum (tolerance: 1e-4 relative).
constexpr int S_MR = 16;          // most rows one pass of the k-contiguous form takes
constexpr int S_MR_AXPY = 8;      // and of the n-contiguous form

// D[m, n] = sum_k A[m, k] * B[n, k], both k-contiguous (a forward layer x · Wᵀ): a warp owns CW output
// columns, its lanes split k in 16-byte pieces; MR rows of A are staged in shared memory (16 KB:
// 4096 / MR floats of each row per pass) and shared by the block's 8 warps, so one pass over the
// weights serves MR rows.  With few column blocks the launch is a cluster of `splits` CTAs per block
// of columns, each taking a slice of k; the slices' sums are added in rank order by the first CTA
// through distributed shared memory (a fixed order: the same bits every launch).
template <int MR, int CW>
__global__ void __launch_bounds__(256) gemm_f32_few_rows_dot(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ d,
                                                              int M, int N, int K, long long a_sm, long long b_sn, int ldd, int vec, int splits) {
    namespace cg = cooperative_groups;
    constexpr int KC = 4096 / MR;
    __shared__ __align__(16) float As[MR][KC];
    __shared__ float mine[MR][8 * CW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = splits > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int nb = ((int)blockIdx.x / splits) * (8 * CW), n0 = nb + warp * CW, m0 = blockIdx.y * MR;
    const int slice = (((K + splits - 1) / splits) + 127) & ~127;
    const int ks0 = rank * slice, ks1 = (ks0 + slice) < K ? (ks0 + slice) : K;
    float acc[MR][CW];
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int c = 0; c < CW; c++) acc[m][c] = 0.0f;
    const float* brow[CW];
#pragma unroll
    for (int c = 0; c < CW; c++) brow[c] = b + (long long)(n0 + c < N ? n0 + c : N - 1) * b_sn;
    for (int k0 = ks0; k0 < ks1; k0 += KC) {
        const int kc = (ks1 - k0) < KC ? (ks1 - k0) : KC;
        const int kc4 = (kc + 3) & ~3;
        for (int i = threadIdx.x; i < MR * kc4; i += 256) {
            const int m = i / kc4, k = i - m * kc4;
            As[m][k] = (m0 + m < M && k < kc) ? a[(long long)(m0 + m) * a_sm + k0 + k] : 0.0f;
        }
        __syncthreads();
        if (vec) {
            constexpr int U = CW >= 4 ? 1 : (CW == 2 ? 2 : 4);      // 16-byte loads in flight per lane: U * CW
            for (int kk = lane * 4; kk < kc; kk += 128 * U) {
                float4 bv[U][CW];
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int c = 0; c < CW; c++)
                        bv[u][c] = (kk + u * 128 < kc) ? __ldg(reinterpret_cast<const float4*>(brow[c] + k0 + kk + u * 128)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (kk + u * 128 >= kc) break;
#pragma unroll
                    for (int m = 0; m < MR; m++) {
                        const float4 av = *reinterpret_cast<const float4*>(&As[m][kk + u * 128]);
#pragma unroll
                        for (int c = 0; c < CW; c++) {
                            acc[m][c] = fmaf(av.x, bv[u][c].x, acc[m][c]); acc[m][c] = fmaf(av.y, bv[u][c].y, acc[m][c]);
                            acc[m][c] = fmaf(av.z, bv[u][c].z, acc[m][c]); acc[m][c] = fmaf(av.w, bv[u][c].w, acc[m][c]);
                        }
                    }
                }
            }
        } else {
            for (int kk = lane; kk < kc; kk += 32) {
                float bv[CW];
#pragma unroll
                for (int c = 0; c < CW; c++) bv[c] = brow[c][k0 + kk];
#pragma unroll
                for (int m = 0; m < MR; m++)
#pragma unroll
                    for (int c = 0; c < CW; c++) acc[m][c] = fmaf(As[m][kk], bv[c], acc[m][c]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int c = 0; c < CW; c++) {
            float v = acc[m][c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                if (splits > 1) mine[m][warp * CW + c] = v;
                else if (n0 + c < N && m0 + m < M) d[(long long)(m0 + m) * ldd + n0 + c] = v;
            }
        }
    if (splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (rank == 0) {
            for (int i = threadIdx.x; i < MR * 8 * CW; i += 256) {
                const int m = i / (8 * CW), c = i - m * (8 * CW);
                float v = 0.0f;
                for (int r = 0; r < splits; r++) v += cluster.map_shared_rank(&mine[0][0], r)[i];
                if (m0 + m < M && nb + c < N) d[(long long)(m0 + m) * ldd + nb + c] = v;
            }
        }
        cluster.sync();           // the other CTAs' shared memory stays until the first has read it
    }
}

// D[m, n] = sum_k A[m, k] * B[k, n]: A k-contiguous, B n-contiguous (an input gradient dY · W).
// A cluster of 8 CTAs owns 128 columns and splits k eight ways, so that a matrix of a few thousand
// columns still spreads over every SM; inside a CTA the 8 warps take every 8th k of the slice, each
// lane four columns.  The warps' partial sums are added in warp order through shared memory, the
// CTAs' in rank order through distributed shared memory by the cluster's first CTA: a fixed order,
// the same bits every launch.
constexpr int S_KA = 128;         // k chunk of the n-contiguous form
constexpr int S_KSPLIT = 8;
template <int MR>
__global__ void __cluster_dims__(S_KSPLIT, 1, 1) __launch_bounds__(256)
gemm_f32_few_rows_axpy(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ d,
                       int M, int N, int K, long long a_sm, long long b_sk, int ldd, int vec) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float As[MR][S_KA];
    __shared__ __align__(16) float part[8][MR][128];
    __shared__ __align__(16) float mine[MR][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster.block_rank();
    const int n0 = (blockIdx.x / S_KSPLIT) * 128, m0 = blockIdx.y * MR;
    const int c0 = n0 + lane * 4;
    const int slice = (((K + S_KSPLIT - 1) / S_KSPLIT) + 7) & ~7;
    const int ks0 = rank * slice, ks1 = (ks0 + slice) < K ? (ks0 + slice) : K;
    float acc[MR][4];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;
    for (int k0 = ks0; k0 < ks1; k0 += S_KA) {
        const int kend = (ks1 - k0) < S_KA ? (ks1 - k0) : S_KA;
        for (int i = threadIdx.x; i < MR * S_KA; i += 256) {
            const int m = i / S_KA, k = i % S_KA;
            As[m][k] = (m0 + m < M && k < kend) ? a[(long long)(m0 + m) * a_sm + k0 + k] : 0.0f;
        }
        __syncthreads();
        for (int k = warp; k < kend; k += 32) {
            // four rows of B in flight per lane
            float4 bv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int kr = k + u * 8;
                bv[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (kr < kend) {
                    const float* brow = b + (long long)(k0 + kr) * b_sk + c0;
                    if (vec) { if (c0 < N) bv[u] = __ldg(reinterpret_cast<const float4*>(brow)); }
                    else {
                        if (c0 < N) bv[u].x = brow[0];
                        if (c0 + 1 < N) bv[u].y = brow[1];
                        if (c0 + 2 < N) bv[u].z = brow[2];
                        if (c0 + 3 < N) bv[u].w = brow[3];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int kr = k + u * 8;
                if (kr >= kend) break;
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    const float av = As[m][kr];
                    acc[m][0] = fmaf(av, bv[u].x, acc[m][0]); acc[m][1] = fmaf(av, bv[u].y, acc[m][1]);
                    acc[m][2] = fmaf(av, bv[u].z, acc[m][2]); acc[m][3] = fmaf(av, bv[u].w, acc[m][3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < MR; m++) *reinterpret_cast<float4*>(&part[warp][m][lane * 4]) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    __syncthreads();
    for (int i = threadIdx.x; i < MR * 128; i += 256) {
        const int m = i >> 7, c = i & 127;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++) v += part[w][m][c];
        mine[m][c] = v;
    }
    cluster.sync();
    if (rank == 0) {
        for (int i = threadIdx.x; i < MR * 128; i += 256) {
            const int m = i >> 7, c = i & 127;
            float v = 0.0f;
#pragma unroll
            for (int r = 0; r < S_KSPLIT; r++) v += cluster.map_shared_rank(&mine[0][0], r)[m * 128 + c];
            if (m0 + m < M && n0 + c < N) d[(long long)(m0 + m) * ldd + n0 + c] = v;
        }
    }
    cluster.sync();               // the other CTAs' shared memory stays until the first has read it
}

// D[m, n] = sum_k A[k, m] * B[k, n] with few terms (a weight gradient at a small batch): every thread
// four consecutive columns of one row, the terms added in ascending k like the reference's loop.
__global__ void __launch_bounds__(256) gemm_f32_few_terms(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ d,
                                                           int M, int N, int K, long long a_sk, long long b_sk, int ldd, int vec) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int n4 = (N + 3) / 4;
    const long long m = t / n4;
    const int n = (int)(t % n4) * 4;
    if (m >= M) return;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int k = 0; k < K; k++) {
        const float av = a[(long long)k * a_sk + m];
        const float* brow = b + (long long)k * b_sk + n;
        if (vec) {
            const float4 bv = *reinterpret_cast<const float4*>(brow);
            acc[0] = fmaf(av, bv.x, acc[0]); acc[1] = fmaf(av, bv.y, acc[1]); acc[2] = fmaf(av, bv.z, acc[2]); acc[3] = fmaf(av, bv.w, acc[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) if (n + j < N) acc[j] = fmaf(av, brow[j], acc[j]);
        }
    }
    float* out = d + m * ldd + n;
    if (vec) *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else for (int j = 0; j < 4; j++) if (n + j < N) out[j] = acc[j];
}

// Which hand-written kernel, if any, finishes a contraction of these extents and strides sooner than
// the generated one-thread-per-output kernel.
enum F32Route { F32_NONE = 0, F32_TILED, F32_FEW_ROWS_DOT, F32_FEW_ROWS_AXPY, F32_FEW_TERMS };
static F32Route f32_route(int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk) {
    if (M <= 0 || N <= 0 || K <= 0) return F32_NONE;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return F32_NONE;
    if (M <= 2 * S_MR && N >= 256 && K >= 128 && (a_sk == 1 || M == 1)) {
        if (b_sk == 1) return F32_FEW_ROWS_DOT;
        if (b_sn == 1) return F32_FEW_ROWS_AXPY;
    }
    if (K <= 64 && a_sm == 1 && b_sn == 1 && M * N >= (1 << 16)) return F32_FEW_TERMS;
    const int64_t tiles = ((M + F_BM - 1) / F_BM) * ((N + F_BN - 1) / F_BN);
    if (M > 2 * S_MR && tiles >= 16 && K >= 64 && tiles < (1ll << 31)) return F32_TILED;
    return F32_NONE;
}
// f32 contractions of more than a few rows are worth the tensor cores in 3 x TF32 form (gemm.cu):
// below 33 rows the few-row kernels above read the other operand once and are bound by that; from
// there on even a mostly empty 256-row tile beats the FP32 pipes.  Operands must be contiguous along
// k or along their row index.
bool gemm_tf32_shape_ok(int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk) {
    if (M <= 2 * S_MR || N < 128 || K < 64) return false;
    if (K <= 64 && a_sm == 1 && b_sn == 1) return false;       // the few-terms kernel: bound by writing the output
    if ((double)M * (double)N * (double)K < 6.4e7) return false;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return false;
    return (a_sk == 1 || a_sm == 1) && (b_sk == 1 || b_sn == 1);
}
bool gemm_f32_worth(int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk) {
    return f32_route(M, N, K, a_sm, a_sk, b_sn, b_sk) != F32_NONE || gemm_tf32_shape_ok(M, N, K, a_sm, a_sk, b_sn, b_sk);
}

int launch_gemm_f32(anl_device* dev, const float* a, const float* b, float* d, int64_t M, int64_t N, int64_t K,
                    int64_t a_sm, int64_t a_sk, int64_t b_sn, int64_t b_sk, cudaStream_t stream) {
    const F32Route route = f32_route(M, N, K, a_sm, a_sk, b_sn, b_sk);
    if (route == F32_FEW_ROWS_DOT || route == F32_FEW_ROWS_AXPY || route == F32_FEW_TERMS) {
        auto pick = [](int64_t rows, int most) { int r = 1; while (r < rows && r < most) r *= 2; return r; };
        auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
        if (route == F32_FEW_ROWS_DOT) {
            const int mr = pick(M, S_MR), groups = (int)((M + mr - 1) / mr);
            const int vec = al16(b) && b_sn % 4 == 0 && K % 4 == 0;
            const int cw = mr >= 8 ? 4 : (mr == 4 ? 2 : 1);
            const int colblocks = (int)((N + 8 * cw - 1) / (8 * cw));
            // enough CTAs for two per SM, by splitting k across a cluster while a slice stays 256 long
            int splits = 1;
            while (splits < 8 && (int64_t)colblocks * groups * splits < 2 * dev->prop.multiProcessorCount && K / (splits * 2) >= 256) splits *= 2;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3((unsigned)(colblocks * splits), (unsigned)groups, 1);
            cfg.blockDim = dim3(256, 1, 1);
            cfg.stream = stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = (unsigned)splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            const int Mi = (int)M, Ni = (int)N, Ki = (int)K, ldd = (int)N;
            cudaError_t le = cudaSuccess;
#define ANL_DOT(R, C) le = cudaLaunchKernelEx(&cfg, gemm_f32_few_rows_dot<R, C>, a, b, d, Mi, Ni, Ki, (long long)a_sm, (long long)b_sn, ldd, vec, splits)
            switch (mr) { case 1: ANL_DOT(1, 1); break; case 2: ANL_DOT(2, 1); break; case 4: ANL_DOT(4, 2); break; case 8: ANL_DOT(8, 4); break; default: ANL_DOT(16, 4); }
#undef ANL_DOT
            if (le != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm f32: launch: ") + cudaGetErrorString(le));
        } else if (route == F32_FEW_ROWS_AXPY) {
            const int mr = pick(M, S_MR_AXPY), groups = (int)((M + mr - 1) / mr);
            const int vec = al16(b) && b_sk % 4 == 0 && N % 4 == 0;
            const dim3 grid((unsigned)(S_KSPLIT * ((N + 127) / 128)), groups);
#define ANL_AXPY(R) gemm_f32_few_rows_axpy<R><<<grid, 256, 0, stream>>>(a, b, d, (int)M, (int)N, (int)K, a_sm, b_sk, (int)N, vec)
            switch (mr) { case 1: ANL_AXPY(1); break; case 2: ANL_AXPY(2); break; case 4: ANL_AXPY(4); break; default: ANL_AXPY(8); }
#undef ANL_AXPY
        }
        else {
            const int vec4 = (N % 4 == 0) && (b_sk % 4 == 0) && (((uintptr_t)b & 15) == 0) && (((uintptr_t)d & 15) == 0);
            const long long threads = M * ((N + 3) / 4);
            gemm_f32_few_terms<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(a, b, d, (int)M, (int)N, (int)K, a_sk, b_sk, (int)N, vec4);
        }
        cudaError_t e0 = cudaGetLastError();
        if (e0 != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm f32: launch: ") + cudaGetErrorString(e0));
        dev->stats.kernels_launched++;
        dev->stats.gemm_launched++;
        return ANL_OK;
    }
    GemmF32Args g;
    g.a = a; g.b = b; g.d = d;
    g.M = (int)M; g.N = (int)N; g.K = (int)K;
    g.a_sm = a_sm; g.a_sk = a_sk; g.b_sn = b_sn; g.b_sk = b_sk;
    g.ldd = (int)N;
    g.tiles_m = (int)((M + F_BM - 1) / F_BM); g.tiles_n = (int)((N + F_BN - 1) / F_BN);
    // staged "k contiguous" unless the row index is the contiguous one; an operand with neither
    // contiguous still works through the scalar loads of the k-contiguous form
    const bool a_kc = a_sm != 1 || M == 1, b_kc = b_sn != 1;
    auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    // 128-bit loads: aligned bases, the strided index a multiple of 4 elements, and the contiguous
    // extent a multiple of 4 so that no vector straddles the edge
    bool vec = al16(a) && al16(b) && al16(d);
    vec = vec && (a_kc ? (a_sk == 1 && a_sm % 4 == 0 && K % 4 == 0) : (a_sk % 4 == 0 && M % 4 == 0));
    vec = vec && (b_kc ? (b_sk == 1 && b_sn % 4 == 0 && K % 4 == 0) : (b_sk % 4 == 0 && N % 4 == 0));
    const unsigned grid = (unsigned)(g.tiles_m * g.tiles_n);
#define ANL_F32_LAUNCH(AK, BK_, V) gemm_f32_simt<AK, BK_, V><<<grid, F_THREADS, 0, stream>>>(g)
    if (vec) {
        if (a_kc && b_kc) ANL_F32_LAUNCH(true, true, true);
        else if (a_kc) ANL_F32_LAUNCH(true, false, true);
        else if (b_kc) ANL_F32_LAUNCH(false, true, true);
        else ANL_F32_LAUNCH(false, false, true);
    } else {
        if (a_kc && b_kc) ANL_F32_LAUNCH(true, true, false);
        else if (a_kc) ANL_F32_LAUNCH(true, false, false);
        else if (b_kc) ANL_F32_LAUNCH(false, true, false);
        else ANL_F32_LAUNCH(false, false, false);
    }
#undef ANL_F32_LAUNCH
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return dev->fail(ANL_ERR_CUDA, std::string("gemm f32: launch: ") + cudaGetErrorString(e));
    dev->stats.kernels_launched++;
    dev->stats.gemm_launched++;
    return ANL_OK;
}

}  // namespace anl
