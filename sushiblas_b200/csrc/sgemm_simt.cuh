// sgemm_simt.cuh -- fp32 FFMA tiled SGEMM for sm_100a (CUDA cores, no tensor cores).
//
// Serves the shapes that cannot fill a tcgen05 tile (the reference's own tests are 2x2,
// 3x3, 8x8 and 32x32: tests/blas/level3/test_gemm.cpp:39-88,
// tests/runtime/test_dependency_stress.cpp:17-18,67-68), arbitrary leading dimensions and
// alignments, and gives the "FP32 SIMT" data point next to the 3xTF32 kernel.
// Arithmetic: exact fp32 products, fp32 accumulation in k order within a thread -- the
// same class of result as the sgemm the reference forwards to (gemm.cpp:58,63).
//
// Data layout: row-major, op(A) is m x k, op(B) is k x n; a CTA owns one BM x BN tile of one
// batch entry; 256 threads, each a (TM x TN) register block split in groups of 4 so that
// every shared-memory read is a conflict-free 128-bit access.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "activation.cuh"

namespace sushi {

struct SimtGemmArgs
{
    const float* a; const float* b; float* c;
    int64_t m, n, k;
    int64_t lda, ldb, ldc;
    int64_t stride_a, stride_b, stride_c;
    int64_t tiles_m, tiles_n;
    float alpha, beta;
    int act;             // epilogue activation (ACT_* of activation.cuh) applied to alpha*acc + beta*C
    float act_param;     // its parameter (leaky_relu, elu)
    int tri;             // 0: full C; 1: only row >= col is written (lower triangle); 2: only row <= col (upper)
};

constexpr int SIMT_THREADS = 256;
constexpr int SIMT_BK = 16;

// Loads one R x BK operand tile into registers.  KC: k is the contiguous index in memory.
template <int R, bool KC>
__device__ __forceinline__ void simt_load_tile(float (&reg)[R * SIMT_BK / SIMT_THREADS],
                                               const float* __restrict__ base, int64_t ld,
                                               int64_t r0, int64_t rmax, int64_t k0, int64_t kmax, int t)
{
    constexpr int PER = R * SIMT_BK / SIMT_THREADS;
#pragma unroll
    for (int j = 0; j < PER; ++j)
    {
        int r, kk;
        if (KC) { kk = t % SIMT_BK; r = t / SIMT_BK + (SIMT_THREADS / SIMT_BK) * j; }
        else    { r = t % R;        kk = t / R + (SIMT_THREADS / R) * j; }
        int64_t gr = r0 + r, gk = k0 + kk;
        float v = 0.0f;
        if (gr < rmax && gk < kmax)
            v = KC ? __ldg(base + gr * ld + gk) : __ldg(base + gk * ld + gr);
        reg[j] = v;
    }
}

template <int R, bool KC>
__device__ __forceinline__ void simt_store_tile(float (*smem)[R + 4],
                                                const float (&reg)[R * SIMT_BK / SIMT_THREADS], int t)
{
    constexpr int PER = R * SIMT_BK / SIMT_THREADS;
#pragma unroll
    for (int j = 0; j < PER; ++j)
    {
        int r, kk;
        if (KC) { kk = t % SIMT_BK; r = t / SIMT_BK + (SIMT_THREADS / SIMT_BK) * j; }
        else    { r = t % R;        kk = t / R + (SIMT_THREADS / R) * j; }
        smem[kk][r] = reg[j];
    }
}

// One BM x BN tile (tm, tn) of batch entry bi.  TA / TB: op(A) = A^T / op(B) = B^T.
// BM == BN in {64, 128}; TM == TN == BM / 16.  As / Bs: shared-memory staging of the caller.
template <int BM, int BN, bool TA, bool TB>
__device__ __forceinline__ void simt_gemm_tile(const SimtGemmArgs& p, int64_t tm, int64_t tn, int64_t bi,
                                               float (*As)[BM + 4], float (*Bs)[BN + 4])
{
    constexpr int TM = BM / 16, TN = BN / 16;
    constexpr int GM = TM / 4, GN = TN / 4;
    const int t = threadIdx.x;
    const int tx = t % 16, ty = t / 16;

    const float* __restrict__ A = p.a + bi * p.stride_a;
    const float* __restrict__ B = p.b + bi * p.stride_b;
    float* __restrict__ C = p.c + bi * p.stride_c;
    const int64_t m0 = tm * BM, n0 = tn * BN;
    // triangular output: a tile wholly outside the triangle has nothing to do (uniform per CTA)
    if (p.tri == 1 && n0 > m0 + BM - 1) return;
    if (p.tri == 2 && m0 > n0 + BN - 1) return;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    float ra[BM * SIMT_BK / SIMT_THREADS], rb[BN * SIMT_BK / SIMT_THREADS];
    // op(A)(i,kk): !TA -> A[i*lda+kk] (k contiguous); TA -> A[kk*lda+i] (row contiguous)
    simt_load_tile<BM, !TA>(ra, A, p.lda, m0, p.m, 0, p.k, t);
    // op(B)(kk,j): !TB -> B[kk*ldb+j] (n contiguous); TB -> B[j*ldb+kk] (k contiguous)
    simt_load_tile<BN, TB>(rb, B, p.ldb, n0, p.n, 0, p.k, t);

    for (int64_t k0 = 0; k0 < p.k; k0 += SIMT_BK)
    {
        simt_store_tile<BM, !TA>(As, ra, t);
        simt_store_tile<BN, TB>(Bs, rb, t);
        __syncthreads();
        if (k0 + SIMT_BK < p.k)
        {
            simt_load_tile<BM, !TA>(ra, A, p.lda, m0, p.m, k0 + SIMT_BK, p.k, t);
            simt_load_tile<BN, TB>(rb, B, p.ldb, n0, p.n, k0 + SIMT_BK, p.k, t);
        }
#pragma unroll
        for (int kk = 0; kk < SIMT_BK; ++kk)
        {
            float av[TM], bv[TN];
#pragma unroll
            for (int g = 0; g < GM; ++g)
            {
                float4 v = *reinterpret_cast<const float4*>(&As[kk][g * (BM / GM) + ty * 4]);
                av[g * 4 + 0] = v.x; av[g * 4 + 1] = v.y; av[g * 4 + 2] = v.z; av[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < GN; ++g)
            {
                float4 v = *reinterpret_cast<const float4*>(&Bs[kk][g * (BN / GN) + tx * 4]);
                bv[g * 4 + 0] = v.x; bv[g * 4 + 1] = v.y; bv[g * 4 + 2] = v.z; bv[g * 4 + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

    // Epilogue: alpha * acc + beta * C; C is not read when beta == 0.
    const bool vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i)
    {
        const int64_t row = m0 + (i / 4) * (BM / GM) + ty * 4 + (i % 4);
        if (row >= p.m) continue;
#pragma unroll
        for (int g = 0; g < GN; ++g)
        {
            const int64_t col = n0 + g * (BN / GN) + tx * 4;
            if (col >= p.n) continue;
            float* dst = C + row * p.ldc + col;
            // triangular output: 4 columns wholly inside -> vector path; straddling -> per element
            const bool tri_all = p.tri == 0 || (p.tri == 1 ? col + 3 <= row : col >= row);
            if (vec_ok && col + 3 < p.n && tri_all)
            {
                float4 o;
                o.x = p.alpha * acc[i][g * 4 + 0]; o.y = p.alpha * acc[i][g * 4 + 1];
                o.z = p.alpha * acc[i][g * 4 + 2]; o.w = p.alpha * acc[i][g * 4 + 3];
                if (p.beta != 0.0f)
                {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    o.x = fmaf(p.beta, old.x, o.x); o.y = fmaf(p.beta, old.y, o.y);
                    o.z = fmaf(p.beta, old.z, o.z); o.w = fmaf(p.beta, old.w, o.w);
                }
                if (p.act)
                {
                    o.x = apply_act(o.x, p.act, p.act_param); o.y = apply_act(o.y, p.act, p.act_param);
                    o.z = apply_act(o.z, p.act, p.act_param); o.w = apply_act(o.w, p.act, p.act_param);
                }
                *reinterpret_cast<float4*>(dst) = o;
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const bool inside = p.tri == 0 || (p.tri == 1 ? col + j <= row : col + j >= row);
                    if (col + j < p.n && inside)
                    {
                        float o = p.alpha * acc[i][g * 4 + j];
                        if (p.beta != 0.0f) o = fmaf(p.beta, dst[j], o);
                        dst[j] = apply_act(o, p.act, p.act_param);
                    }
                }
            }
        }
    }
}

template <int BM, int BN, bool TA, bool TB>
__global__ void __launch_bounds__(SIMT_THREADS)
sgemm_simt_kernel(const SimtGemmArgs p)
{
    __shared__ __align__(16) float As[SIMT_BK][BM + 4];
    __shared__ __align__(16) float Bs[SIMT_BK][BN + 4];
    int64_t tile = blockIdx.x;
    const int64_t tn = tile % p.tiles_n; tile /= p.tiles_n;
    const int64_t tm = tile % p.tiles_m;
    const int64_t bi = tile / p.tiles_m;
    simt_gemm_tile<BM, BN, TA, TB>(p, tm, tn, bi, As, Bs);
}

// Grouped launch: many independent small GEMMs in one grid.  Problem i owns the tiles
// [first_tile, first_tile + tiles_m*tiles_n*batch) of the grid (64 x 64 tiles).
struct GroupedGemm
{
    SimtGemmArgs g;
    int32_t trans_a, trans_b;
    int64_t first_tile;
};

__global__ void __launch_bounds__(SIMT_THREADS)
sgemm_grouped_simt_kernel(const GroupedGemm* __restrict__ problems, int count)
{
    __shared__ __align__(16) float As[SIMT_BK][64 + 4];
    __shared__ __align__(16) float Bs[SIMT_BK][64 + 4];
    __shared__ GroupedGemm prob;
    if (threadIdx.x == 0)
    {
        // last problem whose first tile is <= this CTA's tile
        const int64_t t = blockIdx.x;
        int lo = 0, hi = count - 1;
        while (lo < hi)
        {
            const int mid = (lo + hi + 1) >> 1;
            if (problems[mid].first_tile <= t) lo = mid; else hi = mid - 1;
        }
        prob = problems[lo];
    }
    __syncthreads();
    int64_t tile = (int64_t)blockIdx.x - prob.first_tile;
    const int64_t tn = tile % prob.g.tiles_n; tile /= prob.g.tiles_n;
    const int64_t tm = tile % prob.g.tiles_m;
    const int64_t bi = tile / prob.g.tiles_m;
    if (!prob.trans_a && !prob.trans_b) simt_gemm_tile<64, 64, false, false>(prob.g, tm, tn, bi, As, Bs);
    else if (!prob.trans_a) simt_gemm_tile<64, 64, false, true>(prob.g, tm, tn, bi, As, Bs);
    else if (!prob.trans_b) simt_gemm_tile<64, 64, true, false>(prob.g, tm, tn, bi, As, Bs);
    else simt_gemm_tile<64, 64, true, true>(prob.g, tm, tn, bi, As, Bs);
}

// C <- beta * C (k == 0 or alpha == 0): no operand is read.  One thread per element.
// act != 0 additionally applies that activation.
__global__ void scale_c_kernel(float* c, int64_t m, int64_t n, int64_t ldc, int64_t stride_c,
                               int64_t batch, float beta, int act = 0, float act_param = 0.0f)
{
    const int64_t total = m * n * batch;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
    {
        const int64_t col = i % n;
        const int64_t row = (i / n) % m;
        const int64_t bi = i / (n * m);
        float* dst = c + bi * stride_c + row * ldc + col;
        float v = (beta == 0.0f) ? 0.0f : beta * (*dst);
        *dst = apply_act(v, act, act_param);
    }
}

template <int BT>
inline cudaError_t launch_simt_tile(const SimtGemmArgs& a0, bool ta, bool tb, int64_t batch, cudaStream_t st)
{
    SimtGemmArgs a = a0;
    a.tiles_m = (a.m + BT - 1) / BT;
    a.tiles_n = (a.n + BT - 1) / BT;
    const int64_t blocks = a.tiles_m * a.tiles_n * batch;
    if (blocks <= 0) return cudaSuccess;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    dim3 grid((unsigned)blocks), block(SIMT_THREADS);
    if (!ta && !tb) sgemm_simt_kernel<BT, BT, false, false><<<grid, block, 0, st>>>(a);
    else if (!ta && tb) sgemm_simt_kernel<BT, BT, false, true><<<grid, block, 0, st>>>(a);
    else if (ta && !tb) sgemm_simt_kernel<BT, BT, true, false><<<grid, block, 0, st>>>(a);
    else sgemm_simt_kernel<BT, BT, true, true><<<grid, block, 0, st>>>(a);
    return cudaGetLastError();
}

// Picks the 128-tile when it yields at least one wave of CTAs, else the 64-tile.
inline cudaError_t launch_sgemm_simt(const SimtGemmArgs& a, bool ta, bool tb, int64_t batch,
                                     int sm_count, cudaStream_t st)
{
    const int64_t big = ((a.m + 127) / 128) * ((a.n + 127) / 128) * batch;
    if (big >= sm_count) return launch_simt_tile<128>(a, ta, tb, batch, st);
    return launch_simt_tile<64>(a, ta, tb, batch, st);
}

} // namespace sushi
