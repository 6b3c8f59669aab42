// dgemm_mma.cuh -- fp64 GEMM for sm_100a on the FP64 tensor-core instruction (DMMA m16n8k8).
//
// Serves the FLOAT64 branch of the reference's GEMM front-end (src/ops/blas/level3/gemm.cpp:158-169,
// forwarding to oneapi::mkl::blas::{row,column}_major::gemm[_batch]<double>).  Blackwell's tcgen05
// family has no fp64 kind; fp64 matrix math runs on `mma.sync.m16n8k8.f64`, whose rate on this part
// equals the FP64 FMA rate (128 flop / clk / SM), so the kernel is bound by that pipe (not by
// memory: a 128 x 128 tile moves 32 KB per 16-k step for 0.5 MFLOP).  Arithmetic: exact fp64
// products accumulated in fp64.
//
// A CTA owns one BT x BT tile of one batch entry (BT = 128, or 64 when that fills more SMs);
// 16 warps as 4 (m) x 4 (n), each a (BT/4) x (BT/4) block of 16 x 8 accumulator fragments (the
// 128 x 128 fp64 accumulator is half of the SM's register file, so one CTA per SM).  Operand
// tiles travel global -> shared memory with cp.async (16-byte copies, 8-byte ones for operands
// that are not 16-byte aligned; out-of-range elements are zero-filled by the copy) through a
// ring of four stages guarded by full / empty mbarriers: every thread issues its share of the
// tile three steps ahead and lets the copies' completion arrive on the stage's full barrier,
// every warp releases a stage on its empty barrier after its last fragment load.  No register
// staging and no CTA-wide barrier in the main loop: measured, those cost 15 % and 8 % of the
// DMMA rate.  Every barrier wait is bounded (status word + CTA abort flag, as in the fp32
// kernel).  Two shared-memory layouts, chosen by which index is contiguous in global memory,
// both read conflict-free by the fragment pattern (row = lane / 4, k = lane % 4 (+ 4)):
//     k contiguous:   [row][16 + 4]        (row stride 160 B: four rows cover all 32 banks)
//     row contiguous: [k][BT + 4]          (k stride = 32 B mod 128 B)
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>

namespace sushi {

struct DgemmArgs
{
    const double* a; const double* b; double* c;
    int64_t m, n, k;
    int64_t lda, ldb, ldc;
    int64_t stride_a, stride_b, stride_c;
    int64_t tiles_m, tiles_n;
    double alpha, beta;
    int* status;          // device word for expired bounded waits (may be null)
};

constexpr int DG_THREADS = 512;
constexpr int DG_BK = 16;
constexpr int DG_KSTRIDE = DG_BK + 4;      // doubles per row of a k-contiguous tile
constexpr int DG_STAGES = 4;
constexpr int DG_ST_TIMEOUT_FULL = 21, DG_ST_TIMEOUT_EMPTY = 22;   // status codes of expired waits
constexpr unsigned long long DG_WAIT_LIMIT_NS = 1000000000ull;

template <int R, bool KC>
struct DgTile
{
    static constexpr int P = R * DG_BK / DG_THREADS;                   // doubles per thread per tile
    static constexpr int RS = KC ? DG_KSTRIDE : 1;                     // element (r, kk) lives at r * RS + kk * KS
    static constexpr int KS = KC ? 1 : R + 4;
    static constexpr int SIZE = KC ? R * DG_KSTRIDE : DG_BK * (R + 4); // doubles of shared memory
    __host__ __device__ static constexpr int index(int r, int kk) { return r * RS + kk * KS; }
};

// Shared-memory accesses by 32-bit shared-window address with a compile-time byte offset: no
// per-access address arithmetic in the main loop.
template <int BYTES>
__device__ __forceinline__ double dg_lds(uint32_t addr)
{
    double v;
    asm volatile("ld.shared.f64 %0, [%1+%2];" : "=d"(v) : "r"(addr), "n"(BYTES));
    return v;
}

__device__ __forceinline__ void dg_cp_async16(uint32_t dst, const double* src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void dg_cp_async8(uint32_t dst, const double* src, uint32_t src_bytes)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The executing thread's earlier cp.async copies arrive on the barrier when they have landed.
__device__ __forceinline__ void dg_cp_async_arrive(uint32_t bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void dg_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Issues this thread's share of one R x 16 operand tile per call, 16 k further each time.
// KC: element (r, kk) = base[r * ld + kk], else base[kk * ld + r].  A thread owns P = R / 32
// contiguous doubles of every tile (its valid elements are a prefix of them); elements outside
// the matrix are zero-filled (source size 0, source pointer parked on the operand base).
template <int R, bool KC>
struct DgAsyncLoader
{
    static constexpr int P = DgTile<R, KC>::P;
    static constexpr int TPR = R / P;                                  // threads along the row index (row-contiguous tiles)
    const double* ptr;       // this thread's first element of the next tile
    const double* safe;      // a valid address for zero-size copies
    int64_t step;            // elements between consecutive tiles
    int64_t k_next, kmax;
    int64_t outer, inner0, inner_max;   // KC -> (row, k offset in tile, -); !KC -> (k offset in tile, row, rows)
    bool vec_ok, rows_all, rows_any;

    __device__ __forceinline__ void init(const double* base, int64_t ld, int64_t r0, int64_t rmax, int64_t k_limit, int t, bool vec)
    {
        vec_ok = vec; kmax = k_limit; k_next = 0; safe = base;
        if (KC)
        {
            outer = r0 + t / (16 / P); inner0 = (t % (16 / P)) * P; inner_max = 0;
            ptr = base + outer * ld + inner0; step = DG_BK;
            rows_all = rows_any = outer < rmax;
        }
        else
        {
            outer = t / TPR; inner0 = r0 + (t % TPR) * P; inner_max = rmax;
            ptr = base + outer * ld + inner0; step = DG_BK * ld;
            rows_all = inner0 + P <= rmax; rows_any = inner0 < rmax;
        }
    }

    __device__ __forceinline__ bool valid(int j) const
    {
        return KC ? (rows_any && k_next + inner0 + j < kmax) : (k_next + outer < kmax && inner0 + j < inner_max);
    }

    // dst: shared-window address of this thread's P doubles in the target stage
    __device__ __forceinline__ void issue(uint32_t dst)
    {
        if (vec_ok)
        {
            if (rows_all && k_next + DG_BK <= kmax)
            {
#pragma unroll
                for (int j = 0; j < P; j += 2) dg_cp_async16(dst + 8 * j, ptr + j, 16);
            }
            else
            {
#pragma unroll
                for (int j = 0; j < P; j += 2)
                {
                    const uint32_t bytes = valid(j) ? (valid(j + 1) ? 16u : 8u) : 0u;
                    dg_cp_async16(dst + 8 * j, bytes ? ptr + j : safe, bytes);
                }
            }
        }
        else
        {
#pragma unroll
            for (int j = 0; j < P; ++j)
            {
                const bool ok = valid(j);
                dg_cp_async8(dst + 8 * j, ok ? ptr + j : safe, ok ? 8u : 0u);
            }
        }
        ptr += step; k_next += DG_BK;
    }
};

// Offset (doubles) of a thread's P contiguous, 16-byte aligned doubles inside a tile.
template <int R, bool KC>
__device__ __forceinline__ int dg_store_offset(int t)
{
    constexpr int P = DgTile<R, KC>::P;
    return KC ? DgTile<R, KC>::index(t / (16 / P), (t % (16 / P)) * P) : DgTile<R, KC>::index((t % (R / P)) * P, t / (R / P));
}

// Fragment loads of one k8 step: B fragments of all NB column blocks, A fragments of row block I.
template <typename Tile, int NB, int KS8>
__device__ __forceinline__ void dg_load_b(uint32_t at, double (&bv)[NB][2])
{
    bv[0][0] = dg_lds<8 * Tile::index(0, KS8 * 8)>(at);
    bv[0][1] = dg_lds<8 * Tile::index(0, KS8 * 8 + 4)>(at);
    bv[1][0] = dg_lds<8 * Tile::index(8, KS8 * 8)>(at);
    bv[1][1] = dg_lds<8 * Tile::index(8, KS8 * 8 + 4)>(at);
    if constexpr (NB == 4)
    {
        bv[2][0] = dg_lds<8 * Tile::index(16, KS8 * 8)>(at);
        bv[2][1] = dg_lds<8 * Tile::index(16, KS8 * 8 + 4)>(at);
        bv[3][0] = dg_lds<8 * Tile::index(24, KS8 * 8)>(at);
        bv[3][1] = dg_lds<8 * Tile::index(24, KS8 * 8 + 4)>(at);
    }
}

template <typename Tile, int I, int KS8>
__device__ __forceinline__ void dg_load_a(uint32_t at, double (&av)[4])
{
    av[0] = dg_lds<8 * Tile::index(I * 16, KS8 * 8)>(at);
    av[1] = dg_lds<8 * Tile::index(I * 16 + 8, KS8 * 8)>(at);
    av[2] = dg_lds<8 * Tile::index(I * 16, KS8 * 8 + 4)>(at);
    av[3] = dg_lds<8 * Tile::index(I * 16 + 8, KS8 * 8 + 4)>(at);
}

__device__ __forceinline__ void dmma_m16n8k8(double (&d)[4], const double (&a)[4], const double (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+d"(d[0]), "+d"(d[1]), "+d"(d[2]), "+d"(d[3])
                 : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

// One k8 step of a warp: MB x NB fragments.
template <typename TileA, typename TileB, int MB, int NB, int KS8>
__device__ __forceinline__ void dg_k8_step(uint32_t a_at, uint32_t b_at, double (&acc)[MB][NB][4])
{
    double bv[NB][2];
    dg_load_b<TileB, NB, KS8>(b_at, bv);
    double av[4];
    dg_load_a<TileA, 0, KS8>(a_at, av);
#pragma unroll
    for (int j = 0; j < NB; ++j) dmma_m16n8k8(acc[0][j], av, bv[j]);
    if constexpr (MB == 2)
    {
        dg_load_a<TileA, 1, KS8>(a_at, av);
#pragma unroll
        for (int j = 0; j < NB; ++j) dmma_m16n8k8(acc[1][j], av, bv[j]);
    }
}

template <int BT, bool TA, bool TB>
__global__ void __launch_bounds__(DG_THREADS, 1)
dgemm_mma_kernel(const DgemmArgs p)
{
    // op(A)(i, kk): !TA -> A[i*lda + kk] (k contiguous); TA -> A[kk*lda + i] (row contiguous)
    // op(B)(kk, j): !TB -> B[kk*ldb + j] (column contiguous); TB -> B[j*ldb + kk] (k contiguous)
    using TileA = DgTile<BT, !TA>;
    using TileB = DgTile<BT, TB>;
    constexpr int MB = BT / 64, NB = BT / 32;            // per warp: MB 16-row blocks down, NB 8-column blocks across
    extern __shared__ __align__(16) double dg_smem[];     // DG_STAGES x (A tile | B tile), then the barriers

    const int t = threadIdx.x, lane = t % 32, warp = t / 32;
    const int wm = warp / 4, wn = warp % 4;
    const int gid = lane / 4, tig = lane % 4;
    int64_t tile = blockIdx.x;
    const int64_t tn = tile % p.tiles_n; tile /= p.tiles_n;
    const int64_t tm = tile % p.tiles_m;
    const int64_t bi = tile / p.tiles_m;
    const double* __restrict__ A = p.a + bi * p.stride_a;
    const double* __restrict__ B = p.b + bi * p.stride_b;
    double* __restrict__ C = p.c + bi * p.stride_c;
    const int64_t m0 = tm * BT, n0 = tn * BT;
    const bool vec_a = ((p.lda & 1) == 0) && ((p.stride_a & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0);
    const bool vec_b = ((p.ldb & 1) == 0) && ((p.stride_b & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.b) & 15) == 0);

    // shared-window byte addresses: where this thread's copies land in stage 0, where its fragments start
    constexpr uint32_t A_BYTES = TileA::SIZE * 8, B_BYTES = TileB::SIZE * 8, STAGE_BYTES = A_BYTES + B_BYTES;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(dg_smem));
    const uint32_t a_store = smem_base + 8u * dg_store_offset<BT, !TA>(t);
    const uint32_t b_store = smem_base + A_BYTES + 8u * dg_store_offset<BT, TB>(t);
    const uint32_t a_frag = smem_base + 8u * TileA::index(wm * (BT / 4) + gid, tig);
    const uint32_t b_frag = smem_base + A_BYTES + 8u * TileB::index(wn * (BT / 4) + gid, tig);
    const uint32_t full0 = smem_base + DG_STAGES * STAGE_BYTES;          // full[s] at full0 + 8 s
    const uint32_t empty0 = full0 + 8 * DG_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(reinterpret_cast<char*>(dg_smem) + DG_STAGES * STAGE_BYTES + 16 * DG_STAGES);
    if (t == 0)
    {
        for (int s = 0; s < DG_STAGES; ++s)
        {
            tc3x::mbar_init(full0 + 8 * s, DG_THREADS);      // one asynchronous arrival per thread's copies
            tc3x::mbar_init(empty0 + 8 * s, DG_THREADS / 32); // one arrival per warp
        }
        *abort_flag = 0;
    }
    __syncthreads();

    double acc[MB][NB][4];
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j) { acc[i][j][0] = 0.0; acc[i][j][1] = 0.0; acc[i][j][2] = 0.0; acc[i][j][3] = 0.0; }

    DgAsyncLoader<BT, !TA> load_a;
    DgAsyncLoader<BT, TB> load_b;
    load_a.init(A, p.lda, m0, p.m, p.k, t, vec_a);
    load_b.init(B, p.ldb, n0, p.n, p.k, t, vec_b);
    const int nk = (int)((p.k + DG_BK - 1) / DG_BK);
    for (int s = 0; s < DG_STAGES - 1 && s < nk; ++s)
    {
        load_a.issue(a_store + s * STAGE_BYTES);
        load_b.issue(b_store + s * STAGE_BYTES);
        dg_cp_async_arrive(full0 + 8 * s);
    }

    bool ok = true;
    for (int kt = 0; kt < nk; ++kt)
    {
        const uint32_t s = kt % DG_STAGES;
        ok = tc3x::mbar_wait_bounded(full0 + 8 * s, (kt / DG_STAGES) & 1, abort_flag, p.status, DG_ST_TIMEOUT_FULL, DG_WAIT_LIMIT_NS);
        if (!ok) break;
        const uint32_t a_at = a_frag + s * STAGE_BYTES, b_at = b_frag + s * STAGE_BYTES;
        dg_k8_step<TileA, TileB, MB, NB, 0>(a_at, b_at, acc);
        // this thread's share of the tile three steps ahead goes into the stage read one step ago:
        // by now the other warps have normally released it, so the wait does not stall
        const int kp = kt + DG_STAGES - 1;
        if (kp < nk)
        {
            const uint32_t sp = kp % DG_STAGES;
            if (kt >= 1)
            {
                ok = tc3x::mbar_wait_bounded(empty0 + 8 * sp, ((kt - 1) / DG_STAGES) & 1, abort_flag, p.status, DG_ST_TIMEOUT_EMPTY,
                                             DG_WAIT_LIMIT_NS);
                if (!ok) break;
            }
            load_a.issue(a_store + sp * STAGE_BYTES);
            load_b.issue(b_store + sp * STAGE_BYTES);
            dg_cp_async_arrive(full0 + 8 * sp);
        }
        dg_k8_step<TileA, TileB, MB, NB, 1>(a_at, b_at, acc);
        __syncwarp();
        if (lane == 0) tc3x::mbar_arrive(empty0 + 8 * s);
    }
    dg_cp_async_wait_all();                               // nothing of this thread is in flight past this point
    if (!ok) return;                                      // aborted: the status word tells the host

    // Epilogue: a lane holds columns tig*2, tig*2+1 of rows gid (c0, c1) and gid + 8 (c2, c3) of each block.
    const bool vec_c = ((p.ldc & 1) == 0) && ((p.stride_c & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0);
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h)
        {
            const int64_t row = m0 + wm * (BT / 4) + i * 16 + gid + h * 8;
            if (row >= p.m) continue;
#pragma unroll
            for (int j = 0; j < NB; ++j)
            {
                const int64_t col = n0 + wn * (BT / 4) + j * 8 + tig * 2;
                if (col >= p.n) continue;
                double* dst = C + row * p.ldc + col;
                double o0 = p.alpha * acc[i][j][h * 2 + 0], o1 = p.alpha * acc[i][j][h * 2 + 1];
                if (vec_c && col + 1 < p.n)
                {
                    if (p.beta != 0.0)
                    {
                        const double2 old = *reinterpret_cast<const double2*>(dst);
                        o0 = fma(p.beta, old.x, o0); o1 = fma(p.beta, old.y, o1);
                    }
                    *reinterpret_cast<double2*>(dst) = make_double2(o0, o1);
                }
                else
                {
                    if (p.beta != 0.0) o0 = fma(p.beta, dst[0], o0);
                    dst[0] = o0;
                    if (col + 1 < p.n)
                    {
                        if (p.beta != 0.0) o1 = fma(p.beta, dst[1], o1);
                        dst[1] = o1;
                    }
                }
            }
        }
}

template <int BT, bool TA, bool TB>
inline cudaError_t launch_dgemm_inst(const DgemmArgs& a, unsigned blocks, cudaStream_t st)
{
    constexpr size_t smem = DG_STAGES * sizeof(double) * (DgTile<BT, !TA>::SIZE + DgTile<BT, TB>::SIZE) + 16 * DG_STAGES + 16;
    cudaError_t e = cudaFuncSetAttribute(dgemm_mma_kernel<BT, TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dgemm_mma_kernel<BT, TA, TB><<<blocks, DG_THREADS, smem, st>>>(a);
    return cudaGetLastError();
}

template <int BT>
inline cudaError_t launch_dgemm_tile(const DgemmArgs& a0, bool ta, bool tb, int64_t batch, cudaStream_t st)
{
    DgemmArgs a = a0;
    a.tiles_m = (a.m + BT - 1) / BT;
    a.tiles_n = (a.n + BT - 1) / BT;
    const int64_t blocks = a.tiles_m * a.tiles_n * batch;
    if (blocks <= 0) return cudaSuccess;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (!ta && !tb) return launch_dgemm_inst<BT, false, false>(a, (unsigned)blocks, st);
    if (!ta && tb) return launch_dgemm_inst<BT, false, true>(a, (unsigned)blocks, st);
    if (ta && !tb) return launch_dgemm_inst<BT, true, false>(a, (unsigned)blocks, st);
    return launch_dgemm_inst<BT, true, true>(a, (unsigned)blocks, st);
}

// C <- beta * C (k == 0 or alpha == 0): no operand is read.
__global__ void scale_c_f64_kernel(double* c, int64_t m, int64_t n, int64_t ldc, int64_t stride_c, int64_t batch, double beta)
{
    const int64_t total = m * n * batch;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    {
        const int64_t col = i % n, row = (i / n) % m, bi = i / (n * m);
        double* dst = c + bi * stride_c + row * ldc + col;
        *dst = (beta == 0.0) ? 0.0 : beta * (*dst);
    }
}

// Tile choice by estimated time: whole rounds of 148 CTAs at the measured full-rate throughput of each tile
// (128 x 128: 33.5 TFLOP/s, 64 x 64: 30.4 on B200); a 128-tile does four times the work of a 64-tile.  The small
// tile wins when the large one would leave most of a round idle (1024^3: 64 tiles; 2048^3: 1.73 rounds).
inline cudaError_t launch_dgemm(const DgemmArgs& a, bool ta, bool tb, int64_t batch, int sm_count, cudaStream_t st)
{
    const int64_t t128 = ((a.m + 127) / 128) * ((a.n + 127) / 128) * batch;
    const int64_t t64 = ((a.m + 63) / 64) * ((a.n + 63) / 64) * batch;
    const double cost128 = (double)((t128 + sm_count - 1) / sm_count) * 4.0 / 33.5;
    const double cost64 = (double)((t64 + sm_count - 1) / sm_count) / 30.4;
    if (cost128 <= cost64) return launch_dgemm_tile<128>(a, ta, tb, batch, st);
    return launch_dgemm_tile<64>(a, ta, tb, batch, st);
}

} // namespace sushi
