// split_tf32.cuh -- operand pre-pass of the 3xTF32 GEMM.
//
// fp32 accuracy on TF32 tensor cores needs each operand as hi + lo with
//     hi = rna_tf32(x),  lo = rna_tf32(x - hi)
// so that  x*y ~= hi_x*hi_y + hi_x*lo_y + lo_x*hi_y  (the lo*lo term is below 2^-22 |x y|).
// This pass writes both planes of op(A) (rows = m) and of op(B)^T (rows = n) as K-major,
// zero-padded panels in a layout chosen for the consumer: for every block of 16
// consecutive k all rows lie back to back,
//
//     plane[batch][hi|lo][k_block][row_pad][16]        (fp32; 64 bytes per row per k-block)
//
// so that one pipeline stage of the GEMM (256 rows x 16 k x {hi, lo}) is two contiguous
// 16 KB runs that TMA fetches as one 4-D box.  The transposes of the BLAS call
// (op(A) = A^T, op(B) = B) are absorbed here: the GEMM kernel only ever sees K-major planes.
// Algorithmic traffic: reads the operand once (4 B / element), writes 8 B / element.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace sushi {

constexpr int SPLIT_KB = 16;     // k-block (elements) == GEMM pipeline BK
constexpr int SPLIT_ROWPAD = 256; // rows padded to the GEMM tile

struct SplitArgs
{
    const float* x;      // operand base
    float* planes;       // output base (256-byte aligned)
    int64_t rows, k;     // logical extent of op(X): rows x k
    int64_t ld;          // leading dimension of the stored matrix
    int64_t stride_x;    // batch stride of x (elements)
    int64_t rows_pad;    // rows rounded up to SPLIT_ROWPAD
    int64_t num_kb;      // ceil(k / 16)
    int64_t batch;
};

__device__ __forceinline__ void split_one(float x, float& hi, float& lo)
{
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    float r = x - hi;                 // exact in fp32
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(r));
    // inf / nan inputs: keep them in the hi plane only (inf - inf would poison lo)
    lo = (fabsf(hi) <= 3.402823466e+38f) ? __uint_as_float(l) : 0.0f;
}

__device__ __forceinline__ int64_t plane_offset(const SplitArgs& p, int64_t bi, int plane, int64_t kb, int64_t row)
{
    return (((bi * 2 + plane) * p.num_kb + kb) * p.rows_pad + row) * SPLIT_KB;
}

// k is the contiguous index of the stored operand: element (row, kk) = x[row*ld + kk].
// One CTA per (64 rows, 4 k-blocks = 64 k): sixteen threads read one row's 256 contiguous bytes (128-bit loads
// when the operand is 16-byte aligned), four rows per thread in flight, and every (plane, k-block) receives one
// contiguous 4 KB run.  Neighbouring CTAs take neighbouring k ranges of the same rows.  No index arithmetic
// beyond the CTA's own decomposition: the pass runs at the speed of the memory system.
template <bool VEC>
__global__ void __launch_bounds__(256)
split_tf32_kcontig_kernel(const SplitArgs p)
{
    const int t = threadIdx.x;
    const int64_t row_tiles = p.rows_pad / 64;
    const int64_t k_tiles = (p.num_kb + 3) / 4;
    int64_t blk = blockIdx.x;
    const int64_t kt = blk % k_tiles; blk /= k_tiles;
    const int64_t rt = blk % row_tiles;
    const int64_t bi = blk / row_tiles;
    const int k4 = t % 16;
    const int64_t kk = kt * 64 + k4 * 4;                   // first k of this thread's four
    const int64_t kb = kt * 4 + k4 / 4;
    const int within = (k4 % 4) * 4;
    const int64_t row0 = rt * 64 + t / 16;
    const float* __restrict__ src = p.x + bi * p.stride_x + kk;
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const int64_t row = row0 + 16 * j;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < p.rows && kk < p.k)
        {
            const float* q = src + row * p.ld;
            if (VEC && kk + 3 < p.k) v[j] = __ldg(reinterpret_cast<const float4*>(q));
            else
            {
                v[j].x = __ldg(q);
                if (kk + 1 < p.k) v[j].y = __ldg(q + 1);
                if (kk + 2 < p.k) v[j].z = __ldg(q + 2);
                if (kk + 3 < p.k) v[j].w = __ldg(q + 3);
            }
        }
    }
    if (kb >= p.num_kb) return;
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const int64_t row = row0 + 16 * j;
        float4 hi, lo;
        split_one(v[j].x, hi.x, lo.x); split_one(v[j].y, hi.y, lo.y);
        split_one(v[j].z, hi.z, lo.z); split_one(v[j].w, hi.w, lo.w);
        *reinterpret_cast<float4*>(p.planes + plane_offset(p, bi, 0, kb, row) + within) = hi;
        *reinterpret_cast<float4*>(p.planes + plane_offset(p, bi, 1, kb, row) + within) = lo;
    }
}

// The row index is the contiguous one: element (row, kk) = x[kk*ld + row].
// One CTA per (64 rows, 4 k-blocks = 64 k): reads 64 runs of 64 floats (128-bit loads when the
// operand is 16-byte aligned), transposes through shared memory and writes four contiguous
// 4 KB runs per plane.
template <bool VEC>
__global__ void __launch_bounds__(256)
split_tf32_rcontig_kernel(const SplitArgs p)
{
    constexpr int KT = 4 * SPLIT_KB;                 // 64 k per CTA
    __shared__ float tile[KT][64 + 1];
    const int t = threadIdx.x;
    const int64_t row_tiles = p.rows_pad / 64;
    const int64_t k_tiles = (p.num_kb + 3) / 4;
    int64_t blk = blockIdx.x;
    const int64_t rt = blk % row_tiles; blk /= row_tiles;
    const int64_t kt = blk % k_tiles;
    const int64_t bi = blk / k_tiles;
    const int64_t r0 = rt * 64, k0 = kt * KT;
    const float* __restrict__ src = p.x + bi * p.stride_x;

    if (VEC)
    {
        // 16 threads cover one 64-float run; 16 runs per pass
        const int r4 = (t % 16) * 4, kk0 = t / 16;
#pragma unroll
        for (int j = 0; j < KT / 16; ++j)
        {
            const int kk = kk0 + 16 * j;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + kk < p.k)
            {
                const float* q = src + (k0 + kk) * p.ld + r0 + r4;
                if (r0 + r4 + 3 < p.rows) v = __ldg(reinterpret_cast<const float4*>(q));
                else
                {
                    if (r0 + r4 + 0 < p.rows) v.x = __ldg(q + 0);
                    if (r0 + r4 + 1 < p.rows) v.y = __ldg(q + 1);
                    if (r0 + r4 + 2 < p.rows) v.z = __ldg(q + 2);
                }
            }
            tile[kk][r4 + 0] = v.x; tile[kk][r4 + 1] = v.y; tile[kk][r4 + 2] = v.z; tile[kk][r4 + 3] = v.w;
        }
    }
    else
    {
#pragma unroll
        for (int j = 0; j < KT / 4; ++j)
        {
            const int r = t % 64, kk = t / 64 + 4 * j;
            float v = 0.0f;
            if (r0 + r < p.rows && k0 + kk < p.k) v = __ldg(src + (k0 + kk) * p.ld + r0 + r);
            tile[kk][r] = v;
        }
    }
    __syncthreads();
    const int row = t / 4, q = t % 4;
#pragma unroll
    for (int b = 0; b < 4; ++b)
    {
        const int64_t kb = kt * 4 + b;
        if (kb >= p.num_kb) break;
        float4 hi, lo;
        split_one(tile[b * SPLIT_KB + q * 4 + 0][row], hi.x, lo.x);
        split_one(tile[b * SPLIT_KB + q * 4 + 1][row], hi.y, lo.y);
        split_one(tile[b * SPLIT_KB + q * 4 + 2][row], hi.z, lo.z);
        split_one(tile[b * SPLIT_KB + q * 4 + 3][row], hi.w, lo.w);
        *reinterpret_cast<float4*>(p.planes + plane_offset(p, bi, 0, kb, r0 + row) + q * 4) = hi;
        *reinterpret_cast<float4*>(p.planes + plane_offset(p, bi, 1, kb, r0 + row) + q * 4) = lo;
    }
}

inline size_t split_plane_bytes(int64_t rows, int64_t k, int64_t batch)
{
    const int64_t rows_pad = (rows + SPLIT_ROWPAD - 1) / SPLIT_ROWPAD * SPLIT_ROWPAD;
    const int64_t num_kb = (k + SPLIT_KB - 1) / SPLIT_KB;
    return (size_t)batch * 2 * (size_t)num_kb * (size_t)rows_pad * SPLIT_KB * sizeof(float);
}

// k_contig: the k index is unit stride in memory (A not transposed, or B transposed).
inline cudaError_t launch_split_tf32(const float* x, float* planes, int64_t rows, int64_t k, int64_t ld,
                                     int64_t stride_x, int64_t batch, bool k_contig, int sm_count,
                                     cudaStream_t st)
{
    SplitArgs p;
    p.x = x; p.planes = planes; p.rows = rows; p.k = k; p.ld = ld; p.stride_x = stride_x;
    p.rows_pad = (rows + SPLIT_ROWPAD - 1) / SPLIT_ROWPAD * SPLIT_ROWPAD;
    p.num_kb = (k + SPLIT_KB - 1) / SPLIT_KB;
    p.batch = batch;
    (void)sm_count;
    const int64_t blocks = (p.rows_pad / 64) * ((p.num_kb + 3) / 4) * batch;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (blocks == 0) return cudaSuccess;
    const bool vec = ((ld & 3) == 0) && ((stride_x & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (k_contig)
    {
        if (vec) split_tf32_kcontig_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(p);
        else split_tf32_kcontig_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(p);
    }
    else
    {
        if (vec) split_tf32_rcontig_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(p);
        else split_tf32_rcontig_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(p);
    }
    return cudaGetLastError();
}

} // namespace sushi
