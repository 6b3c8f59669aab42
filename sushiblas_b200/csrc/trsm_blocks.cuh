// trsm_blocks.cuh -- diagonal-block inversion for the blocked triangular solve.
//
// TRSM (reference: src/ops/blas/level3/trsm.cpp:85-202, forwarding to oneMKL trsm[_batch] at
// trsm.cpp:61-79) is run as a recursive blocked substitution: the off-diagonal work is GEMM
// updates on the regular GEMM kernels, and each 512 x 512 diagonal block of op(A) is applied
// through its explicit inverse.  This kernel inverts the 128 x 128 diagonal sub-blocks (the host
// then assembles the 256 and 512 blocks from their halves with batched GEMMs).  One CTA per
// sub-block, thread j owns column j of the inverse and runs the substitution for it out of shared
// memory (reads of T are broadcasts, writes of the column are conflict-free).  Sub-block d is
// written at inv + (d / 4) * 512 * 512 + (d % 4) * (128 * 512 + 128) with leading dimension 512,
// i.e. onto the diagonal of its 512 x 512 block; rows and columns beyond the matrix become identity.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace sushi {

constexpr int TRSM_NB = 128;       // order of the sub-blocks inverted by substitution
constexpr int TRSM_BASE = 512;     // order of the diagonal blocks applied as explicit inverses
constexpr int TRSM_SUBS = TRSM_BASE / TRSM_NB;

struct TrtriArgs
{
    const float* a;        // triangular matrix (dim x dim, leading dimension lda)
    float* inv;            // out: [ceil(dim / 512)][512][512]; this kernel fills the four 128 x 128 diagonal sub-blocks
    int64_t dim, lda;
    int trans;             // op(A) = A^T
    int eff_lower;         // op(A) is lower triangular
    int unit_diag;
};

__global__ void __launch_bounds__(TRSM_NB)
trtri_diag_blocks_kernel(const TrtriArgs p)
{
    extern __shared__ float smem[];
    float (*T)[TRSM_NB + 1] = reinterpret_cast<float (*)[TRSM_NB + 1]>(smem);                    // T[r][c]
    float (*X)[TRSM_NB] = reinterpret_cast<float (*)[TRSM_NB]>(smem + TRSM_NB * (TRSM_NB + 1));   // X[i][j] = inv(i, j)
    const int j = threadIdx.x;
    const int64_t d0 = (int64_t)blockIdx.x * TRSM_NB;
    const int size = (int)((p.dim - d0) < TRSM_NB ? (p.dim - d0) : TRSM_NB);   // <= 0: identity block

    // load op(A)'s block; outside the referenced triangle and beyond the matrix: identity
    for (int r = 0; r < TRSM_NB; ++r)
    {
        const int c = j;
        float v = (r == c) ? 1.0f : 0.0f;
        const bool in_tri = p.eff_lower ? (c <= r) : (c >= r);
        if (r < size && c < size && in_tri && !(p.unit_diag && r == c))
            v = p.trans ? p.a[(d0 + c) * p.lda + d0 + r] : p.a[(d0 + r) * p.lda + d0 + c];
        T[r][c] = v;
    }
    __syncthreads();
    for (int i = 0; i < TRSM_NB; ++i) X[i][j] = 0.0f;
    if (p.eff_lower)
    {
        // column j of inv(L): x_j = 1 / L_jj, x_i = -(sum_{k=j}^{i-1} L_ik x_k) / L_ii for i > j
        X[j][j] = 1.0f / T[j][j];
        for (int i = j + 1; i < TRSM_NB; ++i)
        {
            float s = 0.0f;
            for (int k = j; k < i; ++k) s = fmaf(T[i][k], X[k][j], s);
            X[i][j] = -s / T[i][i];
        }
    }
    else
    {
        // column j of inv(U): x_j = 1 / U_jj, x_i = -(sum_{k=i+1}^{j} U_ik x_k) / U_ii for i < j
        X[j][j] = 1.0f / T[j][j];
        for (int i = j - 1; i >= 0; --i)
        {
            float s = 0.0f;
            for (int k = i + 1; k <= j; ++k) s = fmaf(T[i][k], X[k][j], s);
            X[i][j] = -s / T[i][i];
        }
    }
    __syncthreads();
    float* out = p.inv + (int64_t)(blockIdx.x / TRSM_SUBS) * TRSM_BASE * TRSM_BASE +
                 (int64_t)(blockIdx.x % TRSM_SUBS) * (TRSM_NB * TRSM_BASE + TRSM_NB);
    for (int i = 0; i < TRSM_NB; ++i) out[i * TRSM_BASE + j] = X[i][j];
}

inline size_t trtri_smem_bytes() { return sizeof(float) * (TRSM_NB * (TRSM_NB + 1) + TRSM_NB * TRSM_NB); }

inline cudaError_t launch_trtri_diag_blocks(const TrtriArgs& p, cudaStream_t st)
{
    const int64_t blocks = TRSM_SUBS * ((p.dim + TRSM_BASE - 1) / TRSM_BASE);
    if (blocks <= 0) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(trtri_diag_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)trtri_smem_bytes());
    if (e != cudaSuccess) return e;
    trtri_diag_blocks_kernel<<<(unsigned)blocks, TRSM_NB, trtri_smem_bytes(), st>>>(p);
    return cudaGetLastError();
}

} // namespace sushi
