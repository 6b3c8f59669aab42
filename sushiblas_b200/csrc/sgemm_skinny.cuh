// sgemm_skinny.cuh -- fp32 GEMM for tall-and-skinny products (n <= 32, op(A) = A with k contiguous).
//
// With so few columns the product is bound by reading A once from HBM (65536 x 16 x 256: 7.5 flop
// per byte), which the tiled kernels cannot approach (a 64-wide FFMA tile wastes three quarters of
// its work on padding; the 256-wide tensor tile even more, and its operand pre-pass would triple
// the traffic).  An FFMA version of this kernel turned out issue-bound (685 instructions per
// 16 x 32 block of A); warp-level TF32 MMAs need about 130, and the k reduction happens inside the
// MMA, so no shuffles.  Arithmetic: 3xTF32 like the main tensor path -- x = hi + lo with
// hi = rna_tf32(x), lo = rna_tf32(x - hi); lo*hi + hi*lo + hi*hi accumulated in fp32.
//
// A streams through the SM exactly once.  A warp owns 16 rows; lane (g = lane / 4, t = lane % 4)
// fetches the float4 at k = 4 t (and 16 + 4 t) of rows g and g + 8 -- 64 contiguous bytes per row
// and instruction -- four steps ahead with cp.async into a private ring in shared memory (its own
// copies only, so cp.async.wait_group is all the synchronisation the stream needs; the lookahead
// runs on across row blocks, so the pipe never drains), and splits the values into hi / lo in
// registers.  The MMA's k index is free to be permuted as long as both operands agree: step s of a
// float4 uses components 2s, 2s+1 as k slots t and t + 4, so the natural 128-bit loads feed the
// m16n8k8 fragments directly.  op(B) is small: one 256-k chunk of it sits in shared memory as
// float4 (hi_k, hi_k+1, lo_k, lo_k+1) per column and k pair -- one conflict-free 128-bit load gives
// a lane both B fragments of a step.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "activation.cuh"

namespace sushi {

struct SkinnyArgs
{
    const float* a; const float* b; float* c;
    int64_t m, n, k;
    int64_t lda, ldb, ldc;
    int64_t stride_a, stride_b, stride_c;
    int64_t row_blocks;          // ceil(m / rows per CTA)
    float alpha, beta;
    int trans_b, act;            // act: epilogue activation (ACT_* of activation.cuh)
    float act_param;
};

constexpr int SKINNY_THREADS = 256;
constexpr int SKINNY_ROWS = (SKINNY_THREADS / 32) * 16;   // rows per CTA and row block
constexpr int SKINNY_KC = 256;                            // k per shared-memory chunk of op(B)
constexpr int SKINNY_KPP = SKINNY_KC / 2 + 1;             // float4 per column of the chunk (odd: conflict-free)
constexpr int SKINNY_DEPTH = 4;                           // steps (32 k) of A in flight per lane

__device__ __forceinline__ void skinny_cp_async16(uint32_t dst, const float* src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void skinny_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void skinny_cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ void skinny_split(float x, uint32_t& hi, uint32_t& lo)
{
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    const float r = x - __uint_as_float(hi);          // exact in fp32
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
    if (!(fabsf(__uint_as_float(hi)) <= 3.402823466e+38f)) lo = 0u;   // inf / nan stay in the hi part only
}

__device__ __forceinline__ void skinny_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Position of a lane in the CTA's flattened work: row block, k-chunk, 32-wide step inside the chunk.
struct SkinnyCursor
{
    int64_t rb, k0;
    int ko;
    __device__ __forceinline__ void advance(int64_t k, int64_t rb_step)
    {
        ko += 32;
        const int64_t kc = (k - k0) < SKINNY_KC ? (k - k0) : SKINNY_KC;
        if (ko >= kc) { ko = 0; k0 += SKINNY_KC; if (k0 >= k) { k0 = 0; rb += rb_step; } }
    }
};

template <int NB>                                    // blocks of 8 columns
__global__ void __launch_bounds__(SKINNY_THREADS, 2)
sgemm_skinny_kernel(const SkinnyArgs p)
{
    // dynamic shared memory: op(B) chunk [8 NB][KPP] float4, then the lanes' private ring [DEPTH][4][THREADS] float4
    extern __shared__ __align__(16) float4 skinny_smem[];
    float4* Bq = skinny_smem;
    float4* ring = skinny_smem + 8 * NB * SKINNY_KPP;
    const int t = threadIdx.x, lane = t % 32, warp = t / 32;
    const int gid = lane / 4, tig = lane % 4;
    const int64_t bi = blockIdx.y;
    const float* __restrict__ A = p.a + bi * p.stride_a;
    const float* __restrict__ B = p.b + bi * p.stride_b;
    float* __restrict__ C = p.c + bi * p.stride_c;
    const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring + t));
    const int64_t lane_row = warp * 16 + gid;             // this lane's first row inside a row block (second: + 8)

    // one k-chunk of op(B): (hi_k, hi_k+1, lo_k, lo_k+1) per column and k pair, zeros beyond n and k
    auto load_b_chunk = [&](int64_t k0)
    {
        for (int idx = t; idx < 8 * NB * (SKINNY_KC / 2); idx += SKINNY_THREADS)
        {
            int c, kp;
            if (p.trans_b) { c = idx / (SKINNY_KC / 2); kp = idx % (SKINNY_KC / 2); }   // op(B)(kk, c) = b[c * ldb + kk]
            else           { kp = idx / (8 * NB);        c = idx % (8 * NB); }          // op(B)(kk, c) = b[kk * ldb + c]
            const int64_t kk = k0 + 2 * kp;
            float v0 = 0.0f, v1 = 0.0f;
            if (c < p.n)
            {
                if (kk < p.k) v0 = p.trans_b ? __ldg(B + c * p.ldb + kk) : __ldg(B + kk * p.ldb + c);
                if (kk + 1 < p.k) v1 = p.trans_b ? __ldg(B + c * p.ldb + kk + 1) : __ldg(B + (kk + 1) * p.ldb + c);
            }
            uint32_t h0, l0, h1, l1;
            skinny_split(v0, h0, l0);
            skinny_split(v1, h1, l1);
            Bq[c * SKINNY_KPP + kp] = make_float4(__uint_as_float(h0), __uint_as_float(h1), __uint_as_float(l0), __uint_as_float(l1));
        }
    };
    // this lane's four float4 of one step (rows g, g + 8; k halves 0, 16) into ring slot `slot`;
    // rows or k beyond the matrix arrive as zeros
    auto issue = [&](const SkinnyCursor& cur, int slot)
    {
        if (cur.rb < p.row_blocks)
        {
            const int64_t row0 = cur.rb * SKINNY_ROWS + lane_row;
            const int64_t kk = cur.k0 + cur.ko + 4 * tig;
            const float* src = A + row0 * p.lda + kk;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int q = 0; q < 2; ++q)
                {
                    const bool ok = (row0 + 8 * h < p.m) && (kk + 16 * q < p.k);
                    skinny_cp_async16(ring_addr + (uint32_t)((slot * 4 + h * 2 + q) * SKINNY_THREADS) * 16u,
                                      ok ? src + 8 * h * p.lda + 16 * q : A, ok ? 16u : 0u);
                }
        }
        skinny_cp_async_commit();                     // one group per step, empty past the end
    };

    const bool single_chunk = p.k <= SKINNY_KC;          // then op(B) is prepared once per CTA
    SkinnyCursor ahead{(int64_t)blockIdx.x, 0, 0};
#pragma unroll
    for (int d = 0; d < SKINNY_DEPTH; ++d) { issue(ahead, d); ahead.advance(p.k, gridDim.x); }
    if (single_chunk) { load_b_chunk(0); __syncthreads(); }

    float acc[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
    const bool vec_c = ((p.ldc & 1) == 0) && ((p.stride_c & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 7) == 0);

    int slot = 0;
    for (SkinnyCursor cur{(int64_t)blockIdx.x, 0, 0}; cur.rb < p.row_blocks;)
    {
        if (!single_chunk && cur.ko == 0)
        {
            __syncthreads();                          // the previous chunk has been read by everyone
            load_b_chunk(cur.k0);
            __syncthreads();
        }
        skinny_cp_async_wait<SKINNY_DEPTH - 1>();     // the oldest step of this lane has landed
        float4 av[2][2];                              // [row half][k half]
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int q = 0; q < 2; ++q) av[h][q] = ring[(slot * 4 + h * 2 + q) * SKINNY_THREADS + t];
        issue(ahead, slot);                           // refill the slot just read
        ahead.advance(p.k, gridDim.x);
        slot = (slot + 1) % SKINNY_DEPTH;

        const float4* bq_lane = Bq + gid * SKINNY_KPP + (cur.ko >> 1) + 2 * tig;
#pragma unroll
        for (int q = 0; q < 2; ++q)
        {
            const float x0[4] = {av[0][q].x, av[0][q].y, av[0][q].z, av[0][q].w};      // row g
            const float x1[4] = {av[1][q].x, av[1][q].y, av[1][q].z, av[1][q].w};      // row g + 8
#pragma unroll
            for (int s = 0; s < 2; ++s)
            {
                // k slots t and t + 4 of this MMA are k = 4t + 2s and 4t + 2s + 1 of the 16-k half
                uint32_t ah[4], al[4];
                skinny_split(x0[2 * s], ah[0], al[0]);
                skinny_split(x1[2 * s], ah[1], al[1]);
                skinny_split(x0[2 * s + 1], ah[2], al[2]);
                skinny_split(x1[2 * s + 1], ah[3], al[3]);
#pragma unroll
                for (int j = 0; j < NB; ++j)
                {
                    const float4 bq = bq_lane[j * 8 * SKINNY_KPP + 8 * q + s];
                    const uint32_t bh0 = __float_as_uint(bq.x), bh1 = __float_as_uint(bq.y);
                    const uint32_t bl0 = __float_as_uint(bq.z), bl1 = __float_as_uint(bq.w);
                    skinny_mma(acc[j], al[0], al[1], al[2], al[3], bh0, bh1);
                    skinny_mma(acc[j], ah[0], ah[1], ah[2], ah[3], bl0, bl1);
                    skinny_mma(acc[j], ah[0], ah[1], ah[2], ah[3], bh0, bh1);
                }
            }
        }
        const int64_t rb_done = cur.rb;
        cur.advance(p.k, gridDim.x);
        if (cur.rb == rb_done) continue;              // more k of the same rows to come

        // the row block is complete: a lane holds columns 2t, 2t+1 of rows g and g + 8 in every block
        const int64_t row0 = rb_done * SKINNY_ROWS + lane_row;
#pragma unroll
        for (int j = 0; j < NB; ++j)
        {
#pragma unroll
            for (int h = 0; h < 2; ++h)
            {
                const int64_t row = row0 + 8 * h;
                const int64_t col = 8 * j + 2 * tig;
                float o0 = p.alpha * acc[j][2 * h], o1 = p.alpha * acc[j][2 * h + 1];
                if (row < p.m && col < p.n)
                {
                    float* dst = C + row * p.ldc + col;
                    if (vec_c && col + 1 < p.n)
                    {
                        if (p.beta != 0.0f)
                        {
                            const float2 old = *reinterpret_cast<const float2*>(dst);
                            o0 = fmaf(p.beta, old.x, o0); o1 = fmaf(p.beta, old.y, o1);
                        }
                        if (p.act) { o0 = apply_act(o0, p.act, p.act_param); o1 = apply_act(o1, p.act, p.act_param); }
                        *reinterpret_cast<float2*>(dst) = make_float2(o0, o1);
                    }
                    else
                    {
                        if (p.beta != 0.0f) o0 = fmaf(p.beta, dst[0], o0);
                        dst[0] = apply_act(o0, p.act, p.act_param);
                        if (col + 1 < p.n)
                        {
                            if (p.beta != 0.0f) o1 = fmaf(p.beta, dst[1], o1);
                            dst[1] = apply_act(o1, p.act, p.act_param);
                        }
                    }
                }
                acc[j][2 * h] = 0.0f; acc[j][2 * h + 1] = 0.0f;
            }
        }
    }
    skinny_cp_async_wait<0>();
}

// Shapes this kernel serves: op(A) = A (k contiguous) readable with aligned 128-bit loads, few columns, many rows.
inline bool skinny_eligible(int ta, int64_t m, int64_t n, int64_t k, const float* a, int64_t lda, int64_t stride_a)
{
    return !ta && n >= 1 && n <= 32 && m >= 2048 && k >= 32 && (k % 4) == 0 && (lda % 4) == 0 && (stride_a % 4) == 0 &&
           (reinterpret_cast<uintptr_t>(a) & 15) == 0;
}

template <int NB>
inline cudaError_t launch_sgemm_skinny_inst(const SkinnyArgs& p, dim3 grid, cudaStream_t st)
{
    const size_t smem = sizeof(float4) * (8 * NB * SKINNY_KPP + SKINNY_DEPTH * 4 * SKINNY_THREADS);
    cudaError_t e = cudaFuncSetAttribute(sgemm_skinny_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    sgemm_skinny_kernel<NB><<<grid, SKINNY_THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

inline cudaError_t launch_sgemm_skinny(SkinnyArgs p, int64_t batch, int sm_count, cudaStream_t st)
{
    if (batch <= 0 || batch > 65535) return cudaErrorInvalidValue;
    p.row_blocks = (p.m + SKINNY_ROWS - 1) / SKINNY_ROWS;
    int64_t gx = p.row_blocks;
    const int64_t cap = ((int64_t)sm_count * 2 + batch - 1) / batch;      // two CTAs per SM, grid-stride over the rest
    if (gx > cap) gx = cap > 0 ? cap : 1;
    const dim3 grid((unsigned)gx, (unsigned)batch);
    const int nb = (int)((p.n + 7) / 8);
    if (nb == 1) return launch_sgemm_skinny_inst<1>(p, grid, st);
    if (nb == 2) return launch_sgemm_skinny_inst<2>(p, grid, st);
    if (nb == 3) return launch_sgemm_skinny_inst<3>(p, grid, st);
    return launch_sgemm_skinny_inst<4>(p, grid, st);
}

} // namespace sushi
