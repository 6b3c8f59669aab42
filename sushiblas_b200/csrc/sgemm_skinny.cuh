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
// and instruction -- DEPTH steps ahead with cp.async into a private ring in shared memory (its own
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

constexpr int SKINNY_KC = 256;                            // k per shared-memory chunk of op(B)
constexpr int SKINNY_KPP = SKINNY_KC / 2 + 1;             // float4 per column of the chunk (odd: conflict-free)
// Two shapes of CTA (THREADS, CTAs per SM, DEPTH = steps of 32 k of A in flight per lane; a CTA's row block is
// 16 rows per warp).  The kernel is bound by instruction issue and latency, not by HBM, so what counts is how many
// warps an SM holds and that the row blocks fill the machine in a whole number of rounds:
//   narrow: 256 threads, two CTAs per SM (16 warps per SM, up to 96 registers), DEPTH 4
//   wide:   896 threads, one CTA per SM (28 warps per SM, 72 registers), DEPTH 3 (2 when op(B) has more than 16 columns)
constexpr int SKINNY_THREADS_NARROW = 256, SKINNY_THREADS_WIDE = 896;

__device__ __forceinline__ void skinny_cp_async16(uint32_t dst, const float* src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void skinny_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void skinny_cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// x = hi + lo with hi = rna_tf32(x), lo = rna_tf32(x - hi).  Round-to-nearest-away on the 13 dropped mantissa bits
// is "add half an ulp to the magnitude bits, clear them" -- two integer instructions, the same bits as
// cvt.rna.tf32.f32 for every finite x (a carry into the exponent is the correct rounding, up to infinity) and
// measurably cheaper in this instruction-bound loop.  Where hi is not finite (x is, or rounds to, infinity; NaN)
// lo is 0; a NaN keeps its bits (the carry could otherwise run into the sign of an all-ones payload).
__device__ __forceinline__ void skinny_split(float x, uint32_t& hi, uint32_t& lo)
{
    const uint32_t xb = __float_as_uint(x);
    hi = (xb + 0x1000u) & 0xffffe000u;
    const float r = x - __uint_as_float(hi);          // exact in fp32
    lo = (__float_as_uint(r) + 0x1000u) & 0xffffe000u;
    if (!(fabsf(x) < 0x1.ffep127f)) lo = 0u;          // 0x7f7ff000: the smallest magnitude that rounds to infinity
    if (x != x) hi = xb;
}

__device__ __forceinline__ void skinny_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NB, int SKINNY_THREADS, int SKINNY_DEPTH>       // NB: blocks of 8 columns
__global__ void __launch_bounds__(SKINNY_THREADS, SKINNY_THREADS <= 256 ? 2 : 1)
sgemm_skinny_kernel(const SkinnyArgs p)
{
    constexpr int SKINNY_ROWS = (SKINNY_THREADS / 32) * 16;   // rows per CTA and row block
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
    // The lane walks its CTA's work -- row blocks blockIdx.x, + gridDim.x, ..., each `steps` steps of 32 k -- twice:
    // once DEPTH steps ahead, issuing copies, once consuming.  Both walks keep running pointers (source, ring slot)
    // so that a step costs a handful of instructions besides the arithmetic: the kernel is bound by instruction
    // throughput, not by HBM.
    const int steps = (int)((p.k + 31) / 32);
    const int k_lane = (int)p.k - 4 * tig;               // a float4 at k offset x of this lane is inside iff x < k_lane
    const int64_t lda8 = 8 * p.lda;
    constexpr uint32_t SLOT_BYTES = 4u * SKINNY_THREADS * 16u;
    const uint32_t ring_end = ring_addr + SKINNY_DEPTH * SLOT_BYTES;

    int64_t a_rb = blockIdx.x;                           // walk ahead: row block, step, source of (row g, this step)
    int a_s = 0;
    uint32_t a_dst = ring_addr;
    const float* a_src = A;
    bool a_ok0 = false, a_ok1 = false;
    auto ahead_enter_block = [&]()
    {
        const int64_t row0 = a_rb * SKINNY_ROWS + lane_row;
        const bool live = a_rb < p.row_blocks;
        a_ok0 = live && row0 < p.m;
        a_ok1 = live && row0 + 8 < p.m;
        a_src = A + (a_ok0 ? row0 : 0) * p.lda + 4 * tig;
    };
    // this lane's four float4 of one step (rows g, g + 8; k halves 0, 16) into the ring slot at a_dst; rows or k
    // beyond the matrix arrive as zeros; one group per step, empty past the end
    auto issue = [&]()
    {
        const int kk = 32 * a_s;
#pragma unroll
        for (int q = 0; q < 2; ++q)
        {
            const bool kin = kk + 16 * q < k_lane;
            const bool ok0 = a_ok0 && kin, ok1 = a_ok1 && kin;
            skinny_cp_async16(a_dst + (uint32_t)(q * SKINNY_THREADS) * 16u, ok0 ? a_src + 16 * q : A, ok0 ? 16u : 0u);
            skinny_cp_async16(a_dst + (uint32_t)((2 + q) * SKINNY_THREADS) * 16u, ok1 ? a_src + lda8 + 16 * q : A, ok1 ? 16u : 0u);
        }
        skinny_cp_async_commit();
        a_dst += SLOT_BYTES;
        if (a_dst == ring_end) a_dst = ring_addr;
        a_src += 32;
        if (++a_s == steps) { a_s = 0; a_rb += gridDim.x; ahead_enter_block(); }
    };

    const bool single_chunk = p.k <= SKINNY_KC;          // then op(B) is prepared once per CTA
    ahead_enter_block();
#pragma unroll
    for (int d = 0; d < SKINNY_DEPTH; ++d) issue();
    if (single_chunk) { load_b_chunk(0); __syncthreads(); }

    float acc[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
    const bool vec_c = ((p.ldc & 1) == 0) && ((p.stride_c & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 7) == 0);

    const float4* c_ring = ring + t;                     // consuming walk: ring slot, row block, step
    const float4* const c_ring_end = c_ring + SKINNY_DEPTH * 4 * SKINNY_THREADS;
    int c_s = 0;
    for (int64_t c_rb = blockIdx.x; c_rb < p.row_blocks;)
    {
        if (!single_chunk && (c_s & 7) == 0)
        {
            __syncthreads();                          // the previous chunk has been read by everyone
            load_b_chunk((int64_t)(c_s >> 3) * SKINNY_KC);
            __syncthreads();
        }
        skinny_cp_async_wait<SKINNY_DEPTH - 1>();     // the oldest step of this lane has landed
        float4 av[2][2];                              // [row half][k half]
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int q = 0; q < 2; ++q) av[h][q] = c_ring[(h * 2 + q) * SKINNY_THREADS];
        c_ring += 4 * SKINNY_THREADS;
        if (c_ring == c_ring_end) c_ring = ring + t;
        issue();                                      // refill the slot just read

        const float4* bq_lane = Bq + gid * SKINNY_KPP + 16 * (c_s & 7) + 2 * tig;
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
        if (++c_s < steps) continue;                  // more k of the same rows to come
        const int64_t rb_done = c_rb;
        c_s = 0;
        c_rb += gridDim.x;

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
    return !ta && n >= 1 && n <= 32 && m >= 2048 && k >= 32 && k <= (int64_t(1) << 30) && (k % 4) == 0 && (lda % 4) == 0 && (stride_a % 4) == 0 &&
           (reinterpret_cast<uintptr_t>(a) & 15) == 0;
}

template <int NB, int THREADS, int DEPTH>
inline cudaError_t launch_sgemm_skinny_inst(const SkinnyArgs& p, dim3 grid, cudaStream_t st)
{
    const size_t smem = sizeof(float4) * (8 * NB * SKINNY_KPP + DEPTH * 4 * THREADS);
    cudaError_t e = cudaFuncSetAttribute(sgemm_skinny_kernel<NB, THREADS, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    sgemm_skinny_kernel<NB, THREADS, DEPTH><<<grid, THREADS, smem, st>>>(p);
    return cudaGetLastError();
}

// Rounds the SMs need for `rows * batch` rows when an SM holds `rows_per_sm` of them at a time.
inline int64_t skinny_rounds(int64_t m, int64_t batch, int rows_per_cta, int ctas_per_sm, int sm_count)
{
    const int64_t blocks = ((m + rows_per_cta - 1) / rows_per_cta) * batch;
    const int64_t slots = (int64_t)sm_count * ctas_per_sm;
    return (blocks + slots - 1) / slots;
}

inline cudaError_t launch_sgemm_skinny(SkinnyArgs p, int64_t batch, int sm_count, cudaStream_t st, int shape = 0)
{
    if (batch <= 0 || batch > 65535) return cudaErrorInvalidValue;
    constexpr int ROWS_N = SKINNY_THREADS_NARROW / 32 * 16, ROWS_W = SKINNY_THREADS_WIDE / 32 * 16;
    // a round of the wide shape holds 28 warps per SM against 16: it wins when it does not need more rounds per
    // row than the narrow one, i.e. when the rows keep its larger blocks busy (shape: 1 narrow, 2 wide, 0 by this rule)
    const int64_t work_n = skinny_rounds(p.m, batch, ROWS_N, 2, sm_count) * 2 * ROWS_N;
    const int64_t work_w = skinny_rounds(p.m, batch, ROWS_W, 1, sm_count) * ROWS_W;
    const bool wide = shape ? shape == 2 : work_w <= work_n;
    const int rows = wide ? ROWS_W : ROWS_N;
    p.row_blocks = (p.m + rows - 1) / rows;
    int64_t gx = p.row_blocks;
    const int64_t cap = ((int64_t)sm_count * (wide ? 1 : 2) + batch - 1) / batch;   // co-resident CTAs, grid-stride over the rest
    if (gx > cap) gx = cap > 0 ? cap : 1;
    const dim3 grid((unsigned)gx, (unsigned)batch);
    const int nb = (int)((p.n + 7) / 8);
    if (wide)
    {
        if (nb == 1) return launch_sgemm_skinny_inst<1, SKINNY_THREADS_WIDE, 3>(p, grid, st);
        if (nb == 2) return launch_sgemm_skinny_inst<2, SKINNY_THREADS_WIDE, 3>(p, grid, st);
        if (nb == 3) return launch_sgemm_skinny_inst<3, SKINNY_THREADS_WIDE, 2>(p, grid, st);
        return launch_sgemm_skinny_inst<4, SKINNY_THREADS_WIDE, 2>(p, grid, st);
    }
    if (nb == 1) return launch_sgemm_skinny_inst<1, SKINNY_THREADS_NARROW, 4>(p, grid, st);
    if (nb == 2) return launch_sgemm_skinny_inst<2, SKINNY_THREADS_NARROW, 4>(p, grid, st);
    if (nb == 3) return launch_sgemm_skinny_inst<3, SKINNY_THREADS_NARROW, 4>(p, grid, st);
    return launch_sgemm_skinny_inst<4, SKINNY_THREADS_NARROW, 4>(p, grid, st);
}

} // namespace sushi
