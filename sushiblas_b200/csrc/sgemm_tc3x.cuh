// sgemm_tc3x.cuh -- fp32-accurate GEMM on the sm_100a tensor cores (tcgen05, 3xTF32).
//
// Replaces the closed sgemm the reference forwards to (oneapi::mkl::blas::row_major::gemm /
// gemm_batch, src/ops/blas/level3/gemm.cpp:58,63) for problems large enough to fill tiles.
//
//   C[bi] <- alpha * (Ahi*Bhi + Ahi*Blo + Alo*Bhi) + beta * C[bi]
//
// Operands arrive pre-split by split_tf32.cuh as K-major hi/lo planes
//   plane[batch][hi|lo][k_block][row_pad][16]
// and are fetched by TMA (cp.async.bulk.tensor.4d, SWIZZLE_64B) into a 3-stage ring of
// 64 KB stages: {A: 256 rows x 16 k x 2 planes, B: 256 rows x 16 k x 2 planes}.
// A CTA owns a 256 x 256 tile of C as two 128 x 256 fp32 accumulators in tensor memory
// (2 x 256 of the 512 TMEM columns).  Roles (320 threads, one CTA per SM, persistent):
//   warp 0      TMA producer (one lane issues; waits on empty[], arms full[])
//   warp 1      TMEM allocation + MMA issue: per stage 2 halves x 2 k-steps x 3 products of
//               tcgen05.mma.kind::tf32 (M128 N256 K8); tcgen05.commit frees the stage
//   warps 2..9  epilogue: tcgen05.ld (32 lanes x 32 columns), transpose through swizzled
//               shared memory, then alpha*acc + beta*C with 128-bit stores that are
//               contiguous along each row of C (8 lanes cover one 128-byte row segment)
// In-kernel split: an operand whose k index is contiguous in memory (A not transposed, B
// transposed) and whose leading dimension / base are 16-byte aligned can skip the pre-pass: TMA
// loads its raw fp32 tile (3-D map over the user's matrix, zero fill outside M/N/K) into the hi
// slot of the stage, and the eight epilogue warps -- idle during the main loop -- rewrite it in
// place as hi = rna_tf32(x) and store lo = rna_tf32(x - hi) into the lo slot (element-wise, so the
// TMA swizzle is preserved), fence the generic-proxy writes towards the async proxy and arrive on
// a per-stage "converted" barrier that the MMA warp then waits on instead of the TMA barrier.
// This removes 12 B/element of pre-pass traffic and halves that operand's read traffic.
// An operand stored the other way round (A transposed, B not transposed: the row index of the tile
// is contiguous) is taken raw as well: its tile arrives as eight dense boxes of 32 rows x 16 k, box
// g in the 2 KB of the lo slot that converter warp g rewrites, and that warp transposes while it
// splits -- a lane reads the 16 k values of one row (conflict-free) and writes the row's 64 bytes of
// hi and lo at the positions TMA's SWIZZLE_64B would have used.  The read-before-write hazard
// stays inside one warp, so no cross-warp synchronisation is added.
//
// Why 256 x 256: with both planes of both operands streamed per k-block, a CTA moves
// 8*(BM+BN) bytes per 3*BM*BN tensor-core MACs; 256 x 256 keeps that at ~43 B/clk/SM of L2
// bandwidth at full tensor rate, where 128 x 256 would need 64 B/clk/SM.
//
// Work distribution: whole tiles are dealt round-robin to the CTAs (data-parallel rounds).  The
// tiles of a last, partial round -- or all tiles when there are fewer tiles than SMs -- are cut
// along K into S equal slices ("split-K tail"), and the (slice, tile) items are dealt round-robin
// slice-major, so that the CTAs running at the same time work on the same K range of neighbouring
// tiles and keep sharing A/B panels in L2.  Slices 0 .. S-2 write their raw 256 x 256 fp32
// accumulators to a slot in global scratch and publish an epoch flag (release); the CTA holding
// the last slice owns the tile: it acquires the flags, adds the slots and applies alpha/beta.
// Publishing never waits, an owner only waits for items dealt before its own, and the grid never
// exceeds the SM count, so the exchange cannot deadlock; the flag wait is bounded like every
// other wait.  With so few tiles that S slices of every tile fit the grid at one item per CTA
// (S = 2, 4, 8, 16), the finish is cooperative instead: every slice publishes, then each CTA waits
// for the S flags of its tile and adds and stores rows [q, q+1) * 256/S of it -- every CTA reads
// 256 KB whatever S is, where a single owner would read (S-1) * 256 KB through one SM.
//
// Every wait in this kernel is bounded: on expiry the waiter records a code in *status,
// raises a CTA-wide abort flag, every role leaves its loop, in-flight copies and MMAs are
// drained with bounded waits, TMEM is freed and the kernel returns.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include "activation.cuh"

namespace sushi {
namespace tc3x {


constexpr int BM = 256, BN = 256, BK = 16;
constexpr int STAGES = 3;
constexpr int PLANE_BYTES = 256 * BK * 4;             // one 256-row plane of one k-block: 16 KB
constexpr int OPERAND_BYTES = 2 * PLANE_BYTES;        // hi + lo: 32 KB
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;        // A + B: 64 KB
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;          // 320: launches whose operands are all pre-split planes
// Launches with a raw operand add eight converter warps and lay the roles out by warpgroup (four warps) so that
// setmaxnreg can move registers between them: warps 0..3 producer, MMA issuer and two idle, 4..11 epilogue, 12..19
// converters.  The pool that setmaxnreg trades within is what the CTA was launched with (640 x 96), not the
// register file: an increase that the decreases do not cover would wait for ever.
constexpr int THREADS_RAW = 640;
constexpr int CONV_WARP0 = 12;
constexpr int REGS_COMPILED_RAW = 96, REGS_CTRL = 32, REGS_EPI = 152, REGS_CONV = 72;
static_assert(128 * REGS_CTRL + 256 * REGS_EPI + 256 * REGS_CONV <= THREADS_RAW * REGS_COMPILED_RAW, "setmaxnreg pool");
constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;          // per epilogue warp: 32 rows x 32 cols
constexpr int SMEM_CTRL_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES + SMEM_CTRL_BYTES + 1024;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 12;                           // tile rasterisation group (rows of tiles)
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;  // 1 s per wait
constexpr unsigned long long DRAIN_LIMIT_NS = 2000000ull;    // 2 ms per drain wait

// status codes written to *status (first writer wins)
enum : int { ST_OK = 0, ST_TIMEOUT_PRODUCER = 1, ST_TIMEOUT_MMA_FULL = 2, ST_TIMEOUT_MMA_ACC = 3,
             ST_TIMEOUT_EPILOGUE = 4, ST_TIMEOUT_PARTIAL_FLAG = 5, ST_TIMEOUT_PARTIAL_PUBLISH = 6, ST_TIMEOUT_CONVERT = 7, ST_SELFTEST = 99 };

constexpr int SK_SLOT_FLOATS = BM * BN;               // one raw accumulator tile per published slice
constexpr int SK_MAX_SPLIT = 4;                       // at most this many K slices per tile (owner scheme)
constexpr int SK_COOP_MAX_SPLIT = 16;                 // cooperative scheme: S in {2, 4, 8, 16}
constexpr size_t SK_FLAG_BYTES = 16384;              // flag region at the head of the exchange area
constexpr int SK_MIN_KB = 8;                          // and each slice is at least this many k-blocks

struct Params
{
    float* c;
    int64_t m, n;
    int64_t ldc, stride_c;
    int32_t num_kb;
    int32_t tiles_m, tiles_n;
    int64_t total_tiles;           // tiles_per_mat * batch
    int64_t tiles_per_mat;         // tiles_m * tiles_n, or the tiles of the written triangle (tri_compact)
    int32_t tri_compact;           // 1: tile numbers run over the tiles of the triangle only (square tile grid)
    float alpha, beta;
    int32_t act;                   // epilogue activation (ACT_* of activation.cuh) applied to alpha*acc + beta*C
    float act_param;               // its parameter (leaky_relu, elu)
    int32_t lean_epilogue;         // 1: interior work items use the check-free epilogue path
    int32_t tri;                   // 0: full C; 1: only row >= col is written (lower triangle); 2: only row <= col
    int* status;
    // work distribution
    int64_t dp_tiles;              // tiles [0, dp_tiles) are dealt whole, round-robin over the grid
    int32_t sk_tiles;              // tiles [dp_tiles, dp_tiles + sk_tiles) are cut along K (0: none)
    int32_t sk_split;              // number of K slices per cut tile (>= 2 when sk_tiles > 0)
    int32_t sk_coop;               // 1: every slice publishes and each CTA finishes its own band of rows of the tile
    int32_t n_peers;               // fused all-gather: finished tiles are also stored to peer_c[0 .. n_peers)
    float* peer_c[7];              // the address of `c` inside each peer GPU's buffer
    int32_t raw_mask;              // bit 0: A arrives raw (split in kernel); bit 1: B arrives raw;
                                   // bit 2 / 3: that raw operand is row-contiguous (element (row, kk) at kk*ld + row)
                                   // and is also transposed by the converters
    float* sk_partials;            // [sk_tiles * (sk_split-1)][256*256] raw accumulators of slices 0 .. S-2 (all S when sk_coop)
    unsigned int* sk_flags;        // one per slot: epoch of the slot's last publication
    unsigned int sk_epoch;         // this launch's epoch (never 0)
};

// One unit of work of a CTA: k-blocks [kb0, kb1) of one tile.
struct WorkItem
{
    int64_t tile;
    int32_t kb0, kb1;
    int32_t kind;                  // 0 whole tile; 1 slice that publishes a partial; 2 last slice: owner of a cut tile;
                                   // 3 slice that publishes and then finishes rows [q, q+1) * 256/S of the tile
    int32_t slot;                  // kind 1, 3: slot to publish (q*sk_tiles + t); kind 2: slot of slice 0 (slice q at slot + q*sk_tiles)
};

// idx-th work item of CTA `cta` (identical enumeration in every role); false when exhausted.
// Items are numbered: whole tiles first, then (slice q, cut tile t) at dp_tiles + q*sk_tiles + t;
// item g belongs to CTA g % grid.
__device__ __forceinline__ bool get_work_item(const Params& p, int32_t cta, int32_t grid, int32_t idx, WorkItem& w)
{
    const int64_t g = cta + (int64_t)idx * grid;
    w.slot = 0;
    if (g < p.dp_tiles) { w.tile = g; w.kb0 = 0; w.kb1 = p.num_kb; w.kind = 0; return true; }
    const int64_t i = g - p.dp_tiles;
    if (i >= (int64_t)p.sk_tiles * p.sk_split) return false;
    const int32_t q = (int32_t)(i / p.sk_tiles), t = (int32_t)(i % p.sk_tiles);
    w.tile = p.dp_tiles + t;
    w.kb0 = (int32_t)((int64_t)q * p.num_kb / p.sk_split);
    w.kb1 = (int32_t)((int64_t)(q + 1) * p.num_kb / p.sk_split);
    if (p.sk_coop) { w.kind = 3; w.slot = q * p.sk_tiles + t; }
    else if (q == p.sk_split - 1) { w.kind = 2; w.slot = t; }
    else { w.kind = 1; w.slot = q * p.sk_tiles + t; }
    return true;
}

// Cooperative split-K finish of one warp: rows [q, q+1) * 256/S of a tile are the sum of the S published slots,
// added in slot order.  The reads are L2 round trips, so what matters is how many are in flight: a lane fetches
// sixteen float4 (16 / S positions of the band times S slots) before it adds the first, instead of S per position
// (which made the finish of an S = 2 tile 32 dependent round trips per warp, 35 us of a 150 us GEMM).
template <int S, typename Store>
__device__ __forceinline__ void coop_finish_band(const float* slot0, size_t cstride, int q_idx, int ew, int lane, Store&& store)
{
    constexpr int BAND = 256 / S, ROWS_PER_WARP = BAND / 8, POSITIONS = ROWS_PER_WARP * 2;   // (row, column half) per lane
    constexpr int GROUP = (16 / S) < POSITIONS ? (16 / S) : POSITIONS;
    static_assert(POSITIONS % GROUP == 0, "whole groups");
    for (int p0 = 0; p0 < POSITIONS; p0 += GROUP)
    {
        float4 t4[GROUP][S];
#pragma unroll
        for (int g = 0; g < GROUP; ++g)
        {
            const int trow = q_idx * BAND + ew * ROWS_PER_WARP + ((p0 + g) >> 1), col4 = lane + 32 * ((p0 + g) & 1);
            const float* src = slot0 + (size_t)trow * 256 + col4 * 4;
#pragma unroll
            for (int c = 0; c < S; ++c) t4[g][c] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)c * cstride));
        }
#pragma unroll
        for (int g = 0; g < GROUP; ++g)
        {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int c = 0; c < S; ++c) { sum.x += t4[g][c].x; sum.y += t4[g][c].y; sum.z += t4[g][c].z; sum.w += t4[g][c].w; }
            store(q_idx * BAND + ew * ROWS_PER_WARP + ((p0 + g) >> 1), lane + 32 * ((p0 + g) & 1), sum);
        }
    }
}

// Triangular output (SYRK): true when tile (tm, tn) lies wholly outside the triangle that is
// written, so that every role skips the work item.
__device__ __forceinline__ bool tile_outside_triangle(int32_t tri, int32_t tm, int32_t tn)
{
    if (tri == 1) return (int64_t)tn * BN > (int64_t)tm * BM + BM - 1;
    if (tri == 2) return (int64_t)tm * BM > (int64_t)tn * BN + BN - 1;
    return false;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* ptr)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* ptr, unsigned int v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait for a slot's publication flag (acquire).  Returns false when the CTA is aborting.
__device__ __forceinline__ bool flag_wait_bounded(const unsigned int* flag, unsigned int epoch, volatile int* abort_flag,
                                                  int* status, int code, unsigned long long limit_ns);

// Bounded wait.  Returns false when the CTA is aborting (own expiry or someone else's).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code, unsigned long long limit_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;)
    {
        if (mbar_try_wait(bar, parity)) return true;
        if (((++spins) & 0xFF) == 0)
        {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns)
            {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ bool flag_wait_bounded(const unsigned int* flag, unsigned int epoch, volatile int* abort_flag,
                                                  int* status, int code, unsigned long long limit_ns)
{
    if (ld_acquire_gpu(flag) == epoch) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_gpu(flag) != epoch)
    {
        if (((++spins) & 0x3F) == 0)
        {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns)
            {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2, int32_t c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// hi = rna_tf32(x), lo = rna_tf32(x - hi); inf / nan stay in hi only.
__device__ __forceinline__ void split_tf32_1(float x, float& hi, float& lo)
{
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    const float r = x - hi;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(r));
    lo = (fabsf(hi) <= 3.402823466e+38f) ? __uint_as_float(l) : 0.0f;
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::tf32, issued by one thread.
__device__ __forceinline__ void tcgen05_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tcgen05_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, SWIZZLE_64B: rows of 64 bytes, 8-row groups
// 512 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1.
__device__ __forceinline__ uint64_t make_desc_sw64(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;
    return d;
}

// Instruction descriptor: D fp32, A/B tf32, both K-major, N = 256, M = 128.
constexpr uint32_t IDESC_TF32_M128_N256 =
    (1u << 4) | (2u << 7) | (2u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

struct TileCoord { int64_t bi; int32_t tm, tn; };

__device__ __forceinline__ TileCoord decode_tile(int64_t t, const Params& p)
{
    TileCoord tc;
    tc.bi = t / p.tiles_per_mat;
    const int32_t r = (int32_t)(t % p.tiles_per_mat);
    if (p.tri_compact)
    {
        // r-th tile of the triangle, row by row: row i holds tiles (i, 0 .. i), i (i + 1) / 2 tiles before it
        int32_t i = (int32_t)((sqrtf(8.0f * (float)r + 1.0f) - 1.0f) * 0.5f);
        while ((i + 1) * (i + 2) / 2 <= r) ++i;
        while (i * (i + 1) / 2 > r) --i;
        const int32_t j = r - i * (i + 1) / 2;
        tc.tm = p.tri == 1 ? i : j;                  // lower: column <= row; upper: the mirror image
        tc.tn = p.tri == 1 ? j : i;
        return tc;
    }
    const int32_t tiles_m = p.tiles_m, tiles_n = p.tiles_n;
    const int32_t group = GROUP_M * tiles_n;
    const int32_t gid = r / group;
    const int32_t first_m = gid * GROUP_M;
    const int32_t gm = min(tiles_m - first_m, GROUP_M);
    tc.tm = first_m + (r % group) % gm;
    tc.tn = (r % group) / gm;
    return tc;
}

// Epilogue fast path for one warp's 32 x 256 region of a tile that lies wholly inside its
// destination, with 16-byte aligned rows and no triangle mask: no per-element checks, addresses by
// pointer increments, and the TMEM load of chunk c+1 issued as soon as chunk c has been written
// to the staging buffer, so that it is in flight while chunk c is stored.
// `dst` points at (first row of the warp + lane/8, first column of the tile + 4*(lane%8)) of the
// destination (C, or the slot of a published K slice with ldc = BN, alpha = 1).
// `contrib` (owner of a cut tile): the same position inside the first published slot; n_contrib
// slots, contrib_stride floats apart, are added before alpha/beta.
// ACT: 0 none, 1 ReLU, 2 any activation of activation.cuh (chosen at run time by `act`).
template <bool HAS_BETA, int ACT>
__device__ __forceinline__ void epilogue_fast(uint32_t taddr0, float4* stg, float* __restrict__ dst, int64_t ldc,
                                              float alpha, float beta, int lane,
                                              const float* contrib = nullptr, int n_contrib = 0, size_t contrib_stride = 0,
                                              int act = 0, float act_param = 0.0f)
{
    const int rsub = lane >> 3, c4 = lane & 7;
    const int64_t row_step = 4 * ldc;
    uint32_t v[32];
    tcgen05_ld_32x32b_x32(taddr0, v);
#pragma unroll 1
    for (int chunk = 0; chunk < BN / 32; ++chunk)
    {
        float4 old[8];
        if (HAS_BETA)
        {
            const float* src = dst + chunk * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i) old[i] = *reinterpret_cast<const float4*>(src + i * row_step);
        }
        tcgen05_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            float4 x;
            x.x = __uint_as_float(v[4 * j + 0]); x.y = __uint_as_float(v[4 * j + 1]);
            x.z = __uint_as_float(v[4 * j + 2]); x.w = __uint_as_float(v[4 * j + 3]);
            stg[lane * 8 + (j ^ (lane & 7))] = x;
        }
        if (chunk + 1 < BN / 32) tcgen05_ld_32x32b_x32(taddr0 + (chunk + 1) * 32, v);
        __syncwarp();
        float4 acc4[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const int r = i * 4 + rsub;
            acc4[i] = stg[r * 8 + (c4 ^ (r & 7))];
        }
        for (int c = 0; c < n_contrib; ++c)
        {
            const float* src = contrib + c * contrib_stride + chunk * 32;
            float4 t4[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t4[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)i * 4 * BN));
#pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                acc4[i].x += t4[i].x; acc4[i].y += t4[i].y; acc4[i].z += t4[i].z; acc4[i].w += t4[i].w;
            }
        }
        float* out = dst + chunk * 32;
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            float4 o;
            o.x = alpha * acc4[i].x; o.y = alpha * acc4[i].y; o.z = alpha * acc4[i].z; o.w = alpha * acc4[i].w;
            if (HAS_BETA)
            {
                o.x = fmaf(beta, old[i].x, o.x); o.y = fmaf(beta, old[i].y, o.y);
                o.z = fmaf(beta, old[i].z, o.z); o.w = fmaf(beta, old[i].w, o.w);
            }
            if (ACT == 1)
            {
                o.x = fmaxf(o.x, 0.0f); o.y = fmaxf(o.y, 0.0f); o.z = fmaxf(o.z, 0.0f); o.w = fmaxf(o.w, 0.0f);
            }
            if (ACT == 2)
            {
                o.x = apply_act(o.x, act, act_param); o.y = apply_act(o.y, act, act_param);
                o.z = apply_act(o.z, act, act_param); o.w = apply_act(o.w, act, act_param);
            }
            *reinterpret_cast<float4*>(out + i * row_step) = o;
        }
        __syncwarp();
    }
}

// PRODUCTS: 3 issues lo*hi + hi*lo + hi*hi per k-step (fp32 accuracy); 1 only hi*hi (rate probe, TF32 accuracy).  A
// compile-time choice: the MMA-issuing thread is on the critical path and a run-time test in its loop costs 7 %.
// RAW: the launch has at least one raw operand (640 threads, dedicated converter warps); otherwise 320 threads.
template <int REGS> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS)); }
template <int REGS> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS)); }

template <int PRODUCTS, bool RAW>
__global__ void __launch_bounds__(RAW ? THREADS_RAW : THREADS, 1)
sgemm_tc3x_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap raw_a, const __grid_constant__ CUtensorMap raw_b,
                  const __grid_constant__ Params p)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment keeps every plane base on a swizzle-pattern boundary
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* epi_base = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + EPI_WARPS * EPI_STAGE_BYTES);
    // bars[0..2] full, [3..5] empty, [6] acc_full, [7..8] acc_empty, [9] drain, [10] partial written,
    // [11..13] converted (raw operands split in place)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 15);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const uint32_t full0 = smem_u32(bars + 0), empty0 = smem_u32(bars + 3);
    const uint32_t acc_full = smem_u32(bars + 6), acc_empty0 = smem_u32(bars + 7);
    const uint32_t drain = smem_u32(bars + 9), partial_done = smem_u32(bars + 10), conv0 = smem_u32(bars + 11);
    const bool a_raw = (p.raw_mask & 1) != 0, b_raw = (p.raw_mask & 2) != 0;
    const bool a_mn = (p.raw_mask & 4) != 0, b_mn = (p.raw_mask & 8) != 0;       // raw and row-contiguous

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; ++s)
        {
            mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); mbar_init(conv0 + 8 * s, EPI_WARPS);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty0, EPI_WARPS / 2);
        mbar_init(acc_empty0 + 8, EPI_WARPS / 2);
        mbar_init(drain, 1);
        mbar_init(partial_done, EPI_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int32_t cta = (int32_t)blockIdx.x, grid = (int32_t)gridDim.x;
    constexpr int EPI_WARP0 = RAW ? 4 : 2;       // first epilogue warp (warp & 3 is the TMEM lane quarter either way)

    // With a raw operand every branch below starts with its warpgroup's setmaxnreg (all four warps of a group run it).
    if (RAW && warp >= 2 && warp < 4)
    {
        reg_dec<REGS_CTRL>();                    // the two idle warps of the control group
    }
    else if (warp == 0)
    {
        if (RAW) reg_dec<REGS_CTRL>();
        // ------------------------------------------------------------ TMA producer
        uint32_t it = 0;
        bool ok = true;
        WorkItem w;
        for (int32_t idx = 0; ok && get_work_item(p, cta, grid, idx, w); ++idx)
        {
            const TileCoord tc = decode_tile(w.tile, p);
            if (tile_outside_triangle(p.tri, tc.tm, tc.tn)) continue;
            for (int32_t kb = w.kb0; kb < w.kb1 && ok; ++kb, ++it)
            {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                int okl = 1;
                if (lane == 0)
                {
                    okl = mbar_wait_bounded(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER, WAIT_LIMIT_NS);
                    if (okl)
                    {
                        const uint32_t dst = smem_u32(stage_base + s * STAGE_BYTES);
                        const uint32_t bar = full0 + 8 * s;
                        mbar_arrive_expect_tx(bar, (a_raw ? PLANE_BYTES : OPERAND_BYTES) + (b_raw ? PLANE_BYTES : OPERAND_BYTES));
                        if (a_mn)
                        {
                            // eight boxes of 32 rows x 16 k, box g into the 2 KB of the lo slot that converter warp g rewrites
#pragma unroll
                            for (int g = 0; g < EPI_WARPS; ++g)
                                tma_load_3d(dst + PLANE_BYTES + g * (PLANE_BYTES / EPI_WARPS), &raw_a, bar, tc.tm * BM + 32 * g, kb * BK,
                                            (int32_t)tc.bi);
                        }
                        else if (a_raw) tma_load_3d(dst, &raw_a, bar, kb * BK, tc.tm * BM, (int32_t)tc.bi);
                        else tma_load_4d(dst, &map_a, bar, 0, tc.tm * BM, kb, (int32_t)(tc.bi * 2));
                        if (b_mn)
                        {
#pragma unroll
                            for (int g = 0; g < EPI_WARPS; ++g)
                                tma_load_3d(dst + OPERAND_BYTES + PLANE_BYTES + g * (PLANE_BYTES / EPI_WARPS), &raw_b, bar,
                                            tc.tn * BN + 32 * g, kb * BK, (int32_t)tc.bi);
                        }
                        else if (b_raw) tma_load_3d(dst + OPERAND_BYTES, &raw_b, bar, kb * BK, tc.tn * BN, (int32_t)tc.bi);
                        else tma_load_4d(dst + OPERAND_BYTES, &map_b, bar, 0, tc.tn * BN, kb, (int32_t)(tc.bi * 2));
                    }
                }
                ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
            }
        }
        if (!ok && lane == 0)
        {
            // drain: wait (bounded) for the loads already issued into the ring
            const uint32_t lo = it > STAGES ? it - STAGES : 0;
            for (uint32_t j = lo; j < it; ++j)
            {
                const uint32_t bar = full0 + 8 * (j % STAGES), par = (j / STAGES) & 1;
                const unsigned long long t0 = globaltimer_ns();
                while (!mbar_try_wait(bar, par) && globaltimer_ns() - t0 < DRAIN_LIMIT_NS) {}
            }
        }
        __syncwarp();
    }
    else if (warp == 1)
    {
        if (RAW) reg_dec<REGS_CTRL>();
        // ------------------------------------------------------------ MMA issuer
        uint32_t it = 0, tl = 0;
        bool ok = true;
        WorkItem w;
        for (int32_t idx = 0; ok && get_work_item(p, cta, grid, idx, w); ++idx)
        {
            {
                const TileCoord tc = decode_tile(w.tile, p);
                if (tile_outside_triangle(p.tri, tc.tm, tc.tn)) continue;
            }
            const uint32_t tl_now = tl++;
            for (int32_t kb = w.kb0; kb < w.kb1 && ok; ++kb, ++it)
            {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                int okl = 1;
                if (lane == 0)
                {
                    // raw operands: wait for the converter warps (which waited for the TMA data)
                    okl = mbar_wait_bounded((p.raw_mask ? conv0 : full0) + 8 * s, ph, abort_flag, p.status,
                                            ST_TIMEOUT_MMA_FULL, WAIT_LIMIT_NS);
                    if (okl && kb == w.kb0)
                    {
                        // both accumulator halves must have been drained by the previous tile's epilogue
                        okl = mbar_wait_bounded(acc_empty0, (tl_now & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA_ACC, WAIT_LIMIT_NS) &&
                              mbar_wait_bounded(acc_empty0 + 8, (tl_now & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA_ACC, WAIT_LIMIT_NS);
                    }
                    if (okl)
                    {
                        tcgen05_fence_after();
                        const uint32_t a_addr = smem_u32(stage_base + s * STAGE_BYTES);
                        const uint32_t b_addr = a_addr + OPERAND_BYTES;
                        const uint64_t b_hi = make_desc_sw64(b_addr);
                        const uint64_t b_lo = make_desc_sw64(b_addr + PLANE_BYTES);
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                        {
                            const uint64_t a_hi = make_desc_sw64(a_addr + h * (128 * BK * 4));
                            const uint64_t a_lo = make_desc_sw64(a_addr + PLANE_BYTES + h * (128 * BK * 4));
                            const uint32_t d = tmem_base + h * 256;
#pragma unroll
                            for (int ks = 0; ks < BK / 8; ++ks)
                            {
                                const uint64_t koff = (uint64_t)((ks * 8 * 4) >> 4);   // +32 bytes per k-step
                                const uint32_t acc = (kb > w.kb0 || ks > 0) ? 1u : 0u;   // a run starts from zero
                                // small terms first, then the leading product
                                if (PRODUCTS == 3)
                                {
                                    tcgen05_mma_tf32(d, a_lo + koff, b_hi + koff, IDESC_TF32_M128_N256, acc);
                                    tcgen05_mma_tf32(d, a_hi + koff, b_lo + koff, IDESC_TF32_M128_N256, 1u);
                                    tcgen05_mma_tf32(d, a_hi + koff, b_hi + koff, IDESC_TF32_M128_N256, 1u);
                                }
                                else tcgen05_mma_tf32(d, a_hi + koff, b_hi + koff, IDESC_TF32_M128_N256, acc);
                            }
                        }
                        tcgen05_commit(empty0 + 8 * s);               // stage reusable once these MMAs retire
                        if (kb == w.kb1 - 1) tcgen05_commit(acc_full);     // accumulators of this run complete
                    }
                }
                ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
            }
        }
        if (!ok && lane == 0)
        {
            // drain outstanding MMAs before TMEM is released
            tcgen05_commit(drain);
            const unsigned long long t0 = globaltimer_ns();
            while (!mbar_try_wait(drain, 0) && globaltimer_ns() - t0 < DRAIN_LIMIT_NS) {}
        }
        __syncwarp();
    }
    else if (RAW && warp >= CONV_WARP0)
    {
        reg_dec<REGS_CONV>();
        // ------------------------------------------------------------ converter warps (launches with a raw operand)
        // Split the raw operand tiles of every stage in place: hi = rna_tf32(x) over the raw values, lo beside it.
        const int ew = warp - CONV_WARP0;        // 0..7: the 32 rows of a tile this warp converts
        const int te = ew * 32 + lane;           // 0..255
        uint32_t it = 0;
        bool ok = true;
        WorkItem w;
        for (int32_t idx = 0; ok && get_work_item(p, cta, grid, idx, w); ++idx)
        {
            {
                const TileCoord tc = decode_tile(w.tile, p);
                if (tile_outside_triangle(p.tri, tc.tm, tc.tn)) continue;
            }
            for (int32_t kb = w.kb0; kb < w.kb1 && ok; ++kb, ++it)
            {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                const int okc = mbar_wait_bounded(full0 + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_CONVERT, WAIT_LIMIT_NS);
                ok = __all_sync(0xffffffffu, okc) != 0;
                if (!ok) break;
                uint8_t* stage = stage_base + s * STAGE_BYTES;
#pragma unroll
                for (int op = 0; op < 2; ++op)
                {
                    if (!((p.raw_mask >> op) & 1)) continue;
                    float4* hi = reinterpret_cast<float4*>(stage + op * OPERAND_BYTES);
                    float4* lo = reinterpret_cast<float4*>(stage + op * OPERAND_BYTES + PLANE_BYTES);
                    if ((p.raw_mask >> (op + 2)) & 1)
                    {
                        // Row-contiguous operand: this warp's 32 rows arrived as [16 k][32 rows] in the 2 KB of
                        // the lo slot that hold these rows' lo values afterwards, so reading before writing is
                        // a matter of this warp alone.  A lane takes one row: 16 conflict-free loads, then the
                        // row's 64 bytes of hi and of lo in the MMA's K-major layout (16-byte chunk c of row r
                        // at position c ^ ((r >> 1) & 3): SWIZZLE_64B).
                        const float* raw = reinterpret_cast<const float*>(lo) + ew * (32 * BK);
                        float x[BK];
#pragma unroll
                        for (int kk = 0; kk < BK; ++kk) x[kk] = raw[kk * 32 + lane];
                        __syncwarp();
                        const int r = ew * 32 + lane;
#pragma unroll
                        for (int c = 0; c < BK / 4; ++c)
                        {
                            float4 h4, l4;
                            split_tf32_1(x[4 * c + 0], h4.x, l4.x); split_tf32_1(x[4 * c + 1], h4.y, l4.y);
                            split_tf32_1(x[4 * c + 2], h4.z, l4.z); split_tf32_1(x[4 * c + 3], h4.w, l4.w);
                            const int pos = r * (BK / 4) + (c ^ ((r >> 1) & 3));
                            hi[pos] = h4;
                            lo[pos] = l4;
                        }
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < PLANE_BYTES / 16 / (EPI_WARPS * 32); ++j)
                    {
                        const int e = te + j * (EPI_WARPS * 32);
                        const float4 x = hi[e];
                        float4 h4, l4;
                        split_tf32_1(x.x, h4.x, l4.x); split_tf32_1(x.y, h4.y, l4.y);
                        split_tf32_1(x.z, h4.z, l4.z); split_tf32_1(x.w, h4.w, l4.w);
                        hi[e] = h4;
                        lo[e] = l4;
                    }
                }
                // generic-proxy writes must be visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(conv0 + 8 * s);
            }
        }
    }
    else if (warp >= EPI_WARP0 && warp < EPI_WARP0 + EPI_WARPS)
    {
        if (RAW) reg_inc<REGS_EPI>();
        // ------------------------------------------------------------ epilogue warps
        const int ew = warp - EPI_WARP0;         // 0..7
        const int h = ew >> 2;                   // accumulator half (rows h*128 ..)
        const int q = warp & 3;                  // TMEM lane quarter this warp may access
        float4* stg = reinterpret_cast<float4*>(epi_base + ew * EPI_STAGE_BYTES);   // [32 rows][8 float4]
        const bool has_beta = (p.beta != 0.0f);
        const int rsub = lane >> 3, c4 = lane & 7;
        uint32_t tl = 0, published = 0;
        bool ok = true;
        WorkItem w;
        for (int32_t idx = 0; ok && get_work_item(p, cta, grid, idx, w); ++idx)
        {
            const TileCoord tc = decode_tile(w.tile, p);
            if (tile_outside_triangle(p.tri, tc.tm, tc.tn)) continue;
            const uint32_t tl_now = tl++;
            int okl = mbar_wait_bounded(acc_full, tl_now & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE, WAIT_LIMIT_NS);
            if (okl && w.kind == 2)
            {
                // owner of a cut tile: the earlier slices must have been published
                for (int32_t c = 0; c < p.sk_split - 1 && okl; ++c)
                {
                    const unsigned int* flag = p.sk_flags + (w.slot + c * p.sk_tiles);
                    const unsigned long long t0 = globaltimer_ns();
                    uint32_t spins = 0;
                    while (ld_acquire_gpu(flag) != p.sk_epoch)
                    {
                        if (((++spins) & 0x3F) == 0)
                        {
                            if (*abort_flag) { okl = 0; break; }
                            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS)
                            {
                                *abort_flag = 1;
                                atomicCAS(p.status, 0, (int)ST_TIMEOUT_PARTIAL_FLAG);
                                okl = 0;
                                break;
                            }
                        }
                    }
                }
            }
            ok = __all_sync(0xffffffffu, okl) != 0;
            if (!ok) break;
            tcgen05_fence_after();

            float* __restrict__ cb = p.c + tc.bi * p.stride_c;
            const int64_t row_base = (int64_t)tc.tm * BM + h * 128 + q * 32;   // first row of this warp
            const int64_t col_base = (int64_t)tc.tn * BN;
            const bool vec_ok = ((p.ldc & 3) == 0) && ((p.stride_c & 3) == 0) &&
                                ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0);
            const bool partial = (w.kind == 1 || w.kind == 3);
            // slot element of (tile row, tile col): row-major 256 x 256
            float* my_slot = partial ? p.sk_partials + (size_t)w.slot * SK_SLOT_FLOATS : nullptr;
            const int slot_row0 = h * 128 + q * 32;

            // work items that lie wholly inside their destination take the lean path
            const bool inside_c = p.lean_epilogue && vec_ok && p.tri == 0 && row_base + 32 <= p.m && col_base + BN <= p.n;
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 256);
            const size_t slot_pos = (size_t)(slot_row0 + rsub) * BN + c4 * 4;       // this lane inside a 256 x 256 slot
            if (partial && p.lean_epilogue)
            {
                // raw accumulators into this slice's slot (alpha = 1, no beta, dense 256-wide rows)
                epilogue_fast<false, 0>(taddr0, stg, my_slot + slot_pos, BN, 1.0f, 0.0f, lane);
            }
            else if (inside_c)
            {
                float* dst = cb + (row_base + rsub) * p.ldc + col_base + c4 * 4;
                const float* contrib = w.kind == 2 ? p.sk_partials + (size_t)w.slot * SK_SLOT_FLOATS + slot_pos : nullptr;
                const int n_contrib = w.kind == 2 ? p.sk_split - 1 : 0;
                const size_t cstride = (size_t)p.sk_tiles * SK_SLOT_FLOATS;
                if (has_beta)
                {
                    if (p.act > ACT_RELU)
                        epilogue_fast<true, 2>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride, p.act, p.act_param);
                    else if (p.act) epilogue_fast<true, 1>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride);
                    else epilogue_fast<true, 0>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride);
                }
                else
                {
                    if (p.act > ACT_RELU)
                        epilogue_fast<false, 2>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride, p.act, p.act_param);
                    else if (p.act) epilogue_fast<false, 1>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride);
                    else epilogue_fast<false, 0>(taddr0, stg, dst, p.ldc, p.alpha, p.beta, lane, contrib, n_contrib, cstride);
                }
            }
            else if (partial || row_base < p.m)
            {
                for (int chunk = 0; chunk < BN / 32; ++chunk)
                {
                    const int64_t col0 = col_base + chunk * 32;
                    if (!partial && col0 >= p.n) break;
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 256 + chunk * 32);
                    tcgen05_ld_32x32b_x32(taddr, v);

                    // old C values for the beta term, fetched while the TMEM load is in flight
                    float4 old[8];
                    const int64_t gcol = col0 + c4 * 4;
                    if (!partial && has_beta && vec_ok)
                    {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                        {
                            const int64_t grow = row_base + i * 4 + rsub;
                            old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                            const bool tri_all = p.tri == 0 || (p.tri == 1 ? gcol + 3 <= grow : gcol >= grow);
                            if (grow < p.m && gcol + 3 < p.n && tri_all)
                                old[i] = *reinterpret_cast<const float4*>(cb + grow * p.ldc + gcol);
                        }
                    }
                    tcgen05_wait_ld();

                    // registers (row = lane, 32 columns) -> shared, float4 index XOR-swizzled by row
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                    {
                        float4 x;
                        x.x = __uint_as_float(v[4 * j + 0]); x.y = __uint_as_float(v[4 * j + 1]);
                        x.z = __uint_as_float(v[4 * j + 2]); x.w = __uint_as_float(v[4 * j + 3]);
                        stg[lane * 8 + (j ^ (lane & 7))] = x;
                    }
                    __syncwarp();
                    float4 acc4[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                    {
                        const int r = i * 4 + rsub;
                        acc4[i] = stg[r * 8 + (c4 ^ (r & 7))];
                    }
                    const size_t slot_off0 = (size_t)(slot_row0 + rsub) * BN + chunk * 32 + c4 * 4;   // row r = i*4 + rsub
                    if (partial)
                    {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            __stcg(reinterpret_cast<float4*>(my_slot + slot_off0 + (size_t)i * 4 * BN), acc4[i]);
                    }
                    else
                    {
                        if (w.kind == 2)
                        {
                            // add the published slices; eight independent 128-bit loads in flight per slice
                            for (int32_t c = 0; c < p.sk_split - 1; ++c)
                            {
                                const float* src = p.sk_partials + (size_t)(w.slot + c * p.sk_tiles) * SK_SLOT_FLOATS + slot_off0;
                                float4 t4[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    t4[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)i * 4 * BN));
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                {
                                    acc4[i].x += t4[i].x; acc4[i].y += t4[i].y; acc4[i].z += t4[i].z; acc4[i].w += t4[i].w;
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                        {
                            const float4 a = acc4[i];
                            const int64_t grow = row_base + i * 4 + rsub;
                            if (grow >= p.m || gcol >= p.n) continue;
                            float* dst = cb + grow * p.ldc + gcol;
                            // triangular output: 4 columns wholly inside -> vector path; straddling -> per element
                            const bool tri_all = p.tri == 0 || (p.tri == 1 ? gcol + 3 <= grow : gcol >= grow);
                            if (vec_ok && gcol + 3 < p.n && tri_all)
                            {
                                float4 o;
                                o.x = p.alpha * a.x; o.y = p.alpha * a.y; o.z = p.alpha * a.z; o.w = p.alpha * a.w;
                                if (has_beta)
                                {
                                    o.x = fmaf(p.beta, old[i].x, o.x); o.y = fmaf(p.beta, old[i].y, o.y);
                                    o.z = fmaf(p.beta, old[i].z, o.z); o.w = fmaf(p.beta, old[i].w, o.w);
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
                                const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                {
                                    const bool inside = p.tri == 0 || (p.tri == 1 ? gcol + j <= grow : gcol + j >= grow);
                                    if (gcol + j < p.n && inside)
                                    {
                                        float o = p.alpha * av[j];
                                        if (has_beta) o = fmaf(p.beta, dst[j], o);
                                        dst[j] = apply_act(o, p.act, p.act_param);
                                    }
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            // this warp is done reading accumulator half h of this run
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * h);

            if (p.n_peers > 0 && !partial && vec_ok && row_base < p.m)
            {
                // Fused all-gather: with the accumulators released (the next run's MMAs proceed),
                // copy this warp's 32 x 256 region of the finished tile to every peer.  Each
                // thread re-reads exactly the elements it stored above, so no fence is needed
                // before the loads; the loads hit L2.
                for (int chunk = 0; chunk < BN / 32; ++chunk)
                {
                    const int64_t gcol = col_base + chunk * 32 + c4 * 4;
                    if (col_base + chunk * 32 >= p.n) break;
                    float4 vals[8];
                    bool live[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                    {
                        const int64_t grow = row_base + i * 4 + rsub;
                        live[i] = grow < p.m && gcol + 3 < p.n;
                        if (live[i]) vals[i] = *reinterpret_cast<const float4*>(cb + grow * p.ldc + gcol);
                    }
                    for (int32_t peer = 0; peer < p.n_peers; ++peer)
                    {
                        float* pb = p.peer_c[peer] + tc.bi * p.stride_c;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (live[i])
                                *reinterpret_cast<float4*>(pb + (row_base + i * 4 + rsub) * p.ldc + gcol) = vals[i];
                    }
                }
                __threadfence_system();
            }

            if (partial)
            {
                // publish the slot: every warp fences its stores and arrives; one thread waits
                // (bounded) for all eight and releases the flag
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(partial_done);
                if (ew == 0 && lane == 0)
                {
                    if (mbar_wait_bounded(partial_done, published & 1, abort_flag, p.status, ST_TIMEOUT_PARTIAL_PUBLISH,
                                          WAIT_LIMIT_NS))
                    {
                        __threadfence();
                        st_release_gpu(p.sk_flags + w.slot, p.sk_epoch);
                    }
                }
                ++published;
            }

            if (w.kind == 3)
            {
                // Cooperative finish: when all S slices of the tile are published, this CTA adds rows
                // [q, q+1) * 256/S of the S slots (always in slot order, so the sum does not depend on
                // timing) and applies alpha / beta: every CTA reads 256 KB whatever S is, instead of one
                // owner reading (S-1) * 256 KB.  All S CTAs of a tile are co-resident (the plan deals at
                // most one item per CTA), nobody waits before publishing, and the waits are bounded.
                int okc = 1;
                const int32_t t_idx = w.slot % p.sk_tiles, q_idx = w.slot / p.sk_tiles;
                for (int32_t c = 0; c < p.sk_split && okc; ++c)
                    okc = flag_wait_bounded(p.sk_flags + (c * p.sk_tiles + t_idx), p.sk_epoch, abort_flag, p.status,
                                            ST_TIMEOUT_PARTIAL_FLAG, WAIT_LIMIT_NS) ? 1 : 0;
                ok = __all_sync(0xffffffffu, okc) != 0;
                if (!ok) break;
                const float* slot0 = p.sk_partials + (size_t)t_idx * SK_SLOT_FLOATS;
                const size_t cstride = (size_t)p.sk_tiles * SK_SLOT_FLOATS;
                // one float4 of the finished tile: row `trow` of the tile, columns 4 * col4 ..
                auto finish_store = [&](int trow, int col4, const float4& sum)
                {
                    const int64_t grow = (int64_t)tc.tm * BM + trow;
                    const int64_t gcol = col_base + col4 * 4;
                    if (grow >= p.m || gcol >= p.n) return;
                    float* dst = cb + grow * p.ldc + gcol;
                    const bool tri_all = p.tri == 0 || (p.tri == 1 ? gcol + 3 <= grow : gcol >= grow);
                    if (vec_ok && gcol + 3 < p.n && tri_all)
                    {
                        float4 o;
                        o.x = p.alpha * sum.x; o.y = p.alpha * sum.y; o.z = p.alpha * sum.z; o.w = p.alpha * sum.w;
                        if (has_beta)
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
                        for (int32_t peer = 0; peer < p.n_peers; ++peer)
                            *reinterpret_cast<float4*>(p.peer_c[peer] + tc.bi * p.stride_c + grow * p.ldc + gcol) = o;
                    }
                    else
                    {
                        const float av[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                        {
                            const bool inside = p.tri == 0 || (p.tri == 1 ? gcol + j <= grow : gcol + j >= grow);
                            if (gcol + j < p.n && inside)
                            {
                                float o = p.alpha * av[j];
                                if (has_beta) o = fmaf(p.beta, dst[j], o);
                                o = apply_act(o, p.act, p.act_param);
                                dst[j] = o;
                                for (int32_t peer = 0; peer < p.n_peers; ++peer)
                                    p.peer_c[peer][tc.bi * p.stride_c + grow * p.ldc + gcol + j] = o;
                            }
                        }
                    }
                };
                if (p.sk_split == 2) coop_finish_band<2>(slot0, cstride, q_idx, ew, lane, finish_store);
                else if (p.sk_split == 4) coop_finish_band<4>(slot0, cstride, q_idx, ew, lane, finish_store);
                else if (p.sk_split == 8) coop_finish_band<8>(slot0, cstride, q_idx, ew, lane, finish_store);
                else coop_finish_band<16>(slot0, cstride, q_idx, ew, lane, finish_store);
                if (p.n_peers > 0) __threadfence_system();
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
    {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// One CTA, one thread: the bounded wait on a barrier that never completes (failure-detection
// self-test).  Returns after limit_ns with ST_SELFTEST in *status.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0)
    {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, status, ST_SELFTEST, limit_ns);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn)
    {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Tensor map over plane[batch*2][num_kb][rows_pad][16]; box = {16 k, 256 rows, 1 k-block, 2 planes}.
inline bool make_plane_map(CUtensorMap* map, const float* planes, int64_t rows_pad, int64_t num_kb, int64_t batch)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t gdim[4] = {(cuuint64_t)BK, (cuuint64_t)rows_pad, (cuuint64_t)num_kb, (cuuint64_t)(2 * batch)};
    cuuint64_t gstr[3] = {(cuuint64_t)BK * 4, (cuuint64_t)rows_pad * BK * 4, (cuuint64_t)num_kb * rows_pad * BK * 4};
    cuuint32_t box[4] = {(cuuint32_t)BK, 256u, 1u, 2u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(planes), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Split-K tail plan for `tiles` tiles on `sm_count` SMs (see the header comment).
struct TailPlan { int64_t dp_tiles; int32_t sk_tiles, sk_split; int64_t grid; int32_t coop; };

inline TailPlan plan_tail(int64_t tiles, int64_t num_kb, int sm_count, bool allow_split)
{
    TailPlan t{tiles, 0, 1, tiles < sm_count ? tiles : sm_count, 0};
    // With at least one tile per SM the tail is not cut: measured on B200 (power-capped clocks,
    // fix-up traffic) the gain of a balanced last round does not cover the exchange.
    if (!allow_split || tiles <= 0 || tiles >= sm_count) return t;
    // Few tiles: cut K in S = 2, 4, 8 or 16 slices with one slice per CTA (all co-resident) and let
    // every CTA finish its own band of rows.  The exchange then costs a fixed ~7 us (256 KB written
    // and 256 KB read per CTA) whatever S is, so the largest S that fits the grid wins as long as a
    // slice keeps a few k-blocks: slice main loop 0.9 us per k-block against the fixed cost.
    {
        int s = 1;
        while (s * 2 <= SK_COOP_MAX_SPLIT && tiles * (s * 2) <= sm_count && num_kb / (s * 2) >= SK_MIN_KB) s *= 2;
        if (s >= 2 && (double)num_kb * 0.9 * (1.0 - 1.0 / s) > 8.0)
        {
            t.dp_tiles = 0; t.sk_tiles = (int32_t)tiles; t.sk_split = s; t.grid = tiles * s; t.coop = 1;
            return t;
        }
    }
    // Cost in units of one whole-tile main loop: rounds/S plus the fix-up, which is a fixed
    // time per published slice (slot write + owner's read) and so weighs 7/num_kb of a tile.
    int best_s = 1;
    double best = 1.0;
    for (int s = 2; s <= SK_MAX_SPLIT; ++s)
    {
        if (num_kb / s < SK_MIN_KB) break;
        const double cost = (double)((tiles * s + sm_count - 1) / sm_count) / s + (s - 1) * 7.0 / (double)num_kb;
        if (cost < best - 0.02) { best = cost; best_s = s; }
    }
    if (best_s == 1) return t;
    t.dp_tiles = 0; t.sk_tiles = (int32_t)tiles; t.sk_split = best_s;
    t.grid = tiles * best_s < sm_count ? tiles * best_s : sm_count;
    return t;
}

// Exchange area layout: SK_FLAG_BYTES of epoch flags (one per published slice, at fixed offsets so
// that a flag never aliases old slot data), then one 256 x 256 fp32 slot per published slice.
// The flag region must be zero-filled when the area is allocated.
inline size_t sk_area_bytes(const TailPlan& t)
{
    const size_t slots = (size_t)t.sk_tiles * (size_t)(t.coop ? t.sk_split : t.sk_split - 1);
    return slots ? SK_FLAG_BYTES + slots * (SK_SLOT_FLOATS * sizeof(float)) : 0;
}

// Work items of a problem: tiles (of the written triangle only when `tri` and the tile grid is square, which is
// what SYRK gives: dealing the tiles outside it too would leave the CTAs that drew them idle) and k-blocks.
inline bool triangle_is_compact(int64_t m, int64_t n, int tri)
{
    return tri != 0 && BM == BN && (m + BM - 1) / BM == (n + BN - 1) / BN;
}
inline void tile_counts(int64_t m, int64_t n, int64_t k, int64_t batch, int tri, int64_t* tiles, int64_t* num_kb)
{
    const int64_t tm = (m + BM - 1) / BM, tn = (n + BN - 1) / BN;
    *tiles = (triangle_is_compact(m, n, tri) ? tm * (tm + 1) / 2 : tm * tn) * batch;
    *num_kb = (k + BK - 1) / BK;
}

// planes_a / planes_b as written by launch_split_tf32 for op(A) (rows = m) and op(B)^T (rows = n).
// Tensor map over a user operand whose k index is contiguous: element (row, kk) at
// base[bi*stride + row*ld + kk]; box = {16 k, 256 rows, 1}; outside rows/k reads as zero.
inline bool make_raw_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int64_t stride,
                         int64_t batch)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t gdim[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t gstr[2] = {(cuuint64_t)ld * 4, (cuuint64_t)(batch > 1 ? stride : rows * ld) * 4};
    cuuint32_t box[3] = {(cuuint32_t)BK, 256u, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Raw row-contiguous operand (element (row, kk) at base[kk*ld + row]): boxes of 32 rows x 16 k, dense.
inline bool make_raw_mn_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int64_t stride,
                            int64_t batch)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t gdim[3] = {(cuuint64_t)rows, (cuuint64_t)k, (cuuint64_t)batch};
    cuuint64_t gstr[2] = {(cuuint64_t)ld * 4, (cuuint64_t)(batch > 1 ? stride : k * ld) * 4};
    cuuint32_t box[3] = {32u, (cuuint32_t)BK, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// True when a k-contiguous operand can be fetched raw by TMA: 16-byte aligned base, leading
// dimension and batch stride multiples of 4 floats, extents within the tensor-map limits.
inline bool raw_eligible(const float* base, int64_t rows, int64_t k, int64_t ld, int64_t stride, int64_t batch)
{
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld & 3) != 0) return false;
    if (batch > 1 && ((stride & 3) != 0 || stride <= 0)) return false;
    if (ld * 4 >= (1ll << 40) || (batch > 1 ? stride : rows * ld) * 4 >= (1ll << 40)) return false;
    return rows > 0 && k > 0 && rows < (1ll << 32) && k < (1ll << 32);
}

// One operand of the GEMM kernel: either pre-split planes (split_tf32.cuh) or the raw
// k-contiguous user matrix.
struct OperandSource
{
    const float* planes = nullptr;     // pre-split hi/lo planes, or
    const float* raw = nullptr;        // raw operand: element (row, kk) at raw[bi*stride + row*ld + kk],
    int64_t ld = 0, stride = 0;
    bool row_contig = false;           // ... or, when set, at raw[bi*stride + kk*ld + row]
};

// a / b: op(A) (rows = m) and op(B)^T (rows = n).
// sk_area: zero-initialised exchange area of at least sk_area_bytes(plan) bytes, or nullptr to
// deal whole tiles only; sk_epoch: a value never used before with this area (and never 0).
// products: 3 for the fp32-accurate product; 1 issues only the hi*hi MMAs (rate probe, TF32 accuracy).
inline cudaError_t launch_sgemm_tc3x(const OperandSource& a, const OperandSource& b, float* c,
                                     int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t stride_c, int64_t batch,
                                     float alpha, float beta, int* status, int sm_count, cudaStream_t st,
                                     void* sk_area = nullptr, unsigned int sk_epoch = 0,
                                     float* const* peer_c = nullptr, int n_peers = 0, int act = 0, int tri = 0,
                                     float act_param = 0.0f, int products = 3)
{
    // per-device attribute; cheap enough to set on every launch
    const bool any_raw = a.raw != nullptr || b.raw != nullptr;
    cudaError_t e = products == 1
        ? cudaFuncSetAttribute(sgemm_tc3x_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)
        : any_raw ? cudaFuncSetAttribute(sgemm_tc3x_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)
                  : cudaFuncSetAttribute(sgemm_tc3x_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (products == 1 && any_raw) return cudaErrorInvalidValue;       // the rate probe runs over planes only
    const int64_t m_pad = (m + 255) / 256 * 256, n_pad = (n + 255) / 256 * 256;
    const int64_t num_kb = (k + BK - 1) / BK;
    CUtensorMap map_a, map_b, raw_a, raw_b;
    Params p;
    if (n_peers < 0 || n_peers > 7) return cudaErrorInvalidValue;
    p.n_peers = n_peers;
    for (int i = 0; i < 7; ++i) p.peer_c[i] = (i < n_peers) ? peer_c[i] : nullptr;
    p.raw_mask = (a.raw ? 1 : 0) | (b.raw ? 2 : 0) | (a.raw && a.row_contig ? 4 : 0) | (b.raw && b.row_contig ? 8 : 0);
    if (a.raw && a.row_contig) { if (!make_raw_mn_map(&raw_a, a.raw, m, k, a.ld, a.stride, batch)) return cudaErrorInvalidValue; map_a = raw_a; }
    else if (a.raw) { if (!make_raw_map(&raw_a, a.raw, m, k, a.ld, a.stride, batch)) return cudaErrorInvalidValue; map_a = raw_a; }
    else { if (!make_plane_map(&map_a, a.planes, m_pad, num_kb, batch)) return cudaErrorInvalidValue; raw_a = map_a; }
    if (b.raw && b.row_contig) { if (!make_raw_mn_map(&raw_b, b.raw, n, k, b.ld, b.stride, batch)) return cudaErrorInvalidValue; map_b = raw_b; }
    else if (b.raw) { if (!make_raw_map(&raw_b, b.raw, n, k, b.ld, b.stride, batch)) return cudaErrorInvalidValue; map_b = raw_b; }
    else { if (!make_plane_map(&map_b, b.planes, n_pad, num_kb, batch)) return cudaErrorInvalidValue; raw_b = map_b; }
    p.c = c; p.m = m; p.n = n; p.ldc = ldc; p.stride_c = stride_c;
    p.num_kb = (int32_t)num_kb;
    p.tiles_m = (int32_t)(m_pad / BM); p.tiles_n = (int32_t)(n_pad / BN);
    p.tri_compact = triangle_is_compact(m, n, tri) ? 1 : 0;
    p.tiles_per_mat = p.tri_compact ? (int64_t)p.tiles_m * (p.tiles_m + 1) / 2 : (int64_t)p.tiles_m * p.tiles_n;
    p.total_tiles = p.tiles_per_mat * batch;
    p.alpha = alpha; p.beta = beta; p.status = status; p.act = act; p.act_param = act_param; p.tri = tri;
    p.lean_epilogue = 1;
    const TailPlan plan = plan_tail(p.total_tiles, num_kb, sm_count, sk_area != nullptr && sk_epoch != 0);
    p.dp_tiles = plan.dp_tiles; p.sk_tiles = plan.sk_tiles; p.sk_split = plan.sk_split; p.sk_coop = plan.coop;
    p.sk_flags = static_cast<unsigned int*>(sk_area);
    p.sk_partials = sk_area ? reinterpret_cast<float*>(static_cast<char*>(sk_area) + SK_FLAG_BYTES) : nullptr;
    p.sk_epoch = sk_epoch;
    if (plan.grid <= 0) return cudaSuccess;
    if (products == 1) sgemm_tc3x_kernel<1, false><<<(unsigned)plan.grid, THREADS, SMEM_BYTES, st>>>(map_a, map_b, raw_a, raw_b, p);
    else if (any_raw) sgemm_tc3x_kernel<3, true><<<(unsigned)plan.grid, THREADS_RAW, SMEM_BYTES, st>>>(map_a, map_b, raw_a, raw_b, p);
    else sgemm_tc3x_kernel<3, false><<<(unsigned)plan.grid, THREADS, SMEM_BYTES, st>>>(map_a, map_b, raw_a, raw_b, p);
    return cudaGetLastError();
}

} // namespace tc3x
} // namespace sushi
