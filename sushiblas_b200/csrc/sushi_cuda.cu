// sushi_cuda.cu -- C ABI of the sm_100a backend (declared in include/sushiblas_cuda.h).
//
// Owns: the per-device context (stream, scratch, status word), storage calls
// (cudaMalloc / pinned host + explicit copies, replacing the USM allocator of
// include/SushiRuntime/memory/usm_allocator.hpp:43-71), kernel selection, and the
// NCCL-based multi-GPU layer.  There is no CPU fallback anywhere in this file.
#include "../../include/sushiblas_cuda.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <numeric>
#include <string>
#include <vector>

#include "sgemm_simt.cuh"
#include "sgemm_skinny.cuh"
#include "split_tf32.cuh"
#include "sgemm_tc3x.cuh"
#include "trsm_blocks.cuh"
#include "dgemm_mma.cuh"

namespace {

struct DeviceState
{
    int device = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;        // active stream (own or caller's)
    void* workspace = nullptr;            // 3xTF32 operand planes
    size_t workspace_bytes = 0;
    void* stage[3] = {nullptr, nullptr, nullptr};   // device staging for the *_host entry points
    size_t stage_bytes[3] = {0, 0, 0};
    int* status = nullptr;                // device word written by bounded in-kernel waits
    int* status_host = nullptr;           // pinned mirror
    // host-buffer entry point: copy streams and events of the chunked upload / multiply / download pipeline
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t pipe_events[18] = {};
    // uploads that run ahead of queued work: own stream, fence (work queued so far) and completion events
    cudaStream_t ahead_stream = nullptr;
    cudaEvent_t ahead_fence = nullptr, ahead_done = nullptr;
    bool ahead_fenced = false;
    // downloads that start as soon as their source is final: own stream and completion event
    cudaStream_t behind_stream = nullptr;
    cudaEvent_t behind_done = nullptr;
    void* trsm_buf = nullptr;             // TRSM: inverted diagonal blocks + one block row/column of temporaries
    size_t trsm_bytes = 0;
    void* group_buf = nullptr;            // device copy of the grouped-launch problem list
    size_t group_bytes = 0;
    void* sk_area = nullptr;              // split-K exchange area (epoch flags + slots), flags zeroed at allocation
    size_t sk_area_bytes = 0;
    unsigned int sk_epoch = 0;            // last epoch handed to a launch
    // kernel timing (off by default): event triples {before pre-pass, before GEMM, after GEMM}
    std::vector<cudaEvent_t> timing_events;
    size_t timing_used = 0;
    std::vector<int> timing_prepass_launches;
};

// minimal NCCL surface, resolved at run time
typedef struct ncclComm* ncclComm_t;
struct Id128 { char bytes[128]; };   // ncclUniqueId
struct NcclApi
{
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, Id128, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
constexpr int NCCL_FLOAT32 = 7;

NcclApi g_nccl;
std::mutex g_nccl_mutex;
thread_local std::string g_tls_error;

} // namespace

struct sushi_cuda_ctx
{
    std::vector<DeviceState> devs;
    std::string last_error;
    int variant = SUSHI_GEMM_AUTO;
    std::atomic<int64_t> launches{0};
    std::atomic<uint64_t> h2d_bytes{0}, d2h_bytes{0};   // bytes moved by sushi_cuda_memcpy_h2d / _d2h
    int fail_countdown[4] = {0, 0, 0, 0};   // host-side fault injection: calls left until the site fails (0: off)
    bool timing = false;
    // multi-GPU (one process per GPU: a single communicator bound to one device index)
    ncclComm_t comm = nullptr;
    int comm_dev = -1, nranks = 1, rank = 0;
    cudaStream_t comm_stream = nullptr;
    std::vector<cudaEvent_t> slab_events;
    cudaEvent_t comm_done = nullptr;
    // fused all-gather: every rank's C buffer as addressable from this device (own entry local)
    std::vector<void*> peer_buffers;
    size_t peer_bytes = 0;
    float* barrier_word = nullptr;        // 4-byte operand of the NCCL all-reduce used as a cross-rank barrier
};

namespace {

int set_error(sushi_cuda_ctx* ctx, int code, const std::string& msg)
{
    if (ctx) ctx->last_error = msg; else g_tls_error = msg;
    return code;
}

// Host-side fault injection (sushi_cuda_inject_failure): true when this call of `site` is the one to fail.
bool injected_failure(sushi_cuda_ctx* ctx, int site)
{
    if (!ctx || site < 1 || site > 3 || ctx->fail_countdown[site] == 0) return false;
    return --ctx->fail_countdown[site] == 0;
}

int cuda_fail(sushi_cuda_ctx* ctx, cudaError_t e, const char* what)
{
    std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
    int code = (e == cudaErrorMemoryAllocation) ? SUSHI_CUDA_ERR_OOM
             : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? SUSHI_CUDA_ERR_NO_DEVICE
             : SUSHI_CUDA_ERR_CUDA;
    return set_error(ctx, code, msg);
}

#define SC_CUDA(ctx, call)                                              \
    do { cudaError_t e__ = (call); if (e__ != cudaSuccess) return cuda_fail((ctx), e__, #call); } while (0)

DeviceState* get_dev(sushi_cuda_ctx* ctx, int dev)
{
    if (!ctx || dev < 0 || dev >= (int)ctx->devs.size()) return nullptr;
    return &ctx->devs[dev];
}

int grow(sushi_cuda_ctx* ctx, DeviceState& d, void** buf, size_t* have, size_t need)
{
    if (need <= *have) return SUSHI_CUDA_OK;
    if (*buf)
    {
        SC_CUDA(ctx, cudaStreamSynchronize(d.stream));
        SC_CUDA(ctx, cudaFree(*buf));
        *buf = nullptr; *have = 0;
    }
    if (injected_failure(ctx, SUSHI_CUDA_FAIL_DEVICE_ALLOC))
        return set_error(ctx, SUSHI_CUDA_ERR_OOM, "injected failure: device allocation (library scratch)");
    SC_CUDA(ctx, cudaMalloc(buf, need));
    *have = need;
    return SUSHI_CUDA_OK;
}

int64_t extent(int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t batch)
{
    if (rows <= 0 || cols <= 0 || batch <= 0) return 0;
    return (batch - 1) * stride + (rows - 1) * ld + cols;
}

int validate_gemm(sushi_cuda_ctx* ctx, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda,
                  const void* b, int64_t ldb, const void* c, int64_t ldc, int ta, int tb,
                  int64_t sa, int64_t sb, int64_t sc, int64_t batch)
{
    if (m < 0 || n < 0 || k < 0 || batch < 0)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: negative dimension");
    const int64_t a_cols = ta ? m : k, b_cols = tb ? k : n;
    if (lda < (a_cols > 1 ? a_cols : 1)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: lda too small");
    if (ldb < (b_cols > 1 ? b_cols : 1)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: ldb too small");
    if (ldc < (n > 1 ? n : 1)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: ldc too small");
    if (sa < 0 || sb < 0 || sc < 0) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: negative batch stride");
    if (m > 0 && n > 0 && batch > 0)
    {
        if (!c) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: C is null");
        if (k > 0 && (!a || !b)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: A or B is null");
        if (batch > 1 && sc < extent(m, n, ldc, 0, 1))
            return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: stride_c makes batches of C overlap");
    }
    return SUSHI_CUDA_OK;
}

// Kernel choice for SUSHI_GEMM_AUTO: the tensor-core path pays a pre-pass and works in
// 256 x 256 tiles, so it needs enough k to amortise the split and enough tiles to occupy SMs.
bool prefer_tc3x(int64_t m, int64_t n, int64_t k, int64_t batch, int sm_count, bool allow_split = true)
{
    if (k < 128 || m < 128 || n < 128) return false;
    const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256) * batch;
    const int64_t num_kb = (k + 15) / 16;
    // Tensor path, measured on B200: ~1 us per 16-k block of a 256 x 256 tile on top of ~27 us of fixed cost per
    // launch (prologue, pipeline fill, epilogue, teardown); few tiles are cut along K (plan_tail), which adds
    // the exchange; an operand wider than 2048 in the other dimension goes through the pre-pass (a launch of
    // ~6 us plus 12 B per element at ~5 TB/s), narrower ones are split inside the kernel.
    const sushi::tc3x::TailPlan plan = sushi::tc3x::plan_tail(tiles, num_kb, sm_count, allow_split);
    const int64_t items = plan.sk_split > 1 ? tiles * plan.sk_split : tiles;
    const double rounds = (double)((items + sm_count - 1) / sm_count);
    const double kb_item = (double)((num_kb + plan.sk_split - 1) / plan.sk_split);
    double t_tc = rounds * kb_item * 1.02e-6 + 27e-6 + (plan.sk_split > 1 ? 6e-6 : 0.0);
    if (n > 2048) t_tc += 6e-6 + 12.0 * (double)batch * (double)k * (double)m / 5.0e12;
    if (m > 2048) t_tc += 6e-6 + 12.0 * (double)batch * (double)k * (double)n / 5.0e12;
    // FFMA path, measured: 128 x 128 tiles at ~0.17 TFLOP/s per SM once they fill the GPU; otherwise 64 x 64 tiles,
    // ~0.1 TFLOP/s for a lone CTA and ~0.125 per SM with several resident; ~5 us to launch
    const int64_t big = ((m + 127) / 128) * ((n + 127) / 128) * batch;
    double t_simt;
    if (big >= sm_count)
        t_simt = (double)big / sm_count * (2.0 * 128 * 128 * (double)k) / 0.17e12 + 5e-6;
    else
    {
        const int64_t small = ((m + 63) / 64) * ((n + 63) / 64) * batch;
        const double per_sm = (double)small / sm_count;
        t_simt = (per_sm <= 1.0 ? 1.0 / 0.1e12 : per_sm / 0.125e12) * (2.0 * 64 * 64 * (double)k) + 5e-6;
    }
    return t_tc < t_simt;
}

int check_variant_env(int current)
{
    const char* e = getenv("SUSHI_GEMM_VARIANT");
    if (!e) return current;
    if (!strcmp(e, "simt") || !strcmp(e, "1")) return SUSHI_GEMM_SIMT;
    if (!strcmp(e, "tc3x") || !strcmp(e, "2")) return SUSHI_GEMM_TC3X;
    return current;
}

// Records the next timing event of the current triple (no-op unless timing is enabled).
int timing_mark(sushi_cuda_ctx* ctx, DeviceState& d, int which, int prepass_launches)
{
    if (!ctx->timing) return SUSHI_CUDA_OK;
    if (which == 0)
    {
        while (d.timing_events.size() < d.timing_used + 3)
        {
            cudaEvent_t e;
            SC_CUDA(ctx, cudaEventCreate(&e));
            d.timing_events.push_back(e);
        }
        d.timing_prepass_launches.push_back(prepass_launches);
    }
    SC_CUDA(ctx, cudaEventRecord(d.timing_events[d.timing_used + which], d.stream));
    if (which == 2) d.timing_used += 3;
    return SUSHI_CUDA_OK;
}

// Lets a caller that multiplies several row slabs of A by the same B (the sharded path) keep
// one kernel family for all slabs and split B into planes only once.
struct SlabReuse
{
    int variant = -1;          // -1: choose per call
    bool b_planes_ready = false;
    int64_t max_rows = 0;      // largest slab (sizes the A planes once)
    float* peer_c[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_peers = 0;           // fused all-gather: the GEMM epilogue also stores C to these addresses
    int act = 0;               // epilogue activation (sushi_cuda_activation_kind)
    float act_param = 0.0f;    // its parameter
    int tri = 0;               // triangular output (SYRK): 1 lower, 2 upper
    int products = 3;          // 1: only the hi*hi MMA of every product (rate probe; forces pre-split planes, no K cut)
};

int run_gemm(sushi_cuda_ctx* ctx, DeviceState& d, int ta, int tb, int64_t m, int64_t n, int64_t k, float alpha,
             const float* a, int64_t lda, int64_t sa, const float* b, int64_t ldb, int64_t sb,
             float beta, float* c, int64_t ldc, int64_t sc, int64_t batch, SlabReuse* reuse = nullptr)
{
    if (m == 0 || n == 0 || batch == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d.device));
    const int act = reuse ? reuse->act : 0;
    const float act_param = reuse ? reuse->act_param : 0.0f;
    const int tri = reuse ? reuse->tri : 0;
    if ((k == 0 || alpha == 0.0f) && tri == 0)
    {
        if (beta == 1.0f && !act) return SUSHI_CUDA_OK;
        const int64_t total = m * n * batch;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)d.sm_count * 16) blocks = (int64_t)d.sm_count * 16;
        sushi::scale_c_kernel<<<(unsigned)blocks, 256, 0, d.stream>>>(c, m, n, ldc, sc, batch, beta, act, act_param);
        ctx->launches++;
        SC_CUDA(ctx, cudaGetLastError());
        return SUSHI_CUDA_OK;
    }
    int variant = (reuse && reuse->variant >= 0) ? reuse->variant : ctx->variant;
    if (variant == SUSHI_GEMM_AUTO)
        variant = prefer_tc3x(m, n, k, batch, d.sm_count) ? SUSHI_GEMM_TC3X : SUSHI_GEMM_SIMT;
    // A 3xTF32 product carries up to ~12 * 2^-24 |a b| of error whatever K is, which for K < 4 can exceed
    // the K-scaled tolerance: such products always take the exact-fp32 FFMA kernel.
    if (variant == SUSHI_GEMM_TC3X && k < 4) variant = SUSHI_GEMM_SIMT;
    if (reuse) reuse->variant = variant;

    if (variant == SUSHI_GEMM_TC3X)
    {
        // An operand whose k index is contiguous can be split inside the GEMM kernel instead of
        // by the pre-pass.  The pre-pass costs 12 B per operand element once; the in-kernel split
        // costs ~10 % of the kernel's tensor rate (shared-memory bandwidth) for every tile that
        // uses the operand.  Measured break-even on B200: the operand is reused by about eleven
        // 256-wide tiles, so A is split in-kernel when n <= 2048 and B when m <= 2048
        const int products = reuse ? reuse->products : 3;
        const bool probe = reuse && reuse->products != 3;          // rate probe: both operands as planes, whole tiles
        const bool want_a = n <= 2048 && !probe;
        const bool want_b = m <= 2048 && !probe;
        // either storage order of an operand can be taken raw: k-contiguous tiles are split in place, row-contiguous
        // ones (A^T, or B not transposed) are transposed by the converters on the way
        const bool fuse_a = want_a && sushi::tc3x::raw_eligible(a, m, k, lda, sa, batch);
        const bool fuse_b = want_b && sushi::tc3x::raw_eligible(b, n, k, ldb, sb, batch);
        // workspace: [planes of op(B)^T][planes of op(A)] -- B first so that slabs of A of any
        // size can follow without moving it
        const int64_t a_rows = (reuse && reuse->max_rows > m) ? reuse->max_rows : m;
        const size_t bytes_a = fuse_a ? 0 : sushi::split_plane_bytes(a_rows, k, batch);
        size_t bytes_b = fuse_b ? 0 : sushi::split_plane_bytes(n, k, batch);
        if ((b == a) && (ldb == lda) && (sb == sa) && ((tb != 0) == (ta == 0)) && (m == n) && !(reuse && reuse->max_rows > m))
            bytes_b = 0;           // shares A's planes (see below)
        int rc = SUSHI_CUDA_OK;
        if (bytes_a + bytes_b > 0 && (rc = grow(ctx, d, &d.workspace, &d.workspace_bytes, bytes_a + bytes_b)) != SUSHI_CUDA_OK)
            return rc;
        float* planes_b = static_cast<float*>(d.workspace);
        float* planes_a = reinterpret_cast<float*>(static_cast<char*>(d.workspace) + bytes_b);
        // SYRK-shaped call (op(B)^T is op(A) itself): one set of planes serves both operands
        const bool same_operand = (b == a) && (ldb == lda) && (sb == sa) && ((tb != 0) == (ta == 0)) && (m == n) &&
                                  !(reuse && reuse->max_rows > m);
        const bool split_b = !fuse_b && !same_operand && !(reuse && reuse->b_planes_ready);
        const int prepass_launches = (fuse_a ? 0 : 1) + (split_b ? 1 : 0);
        if ((rc = timing_mark(ctx, d, 0, prepass_launches)) != SUSHI_CUDA_OK) return rc;
        if (!fuse_a)
            SC_CUDA(ctx, sushi::launch_split_tf32(a, planes_a, m, k, lda, sa, batch, /*k_contig=*/!ta, d.sm_count, d.stream));
        if (split_b)
            SC_CUDA(ctx, sushi::launch_split_tf32(b, planes_b, n, k, ldb, sb, batch, /*k_contig=*/tb != 0, d.sm_count, d.stream));
        if (reuse) reuse->b_planes_ready = true;
        void* sk_area = nullptr;
        {
            int64_t tiles = 0, num_kb = 0;
            sushi::tc3x::tile_counts(m, n, k, batch, tri, &tiles, &num_kb);
            const size_t need = sushi::tc3x::sk_area_bytes(sushi::tc3x::plan_tail(tiles, num_kb, d.sm_count, true));
            if (need > d.sk_area_bytes)
            {
                // grown on demand; flags start at zero
                if ((rc = grow(ctx, d, &d.sk_area, &d.sk_area_bytes, need)) != SUSHI_CUDA_OK) return rc;
                SC_CUDA(ctx, cudaMemsetAsync(d.sk_area, 0, sushi::tc3x::SK_FLAG_BYTES, d.stream));
            }
            if (need > 0)
            {
                sk_area = d.sk_area;
                if (++d.sk_epoch == 0)
                {
                    // 2^32 launches later: start the epochs over on clean flags
                    SC_CUDA(ctx, cudaMemsetAsync(d.sk_area, 0, sushi::tc3x::SK_FLAG_BYTES, d.stream));
                    d.sk_epoch = 1;
                }
            }
        }
        sushi::tc3x::OperandSource src_a, src_b;
        if (fuse_a) { src_a.raw = a; src_a.ld = lda; src_a.stride = sa; src_a.row_contig = ta != 0; } else src_a.planes = planes_a;
        if (fuse_b) { src_b.raw = b; src_b.ld = ldb; src_b.stride = sb; src_b.row_contig = tb == 0; }
        else src_b.planes = (same_operand && !fuse_a) ? planes_a : planes_b;
        if ((rc = timing_mark(ctx, d, 1, 0)) != SUSHI_CUDA_OK) return rc;
        SC_CUDA(ctx, sushi::tc3x::launch_sgemm_tc3x(src_a, src_b, c, m, n, k, ldc, sc, batch, alpha, beta,
                                                   d.status, d.sm_count, d.stream, probe ? nullptr : sk_area, d.sk_epoch,
                                                   reuse ? reuse->peer_c : nullptr, reuse ? reuse->n_peers : 0, act, tri, act_param,
                                                   products));
        if ((rc = timing_mark(ctx, d, 2, 0)) != SUSHI_CUDA_OK) return rc;
        ctx->launches += 1 + prepass_launches;
        return SUSHI_CUDA_OK;
    }

    // tall-and-skinny products are bound by reading A once: their own kernel (same arithmetic class)
    if (tri == 0 && batch <= 65535 && sushi::skinny_eligible(ta, m, n, k, a, lda, sa))
    {
        sushi::SkinnyArgs q;
        q.a = a; q.b = b; q.c = c; q.m = m; q.n = n; q.k = k; q.lda = lda; q.ldb = ldb; q.ldc = ldc;
        q.stride_a = sa; q.stride_b = sb; q.stride_c = sc; q.row_blocks = 0; q.alpha = alpha; q.beta = beta;
        q.trans_b = tb != 0; q.act = act; q.act_param = act_param;
        int rcs = timing_mark(ctx, d, 0, 0);
        if (rcs == SUSHI_CUDA_OK) rcs = timing_mark(ctx, d, 1, 0);
        if (rcs != SUSHI_CUDA_OK) return rcs;
        SC_CUDA(ctx, sushi::launch_sgemm_skinny(q, batch, d.sm_count, d.stream));
        if ((rcs = timing_mark(ctx, d, 2, 0)) != SUSHI_CUDA_OK) return rcs;
        ctx->launches++;
        return SUSHI_CUDA_OK;
    }
    sushi::SimtGemmArgs g;
    g.a = a; g.b = b; g.c = c; g.m = m; g.n = n; g.k = k; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
    g.stride_a = sa; g.stride_b = sb; g.stride_c = sc; g.tiles_m = 0; g.tiles_n = 0;
    g.alpha = alpha; g.beta = beta; g.act = act; g.act_param = act_param; g.tri = tri;
    int rc = timing_mark(ctx, d, 0, 0);
    if (rc == SUSHI_CUDA_OK) rc = timing_mark(ctx, d, 1, 0);
    if (rc != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, sushi::launch_sgemm_simt(g, ta != 0, tb != 0, batch, d.sm_count, d.stream));
    if ((rc = timing_mark(ctx, d, 2, 0)) != SUSHI_CUDA_OK) return rc;
    ctx->launches++;
    return SUSHI_CUDA_OK;
}

bool load_nccl(std::string* err)
{
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return true;
    const char* names[] = {getenv("SUSHI_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* nm : names)
    {
        if (!nm) continue;
        h = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) { *err = std::string("cannot load libnccl.so.2: ") + dlerror(); return false; }
    NcclApi api;
    api.handle = h;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
    api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(dlsym(h, "ncclBroadcast"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(dlsym(h, "ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.Broadcast || !api.AllReduce ||
        !api.GroupStart || !api.GroupEnd || !api.GetErrorString)
    {
        *err = "libnccl is missing a required symbol";
        return false;
    }
    g_nccl = api;
    return true;
}

int nccl_fail(sushi_cuda_ctx* ctx, int rc, const char* what)
{
    return set_error(ctx, SUSHI_CUDA_ERR_COMM, std::string(what) + ": " + g_nccl.GetErrorString(rc));
}

#define SC_NCCL(ctx, call)                                              \
    do { int r__ = (call); if (r__ != 0) return nccl_fail((ctx), r__, #call); } while (0)

__global__ void fill_uniform_kernel(float* dst, int64_t count, uint64_t key, int64_t first)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    {
        uint64_t z = ((uint64_t)(first + i) ^ key) + 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z = z ^ (z >> 31);
        const uint32_t u = (uint32_t)(z >> 32) >> 8;
        dst[i] = (float)u * 1.1920928955078125e-07f - 1.0f;   // u * 2^-23 - 1, exact
    }
}

uint64_t splitmix64_host(uint64_t x)
{
    uint64_t z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

} // namespace

// ======================================================================== context
extern "C" int sushi_cuda_device_count(int* count)
{
    if (!count) return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "device_count: null output");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { *count = 0; return cuda_fail(nullptr, e, "cudaGetDeviceCount"); }
    *count = n;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_init(const int* devices, int n_devices, sushi_cuda_ctx** out)
{
    if (!out) return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "init: null output");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
    if (count == 0) return set_error(nullptr, SUSHI_CUDA_ERR_NO_DEVICE, "no CUDA device");

    std::vector<int> ids;
    if (devices && n_devices > 0) ids.assign(devices, devices + n_devices);
    else
    {
        const char* env = getenv("SUSHI_CUDA_DEVICE");
        ids.push_back(env ? atoi(env) : 0);
    }
    sushi_cuda_ctx* ctx = new sushi_cuda_ctx();
    ctx->variant = check_variant_env(SUSHI_GEMM_AUTO);
    for (int id : ids)
    {
        if (id < 0 || id >= count)
        {
            set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "init: device index out of range");
            sushi_cuda_destroy(ctx);
            return SUSHI_CUDA_ERR_INVALID_ARG;
        }
        DeviceState d;
        d.device = id;
        cudaDeviceProp prop;
        bool ok = cudaSetDevice(id) == cudaSuccess && cudaGetDeviceProperties(&prop, id) == cudaSuccess;
        if (ok && prop.major != 10)
        {
            set_error(nullptr, SUSHI_CUDA_ERR_UNSUPPORTED, "this library is built for sm_100a (B200) only");
            sushi_cuda_destroy(ctx);
            return SUSHI_CUDA_ERR_UNSUPPORTED;
        }
        ok = ok && cudaStreamCreateWithFlags(&d.own_stream, cudaStreamNonBlocking) == cudaSuccess;
        ok = ok && cudaMalloc(&d.status, sizeof(int)) == cudaSuccess;
        ok = ok && cudaMemset(d.status, 0, sizeof(int)) == cudaSuccess;
        ok = ok && cudaMallocHost(&d.status_host, sizeof(int)) == cudaSuccess;
        if (!ok)
        {
            cuda_fail(nullptr, cudaGetLastError(), "device set-up");
            ctx->devs.push_back(d);
            sushi_cuda_destroy(ctx);
            return SUSHI_CUDA_ERR_CUDA;
        }
        d.stream = d.own_stream;
        d.sm_count = prop.multiProcessorCount;
        ctx->devs.push_back(d);
    }
    *out = ctx;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_destroy(sushi_cuda_ctx* ctx)
{
    if (!ctx) return SUSHI_CUDA_OK;
    sushi_cuda_comm_destroy(ctx);
    for (DeviceState& d : ctx->devs)
    {
        cudaSetDevice(d.device);
        if (d.own_stream) cudaStreamSynchronize(d.own_stream);
        if (d.workspace) cudaFree(d.workspace);
        if (d.sk_area) cudaFree(d.sk_area);
        if (d.group_buf) cudaFree(d.group_buf);
        if (d.trsm_buf) cudaFree(d.trsm_buf);
        for (void* s : d.stage) if (s) cudaFree(s);
        if (d.status) cudaFree(d.status);
        if (d.status_host) cudaFreeHost(d.status_host);
        for (cudaEvent_t e : d.timing_events) cudaEventDestroy(e);
        if (d.copy_in) { cudaStreamSynchronize(d.copy_in); cudaStreamDestroy(d.copy_in); }
        if (d.copy_out) { cudaStreamSynchronize(d.copy_out); cudaStreamDestroy(d.copy_out); }
        for (cudaEvent_t e : d.pipe_events) if (e) cudaEventDestroy(e);
        if (d.ahead_stream) { cudaStreamSynchronize(d.ahead_stream); cudaStreamDestroy(d.ahead_stream); }
        if (d.ahead_fence) cudaEventDestroy(d.ahead_fence);
        if (d.ahead_done) cudaEventDestroy(d.ahead_done);
        if (d.behind_stream) { cudaStreamSynchronize(d.behind_stream); cudaStreamDestroy(d.behind_stream); }
        if (d.behind_done) cudaEventDestroy(d.behind_done);
        if (d.own_stream) cudaStreamDestroy(d.own_stream);
    }
    delete ctx;
    return SUSHI_CUDA_OK;
}

extern "C" const char* sushi_cuda_last_error(sushi_cuda_ctx* ctx)
{
    return ctx ? ctx->last_error.c_str() : g_tls_error.c_str();
}

extern "C" int sushi_cuda_sync(sushi_cuda_ctx* ctx, int dev)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sync: bad context or device index");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaMemcpyAsync(d->status_host, d->status, sizeof(int), cudaMemcpyDeviceToHost, d->stream));
    SC_CUDA(ctx, cudaStreamSynchronize(d->stream));
    if (ctx->comm_stream && ctx->comm_dev == dev) SC_CUDA(ctx, cudaStreamSynchronize(ctx->comm_stream));
    if (*d->status_host != 0)
    {
        char msg[128];
        snprintf(msg, sizeof msg, "a bounded in-kernel wait expired (code %d)", *d->status_host);
        cudaMemsetAsync(d->status, 0, sizeof(int), d->stream);
        return set_error(ctx, SUSHI_CUDA_ERR_KERNEL_TIMEOUT, msg);
    }
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_selftest_bounded_wait(sushi_cuda_ctx* ctx, int dev, int limit_ms)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || limit_ms < 1 || limit_ms > 2000)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "selftest_bounded_wait: bad argument (limit 1..2000 ms)");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    sushi::tc3x::bounded_wait_selftest_kernel<<<1, 32, 0, d->stream>>>(d->status, (unsigned long long)limit_ms * 1000000ull);
    ctx->launches++;
    SC_CUDA(ctx, cudaGetLastError());
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_set_stream(sushi_cuda_ctx* ctx, int dev, void* cuda_stream)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "set_stream: bad context or device index");
    d->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : d->own_stream;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_get_stream(sushi_cuda_ctx* ctx, int dev, void** cuda_stream)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !cuda_stream) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "get_stream: bad argument");
    *cuda_stream = d->stream;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_set_gemm_variant(sushi_cuda_ctx* ctx, int variant)
{
    if (!ctx || variant < SUSHI_GEMM_AUTO || variant > SUSHI_GEMM_TC3X)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "set_gemm_variant: bad argument");
    ctx->variant = variant;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_launch_count(sushi_cuda_ctx* ctx, int64_t* launches)
{
    if (!ctx || !launches) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "launch_count: bad argument");
    *launches = ctx->launches.load();
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_kernel_timing_enable(sushi_cuda_ctx* ctx, int enable)
{
    if (!ctx) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "kernel_timing_enable: null context");
    ctx->timing = enable != 0;
    for (DeviceState& d : ctx->devs) { d.timing_used = 0; d.timing_prepass_launches.clear(); }
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_kernel_timing_read(sushi_cuda_ctx* ctx, int dev, double* gemm_ms, int64_t* gemm_launches,
                                             double* prepass_ms, int64_t* prepass_launches)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !gemm_ms || !gemm_launches || !prepass_ms || !prepass_launches)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "kernel_timing_read: bad argument");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaStreamSynchronize(d->stream));
    double g = 0.0, p = 0.0;
    int64_t gl = 0, pl = 0;
    for (size_t i = 0; i + 2 < d->timing_used + 1 && i < d->timing_used; i += 3)
    {
        float ms = 0.0f;
        SC_CUDA(ctx, cudaEventElapsedTime(&ms, d->timing_events[i], d->timing_events[i + 1]));
        p += ms;
        SC_CUDA(ctx, cudaEventElapsedTime(&ms, d->timing_events[i + 1], d->timing_events[i + 2]));
        g += ms;
        gl += 1;
        pl += d->timing_prepass_launches[i / 3];
    }
    *gemm_ms = g; *gemm_launches = gl; *prepass_ms = p; *prepass_launches = pl;
    d->timing_used = 0;
    d->timing_prepass_launches.clear();
    return SUSHI_CUDA_OK;
}

// ======================================================================== storage
extern "C" int sushi_cuda_malloc(sushi_cuda_ctx* ctx, int dev, size_t bytes, void** ptr)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !ptr || bytes == 0) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "malloc: bad argument");
    *ptr = nullptr;
    if (injected_failure(ctx, SUSHI_CUDA_FAIL_DEVICE_ALLOC))
        return set_error(ctx, SUSHI_CUDA_ERR_OOM, "injected failure: device allocation");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaMalloc(ptr, bytes));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_inject_failure(sushi_cuda_ctx* ctx, int site, int nth)
{
    if (!ctx || site < 1 || site > 3 || nth < 0)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "inject_failure: bad argument");
    ctx->fail_countdown[site] = nth;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_free(sushi_cuda_ctx* ctx, int dev, void* ptr)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "free: bad context or device index");
    if (!ptr) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaFree(ptr));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_host_alloc(sushi_cuda_ctx* ctx, size_t bytes, void** ptr)
{
    if (!ctx || !ptr || bytes == 0) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "host_alloc: bad argument");
    *ptr = nullptr;
    if (injected_failure(ctx, SUSHI_CUDA_FAIL_HOST_ALLOC))
        return set_error(ctx, SUSHI_CUDA_ERR_OOM, "injected failure: pinned host allocation");
    SC_CUDA(ctx, cudaSetDevice(ctx->devs[0].device));
    SC_CUDA(ctx, cudaHostAlloc(ptr, bytes, cudaHostAllocPortable));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_host_free(sushi_cuda_ctx* ctx, void* ptr)
{
    if (!ctx) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "host_free: null context");
    if (!ptr) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaFreeHost(ptr));
    return SUSHI_CUDA_OK;
}

static int copy_async(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind,
                      const char* what)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, std::string(what) + ": bad context or device index");
    if (bytes == 0) return SUSHI_CUDA_OK;
    if (!dst || !src) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, std::string(what) + ": null pointer");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, kind, d->stream));
    if (kind == cudaMemcpyHostToDevice) ctx->h2d_bytes += bytes;
    if (kind == cudaMemcpyDeviceToHost) ctx->d2h_bytes += bytes;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_copy_bytes(sushi_cuda_ctx* ctx, uint64_t* h2d_bytes, uint64_t* d2h_bytes)
{
    if (!ctx) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "copy_bytes: bad context");
    if (h2d_bytes) *h2d_bytes = ctx->h2d_bytes;
    if (d2h_bytes) *d2h_bytes = ctx->d2h_bytes;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_memcpy_h2d(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes)
{ return copy_async(ctx, dev, dst, src, bytes, cudaMemcpyHostToDevice, "memcpy_h2d"); }
extern "C" int sushi_cuda_memcpy_d2h(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes)
{ return copy_async(ctx, dev, dst, src, bytes, cudaMemcpyDeviceToHost, "memcpy_d2h"); }
extern "C" int sushi_cuda_memcpy_d2d(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes)
{ return copy_async(ctx, dev, dst, src, bytes, cudaMemcpyDeviceToDevice, "memcpy_d2d"); }

static int ensure_ahead_stream(sushi_cuda_ctx* ctx, DeviceState* d)
{
    if (d->ahead_stream) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaEventCreateWithFlags(&d->ahead_fence, cudaEventDisableTiming));
    SC_CUDA(ctx, cudaEventCreateWithFlags(&d->ahead_done, cudaEventDisableTiming));
    SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->ahead_stream, cudaStreamNonBlocking));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_upload_fence(sushi_cuda_ctx* ctx, int dev)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "upload_fence: bad context or device index");
    int rc = ensure_ahead_stream(ctx, d);
    if (rc != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaEventRecord(d->ahead_fence, d->stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->ahead_stream, d->ahead_fence, 0));
    d->ahead_fenced = true;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_upload_ahead(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "upload_ahead: bad context or device index");
    if (bytes == 0) return SUSHI_CUDA_OK;
    if (!dst || !src) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "upload_ahead: null pointer");
    int rc = d->ahead_fenced ? SUSHI_CUDA_OK : sushi_cuda_upload_fence(ctx, dev);   // never ahead of everything
    if (rc != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, d->ahead_stream));
    // a wait takes the event's state at this call, so one event serves every upload
    SC_CUDA(ctx, cudaEventRecord(d->ahead_done, d->ahead_stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, d->ahead_done, 0));
    ctx->h2d_bytes += bytes;
    return SUSHI_CUDA_OK;
}

// A marker is a CUDA event behind an opaque pointer.
extern "C" int sushi_cuda_marker_create(sushi_cuda_ctx* ctx, int dev, sushi_cuda_marker** marker)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !marker) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "marker_create: bad context, device index or pointer");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    cudaEvent_t e = nullptr;
    SC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    *marker = reinterpret_cast<sushi_cuda_marker*>(e);
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_marker_record(sushi_cuda_ctx* ctx, int dev, sushi_cuda_marker* marker)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !marker) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "marker_record: bad context, device index or marker");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaEventRecord(reinterpret_cast<cudaEvent_t>(marker), d->stream));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_marker_destroy(sushi_cuda_ctx* ctx, sushi_cuda_marker* marker)
{
    if (!ctx) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "marker_destroy: bad context");
    if (marker) SC_CUDA(ctx, cudaEventDestroy(reinterpret_cast<cudaEvent_t>(marker)));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_download_behind(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes,
                                          sushi_cuda_marker* after)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !after) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "download_behind: bad context, device index or marker");
    if (bytes == 0) return SUSHI_CUDA_OK;
    if (!dst || !src) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "download_behind: null pointer");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    if (!d->behind_stream)
    {
        SC_CUDA(ctx, cudaEventCreateWithFlags(&d->behind_done, cudaEventDisableTiming));
        SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->behind_stream, cudaStreamNonBlocking));
    }
    SC_CUDA(ctx, cudaStreamWaitEvent(d->behind_stream, reinterpret_cast<cudaEvent_t>(after), 0));
    SC_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, d->behind_stream));
    // the device's stream joins the download: a sync of it covers the copy, and nothing enqueued later
    // overwrites the source under it
    SC_CUDA(ctx, cudaEventRecord(d->behind_done, d->behind_stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, d->behind_done, 0));
    ctx->d2h_bytes += bytes;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_memset(sushi_cuda_ctx* ctx, int dev, void* dst, int byte, size_t bytes)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "memset: bad context or device index");
    if (bytes == 0) return SUSHI_CUDA_OK;
    if (!dst) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "memset: null pointer");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaMemsetAsync(dst, byte, bytes, d->stream));
    return SUSHI_CUDA_OK;
}

// ======================================================================== GEMM
extern "C" int sushi_cuda_sgemm_strided_batched(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                int64_t m, int64_t n, int64_t k, float alpha,
                                                const float* a, int64_t lda, int64_t stride_a,
                                                const float* b, int64_t ldb, int64_t stride_b,
                                                float beta, float* c, int64_t ldc, int64_t stride_c,
                                                int64_t batch)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm: bad context or device index");
    int rc = validate_gemm(ctx, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, stride_a, stride_b, stride_c, batch);
    if (rc != SUSHI_CUDA_OK) return rc;
    return run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b, beta, c, ldc,
                    stride_c, batch);
}

extern "C" int sushi_cuda_dgemm_strided_batched(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                int64_t m, int64_t n, int64_t k, double alpha,
                                                const double* a, int64_t lda, int64_t stride_a,
                                                const double* b, int64_t ldb, int64_t stride_b,
                                                double beta, double* c, int64_t ldc, int64_t stride_c,
                                                int64_t batch)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "dgemm: bad context or device index");
    int rc = validate_gemm(ctx, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, stride_a, stride_b, stride_c, batch);
    if (rc != SUSHI_CUDA_OK) return rc;
    if (m == 0 || n == 0 || batch == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    if (k == 0 || alpha == 0.0)
    {
        if (beta == 1.0) return SUSHI_CUDA_OK;
        int64_t blocks = (m * n * batch + 255) / 256;
        if (blocks > (int64_t)d->sm_count * 16) blocks = (int64_t)d->sm_count * 16;
        sushi::scale_c_f64_kernel<<<(unsigned)blocks, 256, 0, d->stream>>>(c, m, n, ldc, stride_c, batch, beta);
        ctx->launches++;
        SC_CUDA(ctx, cudaGetLastError());
        return SUSHI_CUDA_OK;
    }
    sushi::DgemmArgs g;
    g.a = a; g.b = b; g.c = c; g.m = m; g.n = n; g.k = k; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
    g.stride_a = stride_a; g.stride_b = stride_b; g.stride_c = stride_c; g.tiles_m = 0; g.tiles_n = 0;
    g.alpha = alpha; g.beta = beta;
    g.status = d->status;
    SC_CUDA(ctx, sushi::launch_dgemm(g, trans_a != 0, trans_b != 0, batch, d->sm_count, d->stream));
    ctx->launches++;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_dgemm(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b, int64_t m, int64_t n, int64_t k,
                                double alpha, const double* a, int64_t lda, const double* b, int64_t ldb, double beta,
                                double* c, int64_t ldc)
{
    return sushi_cuda_dgemm_strided_batched(ctx, dev, trans_a, trans_b, m, n, k, alpha, a, lda, 0, b, ldb, 0, beta, c, ldc, 0, 1);
}

extern "C" int sushi_cuda_sgemm_strided_batched_ex(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                   int64_t m, int64_t n, int64_t k, float alpha,
                                                   const float* a, int64_t lda, int64_t stride_a,
                                                   const float* b, int64_t ldb, int64_t stride_b,
                                                   float beta, float* c, int64_t ldc, int64_t stride_c,
                                                   int64_t batch, int epilogue)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_ex: bad context or device index");
    if (epilogue != SUSHI_EPILOGUE_NONE && epilogue != SUSHI_EPILOGUE_RELU)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_ex: unknown epilogue");
    return sushi_cuda_sgemm_strided_batched_act(ctx, dev, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b,
                                                beta, c, ldc, stride_c, batch, epilogue, 0.0f);
}

extern "C" int sushi_cuda_sgemm_strided_batched_act(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                    int64_t m, int64_t n, int64_t k, float alpha,
                                                    const float* a, int64_t lda, int64_t stride_a,
                                                    const float* b, int64_t ldb, int64_t stride_b,
                                                    float beta, float* c, int64_t ldc, int64_t stride_c,
                                                    int64_t batch, int activation, float act_param)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_act: bad context or device index");
    if (activation < 0 || activation >= sushi::ACT_COUNT)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_act: unknown activation");
    int rc = validate_gemm(ctx, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, stride_a, stride_b, stride_c, batch);
    if (rc != SUSHI_CUDA_OK) return rc;
    SlabReuse opts;
    opts.act = activation; opts.act_param = act_param;
    return run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b, beta, c, ldc,
                    stride_c, batch, &opts);
}

extern "C" int sushi_cuda_sgemm_grouped(sushi_cuda_ctx* ctx, int dev, const sushi_cuda_gemm_desc* problems, int64_t count)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || count < 0 || (count > 0 && !problems))
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_grouped: bad argument");
    if (count == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    std::vector<sushi::GroupedGemm> small;
    std::vector<int64_t> large;
    small.reserve((size_t)count);
    int64_t tiles = 0;
    for (int64_t i = 0; i < count; ++i)
    {
        const sushi_cuda_gemm_desc& q = problems[i];
        int rc = validate_gemm(ctx, q.m, q.n, q.k, q.a, q.lda, q.b, q.ldb, q.c, q.ldc, q.trans_a, q.trans_b, q.stride_a,
                               q.stride_b, q.stride_c, q.batch);
        if (rc != SUSHI_CUDA_OK) return rc;
        if (q.epilogue < 0 || q.epilogue >= sushi::ACT_COUNT)
            return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_grouped: unknown epilogue");
        if (q.m == 0 || q.n == 0 || q.batch == 0) continue;
        const bool tensor = ctx->variant == SUSHI_GEMM_TC3X ||
                            (ctx->variant == SUSHI_GEMM_AUTO && prefer_tc3x(q.m, q.n, q.k, q.batch, d->sm_count));
        if (tensor || q.k == 0 || q.alpha == 0.0f) { large.push_back(i); continue; }
        sushi::GroupedGemm g;
        g.g.a = q.a; g.g.b = q.b; g.g.c = q.c; g.g.m = q.m; g.g.n = q.n; g.g.k = q.k;
        g.g.lda = q.lda; g.g.ldb = q.ldb; g.g.ldc = q.ldc;
        g.g.stride_a = q.stride_a; g.g.stride_b = q.stride_b; g.g.stride_c = q.stride_c;
        g.g.tiles_m = (q.m + 63) / 64; g.g.tiles_n = (q.n + 63) / 64;
        g.g.alpha = q.alpha; g.g.beta = q.beta; g.g.act = q.epilogue; g.g.act_param = q.act_param; g.g.tri = 0;
        g.trans_a = q.trans_a != 0; g.trans_b = q.trans_b != 0;
        g.first_tile = tiles;
        tiles += g.g.tiles_m * g.g.tiles_n * q.batch;
        small.push_back(g);
    }
    if (tiles > 0x7fffffffLL) return set_error(ctx, SUSHI_CUDA_ERR_UNSUPPORTED, "sgemm_grouped: too many tiles for one launch");
    if (!small.empty())
    {
        const size_t bytes = small.size() * sizeof(sushi::GroupedGemm);
        int rc = grow(ctx, *d, &d->group_buf, &d->group_bytes, bytes);
        if (rc != SUSHI_CUDA_OK) return rc;
        // pageable source: the runtime stages it before returning, so `small` may go out of scope
        SC_CUDA(ctx, cudaMemcpyAsync(d->group_buf, small.data(), bytes, cudaMemcpyHostToDevice, d->stream));
        sushi::sgemm_grouped_simt_kernel<<<(unsigned)tiles, sushi::SIMT_THREADS, 0, d->stream>>>(
            static_cast<const sushi::GroupedGemm*>(d->group_buf), (int)small.size());
        ctx->launches++;
        SC_CUDA(ctx, cudaGetLastError());
    }
    for (int64_t i : large)
    {
        const sushi_cuda_gemm_desc& q = problems[i];
        SlabReuse opts;
        opts.act = q.epilogue; opts.act_param = q.act_param;
        int rc = run_gemm(ctx, *d, q.trans_a, q.trans_b, q.m, q.n, q.k, q.alpha, q.a, q.lda, q.stride_a, q.b, q.ldb,
                          q.stride_b, q.beta, q.c, q.ldc, q.stride_c, q.batch, &opts);
        if (rc != SUSHI_CUDA_OK) return rc;
    }
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_ssyrk_strided_batched(sushi_cuda_ctx* ctx, int dev, int upper, int trans, int64_t n, int64_t k,
                                                float alpha, const float* a, int64_t lda, int64_t stride_a, float beta,
                                                float* c, int64_t ldc, int64_t stride_c, int64_t batch)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "ssyrk: bad context or device index");
    // C <- alpha * op(A) * op(A)^T + beta * C is the GEMM with B = A and op(B) = op(A)^T
    int rc = validate_gemm(ctx, n, n, k, a, lda, a, lda, c, ldc, trans, !trans, stride_a, stride_a, stride_c, batch);
    if (rc != SUSHI_CUDA_OK) return rc;
    SlabReuse opts;
    opts.tri = upper ? 2 : 1;
    if (k == 0 || alpha == 0.0f)
    {
        // only beta * C on the triangle remains: run the FFMA kernel with k = 0 (it reads no operand)
        opts.variant = SUSHI_GEMM_SIMT;
        if (beta == 1.0f) return SUSHI_CUDA_OK;
        return run_gemm(ctx, *d, trans, !trans, n, n, 0, 1.0f, c, lda > 0 ? lda : 1, stride_a, c, lda > 0 ? lda : 1, stride_a,
                        beta, c, ldc, stride_c, batch, &opts);
    }
    return run_gemm(ctx, *d, trans, !trans, n, n, k, alpha, a, lda, stride_a, a, lda, stride_a, beta, c, ldc, stride_c,
                    batch, &opts);
}

extern "C" int sushi_cuda_ssyrk(sushi_cuda_ctx* ctx, int dev, int upper, int trans, int64_t n, int64_t k, float alpha,
                                const float* a, int64_t lda, float beta, float* c, int64_t ldc)
{
    return sushi_cuda_ssyrk_strided_batched(ctx, dev, upper, trans, n, k, alpha, a, lda, 0, beta, c, ldc, 0, 1);
}

namespace {

// One triangular solve, row-major:  left: op(A) X = alpha B (A m x m);  right: X op(A) = alpha B (A n x n);
// X overwrites B.  Recursive blocked substitution over 512-wide blocks of the triangular dimension:
// a range of blocks is cut in two, the first half is solved, its contribution is removed from the
// second half with ONE GEMM (alpha = -1, beta = 1, in place; at the top level half of all the
// flops), then the second half is solved.  A single block is applied through its explicit inverse
// (a GEMM into a temporary, copied back).  The 512 x 512 inverses come from the substitution
// kernel on the 128 x 128 diagonal sub-blocks, assembled level by level (128 -> 256 -> 512) with
// inv21 = -inv22 * T21 * inv11 (lower; inv12 = -inv11 * T12 * inv22 for upper) as batched GEMMs.
int run_trsm(sushi_cuda_ctx* ctx, DeviceState& d, int left, int upper, int trans, int unit_diag, int64_t m, int64_t n,
             float alpha, const float* a, int64_t lda, float* b, int64_t ldb)
{
    if (m == 0 || n == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d.device));
    constexpr int64_t NB = sushi::TRSM_BASE, HB = sushi::TRSM_NB;
    const int64_t dim = left ? m : n;
    const int64_t nblk = (dim + NB - 1) / NB;
    const bool eff_lower = (upper != 0) == (trans != 0);        // op(A) is lower triangular
    auto scale_b = [&](float f) -> int {
        int64_t blocks = (m * n + 255) / 256;
        if (blocks > (int64_t)d.sm_count * 16) blocks = (int64_t)d.sm_count * 16;
        sushi::scale_c_kernel<<<(unsigned)blocks, 256, 0, d.stream>>>(b, m, n, ldb, 0, 1, f);
        ctx->launches++;
        SC_CUDA(ctx, cudaGetLastError());
        return SUSHI_CUDA_OK;
    };
    if (alpha == 0.0f) return scale_b(0.0f);                    // BLAS convention: B <- 0 without reading A

    // workspace: the inverses, one 256 x 256 product T21 * inv11 per block, one block row / column of temporaries
    constexpr int64_t WB = NB / 2;
    const size_t inv_bytes = (size_t)nblk * NB * NB * sizeof(float);
    const size_t w_bytes = (size_t)nblk * WB * WB * sizeof(float);
    const size_t tmp_bytes = (size_t)NB * (size_t)(left ? n : m) * sizeof(float);
    int rc = grow(ctx, d, &d.trsm_buf, &d.trsm_bytes, inv_bytes + w_bytes + tmp_bytes);
    if (rc != SUSHI_CUDA_OK) return rc;
    float* inv = static_cast<float*>(d.trsm_buf);
    float* w = reinterpret_cast<float*>(static_cast<char*>(d.trsm_buf) + inv_bytes);
    float* tmp = reinterpret_cast<float*>(static_cast<char*>(d.trsm_buf) + inv_bytes + w_bytes);

    SC_CUDA(ctx, cudaMemsetAsync(inv, 0, inv_bytes, d.stream));
    sushi::TrtriArgs t;
    t.a = a; t.inv = inv; t.dim = dim; t.lda = lda; t.trans = trans != 0; t.eff_lower = eff_lower; t.unit_diag = unit_diag != 0;
    SC_CUDA(ctx, sushi::launch_trtri_diag_blocks(t, d.stream));
    ctx->launches++;

    // Inverse of a diagonal block of order 2L from the inverses of its halves of order L:
    //   lower:  inv21 = -inv22 * T21 * inv11        upper:  inv12 = -inv11 * T12 * inv22
    // for `count` consecutive 512-blocks starting at q0, the 2L block sitting `off` rows into each of them and
    // its second half holding r2 <= L rows of the matrix (the rest of that half is identity padding).
    auto pair_up = [&](int64_t L, int64_t off, int64_t q0, int64_t count, int64_t r2) -> int {
        if (count <= 0 || r2 <= 0) return SUSHI_CUDA_OK;
        const int64_t p0 = q0 * NB + off;
        float* i11 = inv + q0 * NB * NB + off * (NB + 1);
        float* i22 = i11 + L * (NB + 1);
        float* wq = w + q0 * WB * WB;
        const int64_t sa = NB * (lda + 1), si = NB * NB, sw = WB * WB;
        int r;
        if (eff_lower)
        {
            // T21 = op(A)[p0 + L .., p0 ..] (r2 x L);  W = T21 * inv11;  inv21 = -inv22 * W
            const float* t21 = trans ? a + p0 * lda + p0 + L : a + (p0 + L) * lda + p0;
            r = run_gemm(ctx, d, trans, 0, r2, L, L, 1.0f, t21, lda, sa, i11, NB, si, 0.0f, wq, L, sw, count);
            if (r != SUSHI_CUDA_OK) return r;
            return run_gemm(ctx, d, 0, 0, r2, L, r2, -1.0f, i22, NB, si, wq, L, sw, 0.0f, i11 + L * NB, NB, si, count);
        }
        // T12 = op(A)[p0 .., p0 + L ..] (L x r2);  W = T12 * inv22;  inv12 = -inv11 * W
        const float* t12 = trans ? a + (p0 + L) * lda + p0 : a + p0 * lda + p0 + L;
        r = run_gemm(ctx, d, trans, 0, L, r2, r2, 1.0f, t12, lda, sa, i22, NB, si, 0.0f, wq, L, sw, count);
        if (r != SUSHI_CUDA_OK) return r;
        return run_gemm(ctx, d, 0, 0, L, r2, L, -1.0f, i11, NB, si, wq, L, sw, 0.0f, i11 + L, NB, si, count);
    };
    for (int64_t L = HB; L < NB; L *= 2)
        for (int64_t off = 0; off < NB; off += 2 * L)
        {
            // 512-blocks whose 2L block at `off` lies wholly inside the matrix run as one batched call,
            // the (at most one) partial one after them on its own
            const int64_t full = dim >= off + 2 * L ? (dim - off - 2 * L) / NB + 1 : 0;
            if ((rc = pair_up(L, off, 0, full, L)) != SUSHI_CUDA_OK) return rc;
            const int64_t p0 = full * NB + off;
            if (p0 + L < dim && (rc = pair_up(L, off, full, 1, dim - p0 - L)) != SUSHI_CUDA_OK) return rc;
        }

    if (alpha != 1.0f) { rc = scale_b(alpha); if (rc != SUSHI_CUDA_OK) return rc; }

    // substitution order: forward when the solved blocks lie before the current one
    const bool forward = left ? eff_lower : !eff_lower;
    auto lim = [&](int64_t blk_index) { const int64_t e = blk_index * NB; return e < dim ? e : dim; };
    // remove the contribution of the solved range [s0, s1) from the target range [r0, r1) (elements)
    auto update = [&](int64_t r0, int64_t r1, int64_t s0, int64_t s1) -> int {
        if (r1 <= r0 || s1 <= s0) return SUSHI_CUDA_OK;
        if (left)
        {
            const float* t_op = trans ? a + s0 * lda + r0 : a + r0 * lda + s0;       // op(A)[r0.., s0..]
            return run_gemm(ctx, d, trans, 0, r1 - r0, n, s1 - s0, -1.0f, t_op, lda, 0, b + s0 * ldb, ldb, 0, 1.0f,
                            b + r0 * ldb, ldb, 0, 1);
        }
        const float* t_op = trans ? a + r0 * lda + s0 : a + s0 * lda + r0;           // op(A)[s0.., r0..]
        return run_gemm(ctx, d, 0, trans, m, r1 - r0, s1 - s0, -1.0f, b + s0, ldb, 0, t_op, lda, 0, 1.0f, b + r0, ldb, 0, 1);
    };
    auto apply_inverse = [&](int64_t blk_index) -> int {
        const int64_t p0 = blk_index * NB, size = lim(blk_index + 1) - p0;
        const float* iv = inv + blk_index * NB * NB;
        if (left)
        {
            float* b_blk = b + p0 * ldb;                                              // size x n
            int r = run_gemm(ctx, d, 0, 0, size, n, size, 1.0f, iv, NB, 0, b_blk, ldb, 0, 0.0f, tmp, n, 0, 1);
            if (r != SUSHI_CUDA_OK) return r;
            SC_CUDA(ctx, cudaMemcpy2DAsync(b_blk, (size_t)ldb * sizeof(float), tmp, (size_t)n * sizeof(float),
                                           (size_t)n * sizeof(float), (size_t)size, cudaMemcpyDeviceToDevice, d.stream));
            return SUSHI_CUDA_OK;
        }
        float* b_blk = b + p0;                                                        // m x size, leading dimension ldb
        int r = run_gemm(ctx, d, 0, 0, m, size, size, 1.0f, b_blk, ldb, 0, iv, NB, 0, 0.0f, tmp, size, 0, 1);
        if (r != SUSHI_CUDA_OK) return r;
        SC_CUDA(ctx, cudaMemcpy2DAsync(b_blk, (size_t)ldb * sizeof(float), tmp, (size_t)size * sizeof(float),
                                       (size_t)size * sizeof(float), (size_t)m, cudaMemcpyDeviceToDevice, d.stream));
        return SUSHI_CUDA_OK;
    };
    // explicit stack instead of recursion: ranges of blocks [lo, hi); kind 0 = solve, 1 = update
    struct Frame { int64_t lo, hi, mid; int kind; };
    std::vector<Frame> stack;
    stack.push_back({0, nblk, 0, 0});
    while (!stack.empty())
    {
        const Frame f = stack.back();
        stack.pop_back();
        if (f.kind == 1)
        {
            // [lo, mid) and [mid, hi): the half solved first feeds the other one
            rc = forward ? update(lim(f.mid), lim(f.hi), lim(f.lo), lim(f.mid))
                         : update(lim(f.lo), lim(f.mid), lim(f.mid), lim(f.hi));
        }
        else if (f.hi - f.lo == 1) rc = apply_inverse(f.lo);
        else
        {
            const int64_t mid = f.lo + (f.hi - f.lo + 1) / 2;
            // pushed in reverse order of execution
            if (forward) { stack.push_back({mid, f.hi, 0, 0}); stack.push_back({f.lo, f.hi, mid, 1}); stack.push_back({f.lo, mid, 0, 0}); }
            else { stack.push_back({f.lo, mid, 0, 0}); stack.push_back({f.lo, f.hi, mid, 1}); stack.push_back({mid, f.hi, 0, 0}); }
        }
        if (rc != SUSHI_CUDA_OK) return rc;
    }
    return SUSHI_CUDA_OK;
}

} // namespace

extern "C" int sushi_cuda_strsm_strided_batched(sushi_cuda_ctx* ctx, int dev, int left, int upper, int trans, int unit_diag,
                                                int64_t m, int64_t n, float alpha, const float* a, int64_t lda,
                                                int64_t stride_a, float* b, int64_t ldb, int64_t stride_b, int64_t batch)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "strsm: bad context or device index");
    const int64_t dim = left ? m : n;
    if (m < 0 || n < 0 || batch < 0 || stride_a < 0 || stride_b < 0)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "strsm: negative dimension or stride");
    if (lda < (dim > 1 ? dim : 1)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "strsm: lda too small");
    if (ldb < (n > 1 ? n : 1)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "strsm: ldb too small");
    if (m > 0 && n > 0 && batch > 0 && (!a || !b)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "strsm: A or B is null");
    for (int64_t i = 0; i < batch; ++i)
    {
        int rc = run_trsm(ctx, *d, left, upper, trans, unit_diag, m, n, alpha, a + i * stride_a, lda, b + i * stride_b, ldb);
        if (rc != SUSHI_CUDA_OK) return rc;
    }
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_strsm(sushi_cuda_ctx* ctx, int dev, int left, int upper, int trans, int unit_diag,
                                int64_t m, int64_t n, float alpha, const float* a, int64_t lda, float* b, int64_t ldb)
{
    return sushi_cuda_strsm_strided_batched(ctx, dev, left, upper, trans, unit_diag, m, n, alpha, a, lda, 0, b, ldb, 0, 1);
}

extern "C" int sushi_cuda_activation(sushi_cuda_ctx* ctx, int dev, int activation, float act_param, float* x, int64_t count)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || count < 0 || (count > 0 && !x)) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "activation: bad argument");
    if (activation < 0 || activation >= sushi::ACT_COUNT)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "activation: unknown activation");
    if (count == 0 || activation == sushi::ACT_NONE) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    int64_t blocks = (count / 4 + 255) / 256 + 1;
    if (blocks > (int64_t)d->sm_count * 16) blocks = (int64_t)d->sm_count * 16;
    sushi::activation_forward_kernel<<<(unsigned)blocks, 256, 0, d->stream>>>(x, count, activation, act_param);
    ctx->launches++;
    SC_CUDA(ctx, cudaGetLastError());
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_activation_backward(sushi_cuda_ctx* ctx, int dev, int activation, float act_param, const float* dy,
                                              const float* saved, float* dx, int64_t count)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || count < 0 || (count > 0 && (!dy || !saved || !dx)))
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "activation_backward: bad argument");
    if (activation <= sushi::ACT_NONE || activation >= sushi::ACT_COUNT)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "activation_backward: unknown activation");
    if (count == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    int64_t blocks = (count / 4 + 255) / 256 + 1;
    if (blocks > (int64_t)d->sm_count * 16) blocks = (int64_t)d->sm_count * 16;
    sushi::activation_backward_kernel<<<(unsigned)blocks, 256, 0, d->stream>>>(dy, saved, dx, count, activation, act_param);
    ctx->launches++;
    SC_CUDA(ctx, cudaGetLastError());
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_relu(sushi_cuda_ctx* ctx, int dev, float* x, int64_t count)
{
    return sushi_cuda_activation(ctx, dev, sushi::ACT_RELU, 0.0f, x, count);
}

extern "C" int sushi_cuda_sgemm(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                int64_t m, int64_t n, int64_t k, float alpha,
                                const float* a, int64_t lda, const float* b, int64_t ldb,
                                float beta, float* c, int64_t ldc)
{
    return sushi_cuda_sgemm_strided_batched(ctx, dev, trans_a, trans_b, m, n, k, alpha, a, lda, 0, b, ldb, 0,
                                            beta, c, ldc, 0, 1);
}

extern "C" int sushi_cuda_sgemm_strided_batched_host(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                     int64_t m, int64_t n, int64_t k, float alpha,
                                                     const float* a, int64_t lda, int64_t stride_a,
                                                     const float* b, int64_t ldb, int64_t stride_b,
                                                     float beta, float* c, int64_t ldc, int64_t stride_c,
                                                     int64_t batch)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_host: bad context or device index");
    int rc = validate_gemm(ctx, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, stride_a, stride_b, stride_c, batch);
    if (rc != SUSHI_CUDA_OK) return rc;
    if (m == 0 || n == 0 || batch == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    const size_t ea = (size_t)extent(trans_a ? k : m, trans_a ? m : k, lda, stride_a, batch) * sizeof(float);
    const size_t eb = (size_t)extent(trans_b ? n : k, trans_b ? k : n, ldb, stride_b, batch) * sizeof(float);
    const size_t ec = (size_t)extent(m, n, ldc, stride_c, batch) * sizeof(float);
    const size_t need[3] = {ea ? ea : 4, eb ? eb : 4, ec};
    for (int i = 0; i < 3; ++i)
        if ((rc = grow(ctx, *d, &d->stage[i], &d->stage_bytes[i], need[i])) != SUSHI_CUDA_OK) return rc;
    float* da = static_cast<float*>(d->stage[0]);
    float* db = static_cast<float*>(d->stage[1]);
    float* dc = static_cast<float*>(d->stage[2]);
    // C goes up when it is read (beta != 0) or when its buffer has gaps the copy back must preserve
    const bool dense_c = (ldc == n) && (batch == 1 || stride_c == m * n);
    const bool upload_c = beta != 0.0f || !dense_c;

    // Large problems are cut into chunks -- row blocks of A and C, or batch entries -- so that the
    // upload of chunk i+1, the multiplication of chunk i and the download of chunk i-1 overlap
    // (PCIe is full duplex and the copies dwarf the arithmetic).  B goes up once and is split
    // into planes once.  Row blocks of a transposed A are column blocks of the stored k x m matrix
    // and go up as strided 2-D copies.  Small problems take the plain sequence.
    const size_t total_bytes = ea + eb + ec;
    int chunks = 1;
    if (total_bytes >= ((size_t)32 << 20))
    {
        if (batch >= 4) chunks = 4;
        else if (batch == 1 && m >= 2048) chunks = 4;
    }
    if (chunks == 1)
    {
        if (ea) SC_CUDA(ctx, cudaMemcpyAsync(da, a, ea, cudaMemcpyHostToDevice, d->stream));
        if (eb) SC_CUDA(ctx, cudaMemcpyAsync(db, b, eb, cudaMemcpyHostToDevice, d->stream));
        if (upload_c) SC_CUDA(ctx, cudaMemcpyAsync(dc, c, ec, cudaMemcpyHostToDevice, d->stream));
        rc = run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, da, lda, stride_a, db, ldb, stride_b, beta, dc, ldc,
                      stride_c, batch);
        if (rc != SUSHI_CUDA_OK) return rc;
        SC_CUDA(ctx, cudaMemcpyAsync(c, dc, ec, cudaMemcpyDeviceToHost, d->stream));
        return SUSHI_CUDA_OK;
    }

    if (!d->copy_in)
    {
        SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->copy_in, cudaStreamNonBlocking));
        SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->copy_out, cudaStreamNonBlocking));
        for (cudaEvent_t& e : d->pipe_events) SC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    cudaEvent_t* ev = d->pipe_events;          // [0] start, [1..4] chunk uploaded, [5..8] chunk multiplied, [9] all downloaded
    SC_CUDA(ctx, cudaEventRecord(ev[0], d->stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_in, ev[0], 0));      // after everything queued before this call
    SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_out, ev[0], 0));
    SlabReuse reuse;
    const bool by_batch = batch > 1;
    const int64_t units = by_batch ? batch : m;
    int64_t per = (units + chunks - 1) / chunks;
    if (!by_batch) per = (per + 255) / 256 * 256;                 // whole tiles per chunk
    if (by_batch)
    {
        // batch entries do not share B: upload and split per chunk
        for (int i = 0; i < chunks; ++i)
        {
            const int64_t u0 = i * per, u1 = (u0 + per < units) ? u0 + per : units;
            if (u1 <= u0) { SC_CUDA(ctx, cudaEventRecord(ev[1 + i], d->copy_in)); SC_CUDA(ctx, cudaEventRecord(ev[5 + i], d->stream)); continue; }
            const int64_t nb = u1 - u0;
            const size_t ca = (size_t)extent(trans_a ? k : m, trans_a ? m : k, lda, stride_a, nb) * sizeof(float);
            const size_t cb = (size_t)extent(trans_b ? n : k, trans_b ? k : n, ldb, stride_b, nb) * sizeof(float);
            const size_t cc = (size_t)extent(m, n, ldc, stride_c, nb) * sizeof(float);
            SC_CUDA(ctx, cudaMemcpyAsync(da + u0 * stride_a, a + u0 * stride_a, ca, cudaMemcpyHostToDevice, d->copy_in));
            SC_CUDA(ctx, cudaMemcpyAsync(db + u0 * stride_b, b + u0 * stride_b, cb, cudaMemcpyHostToDevice, d->copy_in));
            if (upload_c) SC_CUDA(ctx, cudaMemcpyAsync(dc + u0 * stride_c, c + u0 * stride_c, cc, cudaMemcpyHostToDevice, d->copy_in));
            SC_CUDA(ctx, cudaEventRecord(ev[1 + i], d->copy_in));
            SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ev[1 + i], 0));
            rc = run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, da + u0 * stride_a, lda, stride_a, db + u0 * stride_b,
                          ldb, stride_b, beta, dc + u0 * stride_c, ldc, stride_c, nb);
            if (rc != SUSHI_CUDA_OK) return rc;
            SC_CUDA(ctx, cudaEventRecord(ev[5 + i], d->stream));
            SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_out, ev[5 + i], 0));
            SC_CUDA(ctx, cudaMemcpyAsync(c + u0 * stride_c, dc + u0 * stride_c, cc, cudaMemcpyDeviceToHost, d->copy_out));
        }
    }
    else
    {
        if (eb) SC_CUDA(ctx, cudaMemcpyAsync(db, b, eb, cudaMemcpyHostToDevice, d->copy_in));
        reuse.max_rows = per < m ? per : m;
        for (int i = 0; i < chunks; ++i)
        {
            const int64_t r0 = i * per, r1 = (r0 + per < m) ? r0 + per : m;
            if (r1 <= r0) continue;
            const int64_t rows = r1 - r0;
            const size_t ca = (size_t)extent(rows, k, lda, 0, 1) * sizeof(float);
            const size_t cc = (size_t)extent(rows, n, ldc, 0, 1) * sizeof(float);
            const float* a_chunk = trans_a ? da + r0 : da + r0 * lda;
            if (k > 0)
            {
                if (trans_a)
                    SC_CUDA(ctx, cudaMemcpy2DAsync(da + r0, (size_t)lda * sizeof(float), a + r0, (size_t)lda * sizeof(float),
                                                   (size_t)rows * sizeof(float), (size_t)k, cudaMemcpyHostToDevice, d->copy_in));
                else
                    SC_CUDA(ctx, cudaMemcpyAsync(da + r0 * lda, a + r0 * lda, ca, cudaMemcpyHostToDevice, d->copy_in));
            }
            if (upload_c) SC_CUDA(ctx, cudaMemcpyAsync(dc + r0 * ldc, c + r0 * ldc, cc, cudaMemcpyHostToDevice, d->copy_in));
            SC_CUDA(ctx, cudaEventRecord(ev[1 + i], d->copy_in));
            SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ev[1 + i], 0));
            rc = run_gemm(ctx, *d, trans_a, trans_b, rows, n, k, alpha, a_chunk, lda, 0, db, ldb, 0, beta,
                          dc + r0 * ldc, ldc, 0, 1, &reuse);
            if (rc != SUSHI_CUDA_OK) return rc;
            SC_CUDA(ctx, cudaEventRecord(ev[5 + i], d->stream));
            SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_out, ev[5 + i], 0));
            SC_CUDA(ctx, cudaMemcpyAsync(c + r0 * ldc, dc + r0 * ldc, cc, cudaMemcpyDeviceToHost, d->copy_out));
        }
    }
    // the call completes on the caller's stream once the last download has
    SC_CUDA(ctx, cudaEventRecord(ev[9], d->copy_out));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ev[9], 0));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch, size_t* bytes)
{
    if (!bytes || m < 0 || n < 0 || k < 0 || batch < 0)
        return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "gemm_workspace_bytes: bad argument");
    *bytes = sushi::split_plane_bytes(m, k, batch) + sushi::split_plane_bytes(n, k, batch);
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_reserve_workspace(sushi_cuda_ctx* ctx, int dev, size_t bytes)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "reserve_workspace: bad context or device index");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    return grow(ctx, *d, &d->workspace, &d->workspace_bytes, bytes);
}

// ======================================================================== multi-GPU
extern "C" int sushi_cuda_partition(int64_t total, int nranks, int rank, int64_t* first, int64_t* count)
{
    if (total < 0 || nranks <= 0 || rank < 0 || rank >= nranks || !first || !count)
        return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "partition: bad argument");
    const int64_t block = (total + nranks - 1) / nranks;
    int64_t lo = block * rank;
    if (lo > total) lo = total;
    int64_t hi = lo + block;
    if (hi > total) hi = total;
    *first = lo;
    *count = hi - lo;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_comm_unique_id(void* id128)
{
    if (!id128) return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "comm_unique_id: null output");
    std::string err;
    if (!load_nccl(&err)) return set_error(nullptr, SUSHI_CUDA_ERR_COMM, err);
    int rc = g_nccl.GetUniqueId(id128);
    if (rc != 0) return nccl_fail(nullptr, rc, "ncclGetUniqueId");
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_comm_init_rank(sushi_cuda_ctx* ctx, int dev, const void* id128, int nranks, int rank)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !id128 || nranks < 1 || rank < 0 || rank >= nranks)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "comm_init_rank: bad argument");
    if (ctx->comm) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "comm_init_rank: communicator already exists");
    std::string err;
    if (injected_failure(ctx, SUSHI_CUDA_FAIL_COMM_INIT))
        return set_error(ctx, SUSHI_CUDA_ERR_COMM, "injected failure: communicator initialisation");
    if (!load_nccl(&err)) return set_error(ctx, SUSHI_CUDA_ERR_COMM, err);
    SC_CUDA(ctx, cudaSetDevice(d->device));
    Id128 id;
    memcpy(id.bytes, id128, sizeof id.bytes);
    SC_NCCL(ctx, g_nccl.CommInitRank(&ctx->comm, nranks, id, rank));
    ctx->comm_dev = dev; ctx->nranks = nranks; ctx->rank = rank;
    SC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking));
    SC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->comm_done, cudaEventDisableTiming));
    SC_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->barrier_word), 256));
    SC_CUDA(ctx, cudaMemset(ctx->barrier_word, 0, 256));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_comm_destroy(sushi_cuda_ctx* ctx)
{
    if (!ctx) return SUSHI_CUDA_OK;
    if (ctx->comm_stream) { cudaStreamSynchronize(ctx->comm_stream); }
    if (ctx->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->comm);
    ctx->comm = nullptr;
    for (cudaEvent_t e : ctx->slab_events) cudaEventDestroy(e);
    ctx->slab_events.clear();
    if (ctx->comm_done) { cudaEventDestroy(ctx->comm_done); ctx->comm_done = nullptr; }
    if (ctx->comm_stream) { cudaStreamDestroy(ctx->comm_stream); ctx->comm_stream = nullptr; }
    if (ctx->barrier_word) { cudaFree(ctx->barrier_word); ctx->barrier_word = nullptr; }
    ctx->peer_buffers.clear();
    ctx->peer_bytes = 0;
    ctx->comm_dev = -1; ctx->nranks = 1; ctx->rank = 0;
    return SUSHI_CUDA_OK;
}

namespace {

// Exchange `units` owned units (rows or batches; `unit_elems` floats each, contiguous) of every
// rank, restricted to local unit range [u0, u1) of each rank's block.  In place in c_full.
int gather_slab(sushi_cuda_ctx* ctx, float* c_full, int64_t total_units, int64_t unit_elems, int64_t u0, int64_t u1)
{
    const bool even = (total_units % ctx->nranks) == 0;
    const int64_t block = (total_units + ctx->nranks - 1) / ctx->nranks;
    if (even && u0 == 0 && u1 == block)
    {
        // whole blocks of equal size: one in-place all-gather
        SC_NCCL(ctx, g_nccl.AllGather(c_full + (int64_t)ctx->rank * block * unit_elems, c_full,
                                      (size_t)(block * unit_elems), NCCL_FLOAT32, ctx->comm, ctx->comm_stream));
        return SUSHI_CUDA_OK;
    }
    // slab of each rank's block: every rank is the root of its own piece
    SC_NCCL(ctx, g_nccl.GroupStart());
    for (int r = 0; r < ctx->nranks; ++r)
    {
        int64_t first, count;
        sushi_cuda_partition(total_units, ctx->nranks, r, &first, &count);
        const int64_t lo = u0 < count ? u0 : count, hi = u1 < count ? u1 : count;
        if (hi <= lo) continue;
        float* piece = c_full + (first + lo) * unit_elems;
        int rc = g_nccl.Broadcast(piece, piece, (size_t)((hi - lo) * unit_elems), NCCL_FLOAT32, r, ctx->comm,
                                  ctx->comm_stream);
        if (rc != 0) { g_nccl.GroupEnd(); return nccl_fail(ctx, rc, "ncclBroadcast"); }
    }
    SC_NCCL(ctx, g_nccl.GroupEnd());
    return SUSHI_CUDA_OK;
}

int ensure_events(sushi_cuda_ctx* ctx, size_t n)
{
    while (ctx->slab_events.size() < n)
    {
        cudaEvent_t e;
        SC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->slab_events.push_back(e);
    }
    return SUSHI_CUDA_OK;
}

} // namespace

extern "C" int sushi_cuda_ipc_export(sushi_cuda_ctx* ctx, int dev, const void* base_ptr, void* handle64)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !base_ptr || !handle64) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "ipc_export: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    SC_CUDA(ctx, cudaSetDevice(d->device));
    cudaIpcMemHandle_t h;
    SC_CUDA(ctx, cudaIpcGetMemHandle(&h, const_cast<void*>(base_ptr)));
    memcpy(handle64, &h, sizeof h);
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_ipc_open(sushi_cuda_ctx* ctx, int dev, const void* handle64, void** peer_ptr)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || !handle64 || !peer_ptr) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "ipc_open: bad argument");
    *peer_ptr = nullptr;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    SC_CUDA(ctx, cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_ipc_close(sushi_cuda_ctx* ctx, int dev, void* peer_ptr)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "ipc_close: bad context or device index");
    if (!peer_ptr) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    SC_CUDA(ctx, cudaStreamSynchronize(d->stream));
    SC_CUDA(ctx, cudaIpcCloseMemHandle(peer_ptr));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_comm_set_peer_buffers(sushi_cuda_ctx* ctx, int dev, void* const* buffers, int count,
                                                size_t bytes_each)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "comm_set_peer_buffers: bad context or device index");
    if (count == 0) { ctx->peer_buffers.clear(); ctx->peer_bytes = 0; return SUSHI_CUDA_OK; }
    if (!ctx->comm || ctx->comm_dev != dev || !buffers || count != ctx->nranks || count > 8)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG,
                         "comm_set_peer_buffers: needs a communicator on this device and one buffer per rank (at most 8)");
    for (int i = 0; i < count; ++i)
        if (!buffers[i]) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "comm_set_peer_buffers: null buffer");
    ctx->peer_buffers.assign(buffers, buffers + count);
    ctx->peer_bytes = bytes_each;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_row_sharded_exchange(int64_t m, int64_t n, int64_t k, int nranks, int variant, int sm_count,
                                               int gather, int* exchange)
{
    if (!exchange || m < 0 || n < 0 || k < 0 || nranks < 1 || sm_count < 1)
        return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "row_sharded_exchange: bad argument");
    *exchange = 0;
    if (gather == 0 || nranks == 1) return SUSHI_CUDA_OK;
    *exchange = 1;
    if (gather != 2 || (n & 3) != 0 || m == 0) return SUSHI_CUDA_OK;
    // the peer stores live in the tensor-path kernel: it must suit both block sizes that occur, the full block
    // ceil(m / nranks) and the shorter block of the last rank that owns rows
    const int64_t block = (m + nranks - 1) / nranks;
    const int64_t nonempty = (m + block - 1) / block;
    const int64_t last_rows = m - (nonempty - 1) * block;
    auto tensor_for = [&](int64_t rows) {
        return rows > 0 && k >= 4 && (variant == SUSHI_GEMM_TC3X || (variant == SUSHI_GEMM_AUTO && prefer_tc3x(rows, n, k, 1, sm_count)));
    };
    if (tensor_for(block) && tensor_for(last_rows)) *exchange = 2;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_batch_sharded_exchange(int64_t m, int64_t n, int64_t k, int64_t batch, int nranks, int variant,
                                                 int sm_count, int gather, int* exchange)
{
    if (!exchange || m < 0 || n < 0 || k < 0 || batch < 0 || nranks < 1 || sm_count < 1)
        return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG, "batch_sharded_exchange: bad argument");
    *exchange = 0;
    if (gather == 0 || nranks == 1) return SUSHI_CUDA_OK;
    *exchange = 1;
    if (gather != 2 || (n & 3) != 0 || m == 0 || batch == 0) return SUSHI_CUDA_OK;
    // the two block sizes that occur: ceil(batch / nranks) and the shorter block of the last rank that owns entries
    const int64_t block = (batch + nranks - 1) / nranks;
    const int64_t nonempty = (batch + block - 1) / block;
    const int64_t last = batch - (nonempty - 1) * block;
    auto tensor_for = [&](int64_t cnt) {
        return cnt > 0 && k >= 4 && (variant == SUSHI_GEMM_TC3X || (variant == SUSHI_GEMM_AUTO && prefer_tc3x(m, n, k, cnt, sm_count)));
    };
    if (tensor_for(block) && tensor_for(last)) *exchange = 2;
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_sgemm_row_sharded(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                            int64_t m, int64_t n, int64_t k, float alpha,
                                            const float* a_local, int64_t lda,
                                            const float* b, int64_t ldb,
                                            float beta, float* c_full, int64_t ldc, int gather)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_row_sharded: bad context or device index");
    const int nranks = ctx->comm ? ctx->nranks : 1, rank = ctx->comm ? ctx->rank : 0;
    if (ctx->comm && ctx->comm_dev != dev)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_row_sharded: communicator is bound to another device");
    int64_t first, count;
    sushi_cuda_partition(m, nranks, rank, &first, &count);
    // validate against the local block (lda is checked for the stored layout of the local block)
    int rc = validate_gemm(ctx, count, n, k, a_local, lda, b, ldb, c_full, ldc, trans_a, trans_b, 0, 0, 0, 1);
    if (rc != SUSHI_CUDA_OK) return rc;
    const bool do_gather = gather != 0 && nranks > 1;
    if (do_gather && ldc != n)
        return set_error(ctx, SUSHI_CUDA_ERR_UNSUPPORTED, "sgemm_row_sharded: gathering needs ldc == n");
    float* c_block = c_full + first * ldc;
    // Which exchange runs -- and with it which collectives every rank issues -- is decided from quantities all
    // ranks share, never from this rank's own block (sushi_cuda_row_sharded_exchange).
    const int64_t block = (m + nranks - 1) / nranks;
    auto tensor_for = [&](int64_t rows) {
        return rows > 0 && k >= 4 && (ctx->variant == SUSHI_GEMM_TC3X ||
                                      (ctx->variant == SUSHI_GEMM_AUTO && prefer_tc3x(rows, n, k, 1, d->sm_count)));
    };
    int exchange = 0;
    sushi_cuda_row_sharded_exchange(m, n, k, nranks, ctx->variant, d->sm_count, gather, &exchange);
    if (!do_gather)
        return run_gemm(ctx, *d, trans_a, trans_b, count, n, k, alpha, a_local, lda, 0, b, ldb, 0, beta, c_block, ldc, 0, 1);

    // Fused exchange: one launch over the whole block; the epilogue stores C tiles to the peers.
    if (exchange == 2 && !ctx->peer_buffers.empty())
    {
        // what remains is this rank's own registration: a mismatch is an error, not a silent change of path
        if ((int)ctx->peer_buffers.size() != nranks || ctx->peer_buffers[rank] != c_full ||
            (reinterpret_cast<uintptr_t>(c_full) & 15) != 0 || (size_t)m * (size_t)n * sizeof(float) > ctx->peer_bytes)
            return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG,
                             "sgemm_row_sharded: gather == 2 needs c_full to be this rank's registered buffer "
                             "(sushi_cuda_comm_set_peer_buffers), 16-byte aligned and at least m*n*4 bytes");
        SC_CUDA(ctx, cudaSetDevice(d->device));
        // barrier 1: every rank has reached this call, so nobody still reads the previous C
        SC_NCCL(ctx, g_nccl.AllReduce(ctx->barrier_word, ctx->barrier_word, 1, NCCL_FLOAT32, 0, ctx->comm, d->stream));
        if (count > 0)
        {
            SlabReuse fused;
            fused.variant = SUSHI_GEMM_TC3X;
            for (int r = 0; r < nranks; ++r)
                if (r != rank) fused.peer_c[fused.n_peers++] = static_cast<float*>(ctx->peer_buffers[r]) + first * ldc;
            rc = run_gemm(ctx, *d, trans_a, trans_b, count, n, k, alpha, a_local, lda, 0, b, ldb, 0, beta, c_block, ldc, 0, 1,
                          &fused);
            if (rc != SUSHI_CUDA_OK) return rc;
        }
        // barrier 2: every rank's kernel (and with it its stores into this rank's buffer) is complete
        SC_NCCL(ctx, g_nccl.AllReduce(ctx->barrier_word, ctx->barrier_word, 1, NCCL_FLOAT32, 0, ctx->comm, d->stream));
        return SUSHI_CUDA_OK;
    }

    // Slab pipeline: multiply slab s on the compute stream, exchange it on the comm stream.
    int64_t slabs = block / 2048;                 // >= 2048 rows per slab keeps the tile grid full
    if (slabs < 1) slabs = 1;
    if (slabs > 8) slabs = 8;
    int64_t slab_rows = (block + slabs - 1) / slabs;
    slab_rows = (slab_rows + 255) / 256 * 256;
    slabs = (block + slab_rows - 1) / slab_rows;
    if ((rc = ensure_events(ctx, (size_t)slabs)) != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    // one kernel family for the whole block, B split into planes once, A planes sized for a slab
    SlabReuse reuse;
    if (ctx->variant == SUSHI_GEMM_AUTO) reuse.variant = tensor_for(count) ? SUSHI_GEMM_TC3X : SUSHI_GEMM_SIMT;
    reuse.max_rows = slab_rows < count ? slab_rows : count;
    for (int64_t s = 0; s < slabs; ++s)
    {
        const int64_t u0 = s * slab_rows, u1 = (u0 + slab_rows < block) ? u0 + slab_rows : block;
        const int64_t lo = u0 < count ? u0 : count, hi = u1 < count ? u1 : count;
        if (hi > lo)
        {
            const float* a_slab = trans_a ? a_local + lo : a_local + lo * lda;
            rc = run_gemm(ctx, *d, trans_a, trans_b, hi - lo, n, k, alpha, a_slab, lda, 0, b, ldb, 0, beta,
                          c_block + lo * ldc, ldc, 0, 1, &reuse);
            if (rc != SUSHI_CUDA_OK) return rc;
        }
        SC_CUDA(ctx, cudaEventRecord(ctx->slab_events[s], d->stream));
        SC_CUDA(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->slab_events[s], 0));
        if ((rc = gather_slab(ctx, c_full, m, n, u0, u1)) != SUSHI_CUDA_OK) return rc;
    }
    // later work on the compute stream sees the gathered C
    SC_CUDA(ctx, cudaEventRecord(ctx->comm_done, ctx->comm_stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ctx->comm_done, 0));
    return SUSHI_CUDA_OK;
}

// Host-buffer form of the row-sharded GEMM.  Every rank uploads its rows of A and only ITS share of B's k rows;
// the shares are exchanged device to device (NVLink) while A is still going up, the block is multiplied in row
// chunks as they arrive and each chunk of C streams back while the next one multiplies.  One cudaMemcpyAsync per
// piece; the copies run on the device's copy streams, the exchange on the communicator's stream.
extern "C" int sushi_cuda_sgemm_row_sharded_host(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                 int64_t m, int64_t n, int64_t k, float alpha,
                                                 const float* a_local_host, int64_t lda,
                                                 const float* b_host, int64_t ldb,
                                                 float beta, float* c_block_host, int64_t ldc,
                                                 float* a_local_dev, float* b_dev, float* c_block_dev)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_row_sharded_host: bad context or device index");
    const int nranks = ctx->comm ? ctx->nranks : 1, rank = ctx->comm ? ctx->rank : 0;
    if (ctx->comm && ctx->comm_dev != dev)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_row_sharded_host: communicator is bound to another device");
    int64_t first, count;
    sushi_cuda_partition(m, nranks, rank, &first, &count);
    int rc = validate_gemm(ctx, count, n, k, a_local_host, lda, b_host, ldb, c_block_host, ldc, trans_a, trans_b, 0, 0, 0, 1);
    if (rc != SUSHI_CUDA_OK) return rc;
    if (!a_local_dev || !b_dev || !c_block_dev)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_row_sharded_host: null device buffer");
    if (m == 0 || n == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    if (!d->copy_in)
    {
        SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->copy_in, cudaStreamNonBlocking));
        SC_CUDA(ctx, cudaStreamCreateWithFlags(&d->copy_out, cudaStreamNonBlocking));
        for (cudaEvent_t& e : d->pipe_events) SC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    cudaEvent_t* ev = d->pipe_events;          // [0] start, [1..8] chunk uploaded, [9..16] chunk multiplied, [17] all downloaded
    SC_CUDA(ctx, cudaEventRecord(ev[0], d->stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_in, ev[0], 0));      // after everything queued before this call
    SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_out, ev[0], 0));

    // ---- plan (everything that decides which collectives run is a function of what all ranks share)
    // B: this rank's k rows go up, the others' arrive over the interconnect.  That needs B stored k x n with dense
    // rows (a share is then one contiguous run); otherwise every rank uploads all of B.  Each share travels in
    // `pieces` sub-shares so that the first row chunk can start multiplying against the first sub-shares while the
    // later ones are still on their way up.
    const int64_t b_rows = trans_b ? n : k, b_cols = trans_b ? k : n;
    const bool exchange_b = nranks > 1 && !trans_b && ldb == n && k > 0;
    const int64_t k_block = (k + nranks - 1) / nranks;
    // pieces of about 2048 k rows: long enough for the panel GEMMs of the first chunk to run at speed
    const int pieces = exchange_b ? (int)std::min<int64_t>(8, std::max<int64_t>(1, k_block / 2048)) : 1;
    const int64_t piece_rows = ((k_block + pieces - 1) / pieces + 15) / 16 * 16;
    if ((rc = ensure_events(ctx, (size_t)(2 * pieces + 1))) != SUSHI_CUDA_OK) return rc;
    // A and C in row chunks of whole tiles
    const bool upload_c = beta != 0.0f || ldc != n;
    const int chunks = count >= 2048 ? 4 : 1;      // eight chunks measured slower (182 against 176 ms at 32768^3 on two GPUs)
    int64_t per = (count + chunks - 1) / chunks;
    per = (per + 255) / 256 * 256;
    auto upload_chunk = [&](int i) -> int
    {
        const int64_t r0 = i * per, r1 = (r0 + per < count) ? r0 + per : count;
        if (r1 > r0)
        {
            const int64_t rows = r1 - r0;
            if (k > 0)
            {
                if (trans_a)
                    SC_CUDA(ctx, cudaMemcpy2DAsync(a_local_dev + r0, (size_t)lda * sizeof(float), a_local_host + r0, (size_t)lda * sizeof(float),
                                                   (size_t)rows * sizeof(float), (size_t)k, cudaMemcpyHostToDevice, d->copy_in));
                else
                    SC_CUDA(ctx, cudaMemcpyAsync(a_local_dev + r0 * lda, a_local_host + r0 * lda, (size_t)extent(rows, k, lda, 0, 1) * sizeof(float),
                                                 cudaMemcpyHostToDevice, d->copy_in));
            }
            if (upload_c)
                SC_CUDA(ctx, cudaMemcpyAsync(c_block_dev + r0 * ldc, c_block_host + r0 * ldc, (size_t)extent(rows, n, ldc, 0, 1) * sizeof(float),
                                             cudaMemcpyHostToDevice, d->copy_in));
        }
        SC_CUDA(ctx, cudaEventRecord(ev[1 + i], d->copy_in));
        return SUSHI_CUDA_OK;
    };

    // ---- copies and exchange: chunk 0 of A first, then B (piece by piece, each exchanged as soon as it is up), then the rest of A
    if ((rc = upload_chunk(0)) != SUSHI_CUDA_OK) return rc;
    if (k > 0)
    {
        if (exchange_b)
        {
            int64_t k0, kc;
            sushi_cuda_partition(k, nranks, rank, &k0, &kc);
            for (int s_i = 0; s_i < pieces; ++s_i)
            {
                const int64_t u0 = s_i * piece_rows, u1 = (s_i == pieces - 1) ? k_block : u0 + piece_rows;
                const int64_t lo = u0 < kc ? u0 : kc, hi = u1 < kc ? u1 : kc;      // this rank's part of the piece
                if (hi > lo)
                    SC_CUDA(ctx, cudaMemcpyAsync(b_dev + (k0 + lo) * ldb, b_host + (k0 + lo) * ldb, (size_t)(hi - lo) * (size_t)n * sizeof(float),
                                                 cudaMemcpyHostToDevice, d->copy_in));
                SC_CUDA(ctx, cudaEventRecord(ctx->slab_events[s_i], d->copy_in));
                SC_CUDA(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->slab_events[s_i], 0));
                if ((rc = gather_slab(ctx, b_dev, k, n, u0, u1)) != SUSHI_CUDA_OK) return rc;
                SC_CUDA(ctx, cudaEventRecord(ctx->slab_events[pieces + s_i], ctx->comm_stream));
            }
        }
        else
        {
            SC_CUDA(ctx, cudaMemcpyAsync(b_dev, b_host, (size_t)extent(b_rows, b_cols, ldb, 0, 1) * sizeof(float),
                                         cudaMemcpyHostToDevice, d->copy_in));
            SC_CUDA(ctx, cudaEventRecord(ctx->slab_events[pieces], d->copy_in));
        }
    }
    for (int i = 1; i < chunks; ++i)
        if ((rc = upload_chunk(i)) != SUSHI_CUDA_OK) return rc;

    // ---- multiplication
    SlabReuse reuse;
    // one kernel family for the full-K chunks, chosen from what all ranks share (the largest block)
    {
        const int64_t block = (m + nranks - 1) / nranks;
        if (ctx->variant == SUSHI_GEMM_AUTO)
            reuse.variant = (k >= 4 && prefer_tc3x(block, n, k, 1, d->sm_count)) ? SUSHI_GEMM_TC3X : SUSHI_GEMM_SIMT;
    }
    reuse.max_rows = per < count ? per : count;
    for (int i = 0; i < chunks; ++i)
    {
        const int64_t r0 = i * per, r1 = (r0 + per < count) ? r0 + per : count;
        if (r1 <= r0) continue;
        const int64_t rows = r1 - r0;
        const size_t cc = (size_t)extent(rows, n, ldc, 0, 1) * sizeof(float);
        SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ev[1 + i], 0));
        if (i == 0 && exchange_b && pieces > 1)
        {
            // the first chunk is accumulated over the k ranges of the pieces in the order they arrive: piece s_i of
            // every rank's share, i.e. nranks disjoint k ranges per piece
            bool first_panel = true;
            for (int s_i = 0; s_i < pieces; ++s_i)
            {
                SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ctx->slab_events[pieces + s_i], 0));
                const int64_t u0 = s_i * piece_rows, u1 = (s_i == pieces - 1) ? k_block : u0 + piece_rows;
                for (int o = 0; o < nranks; ++o)
                {
                    int64_t o0, oc;
                    sushi_cuda_partition(k, nranks, o, &o0, &oc);
                    const int64_t lo = u0 < oc ? u0 : oc, hi = u1 < oc ? u1 : oc;
                    if (hi <= lo) continue;
                    const int64_t ka = o0 + lo, kw = hi - lo;
                    const float* a_panel = trans_a ? a_local_dev + ka * lda + r0 : a_local_dev + r0 * lda + ka;
                    rc = run_gemm(ctx, *d, trans_a, trans_b, rows, n, kw, alpha, a_panel, lda, 0, b_dev + ka * ldb, ldb, 0,
                                  first_panel ? beta : 1.0f, c_block_dev + r0 * ldc, ldc, 0, 1);
                    if (rc != SUSHI_CUDA_OK) return rc;
                    first_panel = false;
                }
            }
        }
        else
        {
            if (i == 0 && k > 0)
                for (int s_i = 0; s_i < pieces; ++s_i) SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ctx->slab_events[pieces + s_i], 0));
            rc = run_gemm(ctx, *d, trans_a, trans_b, rows, n, k, alpha, trans_a ? a_local_dev + r0 : a_local_dev + r0 * lda, lda, 0,
                          b_dev, ldb, 0, beta, c_block_dev + r0 * ldc, ldc, 0, 1, &reuse);
            if (rc != SUSHI_CUDA_OK) return rc;
        }
        SC_CUDA(ctx, cudaEventRecord(ev[9 + i], d->stream));
        SC_CUDA(ctx, cudaStreamWaitEvent(d->copy_out, ev[9 + i], 0));
        SC_CUDA(ctx, cudaMemcpyAsync(c_block_host + r0 * ldc, c_block_dev + r0 * ldc, cc, cudaMemcpyDeviceToHost, d->copy_out));
    }
    // a rank without rows still owes the main stream the arrival of B (the buffer is the caller's)
    if (count == 0 && k > 0)
        for (int s_i = 0; s_i < pieces; ++s_i) SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ctx->slab_events[pieces + s_i], 0));
    // the call completes on the caller's stream once the last download has
    SC_CUDA(ctx, cudaEventRecord(ev[17], d->copy_out));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ev[17], 0));
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_sgemm_batch_sharded(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                              int64_t m, int64_t n, int64_t k, float alpha,
                                              const float* a_local, int64_t lda, int64_t stride_a,
                                              const float* b_local, int64_t ldb, int64_t stride_b,
                                              float beta, float* c_full, int64_t ldc, int64_t stride_c,
                                              int64_t batch, int gather)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_batch_sharded: bad context or device index");
    const int nranks = ctx->comm ? ctx->nranks : 1, rank = ctx->comm ? ctx->rank : 0;
    if (ctx->comm && ctx->comm_dev != dev)
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_batch_sharded: communicator is bound to another device");
    int64_t first, count;
    if (batch < 0) return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_batch_sharded: negative batch");
    sushi_cuda_partition(batch, nranks, rank, &first, &count);
    int rc = validate_gemm(ctx, m, n, k, a_local, lda, b_local, ldb, c_full, ldc, trans_a, trans_b, stride_a,
                           stride_b, stride_c, count);
    if (rc != SUSHI_CUDA_OK) return rc;
    const bool do_gather = gather != 0 && nranks > 1;
    if (do_gather && (ldc != n || stride_c != m * n))
        return set_error(ctx, SUSHI_CUDA_ERR_UNSUPPORTED, "sgemm_batch_sharded: gathering needs contiguous C");
    // Fused exchange (gather == 2): the epilogue of this rank's GEMM stores its finished tiles into every peer's
    // buffer, as in the row-sharded form (a batch entry is addressed like a row block: bi * stride_c).  Whether it runs
    // is decided from quantities all ranks share -- the largest and the last batch block -- never from this rank's own.
    int exchange = 0;
    sushi_cuda_batch_sharded_exchange(m, n, k, batch, nranks, ctx->variant, d->sm_count, gather, &exchange);
    if (do_gather && exchange == 2 && !ctx->peer_buffers.empty())
    {
        if ((int)ctx->peer_buffers.size() != nranks || ctx->peer_buffers[rank] != c_full ||
            (reinterpret_cast<uintptr_t>(c_full) & 15) != 0 ||
            (size_t)batch * (size_t)m * (size_t)n * sizeof(float) > ctx->peer_bytes)
            return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG,
                             "sgemm_batch_sharded: gather == 2 needs c_full to be this rank's registered buffer "
                             "(sushi_cuda_comm_set_peer_buffers), 16-byte aligned and at least batch*m*n*4 bytes");
        SC_CUDA(ctx, cudaSetDevice(d->device));
        // barrier 1: every rank has reached this call, so nobody still reads the previous C
        SC_NCCL(ctx, g_nccl.AllReduce(ctx->barrier_word, ctx->barrier_word, 1, NCCL_FLOAT32, 0, ctx->comm, d->stream));
        if (count > 0)
        {
            SlabReuse fused;
            fused.variant = SUSHI_GEMM_TC3X;
            for (int r = 0; r < nranks; ++r)
                if (r != rank) fused.peer_c[fused.n_peers++] = static_cast<float*>(ctx->peer_buffers[r]) + first * stride_c;
            rc = run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, a_local, lda, stride_a, b_local, ldb, stride_b, beta,
                          c_full + first * stride_c, ldc, stride_c, count, &fused);
            if (rc != SUSHI_CUDA_OK) return rc;
        }
        // barrier 2: every rank's kernel (and with it its stores into this rank's buffer) is complete
        SC_NCCL(ctx, g_nccl.AllReduce(ctx->barrier_word, ctx->barrier_word, 1, NCCL_FLOAT32, 0, ctx->comm, d->stream));
        return SUSHI_CUDA_OK;
    }
    rc = run_gemm(ctx, *d, trans_a, trans_b, m, n, k, alpha, a_local, lda, stride_a, b_local, ldb, stride_b, beta,
                  c_full + first * stride_c, ldc, stride_c, count);
    if (rc != SUSHI_CUDA_OK || !do_gather) return rc;
    if ((rc = ensure_events(ctx, 1)) != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, cudaEventRecord(ctx->slab_events[0], d->stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->slab_events[0], 0));
    const int64_t block = (batch + nranks - 1) / nranks;
    if ((rc = gather_slab(ctx, c_full, batch, m * n, 0, block)) != SUSHI_CUDA_OK) return rc;
    SC_CUDA(ctx, cudaEventRecord(ctx->comm_done, ctx->comm_stream));
    SC_CUDA(ctx, cudaStreamWaitEvent(d->stream, ctx->comm_done, 0));
    return SUSHI_CUDA_OK;
}

// ======================================================================== harness helper
extern "C" int sushi_cuda_fill_uniform(sushi_cuda_ctx* ctx, int dev, float* dst, int64_t count, uint64_t seed,
                                       int64_t first_index)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || count < 0 || (count > 0 && !dst))
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "fill_uniform: bad argument");
    if (count == 0) return SUSHI_CUDA_OK;
    SC_CUDA(ctx, cudaSetDevice(d->device));
    int64_t blocks = (count + 255) / 256;
    if (blocks > (int64_t)d->sm_count * 32) blocks = (int64_t)d->sm_count * 32;
    fill_uniform_kernel<<<(unsigned)blocks, 256, 0, d->stream>>>(dst, count, splitmix64_host(seed), first_index);
    ctx->launches++;
    SC_CUDA(ctx, cudaGetLastError());
    return SUSHI_CUDA_OK;
}

extern "C" int sushi_cuda_sgemm_tf32_probe(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b, int64_t m, int64_t n,
                                           int64_t k, const float* a, int64_t lda, const float* b, int64_t ldb, float* c,
                                           int64_t ldc, int products)
{
    DeviceState* d = get_dev(ctx, dev);
    if (!d || (products != 1 && products != 3))
        return set_error(ctx, SUSHI_CUDA_ERR_INVALID_ARG, "sgemm_tf32_probe: bad argument (products is 1 or 3)");
    int rc = validate_gemm(ctx, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, 0, 0, 0, 1);
    if (rc != SUSHI_CUDA_OK) return rc;
    if (m == 0 || n == 0 || k == 0) return SUSHI_CUDA_OK;
    SlabReuse probe;
    probe.variant = SUSHI_GEMM_TC3X;
    probe.products = products == 1 ? 1 : 2;       // 2: the regular three products, but on the probe's path (planes, whole tiles)
    return run_gemm(ctx, *d, trans_a, trans_b, m, n, k, 1.0f, a, lda, 0, b, ldb, 0, 0.0f, c, ldc, 0, 1, &probe);
}

// ======================================================================== allocation-free variant
// Scratch for sushi_cuda_sgemm_static_scratch.  In host code these names are host-side stand-ins
// for the device symbols, never device addresses: the addresses handed to kernels come from
// cudaGetSymbolAddress, resolved once per device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[SUSHI_CUDA_STATIC_SCRATCH_BYTES];
static __device__ int g_static_status;

namespace {
struct StaticScratchDevice
{
    bool ready = false;
    float* scratch = nullptr;
    int* status = nullptr;
    int sm_count = 0;
};
constexpr int STATIC_MAX_DEVICES = 64;
StaticScratchDevice g_static_dev[STATIC_MAX_DEVICES];
std::mutex g_static_mutex;
} // namespace

extern "C" int sushi_cuda_sgemm_static_scratch(void* cuda_stream, int trans_a, int trans_b,
                                               int64_t m, int64_t n, int64_t k, float alpha,
                                               const float* a, int64_t lda, const float* b, int64_t ldb,
                                               float beta, float* c, int64_t ldc, int* status_dev)
{
    int rc = validate_gemm(nullptr, m, n, k, a, lda, b, ldb, c, ldc, trans_a, trans_b, 0, 0, 0, 1);
    if (rc != SUSHI_CUDA_OK) return rc;
    int device = -1;
    SC_CUDA(nullptr, cudaGetDevice(&device));
    if (device < 0 || device >= STATIC_MAX_DEVICES)
        return set_error(nullptr, SUSHI_CUDA_ERR_UNSUPPORTED, "sgemm_static_scratch: device index out of range");
    StaticScratchDevice& sd = g_static_dev[device];
    {
        // one-time set-up for this device: resolve the device addresses of the static symbols
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!sd.ready)
        {
            void* p = nullptr;
            SC_CUDA(nullptr, cudaGetSymbolAddress(&p, g_static_scratch));
            sd.scratch = static_cast<float*>(p);
            SC_CUDA(nullptr, cudaGetSymbolAddress(&p, g_static_status));
            sd.status = static_cast<int*>(p);
            SC_CUDA(nullptr, cudaDeviceGetAttribute(&sd.sm_count, cudaDevAttrMultiProcessorCount, device));
            sd.ready = true;
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (st != nullptr && st != cudaStreamLegacy && st != cudaStreamPerThread)
    {
        // a stream of another device would make the kernels address that device's copy of the array
        int stream_device = -1;
        if (cudaStreamGetDevice(st, &stream_device) == cudaSuccess && stream_device != device)
            return set_error(nullptr, SUSHI_CUDA_ERR_INVALID_ARG,
                             "sgemm_static_scratch: the stream belongs to another device than the current one");
        cudaGetLastError();
    }
    int* status = status_dev ? status_dev : sd.status;
    if (m == 0 || n == 0) return SUSHI_CUDA_OK;
    SC_CUDA(nullptr, cudaMemsetAsync(status, 0, sizeof(int), st));       // must start at zero
    if (k == 0 || alpha == 0.0f)
    {
        if (beta == 1.0f) return SUSHI_CUDA_OK;
        int64_t blocks = (m * n + 255) / 256;
        if (blocks > (int64_t)sd.sm_count * 16) blocks = (int64_t)sd.sm_count * 16;
        sushi::scale_c_kernel<<<(unsigned)blocks, 256, 0, st>>>(c, m, n, ldc, 0, 1, beta);
        SC_CUDA(nullptr, cudaGetLastError());
        return SUSHI_CUDA_OK;
    }
    if (k < 4)
    {
        // a 3xTF32 product can miss the K-scaled tolerance below K = 4: exact-fp32 FFMA kernel (needs no scratch)
        sushi::SimtGemmArgs g;
        g.a = a; g.b = b; g.c = c; g.m = m; g.n = n; g.k = k; g.lda = lda; g.ldb = ldb; g.ldc = ldc;
        g.stride_a = 0; g.stride_b = 0; g.stride_c = 0; g.tiles_m = 0; g.tiles_n = 0;
        g.alpha = alpha; g.beta = beta; g.act = 0; g.act_param = 0.0f; g.tri = 0;
        SC_CUDA(nullptr, sushi::launch_sgemm_simt(g, trans_a != 0, trans_b != 0, 1, sd.sm_count, st));
        return SUSHI_CUDA_OK;
    }
    const size_t bytes_a = sushi::split_plane_bytes(m, k, 1);
    const size_t bytes_b = sushi::split_plane_bytes(n, k, 1);
    if (bytes_a + bytes_b > (size_t)SUSHI_CUDA_STATIC_SCRATCH_BYTES)
    {
        char msg[256];
        snprintf(msg, sizeof msg,
                 "sgemm_static_scratch: m=%lld n=%lld k=%lld needs %zu bytes of operand planes, the static scratch "
                 "holds %u; use sushi_cuda_sgemm (context-owned scratch) for this size",
                 (long long)m, (long long)n, (long long)k, bytes_a + bytes_b, (unsigned)SUSHI_CUDA_STATIC_SCRATCH_BYTES);
        return set_error(nullptr, SUSHI_CUDA_ERR_UNSUPPORTED, msg);
    }
    // The pre-pass writes every byte of the planes it hands to the GEMM (padding included), so
    // whatever an earlier call left in the array is never read.
    float* planes_a = sd.scratch;
    float* planes_b = reinterpret_cast<float*>(reinterpret_cast<char*>(sd.scratch) + bytes_a);
    SC_CUDA(nullptr, sushi::launch_split_tf32(a, planes_a, m, k, lda, 0, 1, /*k_contig=*/!trans_a, sd.sm_count, st));
    SC_CUDA(nullptr, sushi::launch_split_tf32(b, planes_b, n, k, ldb, 0, 1, /*k_contig=*/trans_b != 0, sd.sm_count, st));
    sushi::tc3x::OperandSource src_a, src_b;
    src_a.planes = planes_a;
    src_b.planes = planes_b;
    SC_CUDA(nullptr, sushi::tc3x::launch_sgemm_tc3x(src_a, src_b, c, m, n, k, ldc, 0, 1, alpha, beta, status,
                                                   sd.sm_count, st));
    return SUSHI_CUDA_OK;
}
