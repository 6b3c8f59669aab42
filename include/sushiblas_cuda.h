/*
 * sushiblas_cuda.h -- C ABI of the B200 (sm_100a) backend for the SushiBLAS fp32 GEMM path.
 *
 * This is the boundary the C++ Engine dispatches to.  Its GEMM entry points take the
 * argument list of the reference's internal dispatcher
 *     gemm_dispatch<float>(queue, layout, transA, transB, m, n, k, alpha,
 *                          a, lda, str_a, b, ldb, str_b, beta, c, ldc, str_c, batch, deps)
 * (src/ops/blas/level3/gemm.cpp:44-51), i.e. of the two oneMKL calls it forwards to
 * (gemm.cpp:58 gemm_batch, gemm.cpp:63 gemm): element-typed pointers, leading dimensions
 * and batch strides in elements, 64-bit sizes.  The sycl::queue becomes a context handle
 * plus a device index; event dependencies become stream order.
 *
 * Conventions
 *  - plain C types only; every function returns SUSHI_CUDA_OK (0) or a negative code;
 *    nothing throws across this boundary; sushi_cuda_last_error() gives the text;
 *  - matrices are ROW-MAJOR (the column-major case of gemm.cpp:66-78 is served by the
 *    caller swapping operands: C^T = op(B)^T * op(A)^T);
 *  - GEMM pointers are device pointers unless the function name ends in _host;
 *  - GEMM calls are asynchronous on the context's stream of that device; call
 *    sushi_cuda_sync() before reading results on the host;
 *  - there is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef SUSHIBLAS_CUDA_H
#define SUSHIBLAS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define SUSHI_CUDA_API __declspec(dllexport)
#else
#define SUSHI_CUDA_API __attribute__((visibility("default")))
#endif

typedef struct sushi_cuda_ctx sushi_cuda_ctx;

enum sushi_cuda_status
{
    SUSHI_CUDA_OK = 0,
    SUSHI_CUDA_ERR_INVALID_ARG = -1,    /* bad size, leading dimension, pointer or index   */
    SUSHI_CUDA_ERR_CUDA = -2,           /* a CUDA runtime / driver call failed             */
    SUSHI_CUDA_ERR_NO_DEVICE = -3,      /* no usable CUDA device                           */
    SUSHI_CUDA_ERR_OOM = -4,            /* device or pinned-host allocation failed         */
    SUSHI_CUDA_ERR_KERNEL_TIMEOUT = -5, /* a bounded in-kernel wait expired (see _sync)    */
    SUSHI_CUDA_ERR_COMM = -6,           /* NCCL missing or a collective failed             */
    SUSHI_CUDA_ERR_UNSUPPORTED = -7     /* request outside what this build supports        */
};

/* Kernel family used by the GEMM entry points. */
enum sushi_cuda_gemm_variant
{
    SUSHI_GEMM_AUTO = 0,   /* tensor-core 3xTF32 when the problem can fill its tiles, else SIMT */
    SUSHI_GEMM_SIMT = 1,   /* fp32 FFMA tiles (exact fp32 products, fp32 accumulation)          */
    SUSHI_GEMM_TC3X = 2    /* tcgen05 3xTF32 (hi/lo split, fp32 accumulation in TMEM)           */
};

/* ---- context ------------------------------------------------------------------------
 * Replaces the sycl::queue / RuntimeContext pair the reference passes around
 * (include/SushiRuntime/execution/runtime_context.hpp:42-96, get_queue(xpu_index)).
 * devices == NULL or n_devices == 0 selects device 0 (or $SUSHI_CUDA_DEVICE). The `dev`
 * argument of the other calls indexes this list.                                         */
SUSHI_CUDA_API int sushi_cuda_device_count(int* count);
SUSHI_CUDA_API int sushi_cuda_init(const int* devices, int n_devices, sushi_cuda_ctx** out);
SUSHI_CUDA_API int sushi_cuda_destroy(sushi_cuda_ctx* ctx);
SUSHI_CUDA_API const char* sushi_cuda_last_error(sushi_cuda_ctx* ctx);

/* Waits for everything queued on the device's stream (RuntimeContext::wait_all,
 * runtime_context.hpp:90) and reports a kernel-side bounded-wait expiry, if any.          */
SUSHI_CUDA_API int sushi_cuda_sync(sushi_cuda_ctx* ctx, int dev);

/* Run on a caller-owned stream (a cudaStream_t passed as void*; NULL restores the
 * context's own stream).  Lets a host framework time or order the calls with its events. */
SUSHI_CUDA_API int sushi_cuda_set_stream(sushi_cuda_ctx* ctx, int dev, void* cuda_stream);
SUSHI_CUDA_API int sushi_cuda_get_stream(sushi_cuda_ctx* ctx, int dev, void** cuda_stream);

/* Failure-detection self-test: launches one CTA that waits, with the same bounded-wait routine
 * the GEMM kernel uses, on a barrier nothing ever arrives on; after `limit_ms` (1..2000) the
 * wait gives up and records its code.  The next sushi_cuda_sync() must then return
 * SUSHI_CUDA_ERR_KERNEL_TIMEOUT, clear the status and leave the context usable.  Nothing
 * faults, traps or hangs.                                                                    */
SUSHI_CUDA_API int sushi_cuda_selftest_bounded_wait(sushi_cuda_ctx* ctx, int dev, int limit_ms);

/* Host-side fault injection for tests (no counterpart in the reference; nothing on the GPU faults): the
 * `nth` next call (1 = the very next, 0 = cancel) that reaches `site` returns its error code without making the
 * CUDA / NCCL call -- SUSHI_CUDA_ERR_OOM for the two allocation sites (device allocation covers sushi_cuda_malloc
 * and the library's own scratch), SUSHI_CUDA_ERR_COMM for communicator initialisation.  The context stays usable. */
enum sushi_cuda_fail_site
{
    SUSHI_CUDA_FAIL_DEVICE_ALLOC = 1,
    SUSHI_CUDA_FAIL_COMM_INIT = 2,
    SUSHI_CUDA_FAIL_HOST_ALLOC = 3
};
SUSHI_CUDA_API int sushi_cuda_inject_failure(sushi_cuda_ctx* ctx, int site, int nth);

SUSHI_CUDA_API int sushi_cuda_set_gemm_variant(sushi_cuda_ctx* ctx, int variant);
/* Number of kernels this context has launched so far (all devices). */
SUSHI_CUDA_API int sushi_cuda_launch_count(sushi_cuda_ctx* ctx, int64_t* launches);
/* Bytes this context has moved between host and device through sushi_cuda_memcpy_h2d / _d2h and
 * sushi_cuda_upload_ahead so far (either pointer may be NULL).  The Engine's residency tests count PCIe crossings with it; the reference
 * has no counterpart (its shared USM migrates pages without telling anyone).                          */
SUSHI_CUDA_API int sushi_cuda_copy_bytes(sushi_cuda_ctx* ctx, uint64_t* h2d_bytes, uint64_t* d2h_bytes);

/* Optional per-kernel timing for measurement harnesses: when enabled, every GEMM call brackets
 * its operand pre-pass and its main kernel with CUDA events on the launching stream.
 * _read() waits for the stream, returns the accumulated device milliseconds and launch counts
 * since the last read and resets them.  Off by default (the reference has no profiler; its
 * TaskMetadata names exist "for profilers", include/SushiRuntime/graph/task_types.hpp:90-129). */
SUSHI_CUDA_API int sushi_cuda_kernel_timing_enable(sushi_cuda_ctx* ctx, int enable);
SUSHI_CUDA_API int sushi_cuda_kernel_timing_read(sushi_cuda_ctx* ctx, int dev,
                                                 double* gemm_ms, int64_t* gemm_launches,
                                                 double* prepass_ms, int64_t* prepass_launches);

/* ---- storage ------------------------------------------------------------------------
 * Replace USMAllocator::allocate / deallocate (include/SushiRuntime/memory/
 * usm_allocator.hpp:43-71) for AllocStrategy::DEVICE (cudaMalloc) and HOST (pinned), and
 * the queue.memcpy staging the reference uses for DEVICE tensors (src/io.cpp:73-78).
 * Copies are asynchronous on the device's stream.                                         */
SUSHI_CUDA_API int sushi_cuda_malloc(sushi_cuda_ctx* ctx, int dev, size_t bytes, void** ptr);
SUSHI_CUDA_API int sushi_cuda_free(sushi_cuda_ctx* ctx, int dev, void* ptr);
SUSHI_CUDA_API int sushi_cuda_host_alloc(sushi_cuda_ctx* ctx, size_t bytes, void** ptr);
SUSHI_CUDA_API int sushi_cuda_host_free(sushi_cuda_ctx* ctx, void* ptr);
SUSHI_CUDA_API int sushi_cuda_memcpy_h2d(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes);
SUSHI_CUDA_API int sushi_cuda_memcpy_d2h(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes);
SUSHI_CUDA_API int sushi_cuda_memcpy_d2d(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes);
SUSHI_CUDA_API int sushi_cuda_memset(sushi_cuda_ctx* ctx, int dev, void* dst, int byte, size_t bytes);
/* Uploads that overlap queued work (what the reference gets from shared-USM page migration running beside
 * its kernels).  _ahead() copies pinned host memory on the context's upload stream and makes the device's
 * stream wait for it, so everything enqueued afterwards sees the data while work enqueued earlier keeps
 * running.  The upload stream itself only waits for the work that was queued at the last _fence(): call
 * _fence() once nothing enqueued before it may still touch the destinations of the uploads that follow
 * (the Engine does so at the start of every execute() round).                                        */
SUSHI_CUDA_API int sushi_cuda_upload_fence(sushi_cuda_ctx* ctx, int dev);
SUSHI_CUDA_API int sushi_cuda_upload_ahead(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes);
/* Downloads that do not wait for unrelated work.  A marker names a point in the device's stream
 * (_record(): everything enqueued so far).  _download_behind() copies to pinned host memory on the
 * context's download stream as soon as the work before `after` has finished, whatever else is still
 * queued behind it; the device's stream then waits for the copy, so sushi_cuda_sync() covers it and
 * later work cannot overwrite the source under it.  The Engine records a marker after every operation
 * that writes a SHARED/HOST tensor and downloads each written tensor behind its last marker.        */
typedef struct sushi_cuda_marker sushi_cuda_marker;
SUSHI_CUDA_API int sushi_cuda_marker_create(sushi_cuda_ctx* ctx, int dev, sushi_cuda_marker** marker);
SUSHI_CUDA_API int sushi_cuda_marker_record(sushi_cuda_ctx* ctx, int dev, sushi_cuda_marker* marker);
SUSHI_CUDA_API int sushi_cuda_marker_destroy(sushi_cuda_ctx* ctx, sushi_cuda_marker* marker);
SUSHI_CUDA_API int sushi_cuda_download_behind(sushi_cuda_ctx* ctx, int dev, void* dst, const void* src, size_t bytes,
                                              sushi_cuda_marker* after);

/* ---- GEMM ---------------------------------------------------------------------------
 * C <- alpha * op(A) * op(B) + beta * C, row-major, op(X) = X or X^T.
 * Replaces oneapi::mkl::blas::row_major::gemm (call site gemm.cpp:63).
 * C is not read when beta == 0.  lda >= (transA ? m : k), ldb >= (transB ? k : n),
 * ldc >= n (each at least 1).                                                             */
SUSHI_CUDA_API int sushi_cuda_sgemm(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                    int64_t m, int64_t n, int64_t k, float alpha,
                                    const float* a, int64_t lda,
                                    const float* b, int64_t ldb,
                                    float beta, float* c, int64_t ldc);

/* Batch i uses a + i*stride_a, b + i*stride_b, c + i*stride_c.
 * Replaces oneapi::mkl::blas::row_major::gemm_batch (call site gemm.cpp:58).              */
SUSHI_CUDA_API int sushi_cuda_sgemm_strided_batched(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                    int64_t m, int64_t n, int64_t k, float alpha,
                                                    const float* a, int64_t lda, int64_t stride_a,
                                                    const float* b, int64_t ldb, int64_t stride_b,
                                                    float beta, float* c, int64_t ldc, int64_t stride_c,
                                                    int64_t batch);

/* GEMM with a fused epilogue activation (no counterpart call in the reference, which runs
 * ReLU as a separate element-wise task after the GEMM: tests/runtime/test_framework_sim.cpp:47-58,
 * src/ops/math/nonlinear/relu.cpp:36-40).  epilogue: SUSHI_EPILOGUE_NONE or SUSHI_EPILOGUE_RELU,
 * C <- act(alpha * op(A) * op(B) + beta * C).                                                 */
enum sushi_cuda_epilogue { SUSHI_EPILOGUE_NONE = 0, SUSHI_EPILOGUE_RELU = 1 };
SUSHI_CUDA_API int sushi_cuda_sgemm_strided_batched_ex(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                       int64_t m, int64_t n, int64_t k, float alpha,
                                                       const float* a, int64_t lda, int64_t stride_a,
                                                       const float* b, int64_t ldb, int64_t stride_b,
                                                       float beta, float* c, int64_t ldc, int64_t stride_c,
                                                       int64_t batch, int epilogue);

/* Symmetric rank-k update, row-major:  C <- alpha * op(A) * op(A)^T + beta * C  on the upper
 * (upper != 0) or lower triangle of the n x n matrix C; the other triangle is neither read nor
 * written.  op(A) = A (n x k, trans == 0) or A^T (A stored k x n, trans != 0).
 * Replaces oneapi::mkl::blas::row_major::syrk / syrk_batch (call sites
 * src/ops/blas/level3/syrk.cpp:60-78).  Runs on the GEMM main loop: tiles outside the triangle
 * are skipped, diagonal tiles store under a mask, and A's hi/lo planes serve as both operands.  */
SUSHI_CUDA_API int sushi_cuda_ssyrk(sushi_cuda_ctx* ctx, int dev, int upper, int trans, int64_t n, int64_t k,
                                    float alpha, const float* a, int64_t lda, float beta, float* c, int64_t ldc);
SUSHI_CUDA_API int sushi_cuda_ssyrk_strided_batched(sushi_cuda_ctx* ctx, int dev, int upper, int trans,
                                                    int64_t n, int64_t k, float alpha,
                                                    const float* a, int64_t lda, int64_t stride_a, float beta,
                                                    float* c, int64_t ldc, int64_t stride_c, int64_t batch);

/* fp64 GEMM, same argument meaning as sushi_cuda_sgemm[_strided_batched] with double data:
 * replaces oneapi::mkl::blas::row_major::gemm / gemm_batch<double> (FLOAT64 branch of the
 * front-end, src/ops/blas/level3/gemm.cpp:158-169).  Runs on the FP64 tensor-core instruction
 * (mma.sync m16n8k8.f64): exact fp64 products, fp64 accumulation.                              */
SUSHI_CUDA_API int sushi_cuda_dgemm(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                    int64_t m, int64_t n, int64_t k, double alpha,
                                    const double* a, int64_t lda, const double* b, int64_t ldb,
                                    double beta, double* c, int64_t ldc);
SUSHI_CUDA_API int sushi_cuda_dgemm_strided_batched(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                    int64_t m, int64_t n, int64_t k, double alpha,
                                                    const double* a, int64_t lda, int64_t stride_a,
                                                    const double* b, int64_t ldb, int64_t stride_b,
                                                    double beta, double* c, int64_t ldc, int64_t stride_c,
                                                    int64_t batch);

/* Triangular solve with multiple right-hand sides, row-major; X overwrites B (m x n):
 *     left != 0:  op(A) * X = alpha * B,  A is m x m        left == 0:  X * op(A) = alpha * B,  A is n x n
 * A is upper (upper != 0) or lower triangular; only that triangle is read, and its diagonal is
 * taken as 1 when unit_diag != 0.  Replaces oneapi::mkl::blas::row_major::trsm / trsm_batch (call
 * sites src/ops/blas/level3/trsm.cpp:61-79).  Recursive blocked substitution: ranges of 512-wide
 * blocks of the triangular dimension are halved, each halving costing one GEMM update on the
 * regular GEMM kernels, and single blocks are applied through their explicit inverses (a small
 * substitution kernel plus two batched GEMMs), so large solves run on the tensor cores.
 * Accuracy is that of inverse-based blocked solvers: backward stable for well-conditioned diagonal
 * blocks.                                                                                       */
SUSHI_CUDA_API int sushi_cuda_strsm(sushi_cuda_ctx* ctx, int dev, int left, int upper, int trans, int unit_diag,
                                    int64_t m, int64_t n, float alpha, const float* a, int64_t lda,
                                    float* b, int64_t ldb);
SUSHI_CUDA_API int sushi_cuda_strsm_strided_batched(sushi_cuda_ctx* ctx, int dev, int left, int upper, int trans,
                                                    int unit_diag, int64_t m, int64_t n, float alpha,
                                                    const float* a, int64_t lda, int64_t stride_a,
                                                    float* b, int64_t ldb, int64_t stride_b, int64_t batch);

/* Many independent GEMMs in one call (no counterpart call in the reference; it is what its
 * scheduler stress tests submit per execute(): 5000 GEMMs of 32^3 and 3000 of 8^3,
 * tests/runtime/test_dependency_stress.cpp:17-45,67-83).  No output of one problem may overlap
 * an input or output of another.  Small problems run as ONE grouped kernel launch (64 x 64 FFMA
 * tiles); problems large enough for the tensor-core path run one by one after it.             */
typedef struct sushi_cuda_gemm_desc
{
    int32_t trans_a, trans_b;
    int64_t m, n, k;
    float alpha;
    const float* a; int64_t lda, stride_a;
    const float* b; int64_t ldb, stride_b;
    float beta;
    float* c; int64_t ldc, stride_c;
    int64_t batch;
    int32_t epilogue;          /* sushi_cuda_epilogue or sushi_cuda_activation_kind */
    float act_param;           /* parameter of the activation (leaky_relu, elu) */
} sushi_cuda_gemm_desc;
SUSHI_CUDA_API int sushi_cuda_sgemm_grouped(sushi_cuda_ctx* ctx, int dev, const sushi_cuda_gemm_desc* problems,
                                            int64_t count);

/* In-place ReLU on `count` contiguous floats (replaces the element-wise kernel of
 * src/ops/math/nonlinear/relu.cpp:36-40 for FLOAT32).                                         */
SUSHI_CUDA_API int sushi_cuda_relu(sushi_cuda_ctx* ctx, int dev, float* x, int64_t count);

/* The activations of the reference's non-linear family, FLOAT32 (the .cpp files of src/ops/math/nonlinear;
 * element-wise driver nonlinear_internal.hpp:50-92).  Values 0 and 1 coincide with
 * sushi_cuda_epilogue.  `act_param` is leaky_relu's slope (reference default 0.01) or elu's alpha
 * (default 1.0); ignored by the others.  gelu is the tanh form the reference uses
 * (gelu.cpp:38-44).                                                                            */
typedef enum sushi_cuda_activation_kind
{
    SUSHI_ACT_NONE = 0,
    SUSHI_ACT_RELU = 1,
    SUSHI_ACT_LEAKY_RELU = 2,
    SUSHI_ACT_SIGMOID = 3,
    SUSHI_ACT_TANH = 4,
    SUSHI_ACT_ELU = 5,
    SUSHI_ACT_SILU = 6,
    SUSHI_ACT_GELU = 7,
    SUSHI_ACT_SOFTPLUS = 8
} sushi_cuda_activation_kind;

/* x <- f(x) in place on `count` contiguous floats (the forward lambdas of the files above).   */
SUSHI_CUDA_API int sushi_cuda_activation(sushi_cuda_ctx* ctx, int dev, int activation, float act_param, float* x,
                                         int64_t count);
/* dx <- dy * f'(.), the backward lambdas of the same files: `saved` is the forward INPUT x, except
 * for sigmoid and tanh, which take the forward OUTPUT y (sigmoid.cpp, tanh.cpp).              */
SUSHI_CUDA_API int sushi_cuda_activation_backward(sushi_cuda_ctx* ctx, int dev, int activation, float act_param,
                                                  const float* dy, const float* saved, float* dx, int64_t count);
/* GEMM with any of these activations applied to alpha*op(A)*op(B) + beta*C in the epilogue (one
 * pass over C instead of two).                                                                 */
SUSHI_CUDA_API int sushi_cuda_sgemm_strided_batched_act(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                        int64_t m, int64_t n, int64_t k, float alpha,
                                                        const float* a, int64_t lda, int64_t stride_a,
                                                        const float* b, int64_t ldb, int64_t stride_b,
                                                        float beta, float* c, int64_t ldc, int64_t stride_c,
                                                        int64_t batch, int activation, float act_param);

/* Same operation on HOST buffers (the SHARED / HOST strategies of the reference, whose
 * tensors callers fill and read on the host: tests/test_common.hpp:36-58): stages A, B
 * (and C when beta != 0) to the device, runs the GEMM, stages C back; all queued on the
 * stream.  Buffers should be pinned (sushi_cuda_host_alloc) for the copies to overlap.    */
SUSHI_CUDA_API int sushi_cuda_sgemm_strided_batched_host(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                         int64_t m, int64_t n, int64_t k, float alpha,
                                                         const float* a, int64_t lda, int64_t stride_a,
                                                         const float* b, int64_t ldb, int64_t stride_b,
                                                         float beta, float* c, int64_t ldc, int64_t stride_c,
                                                         int64_t batch);

/* Bytes of device scratch the 3xTF32 path would use for this problem (0 for SIMT). The
 * context grows its scratch on demand; sushi_cuda_reserve_workspace() does it up front so
 * that no allocation happens inside a timed or latency-critical region.                   */
SUSHI_CUDA_API int sushi_cuda_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch, size_t* bytes);
SUSHI_CUDA_API int sushi_cuda_reserve_workspace(sushi_cuda_ctx* ctx, int dev, size_t bytes);

/* Allocation-free variant of sushi_cuda_sgemm (no counterpart in the reference).
 *
 * Some hosts cannot let a library allocate device memory at call time: an application whose own
 * pool already owns the whole GPU, a thread running while another one is capturing a CUDA graph
 * (cudaMalloc is refused during a global-mode capture), or a latency-critical loop that cannot
 * afford the device-wide synchronisation an allocation implies.  This entry point needs no
 * context and calls no cudaMalloc / cudaFree / allocating routine: the hi/lo operand planes of
 * the 3xTF32 kernel live in a fixed SUSHI_CUDA_STATIC_SCRATCH_BYTES array that is part of the
 * library image (every GPU that loads the library holds it until the process exits).
 *
 *  - Runs on the CURRENT device, on `cuda_stream` (a cudaStream_t as void*; NULL = default
 *    stream), asynchronously; the tensor-core 3xTF32 kernel for k >= 4, the exact-fp32 FFMA kernel
 *    (no scratch) below that, where a 3xTF32 product could miss the K-scaled tolerance.  A stream
 *    that belongs to another device is refused (SUSHI_CUDA_ERR_INVALID_ARG).
 *  - Limit: 8 * (pad256(m) + pad256(n)) * pad16(k) bytes must fit the scratch (pad = round up);
 *    e.g. 1024 x 1024 x 2048 fits, 2048^3 does not.  Larger problems return
 *    SUSHI_CUDA_ERR_UNSUPPORTED with the sizes in sushi_cuda_last_error(NULL).
 *  - The first call on each device resolves the scratch address (one-time set-up); make that
 *    call before any stream capture begins.
 *  - All calls on a device share the one scratch array: calls that may overlap on the GPU
 *    (different streams, no ordering between them) race and give wrong results; order them.
 *    Nothing is assumed about the array's previous contents.
 *  - `status_dev` (optional, device memory, 4 bytes): set to 0 by the call and to a non-zero
 *    code by the kernel if one of its bounded waits expired (C is then incomplete).  With
 *    status_dev == NULL the word is one per device, shared by every call and zeroed by each, so
 *    a later or overlapping call can clear a code before the host reads it: callers that need
 *    failure detection pass their own word.                                                 */
#define SUSHI_CUDA_STATIC_SCRATCH_BYTES (32u << 20)
SUSHI_CUDA_API int sushi_cuda_sgemm_static_scratch(void* cuda_stream, int trans_a, int trans_b,
                                                   int64_t m, int64_t n, int64_t k, float alpha,
                                                   const float* a, int64_t lda,
                                                   const float* b, int64_t ldb,
                                                   float beta, float* c, int64_t ldc,
                                                   int* status_dev);

/* ---- multi-GPU layer (one process per GPU) --------------------------------------------
 * No counterpart in the reference (it has no collective call site); the partitioning
 * follows the independence of C's row blocks / batch entries in the calls above.
 * sushi_cuda_partition(): contiguous block [first, first+count) of `total` owned by
 * `rank` of `nranks` (block size ceil(total/nranks), trailing ranks may be short/empty). */
SUSHI_CUDA_API int sushi_cuda_partition(int64_t total, int nranks, int rank, int64_t* first, int64_t* count);

/* NCCL bootstrap: rank 0 creates a 128-byte id, the host program broadcasts it by any
 * means, every rank then joins.  NCCL is loaded at run time (dlopen of libnccl.so.2).     */
SUSHI_CUDA_API int sushi_cuda_comm_unique_id(void* id128);
SUSHI_CUDA_API int sushi_cuda_comm_init_rank(sushi_cuda_ctx* ctx, int dev, const void* id128, int nranks, int rank);
SUSHI_CUDA_API int sushi_cuda_comm_destroy(sushi_cuda_ctx* ctx);

/* Peer-memory exchange for the fused GEMM + all-gather (gather == 2 below).  Each rank exports
 * the buffer that will hold the full C (it must be the base of a sushi_cuda_malloc allocation),
 * the host program exchanges the 64-byte handles, every rank opens its peers' handles and
 * registers the nranks addresses (its own entry = its local pointer) and their common size with
 * the context; a fused call whose m*n*4 exceeds that size falls back to the NCCL exchange.     */
SUSHI_CUDA_API int sushi_cuda_ipc_export(sushi_cuda_ctx* ctx, int dev, const void* base_ptr, void* handle64);
SUSHI_CUDA_API int sushi_cuda_ipc_open(sushi_cuda_ctx* ctx, int dev, const void* handle64, void** peer_ptr);
SUSHI_CUDA_API int sushi_cuda_ipc_close(sushi_cuda_ctx* ctx, int dev, void* peer_ptr);
SUSHI_CUDA_API int sushi_cuda_comm_set_peer_buffers(sushi_cuda_ctx* ctx, int dev, void* const* buffers, int count,
                                                    size_t bytes_each);

/* Row-block sharded GEMM (A NN/TN..., B replicated).  Global problem m x n x k.  `a_local`
 * holds this rank's rows of op(A): for trans_a == 0 the rows [first, first+count) of A
 * (count x k, leading dimension lda); for trans_a != 0 the matching columns of the stored
 * k x m matrix, i.e. a k x count block with leading dimension lda.  `c_full` is the whole
 * m x n result buffer on this rank: the rank computes its own row block in place and the
 * blocks are all-gathered (NCCL over NVLink) slab by slab so that the exchange of one slab
 * overlaps the multiplication of the next.  With beta != 0 only the rank's own block of
 * c_full needs valid input.  gather == 0 skips the exchange (C stays sharded).
 * gather == 2: fused exchange -- one GEMM launch over the whole block whose epilogue warps copy
 * every finished 256 x 256 tile of C into the peers' buffers with plain NVLink stores while the
 * next tile is being multiplied, followed by a 4-byte NCCL all-reduce as the cross-rank barrier.
 * Taken when ldc == n, n % 4 == 0, the tensor path suits every rank's block
 * (sushi_cuda_row_sharded_exchange) and peer buffers are registered (on every rank alike); otherwise
 * the call runs gather == 1.  With buffers registered, c_full must be this rank's registered entry,
 * 16-byte aligned and large enough: a mismatch is SUSHI_CUDA_ERR_INVALID_ARG, never a silent
 * change of path.  Ranks whose block is empty still take part in the two barriers.             */
/* Which exchange sushi_cuda_sgemm_row_sharded runs for a problem: 0 none, 1 NCCL slabs, 2 peer stores fused
 * into the GEMM epilogue.  Pure host arithmetic over quantities every rank shares (no rank, no pointer): the
 * ranks of an uneven partition -- short or empty trailing blocks -- therefore always issue the same
 * collectives.  `variant` is the kernel-family setting (sushi_cuda_gemm_variant), which the ranks must set
 * alike, as they must register peer buffers alike; `sm_count` the SM count of the (homogeneous) GPUs.     */
SUSHI_CUDA_API int sushi_cuda_row_sharded_exchange(int64_t m, int64_t n, int64_t k, int nranks, int variant, int sm_count,
                                                   int gather, int* exchange);

SUSHI_CUDA_API int sushi_cuda_sgemm_row_sharded(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                int64_t m, int64_t n, int64_t k, float alpha,
                                                const float* a_local, int64_t lda,
                                                const float* b, int64_t ldb,
                                                float beta, float* c_full, int64_t ldc, int gather);

/* Host-buffer form of the row-block sharded GEMM (host staging of device tensors: reference src/io.cpp:73-78,
 * 103-108; host-resident inputs and outputs are what the reference's callers hold, include/SushiBLAS/engine.hpp:
 * 156-168).  `a_local_host` holds this rank's rows of op(A) and `c_block_host` receives this rank's rows of C,
 * both laid out as for sushi_cuda_sgemm_row_sharded's local block; `b_host` is the whole B, of which every rank
 * needs only its share of the k rows to be valid when B is stored k x n with ldb == n: the rank uploads that
 * share and the others arrive device to device through the communicator, under the upload of A.  (A transposed
 * or padded B goes up whole on every rank.)  The block is multiplied in row chunks as they arrive and each
 * chunk of C streams back while the next multiplies; C goes up first only when beta != 0 or ldc != n.
 * `a_local_dev`, `b_dev` (whole B) and `c_block_dev` are caller-owned device buffers of the same layouts; the
 * call allocates nothing of that size.  It is collective over the communicator and completes in stream order
 * on the context's stream; the host buffers should be pinned (sushi_cuda_host_alloc) for the copies to overlap. */
SUSHI_CUDA_API int sushi_cuda_sgemm_row_sharded_host(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                     int64_t m, int64_t n, int64_t k, float alpha,
                                                     const float* a_local_host, int64_t lda,
                                                     const float* b_host, int64_t ldb,
                                                     float beta, float* c_block_host, int64_t ldc,
                                                     float* a_local_dev, float* b_dev, float* c_block_dev);

/* Batch-index sharded strided-batched GEMM: the rank owns batches [first, first+count) of
 * the global `batch`; a_local / b_local point at its first owned batch; c_full is the whole
 * batch x m x n result (contiguous: ldc == n, stride_c == m*n is required when gather != 0).
 * gather == 1: one in-place NCCL all-gather of the batch blocks after the GEMM.  gather == 2: the exchange is
 * fused into the GEMM epilogue (peer stores over NVLink between two 4-byte all-reduce barriers), under the
 * conditions of the row-sharded form: registered peer buffers with c_full this rank's own, n % 4 == 0 and the
 * tensor path suiting the largest and the last batch block; otherwise the call runs gather == 1.            */
/* Which exchange sushi_cuda_sgemm_batch_sharded runs: 0 none, 1 NCCL all-gather, 2 peer stores fused into the GEMM
 * epilogue -- like sushi_cuda_row_sharded_exchange, pure host arithmetic over what every rank knows.            */
SUSHI_CUDA_API int sushi_cuda_batch_sharded_exchange(int64_t m, int64_t n, int64_t k, int64_t batch, int nranks, int variant,
                                                     int sm_count, int gather, int* exchange);

SUSHI_CUDA_API int sushi_cuda_sgemm_batch_sharded(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b,
                                                  int64_t m, int64_t n, int64_t k, float alpha,
                                                  const float* a_local, int64_t lda, int64_t stride_a,
                                                  const float* b_local, int64_t ldb, int64_t stride_b,
                                                  float beta, float* c_full, int64_t ldc, int64_t stride_c,
                                                  int64_t batch, int gather);

/* ---- harness helper --------------------------------------------------------------------
 * Counter-based uniform [-1,1) fill: element i = ((hash(seed, first_index+i) >> 8) * 2^-23) - 1,
 * bit-identical to the host generator used by the tests.  The reference fills benchmark
 * inputs with oneMKL philox (src/ops/math/random/uniform.cpp:41-65), whose stream no test
 * pins; only the distribution is matched.                                                 */
SUSHI_CUDA_API int sushi_cuda_fill_uniform(sushi_cuda_ctx* ctx, int dev, float* dst, int64_t count,
                                           uint64_t seed, int64_t first_index);

/* Rate probe of the tensor-core kernel (measurement only; no counterpart in the reference): C <- op(A)*op(B)
 * through the regular pipeline with both operands pre-split into planes and whole tiles only (no split-K), with
 * `products` = 3 (the fp32-accurate 3xTF32 product) or 1 (only the hi*hi MMA of every product: a TF32-accurate
 * result at the kernel's 1xTF32 rate, which bounds what the three-MMA product can reach).                      */
SUSHI_CUDA_API int sushi_cuda_sgemm_tf32_probe(sushi_cuda_ctx* ctx, int dev, int trans_a, int trans_b, int64_t m, int64_t n,
                                               int64_t k, const float* a, int64_t lda, const float* b, int64_t ldb, float* c,
                                               int64_t ldc, int products);

#ifdef __cplusplus
}
#endif
#endif /* SUSHIBLAS_CUDA_H */
