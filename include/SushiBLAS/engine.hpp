// engine.hpp -- entry object of the library (reference: include/SushiBLAS/engine.hpp:61-194,
// src/engine.cpp:35-69): holds the runtime context, the deferred task graph, the default
// layout and the RNG seed; hands out tensors and the op facades.  Provided: blas() (Level 3:
// GEMM, SYRK, TRSM), nonlinear() (the activations, fusable into a GEMM) and io() (.npy / raw files); the
// other op families of the reference are outside the GEMM path.
#pragma once

#include <atomic>
#include <cmath>
#include <sstream>
#include <iomanip>
#include <functional>
#include <cstdio>
#include <cstdint>
#include <initializer_list>
#include <vector>

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiBLAS/io.hpp>
#include <SushiBLAS/ops/blas.hpp>
#include <SushiBLAS/ops/math/nonlinear.hpp>
#include <SushiBLAS/storage.hpp>
#include <SushiBLAS/tensor.hpp>
#include <SushiRuntime/SushiRuntime.h>

namespace SushiBLAS
{
    class Engine
    {
        public:
            Engine(SushiRuntime::Execution::RuntimeContext& ctx, Core::Layout layout = Core::Layout::ROW_MAJOR)
                : context_(ctx), graph_(ctx), default_layout_(layout)
            {
                SB_LOG_INFO("SushiBLAS Engine initialized with {} layout.",
                            layout == Core::Layout::ROW_MAJOR ? "Row-Major" : "Column-Major");
            }

            Core::Layout get_layout() const { return default_layout_; }

            BLASOps blas() { return BLASOps(*this); }
            NonLinearOps nonlinear() { return NonLinearOps(*this); }
            IO io() { return IO(*this); }

            SushiRuntime::Execution::RuntimeContext& get_context() { return context_; }
            SushiRuntime::Graph::TaskGraph& get_graph() { return graph_; }

            /// Enqueues every recorded task on the device stream.  wait() on the result blocks
            /// until they have run and throws std::runtime_error if any failed.
            SushiRuntime::Execution::Event execute() { return graph_.execute(); }

            /// New FLOAT32 tensor; memory is not initialised (engine.cpp:42-46).
            Tensor create_tensor(std::initializer_list<int64_t> dims,
                                 SushiRuntime::Memory::AllocStrategy strat = SushiRuntime::Memory::AllocStrategy::SHARED)
            {
                return create_tensor(dims, Core::DataType::FLOAT32, strat);
            }

            /// New tensor of `dtype`: one Storage of prod(dims) * bytes-per-element, contiguous in
            /// the engine's default layout (engine.cpp:48-69).
            Tensor create_tensor(std::initializer_list<int64_t> dims, Core::DataType dtype,
                                 SushiRuntime::Memory::AllocStrategy strat = SushiRuntime::Memory::AllocStrategy::SHARED)
            {
                std::size_t elements = 1;
                for (int64_t d : dims) elements *= static_cast<std::size_t>(d);
                std::size_t bytes_per_element = 4;
                if (dtype == Core::DataType::FLOAT64 || dtype == Core::DataType::COMPLEX32) bytes_per_element = 8;
                else if (dtype == Core::DataType::COMPLEX64) bytes_per_element = 16;
                else if (dtype == Core::DataType::HALF) bytes_per_element = 2;
                auto storage = SushiRuntime::make_sushi<Storage>(context_.get_allocator(), elements * bytes_per_element, strat);
                Tensor t(storage, dims, 0, default_layout_);
                t.dtype = dtype;
                return t;
            }

            void set_seed(uint64_t s) { seed_ = s; }
            uint64_t get_seed() const { return seed_; }
            uint64_t get_and_increment_rng_offset() { return rng_offset_++; }

        private:
            SushiRuntime::Execution::RuntimeContext& context_;
            SushiRuntime::Graph::TaskGraph graph_;
            Core::Layout default_layout_;
            uint64_t seed_ = 0;
            std::atomic<uint64_t> rng_offset_{0};
    };

    namespace detail
    {
        /// Device address of `ptr` (which lies inside `storage`) for an operation that is being enqueued.
        /// `reads`: the operation reads the range or needs what it does not overwrite; a range that does
        /// not cover the whole storage always keeps the rest, so the storage's contents are brought up too.
        template <typename T>
        inline int stage_in(const SushiRuntime::sushi_ptr<Storage>& storage, T* ptr, int64_t extent, bool reads, T** out)
        {
            const bool whole = static_cast<void*>(ptr) == storage->data_ptr &&
                               static_cast<std::size_t>(extent) * sizeof(T) >= storage->requested_bytes;
            int rc = SUSHI_CUDA_OK;
            char* base = static_cast<char*>(storage->allocator->device_for_operation(storage->data_ptr, reads || !whole, &rc));
            if (!base) return rc != SUSHI_CUDA_OK ? rc : SUSHI_CUDA_ERR_OOM;
            *out = reinterpret_cast<T*>(base + (reinterpret_cast<char*>(ptr) - static_cast<char*>(storage->data_ptr)));
            return SUSHI_CUDA_OK;
        }
        /// The operation just enqueued writes `storage` on the device.
        inline void stage_out(const SushiRuntime::sushi_ptr<Storage>& storage)
        {
            storage->allocator->mark_device_written(storage->data_ptr);
        }
    } // namespace detail

    // ---------------------------------------------------------------- Level3::gemm
    inline SushiRuntime::Execution::Event Level3::gemm(const Tensor& A, const Tensor& B, Tensor& C, bool transA,
                                                       bool transB, float alpha, float beta)
    {
        using namespace SushiRuntime::Graph::Literals;
        const detail::GemmCall user = detail::derive_gemm_call(A, B, C, transA, transB, alpha, beta);
        if (A.dtype == Core::DataType::FLOAT64) return gemm_f64(A, B, C, transA, transB, alpha, beta);
        SB_THROW_IF(A.dtype != Core::DataType::FLOAT32,
                    "Unsupported data type for GEMM operation (the CUDA backend serves FLOAT32 and FLOAT64).");

        bool swapped = false;
        const detail::GemmCall g = detail::row_major_equivalent(user, &swapped);
        const Tensor& first = swapped ? B : A;       // operand in the "A" position of the row-major call
        const Tensor& second = swapped ? A : B;

        struct Operand
        {
            SushiRuntime::sushi_ptr<Storage> storage;   // keeps the block alive until the task has run
            float* ptr;                                 // tensor.data(): host (SHARED/HOST) or device (DEVICE)
            int64_t extent;                             // elements the call may touch from ptr
            bool host;
        };
        auto describe = [](const Tensor& t, int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t batch) {
            Operand o{t.storage, t.data_as<float>(), detail::operand_extent(rows, cols, ld, stride, batch), false};
            o.host = t.storage->host_resident();
            const std::size_t need = (static_cast<std::size_t>(t.storage_offset) + static_cast<std::size_t>(o.extent)) * sizeof(float);
            SB_THROW_IF(need > t.storage->size_bytes,
                        "GEMM operand does not fit its storage (needs {} bytes, has {}).", need, t.storage->size_bytes);
            return o;
        };
        Operand oa = describe(first, g.trans_a ? g.k : g.m, g.trans_a ? g.m : g.k, g.lda, g.stride_a, g.batch);
        Operand ob = describe(second, g.trans_b ? g.n : g.k, g.trans_b ? g.k : g.n, g.ldb, g.stride_b, g.batch);
        Operand oc = describe(C, g.m, g.n, g.ldc, g.stride_c, g.batch);

        // dependency sets name the storage base pointers, as in gemm.cpp:112-120
        std::vector<void*> reads = {A.storage->data_ptr, B.storage->data_ptr};
        std::vector<void*> writes = {C.storage->data_ptr};

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = "blas.lvl3.gemm";
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = "blas.lvl3.gemm"_op;
        meta.set_param(0, alpha);
        meta.set_param(1, beta);
        meta.set_param(2, transA);
        meta.set_param(3, transB);

        // a later relu(C) can be folded into this GEMM when C is written densely
        const bool dense_out = (g.ldc == g.n) && (g.batch == 1 || g.stride_c == g.m * g.n);
        SushiRuntime::Graph::FusionInfo producer;
        producer.slot = std::make_shared<SushiRuntime::Graph::EpilogueSlot>();
        if (dense_out) { producer.out_ptr = C.data(); producer.out_count = g.m * g.n * g.batch; }
        auto slot = producer.slot;

        // stage inputs and describe the call with device addresses
        auto prepare = [g, oa, ob, oc, slot](SushiRuntime::Execution::RuntimeContext& rt, sushi_cuda_gemm_desc& q) -> int
        {
            sushi_cuda_ctx* ctx = rt.native_handle();
            // device address of an operand; host-resident operands live in their mirror (uploaded when stale)
            (void)ctx;
            auto on_device = [](const Operand& o, bool reads, float** out) -> int
            { return detail::stage_in(o.storage, o.ptr, o.extent, reads, out); };
            float *da = nullptr, *db = nullptr, *dc = nullptr;
            int rc = on_device(oa, true, &da);
            if (rc == SUSHI_CUDA_OK) rc = on_device(ob, true, &db);
            // C goes up when it is read (beta != 0) or when the call leaves gaps in it
            const bool dense_c = (g.ldc == g.n) && (g.batch == 1 || g.stride_c == g.m * g.n);
            if (rc == SUSHI_CUDA_OK) rc = on_device(oc, g.beta != 0.0f || !dense_c, &dc);
            if (rc != SUSHI_CUDA_OK) return rc;
            q.trans_a = g.trans_a; q.trans_b = g.trans_b; q.m = g.m; q.n = g.n; q.k = g.k; q.alpha = g.alpha;
            q.a = da; q.lda = g.lda; q.stride_a = g.stride_a;
            q.b = db; q.ldb = g.ldb; q.stride_b = g.stride_b;
            q.beta = g.beta; q.c = dc; q.ldc = g.ldc; q.stride_c = g.stride_c; q.batch = g.batch;
            q.epilogue = slot->activation;
            q.act_param = slot->param;
            return SUSHI_CUDA_OK;
        };
        // host-resident C: its host image is stale until the caller waits
        auto finish = [oc](SushiRuntime::Execution::RuntimeContext&) -> int
        {
            detail::stage_out(oc.storage);
            return SUSHI_CUDA_OK;
        };
        auto work = [g, prepare, finish](SushiRuntime::Execution::RuntimeContext& rt) -> int
        {
            sushi_cuda_gemm_desc q{};
            int rc = prepare(rt, q);
            if (rc != SUSHI_CUDA_OK) return rc;
            SB_LOG_INFO("CUDA GEMM [Row-Major]: {}x[{}x{}x{}]", g.batch, g.m, g.n, g.k);
            rc = sushi_cuda_sgemm_strided_batched_act(rt.native_handle(), 0, q.trans_a, q.trans_b, q.m, q.n, q.k, q.alpha,
                                                      q.a, q.lda, q.stride_a, q.b, q.ldb, q.stride_b, q.beta, q.c, q.ldc,
                                                      q.stride_c, q.batch, q.epilogue, q.act_param);
            return rc == SUSHI_CUDA_OK ? finish(rt) : rc;
        };
        // small problems may be batched with their neighbours into one grouped launch at execute()
        SushiRuntime::Graph::GroupableGemm groupable;
        if (g.m <= 128 && g.n <= 128 && g.k <= 1024 && g.batch <= 8)
        {
            groupable.prepare = prepare;
            groupable.finish = finish;
        }
        engine_.get_graph().add_task(meta, reads, writes, work, producer, groupable);
        return SushiRuntime::Execution::Event();
    }

    // ---------------------------------------------------------------- Level3::gemm, FLOAT64
    inline SushiRuntime::Execution::Event Level3::gemm_f64(const Tensor& A, const Tensor& B, Tensor& C, bool transA,
                                                           bool transB, float alpha, float beta)
    {
        using namespace SushiRuntime::Graph::Literals;
        const detail::GemmCall user = detail::derive_gemm_call(A, B, C, transA, transB, alpha, beta);
        bool swapped = false;
        const detail::GemmCall g = detail::row_major_equivalent(user, &swapped);
        const Tensor& first = swapped ? B : A;
        const Tensor& second = swapped ? A : B;

        struct Operand { SushiRuntime::sushi_ptr<Storage> storage; double* ptr; int64_t extent; bool host; };
        auto describe = [](const Tensor& t, int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t batch) {
            Operand o{t.storage, t.data_as<double>(), detail::operand_extent(rows, cols, ld, stride, batch), false};
            o.host = t.storage->host_resident();
            const std::size_t need = (static_cast<std::size_t>(t.storage_offset) + static_cast<std::size_t>(o.extent)) * sizeof(double);
            SB_THROW_IF(need > t.storage->size_bytes,
                        "GEMM operand does not fit its storage (needs {} bytes, has {}).", need, t.storage->size_bytes);
            return o;
        };
        Operand oa = describe(first, g.trans_a ? g.k : g.m, g.trans_a ? g.m : g.k, g.lda, g.stride_a, g.batch);
        Operand ob = describe(second, g.trans_b ? g.n : g.k, g.trans_b ? g.k : g.n, g.ldb, g.stride_b, g.batch);
        Operand oc = describe(C, g.m, g.n, g.ldc, g.stride_c, g.batch);

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = "blas.lvl3.gemm";
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = "blas.lvl3.gemm"_op;
        meta.set_param(0, alpha); meta.set_param(1, beta); meta.set_param(2, transA); meta.set_param(3, transB);
        engine_.get_graph().add_task(meta, {A.storage->data_ptr, B.storage->data_ptr}, {C.storage->data_ptr},
            [=](SushiRuntime::Execution::RuntimeContext& rt) -> int
            {
                sushi_cuda_ctx* ctx = rt.native_handle();
                auto on_device = [](const Operand& o, bool reads, double** out) -> int
                { return detail::stage_in(o.storage, o.ptr, o.extent, reads, out); };
                double *da = nullptr, *db = nullptr, *dc = nullptr;
                int rc = on_device(oa, true, &da);
                if (rc == SUSHI_CUDA_OK) rc = on_device(ob, true, &db);
                const bool dense_c = (g.ldc == g.n) && (g.batch == 1 || g.stride_c == g.m * g.n);
                if (rc == SUSHI_CUDA_OK) rc = on_device(oc, g.beta != 0.0f || !dense_c, &dc);
                if (rc != SUSHI_CUDA_OK) return rc;
                SB_LOG_INFO("CUDA GEMM f64 [Row-Major]: {}x[{}x{}x{}]", g.batch, g.m, g.n, g.k);
                rc = sushi_cuda_dgemm_strided_batched(ctx, 0, g.trans_a, g.trans_b, g.m, g.n, g.k, static_cast<double>(g.alpha),
                                                      da, g.lda, g.stride_a, db, g.ldb, g.stride_b, static_cast<double>(g.beta),
                                                      dc, g.ldc, g.stride_c, g.batch);
                if (rc == SUSHI_CUDA_OK) detail::stage_out(oc.storage);
                return rc;
            });
        return SushiRuntime::Execution::Event();
    }

    // ---------------------------------------------------------------- Level3::syrk
    inline SushiRuntime::Execution::Event Level3::syrk(const Tensor& A, Tensor& C, bool upper, bool transA, float alpha,
                                                       float beta)
    {
        using namespace SushiRuntime::Graph::Literals;
        SB_THROW_IF(A.rank < 2 || C.rank < 2, "SYRK requires at least 2D tensors.");
        SB_THROW_IF(A.dtype != C.dtype, "Data type mismatch in SYRK operation.");
        SB_THROW_IF(A.dtype != Core::DataType::FLOAT32,
                    "Unsupported data type for SYRK operation (the CUDA backend serves FLOAT32 only).");
        const int32_t ra = A.rank, rc = C.rank;
        const int64_t n = C.shape[rc - 2];
        SB_THROW_IF(C.shape[rc - 1] != n, "SYRK requires C to be a square matrix.");
        const int64_t inner_n = transA ? A.shape[ra - 1] : A.shape[ra - 2];
        const int64_t k = transA ? A.shape[ra - 2] : A.shape[ra - 1];
        SB_THROW_IF(inner_n != n, "Dimension mismatch in SYRK: A does not match C dimension.");
        int64_t batch = 1;
        for (int i = 0; i < rc - 2; ++i) batch *= C.shape[i];
        const bool row = A.layout == Core::Layout::ROW_MAJOR;
        const int64_t lda = row ? A.shape[ra - 1] : A.shape[ra - 2];
        const int64_t ldc = (C.layout == Core::Layout::ROW_MAJOR) ? C.shape[rc - 1] : C.shape[rc - 2];
        int64_t stride_a = 0, stride_c = 0;
        if (batch > 1)
        {
            SB_THROW_IF(ra < 3, "Batched SYRK requires A of rank >= 3 (got {}).", ra);
            stride_a = A.strides[ra - 3];
            stride_c = C.strides[rc - 3];
        }
        // a column-major update is the row-major update of the other triangle with the other transpose
        const bool rm_upper = row ? upper : !upper;
        const bool rm_trans = row ? transA : !transA;

        struct Operand { SushiRuntime::sushi_ptr<Storage> storage; float* ptr; int64_t extent; bool host; };
        auto describe = [](const Tensor& t, int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t nb) {
            Operand o{t.storage, t.data_as<float>(), detail::operand_extent(rows, cols, ld, stride, nb), false};
            o.host = t.storage->host_resident();
            const std::size_t need = (static_cast<std::size_t>(t.storage_offset) + static_cast<std::size_t>(o.extent)) * sizeof(float);
            SB_THROW_IF(need > t.storage->size_bytes, "SYRK operand does not fit its storage (needs {} bytes, has {}).", need,
                        t.storage->size_bytes);
            return o;
        };
        Operand oa = describe(A, rm_trans ? k : n, rm_trans ? n : k, lda, stride_a, batch);
        Operand oc = describe(C, n, n, ldc, stride_c, batch);

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = "blas.lvl3.syrk";
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = "blas.lvl3.syrk"_op;
        meta.set_param(0, alpha); meta.set_param(1, beta); meta.set_param(2, upper); meta.set_param(3, transA);
        engine_.get_graph().add_task(meta, {A.storage->data_ptr}, {C.storage->data_ptr},
            [=](SushiRuntime::Execution::RuntimeContext& rt) -> int
            {
                sushi_cuda_ctx* ctx = rt.native_handle();
                auto on_device = [](const Operand& o, bool reads, float** out) -> int
                { return detail::stage_in(o.storage, o.ptr, o.extent, reads, out); };
                float *da = nullptr, *dc = nullptr;
                int rc2 = on_device(oa, true, &da);
                // the untouched triangle must survive the copy back: host-resident C always goes up
                if (rc2 == SUSHI_CUDA_OK) rc2 = on_device(oc, true, &dc);
                if (rc2 != SUSHI_CUDA_OK) return rc2;
                rc2 = sushi_cuda_ssyrk_strided_batched(ctx, 0, rm_upper, rm_trans, n, k, alpha, da, lda, stride_a, beta, dc, ldc,
                                                       stride_c, batch);
                if (rc2 == SUSHI_CUDA_OK) detail::stage_out(oc.storage);
                return rc2;
            });
        return SushiRuntime::Execution::Event();
    }

    // ---------------------------------------------------------------- Level3::trsm
    inline SushiRuntime::Execution::Event Level3::trsm(const Tensor& A, Tensor& B, bool left_side, bool upper, bool transA,
                                                       bool unit_diag, float alpha)
    {
        using namespace SushiRuntime::Graph::Literals;
        SB_THROW_IF(A.rank < 2 || B.rank < 2, "TRSM requires at least 2D tensors.");
        SB_THROW_IF(A.dtype != B.dtype, "Data type mismatch in TRSM operation.");
        SB_THROW_IF(A.dtype != Core::DataType::FLOAT32,
                    "Unsupported data type for TRSM operation (the CUDA backend serves FLOAT32 only).");
        const int32_t ra = A.rank, rb = B.rank;
        const int64_t m = B.shape[rb - 2], n = B.shape[rb - 1];
        const int64_t a_rows = A.shape[ra - 2], a_cols = A.shape[ra - 1];
        SB_THROW_IF(a_rows != a_cols, "TRSM requires matrix A to be square.");
        if (left_side) SB_THROW_IF(a_rows != m, "Left-sided TRSM: dimensions of A must match rows of B.");
        else SB_THROW_IF(a_rows != n, "Right-sided TRSM: dimensions of A must match cols of B.");
        int64_t batch = 1;
        for (int i = 0; i < rb - 2; ++i) batch *= B.shape[i];
        const bool row = A.layout == Core::Layout::ROW_MAJOR;
        const int64_t lda = row ? A.shape[ra - 1] : A.shape[ra - 2];
        const int64_t ldb = (B.layout == Core::Layout::ROW_MAJOR) ? B.shape[rb - 1] : B.shape[rb - 2];
        int64_t stride_a = 0, stride_b = 0;
        if (batch > 1)
        {
            SB_THROW_IF(ra < 3, "Batched TRSM requires A of rank >= 3 (got {}).", ra);
            stride_a = A.strides[ra - 3];
            stride_b = B.strides[rb - 3];
        }
        // A column-major solve is the row-major solve of the transposed equation: the memory of a
        // column-major B (m x n) is a row-major n x m matrix, A's memory is the other triangle, and
        // op(A) moves to the other side:  op(A) X = aB  <=>  X^T op(A)^T = aB^T.
        const bool rm_left = row ? left_side : !left_side;
        const bool rm_upper = row ? upper : !upper;
        const int64_t rm_m = row ? m : n, rm_n = row ? n : m;
        const int64_t dim = left_side ? m : n;

        struct Operand { SushiRuntime::sushi_ptr<Storage> storage; float* ptr; int64_t extent; bool host; };
        auto describe = [](const Tensor& t, int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t nb) {
            Operand o{t.storage, t.data_as<float>(), detail::operand_extent(rows, cols, ld, stride, nb), false};
            o.host = t.storage->host_resident();
            const std::size_t need = (static_cast<std::size_t>(t.storage_offset) + static_cast<std::size_t>(o.extent)) * sizeof(float);
            SB_THROW_IF(need > t.storage->size_bytes, "TRSM operand does not fit its storage (needs {} bytes, has {}).", need,
                        t.storage->size_bytes);
            return o;
        };
        Operand oa = describe(A, dim, dim, lda, stride_a, batch);
        Operand ob = describe(B, rm_m, rm_n, ldb, stride_b, batch);

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = "blas.lvl3.trsm";
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = "blas.lvl3.trsm"_op;
        meta.set_param(0, alpha); meta.set_param(1, left_side); meta.set_param(2, upper); meta.set_param(3, transA);
        meta.set_param(4, unit_diag);
        engine_.get_graph().add_task(meta, {A.storage->data_ptr}, {B.storage->data_ptr},
            [=](SushiRuntime::Execution::RuntimeContext& rt) -> int
            {
                sushi_cuda_ctx* ctx = rt.native_handle();
                auto on_device = [](const Operand& o, float** out) -> int
                { return detail::stage_in(o.storage, o.ptr, o.extent, true, out); };
                float *da = nullptr, *db = nullptr;
                int rc2 = on_device(oa, &da);
                if (rc2 == SUSHI_CUDA_OK) rc2 = on_device(ob, &db);
                if (rc2 != SUSHI_CUDA_OK) return rc2;
                rc2 = sushi_cuda_strsm_strided_batched(ctx, 0, rm_left, rm_upper, transA, unit_diag, rm_m, rm_n, alpha, da, lda,
                                                       stride_a, db, ldb, stride_b, batch);
                if (rc2 == SUSHI_CUDA_OK) detail::stage_out(ob.storage);
                return rc2;
            });
        return SushiRuntime::Execution::Event();
    }

    // ---------------------------------------------------------------- Level3::gemm_row_sharded
    inline SushiRuntime::Execution::Event Level3::gemm_row_sharded(const Tensor& A_local, const Tensor& B, Tensor& C_full,
                                                                   bool transA, bool transB, float alpha, float beta)
    {
        using namespace SushiRuntime::Graph::Literals;
        SB_THROW_IF(A_local.rank != 2 || B.rank != 2 || C_full.rank != 2, "Sharded GEMM requires 2D tensors.");
        SB_THROW_IF(A_local.dtype != B.dtype || A_local.dtype != C_full.dtype, "Data type mismatch in GEMM operation.");
        SB_THROW_IF(A_local.dtype != Core::DataType::FLOAT32,
                    "Unsupported data type for GEMM operation (the CUDA backend serves FLOAT32 only).");
        SB_THROW_IF(A_local.layout != Core::Layout::ROW_MAJOR || B.layout != Core::Layout::ROW_MAJOR ||
                    C_full.layout != Core::Layout::ROW_MAJOR, "Sharded GEMM serves row-major tensors only.");
        for (const Tensor* t : {&A_local, &B, static_cast<const Tensor*>(&C_full)})
            SB_THROW_IF(!t->storage || t->storage->host_resident(), "Sharded GEMM requires DEVICE tensors.");
        auto& rt = engine_.get_context();
        const int64_t m = C_full.shape[0], n = C_full.shape[1];
        const int64_t k = transB ? B.shape[1] : B.shape[0];
        int64_t first = 0, count = 0;
        sushi_cuda_partition(m, rt.nranks(), rt.rank(), &first, &count);
        const int64_t a_rows = transA ? A_local.shape[1] : A_local.shape[0];
        const int64_t a_k = transA ? A_local.shape[0] : A_local.shape[1];
        SB_THROW_IF(a_rows != count || a_k != k, "A_local must hold this rank's {} rows of op(A) with k = {} (got {} x {}).",
                    count, k, a_rows, a_k);
        SB_THROW_IF((transB ? B.shape[0] : B.shape[1]) != n, "B does not match C ({} columns expected).", n);

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = "blas.lvl3.gemm_row_sharded";
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = "blas.lvl3.gemm_row_sharded"_op;
        meta.set_param(0, alpha); meta.set_param(1, beta); meta.set_param(2, transA); meta.set_param(3, transB);
        auto sa = A_local.storage; auto sb_ = B.storage; auto sc = C_full.storage;
        const float* pa = A_local.data_as<float>(); const float* pb = B.data_as<float>(); float* pc = C_full.data_as<float>();
        const int64_t lda = A_local.shape[1], ldb = B.shape[1], ldc = n;
        engine_.get_graph().add_task(meta, {sa->data_ptr, sb_->data_ptr}, {sc->data_ptr},
            [=](SushiRuntime::Execution::RuntimeContext& ctx) -> int
            {
                (void)sa; (void)sb_; (void)sc;       // keep the storages alive until the task has run
                return sushi_cuda_sgemm_row_sharded(ctx.native_handle(), 0, transA, transB, m, n, k, alpha, pa, lda, pb, ldb,
                                                    beta, pc, ldc, /*gather=*/1);
            });
        return SushiRuntime::Execution::Event();
    }

    // ---------------------------------------------------------------- NonLinearOps
    inline SushiRuntime::Execution::Event NonLinearOps::forward(Tensor& t, const char* name, SushiRuntime::Graph::OpID op,
                                                                int activation, float param)
    {
        SB_THROW_IF(t.dtype != Core::DataType::FLOAT32, "Unsupported data type for {} (the CUDA backend serves FLOAT32 only).", name);
        SB_THROW_IF(!t.is_contiguous(), "Tensor must be contiguous for this operation");
        float* ptr = t.data_as<float>();
        const int64_t count = t.num_elements;
        if (engine_.get_graph().try_fuse_activation(ptr, count, activation, param)) return SushiRuntime::Execution::Event();

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = name;
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = op;
        meta.set_param(0, param);
        auto storage = t.storage;
        const bool host = storage->host_resident();
        engine_.get_graph().add_task(meta, {storage->data_ptr}, {storage->data_ptr},
            [storage, ptr, count, host, activation, param](SushiRuntime::Execution::RuntimeContext& rt) -> int
            {
                sushi_cuda_ctx* ctx = rt.native_handle();
                (void)host;
                float* dptr = nullptr;
                int rc = detail::stage_in(storage, ptr, count, true, &dptr);
                if (rc == SUSHI_CUDA_OK) rc = sushi_cuda_activation(ctx, 0, activation, param, dptr, count);
                if (rc == SUSHI_CUDA_OK) detail::stage_out(storage);
                return rc;
            });
        return SushiRuntime::Execution::Event();
    }

    inline SushiRuntime::Execution::Event NonLinearOps::backward(const Tensor& dy, const Tensor& saved, Tensor& dx, const char* name,
                                                                 SushiRuntime::Graph::OpID op, int activation, float param)
    {
        SB_THROW_IF(dy.dtype != saved.dtype || dy.dtype != dx.dtype, "Data type mismatch in {}.", name);
        SB_THROW_IF(dy.dtype != Core::DataType::FLOAT32, "Unsupported data type for {} (the CUDA backend serves FLOAT32 only).", name);
        SB_THROW_IF(dy.num_elements != saved.num_elements || dy.num_elements != dx.num_elements, "Size mismatch in {}.", name);
        SB_THROW_IF(!dy.is_contiguous() || !saved.is_contiguous() || !dx.is_contiguous(), "Tensor must be contiguous for this operation");
        struct Operand { SushiRuntime::sushi_ptr<Storage> storage; float* ptr; bool host; };
        const Operand od{dy.storage, dy.data_as<float>(), dy.storage->host_resident()};
        const Operand os{saved.storage, saved.data_as<float>(), saved.storage->host_resident()};
        const Operand ox{dx.storage, dx.data_as<float>(), dx.storage->host_resident()};
        const int64_t count = dy.num_elements;

        SushiRuntime::Graph::TaskMetadata meta;
        meta.name = name;
        meta.task_type = SushiRuntime::Graph::TaskType::MATH_OP;
        meta.op_id = op;
        meta.set_param(0, param);
        engine_.get_graph().add_task(meta, {dy.storage->data_ptr, saved.storage->data_ptr}, {dx.storage->data_ptr},
            [od, os, ox, count, activation, param](SushiRuntime::Execution::RuntimeContext& rt) -> int
            {
                sushi_cuda_ctx* ctx = rt.native_handle();
                const std::size_t bytes = static_cast<std::size_t>(count) * sizeof(float);
                (void)bytes;
                auto on_device = [count](const Operand& o, bool reads, float** out) -> int
                { return detail::stage_in(o.storage, o.ptr, count, reads, out); };
                float *d_dy = nullptr, *d_s = nullptr, *d_dx = nullptr;
                int rc = on_device(od, true, &d_dy);
                if (rc == SUSHI_CUDA_OK) rc = on_device(os, true, &d_s);
                if (rc == SUSHI_CUDA_OK) rc = on_device(ox, false, &d_dx);
                if (rc == SUSHI_CUDA_OK) rc = sushi_cuda_activation_backward(ctx, 0, activation, param, d_dy, d_s, d_dx, count);
                if (rc == SUSHI_CUDA_OK) detail::stage_out(ox.storage);
                return rc;
            });
        return SushiRuntime::Execution::Event();
    }

#define SUSHI_NONLINEAR_OP(fn, dotted, kind)                                                                                   \
    inline SushiRuntime::Execution::Event NonLinearOps::fn(Tensor& t)                                                          \
    {                                                                                                                          \
        using namespace SushiRuntime::Graph::Literals;                                                                         \
        return forward(t, "math.nonlinear." dotted, "math.nonlinear." dotted ""_op, kind, 0.0f);                               \
    }                                                                                                                          \
    inline SushiRuntime::Execution::Event NonLinearOps::fn##_backward(const Tensor& dy, const Tensor& s, Tensor& dx)           \
    {                                                                                                                          \
        using namespace SushiRuntime::Graph::Literals;                                                                         \
        return backward(dy, s, dx, "math.nonlinear." dotted "_backward", "math.nonlinear." dotted "_backward"_op, kind, 0.0f); \
    }
#define SUSHI_NONLINEAR_OP_PARAM(fn, dotted, kind)                                                                             \
    inline SushiRuntime::Execution::Event NonLinearOps::fn(Tensor& t, float alpha)                                             \
    {                                                                                                                          \
        using namespace SushiRuntime::Graph::Literals;                                                                         \
        return forward(t, "math.nonlinear." dotted, "math.nonlinear." dotted ""_op, kind, alpha);                              \
    }                                                                                                                          \
    inline SushiRuntime::Execution::Event NonLinearOps::fn##_backward(const Tensor& dy, const Tensor& s, Tensor& dx,           \
                                                                      float alpha)                                             \
    {                                                                                                                          \
        using namespace SushiRuntime::Graph::Literals;                                                                         \
        return backward(dy, s, dx, "math.nonlinear." dotted "_backward", "math.nonlinear." dotted "_backward"_op, kind, alpha);\
    }
    SUSHI_NONLINEAR_OP(relu, "relu", SUSHI_ACT_RELU)
    SUSHI_NONLINEAR_OP(sigmoid, "sigmoid", SUSHI_ACT_SIGMOID)
    SUSHI_NONLINEAR_OP(tanh, "tanh", SUSHI_ACT_TANH)
    SUSHI_NONLINEAR_OP(silu, "silu", SUSHI_ACT_SILU)
    SUSHI_NONLINEAR_OP(gelu, "gelu", SUSHI_ACT_GELU)
    SUSHI_NONLINEAR_OP(softplus, "softplus", SUSHI_ACT_SOFTPLUS)
    SUSHI_NONLINEAR_OP_PARAM(leaky_relu, "leaky_relu", SUSHI_ACT_LEAKY_RELU)
    SUSHI_NONLINEAR_OP_PARAM(elu, "elu", SUSHI_ACT_ELU)
#undef SUSHI_NONLINEAR_OP
#undef SUSHI_NONLINEAR_OP_PARAM

    // ---------------------------------------------------------------- IO
    // The file formats themselves live in detail:: functions that take no Engine, so that they can be
    // exercised with host-resident tensors on a machine without a GPU; IO adds the flush of pending work.
    namespace detail
    {
        inline void write_payload(std::ofstream& ofs, const Tensor& t)
        {
            SB_THROW_IF(!t.storage, "Accessing data of a tensor with no storage");
            SB_THROW_IF(!t.is_contiguous(), "Tensor must be contiguous for this operation");
            const std::size_t bytes = static_cast<std::size_t>(t.num_elements) * io_bytes_per_element(t.dtype);
            if (bytes == 0) return;
            if (t.storage->host_resident())
                ofs.write(static_cast<const char*>(t.data()), static_cast<std::streamsize>(bytes));
            else
            {
                std::vector<char> buf(bytes);
                t.to_host(buf.data());
                ofs.write(buf.data(), static_cast<std::streamsize>(bytes));
            }
            SB_THROW_IF(!ofs.good(), "Failed while writing {} bytes of tensor data", bytes);
        }

        inline void read_payload(std::ifstream& ifs, Tensor& t, const std::string& path)
        {
            SB_THROW_IF(!t.storage, "Accessing data of a tensor with no storage");
            SB_THROW_IF(!t.is_contiguous(), "Tensor must be contiguous for this operation");
            const std::size_t bytes = static_cast<std::size_t>(t.num_elements) * io_bytes_per_element(t.dtype);
            if (bytes == 0) return;
            if (t.storage->host_resident())
            {
                ifs.read(static_cast<char*>(t.data()), static_cast<std::streamsize>(bytes));
                SB_THROW_IF(static_cast<std::size_t>(ifs.gcount()) != bytes, "File is shorter than the tensor ({} bytes): {}", bytes, path);
                // the device mirror of a host-resident tensor is refreshed by the next operation that reads it
            }
            else
            {
                std::vector<char> buf(bytes);
                ifs.read(buf.data(), static_cast<std::streamsize>(bytes));
                SB_THROW_IF(static_cast<std::size_t>(ifs.gcount()) != bytes, "File is shorter than the tensor ({} bytes): {}", bytes, path);
                t.from_host(buf.data());
            }
        }

        inline void save_npy_file(const Tensor& t, const std::string& path)
        {
            SB_THROW_IF(npy_descr(t.dtype)[0] == '\0', "Unsupported data type for .npy export.");
            std::ofstream ofs(path, std::ios::binary);
            SB_THROW_IF(!ofs.is_open(), "Failed to open file: {}", path);
            const std::string dict = npy_header_dict(t.dtype, t.layout, t.shape.data(), t.rank);
            SB_THROW_IF(dict.size() > 65535, "Tensor shape does not fit a version 1.0 .npy header");
            const unsigned char preamble[10] = {0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0,
                                                static_cast<unsigned char>(dict.size() & 0xff),
                                                static_cast<unsigned char>(dict.size() >> 8)};
            ofs.write(reinterpret_cast<const char*>(preamble), 10);
            ofs.write(dict.data(), static_cast<std::streamsize>(dict.size()));
            write_payload(ofs, t);
        }

        inline void load_npy_file(Tensor& t, const std::string& path)
        {
            std::ifstream ifs(path, std::ios::binary);
            SB_THROW_IF(!ifs.is_open(), "Failed to open file for reading: {}", path);
            unsigned char pre[8] = {0};
            ifs.read(reinterpret_cast<char*>(pre), 8);
            SB_THROW_IF(ifs.gcount() != 8 || std::memcmp(pre, "\x93NUMPY", 6) != 0, "Invalid .npy file magic.");
            const int major = pre[6];
            SB_THROW_IF(major < 1 || major > 3, "Unsupported .npy format version {}.{}", major, int(pre[7]));
            unsigned char len_bytes[4] = {0};
            const int len_size = (major == 1) ? 2 : 4;
            ifs.read(reinterpret_cast<char*>(len_bytes), len_size);
            SB_THROW_IF(ifs.gcount() != len_size, "Truncated .npy header: {}", path);
            const std::size_t header_len = std::size_t(len_bytes[0]) | (std::size_t(len_bytes[1]) << 8) |
                                           (std::size_t(len_bytes[2]) << 16) | (std::size_t(len_bytes[3]) << 24);
            std::string header(header_len, ' ');
            ifs.read(header.data(), static_cast<std::streamsize>(header_len));
            SB_THROW_IF(static_cast<std::size_t>(ifs.gcount()) != header_len, "Truncated .npy header: {}", path);
            const NpyInfo info = parse_npy_header(header);

            std::string want = npy_descr(t.dtype);
            std::string have = info.descr;
            if (!have.empty() && (have[0] == '=' || have[0] == '|')) have[0] = '<';     // native order on this host is little-endian
            SB_THROW_IF(have != want, "Data type mismatch in .npy header: file has '{}', tensor needs '{}'.", info.descr, want);
            SB_THROW_IF(static_cast<int32_t>(info.shape.size()) != t.rank, "Rank mismatch in .npy header: file has {}, tensor has {}.",
                        info.shape.size(), t.rank);
            for (int i = 0; i < t.rank; ++i)
                SB_THROW_IF(info.shape[static_cast<std::size_t>(i)] != t.shape[i], "Shape dimension {} mismatch in .npy header.", i);
            int wide_dims = 0;
            for (int i = 0; i < t.rank; ++i) wide_dims += t.shape[i] > 1;
            SB_THROW_IF(wide_dims > 1 && info.fortran_order != (t.layout == Core::Layout::COLUMN_MAJOR),
                        "Memory order mismatch in .npy header: fortran_order is {}.", info.fortran_order ? "True" : "False");
            read_payload(ifs, t, path);
        }
        // Native ".sushi" container (src/io.cpp:40-109): the reference dumps a struct
        //   { char magic[6] = "SUSHI"; uint32 version = 1; int32 rank; int64 shape[6]; int32 dtype; int32 layout; }
        // as the compiler lays it out on x86-64 -- magic at 0, version at 8, rank at 12, shape at 16, dtype at 64,
        // layout at 68, 72 bytes in all -- followed by the raw elements.  Written here field by field at those
        // offsets (padding and unused extents zero); the loader checks what the reference checks: magic, rank
        // and the first `rank` extents.
        constexpr std::size_t SUSHI_HEADER_BYTES = 72;

        inline void save_sushi_file(const Tensor& t, const std::string& path)
        {
            unsigned char h[SUSHI_HEADER_BYTES] = {0};
            std::memcpy(h, "SUSHI", 6);
            const std::uint32_t version = 1;
            const std::int32_t rank = t.rank, dtype = static_cast<std::int32_t>(t.dtype), layout = static_cast<std::int32_t>(t.layout);
            std::memcpy(h + 8, &version, 4);
            std::memcpy(h + 12, &rank, 4);
            for (int i = 0; i < t.rank; ++i) std::memcpy(h + 16 + 8 * i, &t.shape[i], 8);
            std::memcpy(h + 64, &dtype, 4);
            std::memcpy(h + 68, &layout, 4);
            std::ofstream ofs(path, std::ios::binary);
            SB_THROW_IF(!ofs.is_open(), "Failed to open file for writing: {}", path);
            ofs.write(reinterpret_cast<const char*>(h), SUSHI_HEADER_BYTES);
            write_payload(ofs, t);
        }

        inline void load_sushi_file(Tensor& t, const std::string& path)
        {
            std::ifstream ifs(path, std::ios::binary);
            SB_THROW_IF(!ifs.is_open(), "Failed to open file for reading: {}", path);
            unsigned char h[SUSHI_HEADER_BYTES] = {0};
            ifs.read(reinterpret_cast<char*>(h), SUSHI_HEADER_BYTES);
            SB_THROW_IF(static_cast<std::size_t>(ifs.gcount()) != SUSHI_HEADER_BYTES || std::memcmp(h, "SUSHI", 5) != 0,
                        "Invalid .sushi file magic.");
            std::int32_t rank = 0;
            std::memcpy(&rank, h + 12, 4);
            SB_THROW_IF(rank != t.rank, "Rank mismatch in .sushi file.");
            for (int i = 0; i < t.rank; ++i)
            {
                std::int64_t extent = 0;
                std::memcpy(&extent, h + 16 + 8 * i, 8);
                SB_THROW_IF(extent != t.shape[i], "Dimension mismatch at index {}", i);
            }
            read_payload(ifs, t, path);
        }
    } // namespace detail

    namespace detail
    {
        // Text form of a tensor (src/io.cpp:242-359): "Tensor(shape=[..], dtype=f32):" and the nested rows with
        // `precision` fixed decimals; a dimension longer than 2 * edge_items shows its first and last edge_items
        // entries around "...".  Elements are addressed through the tensor's strides, so views print as they index.
        inline std::string format_tensor(const Tensor& t, int precision, int edge_items)
        {
            SB_THROW_IF(!t.storage, "Accessing data of a tensor with no storage");
            const bool cplx = t.dtype == Core::DataType::COMPLEX32 || t.dtype == Core::DataType::COMPLEX64;
            const bool wide = t.dtype == Core::DataType::FLOAT64 || t.dtype == Core::DataType::COMPLEX64;
            SB_THROW_IF(t.dtype == Core::DataType::HALF, "Unsupported data type for printing.");
            // elements spanned from data(): 1 + sum (extent - 1) * stride
            std::int64_t span = t.num_elements > 0 ? 1 : 0;
            for (int i = 0; i < t.rank && span > 0; ++i) span += (t.shape[i] - 1) * t.strides[i];
            const std::size_t elem = io_bytes_per_element(t.dtype);
            std::vector<char> host(static_cast<std::size_t>(span) * elem);
            if (span > 0)
            {
                if (t.storage->host_resident()) std::memcpy(host.data(), t.data(), host.size());
                else
                {
                    SB_THROW_IF(!t.is_contiguous(), "Tensor must be contiguous for this operation");
                    t.to_host(host.data());
                }
            }
            auto value = [&](std::int64_t idx) -> std::string
            {
                double re = 0.0, im = 0.0;
                if (wide) { const double* p = reinterpret_cast<const double*>(host.data()) + idx * (cplx ? 2 : 1); re = p[0]; if (cplx) im = p[1]; }
                else { const float* p = reinterpret_cast<const float*>(host.data()) + idx * (cplx ? 2 : 1); re = p[0]; if (cplx) im = p[1]; }
                std::ostringstream v;
                v << std::fixed << std::setprecision(precision);
                // the reference converts to float before printing
                if (std::abs(static_cast<float>(im)) < 1e-9) v << static_cast<float>(re);
                else v << "(" << static_cast<float>(re) << (im >= 0 ? "+" : "") << static_cast<float>(im) << "j)";
                return v.str();
            };
            std::ostringstream os;
            os << "Tensor(shape=[";
            for (int i = 0; i < t.rank; ++i) os << t.shape[i] << (i == t.rank - 1 ? "" : ", ");
            os << "], dtype=" << (t.dtype == Core::DataType::FLOAT32 ? "f32" : t.dtype == Core::DataType::FLOAT64 ? "f64"
                                  : t.dtype == Core::DataType::COMPLEX32 ? "c32" : "c64") << "):\n";
            std::function<void(int, std::int64_t)> emit = [&](int dim, std::int64_t offset)
            {
                const std::int64_t extent = t.shape[dim], stride = t.strides[dim];
                const bool last = dim == t.rank - 1;
                const std::string indent(static_cast<std::size_t>(dim) + 1, ' ');
                os << "[";
                for (std::int64_t i = 0; i < extent; ++i)
                {
                    if (extent > 2 * edge_items && i == edge_items)
                    {
                        if (last) os << "... "; else os << "\n" << indent << "...\n" << indent;
                        i = extent - edge_items - 1;        // resumes at extent - edge_items
                        continue;
                    }
                    if (last) os << value(offset + i * stride) << (i == extent - 1 ? "" : ", ");
                    else
                    {
                        emit(dim + 1, offset + i * stride);
                        if (i < extent - 1) os << ",\n" << indent;
                    }
                }
                os << "]";
                if (dim == 0 && !last) os << "\n";
            };
            if (t.rank > 0) emit(0, 0);
            return os.str();
        }
    } // namespace detail

    inline std::string IO::to_string(const Tensor& t, int precision, int edge_items)
    {
        engine_.execute().wait();
        return detail::format_tensor(t, precision, edge_items);
    }

    inline void IO::print(const Tensor& t, int precision, int edge_items)
    {
        std::fputs(to_string(t, precision, edge_items).c_str(), stdout);
    }

    inline void IO::save(const Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        detail::save_sushi_file(t, path);
        SB_LOG_INFO("Saved native SushiBLAS file: {}", path);
    }

    inline void IO::load(Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        detail::load_sushi_file(t, path);
    }

    inline void IO::save_npy(const Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        detail::save_npy_file(t, path);
        SB_LOG_INFO("Exported NumPy file: {}", path);
    }

    inline void IO::load_npy(Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        detail::load_npy_file(t, path);
        SB_LOG_INFO("Loaded NumPy file: {}", path);
    }

    inline void IO::save_bin(const Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        std::ofstream ofs(path, std::ios::binary);
        SB_THROW_IF(!ofs.is_open(), "Failed to open file: {}", path);
        detail::write_payload(ofs, t);
    }

    inline void IO::load_bin(Tensor& t, const std::string& path)
    {
        engine_.execute().wait();
        std::ifstream ifs(path, std::ios::binary);
        SB_THROW_IF(!ifs.is_open(), "Failed to open file: {}", path);
        detail::read_payload(ifs, t, path);
    }

} // namespace SushiBLAS
