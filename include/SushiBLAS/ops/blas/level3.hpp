// ops/blas/level3.hpp -- Level-3 BLAS front-end: GEMM (reference declaration:
// include/SushiBLAS/ops/blas/level3.hpp:71-73; definition src/ops/blas/level3/gemm.cpp:82-198).
//
//   C <- alpha * op(A) * op(B) + beta * C        op(X) = X or X^T, batched when rank > 2
//
// The record phase is the reference's: validate, derive m/n/k/ld/stride/batch from the Tensor
// metadata, build TaskMetadata, add a task.  The task body calls the C ABI instead of oneMKL.
// GEMM serves FLOAT32 (tcgen05 3xTF32 / FFMA kernels) and FLOAT64 (DMMA kernel); SYRK and TRSM
// (FLOAT32) run on the fp32 GEMM kernels.
#pragma once

#include <cstdint>
#include <vector>

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiBLAS/tensor.hpp>
#include <SushiRuntime/SushiRuntime.h>

namespace SushiBLAS
{
    class Engine;

    namespace detail
    {
        /// BLAS parameters of one GEMM call as gemm.cpp:91-105 derives them.
        struct GemmCall
        {
            bool trans_a = false, trans_b = false;
            int64_t m = 0, n = 0, k = 0, batch = 1;
            int64_t lda = 0, ldb = 0, ldc = 0;
            int64_t stride_a = 0, stride_b = 0, stride_c = 0;
            float alpha = 1.0f, beta = 0.0f;
            Core::Layout layout = Core::Layout::ROW_MAJOR;
        };

        /// Validation and parameter derivation of Level3::gemm (pure host logic, no device).
        ///  - rank >= 2 and equal dtypes, else std::runtime_error (gemm.cpp:87-88);
        ///  - m, n from C; k from A (gemm.cpp:91-93); batch = product of C's leading dims (96-97);
        ///  - leading dimensions from the SHAPE (last dim for row-major, second-to-last for
        ///    column-major), not from strides (99-101); layout taken from A (111);
        ///  - batch strides = strides[rank-3] when batch > 1, else 0 (103-105).
        /// Where the reference would index strides[-1] (a rank-2 operand under a batched C) this
        /// throws instead.
        inline GemmCall derive_gemm_call(const Tensor& A, const Tensor& B, const Tensor& C, bool transA, bool transB,
                                         float alpha, float beta)
        {
            SB_THROW_IF(A.rank < 2 || B.rank < 2 || C.rank < 2, "GEMM requires at least 2D tensors.");
            SB_THROW_IF(A.dtype != B.dtype || A.dtype != C.dtype, "Data type mismatch in GEMM operation.");
            GemmCall g;
            g.trans_a = transA; g.trans_b = transB; g.alpha = alpha; g.beta = beta; g.layout = A.layout;
            const int32_t ra = A.rank, rb = B.rank, rc = C.rank;
            g.m = C.shape[rc - 2];
            g.n = C.shape[rc - 1];
            g.k = transA ? A.shape[ra - 2] : A.shape[ra - 1];
            for (int i = 0; i < rc - 2; ++i) g.batch *= C.shape[i];
            g.lda = (A.layout == Core::Layout::ROW_MAJOR) ? A.shape[ra - 1] : A.shape[ra - 2];
            g.ldb = (B.layout == Core::Layout::ROW_MAJOR) ? B.shape[rb - 1] : B.shape[rb - 2];
            g.ldc = (C.layout == Core::Layout::ROW_MAJOR) ? C.shape[rc - 1] : C.shape[rc - 2];
            if (g.batch > 1)
            {
                SB_THROW_IF(ra < 3 || rb < 3, "Batched GEMM requires operands of rank >= 3 (got {} and {}).", ra, rb);
                g.stride_a = A.strides[ra - 3];
                g.stride_b = B.strides[rb - 3];
                g.stride_c = C.strides[rc - 3];
            }
            return g;
        }

        /// The row-major call that computes `g`.  A column-major product C = op(A) op(B) is the
        /// row-major product C^T = op(B)^T op(A)^T on the same memory: operands and m/n swap
        /// (the reference reaches oneMKL's column_major::gemm instead, gemm.cpp:66-78).
        inline GemmCall row_major_equivalent(const GemmCall& g, bool* swapped)
        {
            *swapped = (g.layout != Core::Layout::ROW_MAJOR);
            if (!*swapped) return g;
            GemmCall r = g;
            r.layout = Core::Layout::ROW_MAJOR;
            r.trans_a = g.trans_b; r.trans_b = g.trans_a;
            r.m = g.n; r.n = g.m;
            r.lda = g.ldb; r.ldb = g.lda;
            r.stride_a = g.stride_b; r.stride_b = g.stride_a;
            return r;
        }

        /// Elements spanned by a strided-batched row-major operand.
        inline int64_t operand_extent(int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t batch)
        {
            if (rows <= 0 || cols <= 0 || batch <= 0) return 0;
            return (batch - 1) * stride + (rows - 1) * ld + cols;
        }
    } // namespace detail

    class Level3
    {
        protected:
            explicit Level3(Engine& e) : engine_(e) {}
            Engine& engine_;

        private:
            /// FLOAT64 branch of gemm() (gemm.cpp:158-169): same derivation, alpha / beta widened.
            inline SushiRuntime::Execution::Event gemm_f64(const Tensor& A, const Tensor& B, Tensor& C, bool transA,
                                                           bool transB, float alpha, float beta);

        public:
            /// Records C <- alpha*op(A)*op(B) + beta*C on the engine's task graph; it runs at
            /// Engine::execute().  Returns an already-complete event (as the reference does,
            /// gemm.cpp:197): wait on execute().  C is not read when beta == 0.
            /// FLOAT32 and FLOAT64 tensors are served.  Throws std::runtime_error on rank < 2, dtype
            /// mismatch, any other dtype, a tensor without storage, or operands that do not fit
            /// their storage.
            inline SushiRuntime::Execution::Event gemm(const Tensor& A, const Tensor& B, Tensor& C,
                                                       bool transA = false, bool transB = false,
                                                       float alpha = 1.0f, float beta = 0.0f);

            /// Symmetric rank-k update C <- alpha*op(A)*op(A)^T + beta*C on the upper or lower triangle
            /// of the square C; the other triangle is left untouched (reference declaration
            /// level3.hpp syrk, definition src/ops/blas/level3/syrk.cpp:84-193).  n comes from C, k from
            /// A (A is n x k, or k x n when transA), leading dimensions from the shapes, batch strides
            /// from strides[rank-3].  FLOAT32 only.  Throws std::runtime_error on rank < 2, dtype
            /// mismatch, a non-square C or A not matching C.
            inline SushiRuntime::Execution::Event syrk(const Tensor& A, Tensor& C, bool upper = false, bool transA = false,
                                                       float alpha = 1.0f, float beta = 0.0f);

            /// Triangular solve with multiple right-hand sides, X overwriting B: op(A)*X = alpha*B
            /// (left_side) or X*op(A) = alpha*B (reference declaration level3.hpp trsm, definition
            /// src/ops/blas/level3/trsm.cpp:85-202).  m and n come from B, A must be square and match
            /// m (left) or n (right); leading dimensions from the shapes, batch count from B, batch
            /// strides from strides[rank-3]; A's layout selects row- or column-major for both tensors
            /// (trsm.cpp:129).  FLOAT32 only.  Throws std::runtime_error on rank < 2, dtype mismatch,
            /// a non-square A or A not matching B.
            inline SushiRuntime::Execution::Event trsm(const Tensor& A, Tensor& B, bool left_side = true, bool upper = false,
                                                       bool transA = false, bool unit_diag = false, float alpha = 1.0f);

            /// Multi-GPU GEMM, one process per GPU (no counterpart in the reference).  The global
            /// problem is C (m x n, the shape of C_full) = alpha*op(A)*op(B) + beta*C with A cut into
            /// row blocks of op(A): this rank passes its block A_local (rows
            /// [first, first+count) of op(A) as sushi_cuda_partition(m, nranks, rank) gives them; a
            /// count x k tensor, or k x count when transA), the whole B, and a full-size C_full in
            /// which it computes its own rows; the blocks are then exchanged so that every rank ends
            /// with the complete C (NCCL over NVLink).  Row-major DEVICE tensors only.
            inline SushiRuntime::Execution::Event gemm_row_sharded(const Tensor& A_local, const Tensor& B, Tensor& C_full,
                                                                   bool transA = false, bool transB = false,
                                                                   float alpha = 1.0f, float beta = 0.0f);
    };
} // namespace SushiBLAS
