// ops/math/nonlinear.hpp -- in-place ReLU (reference: include/SushiBLAS/ops/math/nonlinear.hpp:63,
// src/ops/math/nonlinear/relu.cpp:36-40: x > 0 ? x : 0, FLOAT32 here).  The reference's only
// multi-op workloads are GEMM -> ReLU chains (tests/runtime/test_framework_sim.cpp:47-58,107-111);
// when relu(t) is recorded right after a GEMM that wrote exactly t, it is folded into that GEMM's
// epilogue and no separate kernel runs.  The other activations of the reference are not part of
// this build.
#pragma once

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiBLAS/tensor.hpp>
#include <SushiRuntime/SushiRuntime.h>

namespace SushiBLAS
{
    class Engine;

    class NonLinearOps
    {
        public:
            explicit NonLinearOps(Engine& e) : engine_(e) {}

            /// t <- max(t, 0) element-wise, in place.  Recorded on the task graph (or folded into
            /// the preceding GEMM); runs at Engine::execute().
            inline SushiRuntime::Execution::Event relu(Tensor& t);

        private:
            Engine& engine_;
    };
} // namespace SushiBLAS
