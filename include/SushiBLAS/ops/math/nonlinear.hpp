// ops/math/nonlinear.hpp -- the activation family (reference: include/SushiBLAS/ops/math/nonlinear.hpp:55-205,
// src/ops/math/nonlinear/*.cpp, element-wise driver nonlinear_internal.hpp:50-92), FLOAT32 here.  Forward
// ops work in place; backward ops write dx = dy * f'(.) from the forward INPUT x -- sigmoid and tanh
// from the forward OUTPUT y -- with the reference's argument order.  The reference's only multi-op
// workloads are GEMM -> activation chains (tests/runtime/test_framework_sim.cpp:47-58,107-111): a
// forward op recorded right after a GEMM that wrote exactly that tensor is folded into the GEMM's
// epilogue and no separate kernel runs.
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

            /// t <- f(t) element-wise, in place.  Recorded on the task graph (or folded into the
            /// preceding GEMM); runs at Engine::execute().
            inline SushiRuntime::Execution::Event relu(Tensor& t);                       ///< x > 0 ? x : 0
            inline SushiRuntime::Execution::Event leaky_relu(Tensor& t, float alpha = 0.01f);   ///< x > 0 ? x : alpha x
            inline SushiRuntime::Execution::Event sigmoid(Tensor& t);                    ///< 1 / (1 + exp(-x))
            inline SushiRuntime::Execution::Event tanh(Tensor& t);
            inline SushiRuntime::Execution::Event elu(Tensor& t, float alpha = 1.0f);    ///< x > 0 ? x : alpha (exp(x) - 1)
            inline SushiRuntime::Execution::Event silu(Tensor& t);                       ///< x / (1 + exp(-x))
            inline SushiRuntime::Execution::Event gelu(Tensor& t);                       ///< tanh form (gelu.cpp:38-44)
            inline SushiRuntime::Execution::Event softplus(Tensor& t);                   ///< log(1 + exp(x))

            /// dx <- dy * f'(x); the third argument of the reference's signatures is the forward input x,
            /// for sigmoid and tanh the forward output y.
            inline SushiRuntime::Execution::Event relu_backward(const Tensor& dy, const Tensor& x, Tensor& dx);
            inline SushiRuntime::Execution::Event leaky_relu_backward(const Tensor& dy, const Tensor& x, Tensor& dx, float alpha = 0.01f);
            inline SushiRuntime::Execution::Event sigmoid_backward(const Tensor& dy, const Tensor& y, Tensor& dx);
            inline SushiRuntime::Execution::Event tanh_backward(const Tensor& dy, const Tensor& y, Tensor& dx);
            inline SushiRuntime::Execution::Event elu_backward(const Tensor& dy, const Tensor& x, Tensor& dx, float alpha = 1.0f);
            inline SushiRuntime::Execution::Event silu_backward(const Tensor& dy, const Tensor& x, Tensor& dx);
            inline SushiRuntime::Execution::Event gelu_backward(const Tensor& dy, const Tensor& x, Tensor& dx);
            inline SushiRuntime::Execution::Event softplus_backward(const Tensor& dy, const Tensor& x, Tensor& dx);

        private:
            inline SushiRuntime::Execution::Event forward(Tensor& t, const char* name, SushiRuntime::Graph::OpID op, int activation,
                                                          float param);
            inline SushiRuntime::Execution::Event backward(const Tensor& dy, const Tensor& saved, Tensor& dx, const char* name,
                                                           SushiRuntime::Graph::OpID op, int activation, float param);
            Engine& engine_;
    };
} // namespace SushiBLAS
