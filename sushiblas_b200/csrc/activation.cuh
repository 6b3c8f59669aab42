// activation.cuh -- the element-wise activations of the reference's non-linear family
// (src/ops/math/nonlinear/{relu,leaky_relu,sigmoid,tanh,elu,silu,gelu,softplus}.cpp), as a GEMM
// epilogue stage and as stand-alone forward / backward kernels.  Formulas as the reference states
// them: relu x > 0 ? x : 0; leaky_relu x > 0 ? x : a x; sigmoid 1 / (1 + exp(-x)); tanh;
// elu x > 0 ? x : a (exp(x) - 1); silu x / (1 + exp(-x)); gelu 0.5 x (1 + tanh(0.79788456 (x +
// 0.044715 x^3))); softplus log(1 + exp(x)).  Backward forms take the upstream gradient and the
// forward INPUT x -- except sigmoid and tanh, which take the forward OUTPUT y, as the reference does.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace sushi {

enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY_RELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4, ACT_ELU = 5, ACT_SILU = 6,
             ACT_GELU = 7, ACT_SOFTPLUS = 8, ACT_COUNT = 9 };

__device__ __forceinline__ float apply_act(float v, int act, float a)
{
    switch (act)
    {
        case ACT_RELU: return fmaxf(v, 0.0f);                       // NaN -> 0, like x > 0 ? x : 0
        case ACT_LEAKY_RELU: return v > 0.0f ? v : v * a;
        case ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
        case ACT_TANH: return tanhf(v);
        case ACT_ELU: return v > 0.0f ? v : a * (expf(v) - 1.0f);
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_GELU:
        {
            // explicit roundings: the value must not depend on how a caller's context contracts mul + add
            const float v3 = __fmul_rn(__fmul_rn(v, v), v);
            const float inner = __fmul_rn(0.7978845608028654f, __fmaf_rn(0.044715f, v3, v));
            return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
        }
        case ACT_SOFTPLUS: return logf(1.0f + expf(v));
        default: return v;
    }
}

// dx = dy * f'(.), with `s` the forward input x (the forward output y for sigmoid and tanh)
__device__ __forceinline__ float apply_act_backward(float dy, float s, int act, float a)
{
    switch (act)
    {
        case ACT_RELU: return s > 0.0f ? dy : 0.0f;
        case ACT_LEAKY_RELU: return dy * (s > 0.0f ? 1.0f : a);
        case ACT_SIGMOID: return dy * s * (1.0f - s);
        case ACT_TANH: return dy * (1.0f - s * s);
        case ACT_ELU: return dy * (s > 0.0f ? 1.0f : a * expf(s));
        case ACT_SILU:
        {
            const float sig = 1.0f / (1.0f + expf(-s));
            return dy * (sig + s * sig * (1.0f - sig));
        }
        case ACT_GELU:
        {
            const float inner = 0.7978845608028654f * (s + 0.044715f * s * s * s);
            const float t = tanhf(inner);
            const float d_inner = 0.7978845608028654f * (1.0f + 0.134145f * s * s);
            return dy * (0.5f * (1.0f + t) + 0.5f * s * (1.0f - t * t) * d_inner);
        }
        case ACT_SOFTPLUS: return dy * (1.0f - 1.0f / (1.0f + expf(s)));
        default: return dy;
    }
}

// In place, one float4 per thread where the array allows it: HBM-bound (4 B read + 4 B written per element).
__global__ void activation_forward_kernel(float* __restrict__ x, int64_t count, int act, float a)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0)
    {
        const int64_t n4 = count / 4;
        float4* x4 = reinterpret_cast<float4*>(x);
        for (int64_t i = tid; i < n4; i += stride)
        {
            float4 v = x4[i];
            v.x = apply_act(v.x, act, a); v.y = apply_act(v.y, act, a); v.z = apply_act(v.z, act, a); v.w = apply_act(v.w, act, a);
            x4[i] = v;
        }
        for (int64_t i = n4 * 4 + tid; i < count; i += stride) x[i] = apply_act(x[i], act, a);
    }
    else
        for (int64_t i = tid; i < count; i += stride) x[i] = apply_act(x[i], act, a);
}

__global__ void activation_backward_kernel(const float* __restrict__ dy, const float* __restrict__ s, float* __restrict__ dx,
                                           int64_t count, int act, float a)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
    if (vec)
    {
        const int64_t n4 = count / 4;
        for (int64_t i = tid; i < n4; i += stride)
        {
            const float4 g = __ldg(reinterpret_cast<const float4*>(dy) + i);
            const float4 v = __ldg(reinterpret_cast<const float4*>(s) + i);
            float4 o;
            o.x = apply_act_backward(g.x, v.x, act, a); o.y = apply_act_backward(g.y, v.y, act, a);
            o.z = apply_act_backward(g.z, v.z, act, a); o.w = apply_act_backward(g.w, v.w, act, a);
            reinterpret_cast<float4*>(dx)[i] = o;
        }
        for (int64_t i = n4 * 4 + tid; i < count; i += stride) dx[i] = apply_act_backward(dy[i], s[i], act, a);
    }
    else
        for (int64_t i = tid; i < count; i += stride) dx[i] = apply_act_backward(dy[i], s[i], act, a);
}

} // namespace sushi
