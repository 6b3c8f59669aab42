"""CPU oracle of the activation family -- TEST INFRASTRUCTURE ONLY (imported by tests and smoke checks,
never by the product path).

Restates, in float64 numpy, the element-wise lambdas of the reference's
src/ops/math/nonlinear/{relu,leaky_relu,sigmoid,tanh,elu,silu,gelu,softplus}.cpp (forward and
backward), and holds the known answers of the reference's own tests
(tests/math/nonlinear/test_*.cpp: Forward and Backward of each file, verified there to 1e-4),
which pin these restatements.
"""
from __future__ import annotations

import numpy as np

NONE, RELU, LEAKY_RELU, SIGMOID, TANH, ELU, SILU, GELU, SOFTPLUS = range(9)
NAMES = {RELU: "relu", LEAKY_RELU: "leaky_relu", SIGMOID: "sigmoid", TANH: "tanh", ELU: "elu", SILU: "silu", GELU: "gelu",
         SOFTPLUS: "softplus"}
_C = 0.7978845608028654


def forward(kind: int, x, a: float = 0.0):
    x = np.asarray(x, dtype=np.float64)
    if kind == NONE:
        return x.copy()
    if kind == RELU:                       # relu.cpp:36-40
        return np.where(x > 0, x, 0.0)
    if kind == LEAKY_RELU:                 # leaky_relu.cpp:38-40
        return np.where(x > 0, x, x * a)
    if kind == SIGMOID:                    # sigmoid.cpp:38-39
        return 1.0 / (1.0 + np.exp(-x))
    if kind == TANH:                       # tanh.cpp:38-39
        return np.tanh(x)
    if kind == ELU:                        # elu.cpp:38-40
        return np.where(x > 0, x, a * (np.exp(np.minimum(x, 0.0)) - 1.0))
    if kind == SILU:                       # silu.cpp:38-39
        return x / (1.0 + np.exp(-x))
    if kind == GELU:                       # gelu.cpp:38-44
        return 0.5 * x * (1.0 + np.tanh(_C * (x + 0.044715 * x ** 3)))
    if kind == SOFTPLUS:                   # softplus.cpp:38-43
        return np.log(1.0 + np.exp(x))
    raise ValueError(kind)


def backward(kind: int, dy, s, a: float = 0.0):
    """dx = dy * f'(.): `s` is the forward input x, for sigmoid and tanh the forward output y."""
    dy = np.asarray(dy, dtype=np.float64)
    s = np.asarray(s, dtype=np.float64)
    if kind == RELU:
        return np.where(s > 0, dy, 0.0)
    if kind == LEAKY_RELU:
        return dy * np.where(s > 0, 1.0, a)
    if kind == SIGMOID:
        return dy * s * (1.0 - s)
    if kind == TANH:
        return dy * (1.0 - s * s)
    if kind == ELU:
        return dy * np.where(s > 0, 1.0, a * np.exp(np.minimum(s, 0.0)))
    if kind == SILU:
        sig = 1.0 / (1.0 + np.exp(-s))
        return dy * (sig + s * sig * (1.0 - sig))
    if kind == GELU:                       # gelu.cpp:47-58
        t = np.tanh(_C * (s + 0.044715 * s ** 3))
        d_inner = _C * (1.0 + 0.134145 * s * s)
        return dy * (0.5 * (1.0 + t) + 0.5 * s * (1.0 - t * t) * d_inner)
    if kind == SOFTPLUS:
        return dy * (1.0 - 1.0 / (1.0 + np.exp(s)))
    raise ValueError(kind)


# (kind, param, input, expected output) and (kind, param, dy, saved, expected dx) of the reference's tests
REFERENCE_FORWARD = [
    (RELU, 0.0, [-2.0, -0.5, 0.0, 3.5], [0.0, 0.0, 0.0, 3.5]),
    (LEAKY_RELU, 0.01, [-2.0, -0.5, 0.0, 3.5], [-0.02, -0.005, 0.0, 3.5]),
    (SIGMOID, 0.0, [0.0, 1.0, -1.0, 2.0], [0.5, 0.731058, 0.268941, 0.880797]),
    (TANH, 0.0, [0.0, 1.0, -1.0, 2.0], [0.0, 0.761594, -0.761594, 0.964028]),
    (ELU, 1.0, [-1.0, 0.0, 1.0, 2.0], [-0.632121, 0.0, 1.0, 2.0]),
    (SILU, 0.0, [-1.0, 0.0, 1.0, 2.0], [-0.268941, 0.0, 0.731059, 1.761594]),
    (GELU, 0.0, [-1.0, 0.0, 1.0, 2.0], [-0.158865, 0.0, 0.841135, 1.954598]),
    (SOFTPLUS, 0.0, [-1.0, 0.0, 1.0, 2.0], [0.313262, 0.693147, 1.313262, 2.126928]),
]
REFERENCE_BACKWARD = [
    (RELU, 0.0, [1.0, 2.0, 3.0, 4.0], [-1.0, 0.0, 1.0, 2.0], [0.0, 0.0, 3.0, 4.0]),
    (LEAKY_RELU, 0.01, [1.0, 2.0, 3.0, 4.0], [-1.0, -0.5, 1.0, 2.0], [0.01, 0.02, 3.0, 4.0]),
    (SIGMOID, 0.0, [1.0] * 4, [0.5, 0.731058, 0.268941, 0.880797], [0.25, 0.196612, 0.196612, 0.104994]),
    (TANH, 0.0, [1.0] * 4, [0.0, 0.761594, -0.761594, 0.964028], [1.0, 0.419974, 0.419974, 0.070651]),
    (ELU, 1.0, [1.0] * 4, [-1.0, 0.0, 1.0, 2.0], [0.367879, 1.0, 1.0, 1.0]),
    (SILU, 0.0, [1.0] * 4, [-1.0, 0.0, 1.0, 2.0], [0.072329, 0.5, 0.927671, 1.090784]),
    (GELU, 0.0, [1.0] * 4, [-1.0, 0.0, 1.0, 2.0], [-0.082937, 0.5, 1.082937, 1.086099]),
    (SOFTPLUS, 0.0, [1.0] * 4, [-1.0, 0.0, 1.0, 2.0], [0.268941, 0.5, 0.731059, 0.880797]),
]
