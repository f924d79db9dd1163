// Epilogue arithmetic shared by the matrix-product kernels: bias, activation, residual.
#pragma once

#include "common.cuh"

enum SandyAct : int { SANDY_ACT_NONE = 0, SANDY_ACT_GELU_TANH = 1, SANDY_ACT_GELU_ERF = 2 };

// gelu_new, in the reference's order of operations (src/ir/BuiltinLowering.cpp:116-140):
//   x2 = u*u; x3 = x2*u; inner = u + 0.044715*x3; t = tanh(0.7978845608028654*inner);
//   (0.5*u) * (1 + t)
__device__ __forceinline__ float gelu_tanh(float u) {
    const float x2 = u * u;
    const float x3 = x2 * u;
    const float inner = u + 0.044715f * x3;
    const float t = tanhf(0.7978845608028654f * inner);
    return (0.5f * u) * (1.0f + t);
}

// Exact gelu: 0.5*u*(1 + erf(u / sqrt(2))).  The reference has no erf op
// (ScalarOp list, src/ir/KernelIR.h:317-337); this follows the formula.
__device__ __forceinline__ float gelu_erf(float u) {
    return 0.5f * u * (1.0f + erff(u * 0.70710678118654752440f));
}

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == SANDY_ACT_GELU_TANH) return gelu_tanh(v);
    if (act == SANDY_ACT_GELU_ERF) return gelu_erf(v);
    return v;
}
