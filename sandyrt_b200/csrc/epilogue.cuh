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

// gelu_new with tanh(y) = 1 - 2 / (exp(2y) + 1) on the fast exponential and division: a third
// of tanhf's instructions, absolute error below 1e-6 (exp(2y) overflows to inf for large y,
// giving exactly 1; underflows to 0 for very negative y, giving exactly -1).  For write-backs
// that round to bfloat16 or sit in a tensor-core kernel's critical path; the 32-bit path keeps
// tanhf.
__device__ __forceinline__ float gelu_tanh_fast(float u) {
    const float x2 = u * u;
    const float inner = u + 0.044715f * (x2 * u);
    const float e = __expf(1.5957691216057308f * inner);        // exp(2 * 0.79788456 * inner)
    const float t = 1.0f - __fdividef(2.0f, e + 1.0f);
    return (0.5f * u) * (1.0f + t);
}

__device__ __forceinline__ float apply_act_fast(float v, int act) {
    if (act == SANDY_ACT_GELU_TANH) return gelu_tanh_fast(v);
    if (act == SANDY_ACT_GELU_ERF) return gelu_erf(v);
    return v;
}

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == SANDY_ACT_GELU_TANH) return gelu_tanh(v);
    if (act == SANDY_ACT_GELU_ERF) return gelu_erf(v);
    return v;
}
