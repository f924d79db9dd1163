// Shared helpers of the sm_100a kernels: storage types, 32-bit conversion, reductions.
//
// Policy (as the reference's kernels do through load_float/store_float,
// src/device/cuda/CudaKernelUtils.cuh:148-154,247-254): a value is converted to float
// when it is read, every sum is carried in float, and the result is rounded to the
// storage type once, when it is written.  bfloat16 rounding is round-to-nearest-even
// (src/core/Tensor.h:43-49).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SANDY_API extern "C" __attribute__((visibility("default")))

// dtype codes that cross the C boundary
enum SandyDType : int { SANDY_F32 = 0, SANDY_BF16 = 1 };

// Error codes returned by the entry points.  Non-negative values are cudaError_t.
enum SandyStatus : int {
    SANDY_OK = 0,
    SANDY_ERR_UNSUPPORTED = -1,   // sizes or dtypes this kernel refuses
    SANDY_ERR_ARGUMENT = -2,      // a null pointer or an impossible size
};

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads.  `scratch` holds 32 floats.  Every thread
// gets the total; the order of the additions is fixed by the thread layout, so the
// result for a row does not depend on what else runs beside it.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

static inline int sandy_launch_status() {
    return (int)cudaGetLastError();
}
