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

// Streaming multiprocessors of the current device, asked once per library (grids and split
// counts are sized by it; no kernel assumes a particular GPU's count).
static inline int sandy_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess)
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms = n > 0 ? n : 1;
    }
    return sms;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// A decode step is a chain of ~70 short kernels, each only a few microseconds long, so what
// a kernel costs is mostly getting started: launch latency and the first trip to memory.
// Launched with the programmatic-serialization attribute, a kernel may start while its
// predecessor in the stream is still running (as soon as every block of the predecessor has
// called pdl_launch_dependents() or exited).  It must then call pdl_wait() before it reads
// anything an earlier kernel wrote or writes anything an earlier kernel may still read;
// pdl_wait() returns when the predecessor has completed and its writes are visible.  What may
// go before pdl_wait() is work on data no kernel writes: index arithmetic and, above all, the
// first loads of the weights.  Both calls do nothing in a kernel launched the ordinary way.
//
// What earlier STEPS wrote may also be read before pdl_wait() -- cache pages of older positions, the
// step's index arrays (a burst's sampler advances them at the end of the step before) -- because a
// step's first kernel (the embedding) calls pdl_launch_dependents() only after its own pdl_wait() has
// returned: no later kernel of the step can start before that, and by then every kernel of the steps
// before has completed (a kernel completes only after its wait, which needs its predecessor complete).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
#include <utility>

// SANDYRT_PDL=0 turns the attribute off (every kernel then waits for its predecessor to end).
static inline bool sandy_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = std::getenv("SANDYRT_PDL");
        enabled = (e && e[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline int sandy_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sandy_pdl_enabled() ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
