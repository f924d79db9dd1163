// LayerNorm over the last dimension, statistics in 32-bit.
//
// Per row, as the reference computes it (src/core/TensorCalc.cpp:2048-2072; its CUDA
// twin src/device/cuda/CudaNormKernels.cu:172-206):
//   mean = sum(x) / E;  var = sum((x - mean)^2) / E   (biased, two passes)
//   y = (x - mean) * (1 / sqrt(var + eps)) * gamma + beta
// The reference reads the row from global memory three times; here the row is staged in
// shared memory once as floats and all three passes read that copy.
//
// `rows` (optional) selects which input rows are normalised: output row r is the norm of
// input row rows[r].  The engine uses it to run the final norm only at the positions
// whose logits were asked for.
#include "common.cuh"

template <typename TI, typename TW, typename TO>
__global__ void layernorm_kernel(const TI* __restrict__ x, const TW* __restrict__ gamma,
                                 const TW* __restrict__ beta, TO* __restrict__ out,
                                 const int* __restrict__ rows, int width, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    const TI* xr = x + src * width;
    float s = 0.0f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = to_f32(xr[e]);
        row[e] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)width;
    float q = 0.0f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float c = row[e] - mean;
        q += c * c;
    }
    const float var = block_sum(q, scratch) / (float)width;
    const float inv = 1.0f / sqrtf(var + eps);
    TO* orow = out + (size_t)r * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = (row[e] - mean) * inv * to_f32(gamma[e]);
        if (beta) v += to_f32(beta[e]);
        orow[e] = from_f32<TO>(v);
    }
}

// x: [*, width] of in_dtype; gamma, beta: [width] of w_dtype (beta may be null);
// out: [n_rows, width] of out_dtype; rows: int32[n_rows] or null.
SANDY_API int sandy_layernorm(const void* x, const void* gamma, const void* beta, void* out,
                              const int* rows, int n_rows, int width, float eps,
                              int in_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
    if (n_rows == 0) return SANDY_OK;
    if (!x || !gamma || !out || width <= 0) return SANDY_ERR_ARGUMENT;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return SANDY_ERR_UNSUPPORTED;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define LAUNCH(TI, TW, TO)                                                                      \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(layernorm_kernel<TI, TW, TO>,                                  \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        return sandy_launch(layernorm_kernel<TI, TW, TO>, dim3(n_rows), dim3(threads), smem, stream, \
                            (const TI*)x, (const TW*)gamma, (const TW*)beta, (TO*)out, rows, width, eps); \
    } while (0)
    if (in_dtype == SANDY_F32 && w_dtype == SANDY_F32 && out_dtype == SANDY_F32) LAUNCH(float, float, float);
    if (in_dtype == SANDY_F32 && w_dtype == SANDY_BF16 && out_dtype == SANDY_BF16) LAUNCH(float, bf16, bf16);
    if (in_dtype == SANDY_BF16 && w_dtype == SANDY_BF16 && out_dtype == SANDY_BF16) LAUNCH(bf16, bf16, bf16);
    if (in_dtype == SANDY_F32 && w_dtype == SANDY_F32 && out_dtype == SANDY_BF16) LAUNCH(float, float, bf16);
#undef LAUNCH
    return SANDY_ERR_UNSUPPORTED;
}
