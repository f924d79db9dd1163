// LayerNorm over the last dimension, statistics in 32-bit.
//
// Per row, as the reference computes it (src/core/TensorCalc.cpp:2048-2072; its CUDA
// twin src/device/cuda/CudaNormKernels.cu:172-206):
//   mean = sum(x) / E;  var = sum((x - mean)^2) / E   (biased, two passes)
//   y = (x - mean) * (1 / sqrt(var + eps)) * gamma + beta
// The reference gives every row a block of 256 threads and reads the row from global memory
// three times.  Here a row belongs to ONE WARP and lives in its registers between the passes
// (rows up to 4096 wide; wider rows take the block-per-row kernel that stages the row in
// shared memory), so the two reductions are warp shuffles and a block handles eight rows.
// Where the width is a multiple of 4 and the rows are aligned, a lane moves its four
// consecutive elements with one 16-byte (float) or 8-byte (bfloat16) access.
//
// `rows` (optional) selects which input rows are normalised: output row r is the norm of
// input row rows[r].  The engine uses it to run the final norm only at the positions
// whose logits were asked for.
#include "common.cuh"

namespace {

constexpr int ROWS_PER_BLOCK = 8;

// Four consecutive elements with one access.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

// A lane holds 4 consecutive elements per round; NV: rounds (width <= 32*4*NV).  vec: the width is
// a multiple of 4 and every pointer is aligned for 4-element accesses.
template <typename TI, typename TW, typename TO, int NV>
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
layernorm_warp_kernel(const TI* __restrict__ x, const TW* __restrict__ gamma, const TW* __restrict__ beta,
                      TO* __restrict__ out, const int* __restrict__ rows, int n_rows, int width, float eps, int vec) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + warp;
    // Gain and offset are weights, which no kernel writes: they are asked for before the wait for
    // the kernel that produces x, not after the two reductions: into registers for rows up to 1,024 wide,
    // into shared memory (once for the block's eight rows) beyond.  (Read from global memory where they are
    // used, a row of 1,600 cost 16 trips to memory, one after the other: 10 us a launch.)
    constexpr bool EARLY = NV <= 8;
    extern __shared__ __align__(16) uint8_t params_raw[];      // !EARLY && vec: gain [width], offset [width]
    TW* g_sm = reinterpret_cast<TW*>(params_raw);
    TW* b_sm = g_sm + width;
    if (!EARLY && vec) {
        for (int e = threadIdx.x * 4; e < width; e += ROWS_PER_BLOCK * 32 * 4) {
            float t4[4];
            load4(gamma + e, t4);
            store4(g_sm + e, t4);
            if (beta) {
                load4(beta + e, t4);
                store4(b_sm + e, t4);
            }
        }
    }
    float g[EARLY ? NV : 1][4], b[EARLY ? NV : 1][4];
    if (EARLY && vec && r < n_rows) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int e = (i * 32 + lane) * 4;
            g[i][0] = g[i][1] = g[i][2] = g[i][3] = 0.0f;
            b[i][0] = b[i][1] = b[i][2] = b[i][3] = 0.0f;
            if (e < width) {
                load4(gamma + e, g[i]);
                if (beta) load4(beta + e, b[i]);
            }
        }
    }
    pdl_wait();
    if (!EARLY && vec) __syncthreads();      // gain and offset are in shared memory (every warp comes by here)
    if (r >= n_rows) return;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    const TI* xr = x + src * width;
    float v[NV][4];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = (i * 32 + lane) * 4;
        if (vec) {
            if (e < width) load4(xr + e, v[i]);
            else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.0f;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) v[i][j] = (e + j < width) ? to_f32(xr[e + j]) : 0.0f;
        }
        s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
    }
    const float mean = warp_sum(s) / (float)width;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = (i * 32 + lane) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float c = v[i][j] - mean;
            if (e + j < width) q += c * c;
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(q) / (float)width + eps);
    TO* orow = out + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int e = (i * 32 + lane) * 4;
        if (vec) {
            if (e < width) {
                float gg[4], bb[4] = {0.0f, 0.0f, 0.0f, 0.0f}, y[4];
                if (EARLY) {
#pragma unroll
                    for (int j = 0; j < 4; j++) { gg[j] = g[i][j]; bb[j] = b[i][j]; }
                } else {
                    load4(g_sm + e, gg);
                    if (beta) load4(b_sm + e, bb);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) y[j] = (v[i][j] - mean) * inv * gg[j] + bb[j];
                store4(orow + e, y);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (e + j < width) {
                    float y = (v[i][j] - mean) * inv * to_f32(gamma[e + j]);
                    if (beta) y += to_f32(beta[e + j]);
                    orow[e + j] = from_f32<TO>(y);
                }
            }
        }
    }
}

template <typename TI, typename TW, typename TO>
__global__ void layernorm_block_kernel(const TI* __restrict__ x, const TW* __restrict__ gamma,
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

template <typename TI, typename TW, typename TO>
int launch(const void* x, const void* gamma, const void* beta, void* out, const int* rows, int n_rows, int width,
           float eps, cudaStream_t stream) {
    const dim3 grid((n_rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK), block(ROWS_PER_BLOCK * 32);
    auto aligned = [](const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0; };
    const int vec = width % 4 == 0 && aligned(x, 4 * sizeof(TI)) && aligned(gamma, 4 * sizeof(TW)) &&
                    (!beta || aligned(beta, 4 * sizeof(TW))) && aligned(out, 4 * sizeof(TO));
    // rows wider than 1,024: gain and offset wait in shared memory (at most 2 x 4,096 floats)
#define WARP_CASE(NV)                                                                                          \
    if (width <= 128 * NV)                                                                                     \
        return sandy_launch(layernorm_warp_kernel<TI, TW, TO, NV>, grid, block,                                \
                            (NV > 8 && vec) ? 2 * (size_t)width * sizeof(TW) : 0, stream, (const TI*)x,         \
                            (const TW*)gamma, (const TW*)beta, (TO*)out, rows, n_rows, width, eps, vec)
    WARP_CASE(1); WARP_CASE(2); WARP_CASE(4); WARP_CASE(6); WARP_CASE(8); WARP_CASE(12); WARP_CASE(16);
    WARP_CASE(32);
#undef WARP_CASE
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return SANDY_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(layernorm_block_kernel<TI, TW, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return sandy_launch(layernorm_block_kernel<TI, TW, TO>, dim3(n_rows), dim3(512), smem, stream, (const TI*)x,
                        (const TW*)gamma, (const TW*)beta, (TO*)out, rows, width, eps);
}

}  // namespace

// x: [*, width] of in_dtype; gamma, beta: [width] of w_dtype (beta may be null);
// out: [n_rows, width] of out_dtype; rows: int32[n_rows] or null.
SANDY_API int sandy_layernorm(const void* x, const void* gamma, const void* beta, void* out,
                              const int* rows, int n_rows, int width, float eps,
                              int in_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
    if (n_rows == 0) return SANDY_OK;
    if (!x || !gamma || !out || width <= 0) return SANDY_ERR_ARGUMENT;
#define CASE(DI, DW, DO, TI, TW, TO)                                                                 \
    if (in_dtype == DI && w_dtype == DW && out_dtype == DO)                                          \
        return launch<TI, TW, TO>(x, gamma, beta, out, rows, n_rows, width, eps, stream)
    CASE(SANDY_F32, SANDY_F32, SANDY_F32, float, float, float);
    CASE(SANDY_F32, SANDY_BF16, SANDY_BF16, float, bf16, bf16);
    CASE(SANDY_BF16, SANDY_BF16, SANDY_BF16, bf16, bf16, bf16);
    CASE(SANDY_F32, SANDY_F32, SANDY_BF16, float, float, bf16);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}
