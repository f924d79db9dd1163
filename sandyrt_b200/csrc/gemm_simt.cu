// Matrix product on the ordinary 32-bit pipes (FFMA), with bias / activation / residual
// folded into the write-back.
//
//   out[m, n] = act( sum_k a[m, k] * w(k, n) + bias[n] ) + residual[m, n]
//
// This is the kernel of the true 32-bit path: operands are read as they are stored
// (float, or bfloat16 widened exactly), every product and sum is an IEEE float operation,
// no tensor-core or reduced-precision matrix mode is involved.  It also serves bfloat16
// operands whose sizes the tensor-core kernel refuses.  The reference computes the same
// thing with a scalar triple loop (src/core/TensorCalc.cpp:759-770) or one cuBLAS call
// with CUBLAS_COMPUTE_32F (src/device/cuda/CudaMatMulKernels.cu:196-215).
//
// Each output element is the sum over k = 0..K-1 in ascending order, carried by one
// thread, so its value does not depend on M, on the tile it falls in, or on what other
// rows are in the batch.
//
// The weight may be stored [K, N] ("in_out": GPT-2's Conv1D layout, the file's own) or
// [N, K] ("out_in": a Linear weight, or the token table used as the output head).
#include "epilogue.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int THREADS = (BM / TM) * (BN / TN);  // 256

template <typename TA, typename TW, typename TC, bool W_OUT_IN>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TA* __restrict__ a, const TW* __restrict__ w, const TW* __restrict__ bias,
                 const float* residual, TC* out,
                 int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // A tile: BM x BK, threads run along k (contiguous in memory)
#pragma unroll
        for (int i = tid; i < BM * BK; i += THREADS) {
            const int m = i / BK, k = i % BK;
            const int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? to_f32(a[(size_t)gm * lda + gk]) : 0.0f;
        }
        if (W_OUT_IN) {
#pragma unroll
            for (int i = tid; i < BN * BK; i += THREADS) {
                const int n = i / BK, k = i % BK;
                const int gn = n0 + n, gk = k0 + k;
                Ws[k][n] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * ldw + gk]) : 0.0f;
            }
        } else {
#pragma unroll
            for (int i = tid; i < BN * BK; i += THREADS) {
                const int k = i / BN, n = i % BN;
                const int gn = n0 + n, gk = k0 + k;
                Ws[k][n] = (gn < N && gk < K) ? to_f32(w[(size_t)gk * ldw + gn]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) av[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) wv[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += to_f32(bias[gn]);
            v = apply_act(v, act);
            if (residual) v += residual[(size_t)gm * ldr + gn];
            out[(size_t)gm * ldc + gn] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(const void* a, const void* w, const void* bias, const float* residual, void* out,
           int M, int N, int K, int lda, int ldw, int ldr, int ldc, int w_out_in, int act,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (w_out_in)
        gemm_simt_kernel<TA, TW, TC, true><<<grid, THREADS, 0, stream>>>(
            (const TA*)a, (const TW*)w, (const TW*)bias, residual, (TC*)out, M, N, K, lda, ldw, ldr, ldc, act);
    else
        gemm_simt_kernel<TA, TW, TC, false><<<grid, THREADS, 0, stream>>>(
            (const TA*)a, (const TW*)w, (const TW*)bias, residual, (TC*)out, M, N, K, lda, ldw, ldr, ldc, act);
    return sandy_launch_status();
}

}  // namespace

// a: [M, K] (row stride lda) of a_dtype; w: [K, N] or, with w_out_in, [N, K] (row stride
// ldw) of w_dtype; bias: [N] of w_dtype or null; residual: float [M, N] (row stride ldr)
// or null; out: [M, N] (row stride ldc) of out_dtype.  Strides are in elements.
SANDY_API int sandy_gemm_simt(const void* a, const void* w, const void* bias, const float* residual,
                              void* out, int M, int N, int K, int lda, int ldw, int ldr, int ldc,
                              int w_out_in, int act, int a_dtype, int w_dtype, int out_dtype,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
#define CASE(da, dw, dc, TA, TW, TC)                                                              \
    if (a_dtype == da && w_dtype == dw && out_dtype == dc)                                        \
        return launch<TA, TW, TC>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, w_out_in, act, stream)
    CASE(SANDY_F32, SANDY_F32, SANDY_F32, float, float, float);
    CASE(SANDY_BF16, SANDY_BF16, SANDY_BF16, bf16, bf16, bf16);
    CASE(SANDY_BF16, SANDY_BF16, SANDY_F32, bf16, bf16, float);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}
