// bfloat16 matrix product for a few rows (a decode step: 1 to 64 tokens), shaped for
// reading the weight once at memory speed rather than for arithmetic.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) + residual[m, n]
//
// a: [M, K] bfloat16 (M <= 64), w: [N, K] bfloat16 (K contiguous), as in gemm_tc.cu.  With so
// few rows the product is bound by streaming w from HBM, and a 128-row tensor-memory tile
// would leave most SMs idle; here every block owns just 8 output columns and its eight warps
// split K between them, so a 768 x 768 weight is read by 96 blocks of eight warps at once.  The arithmetic
// runs on the warp-level tensor-core instruction (mma.sync m16n8k16: 16 tokens x 8 columns),
// which is far more than this bandwidth-bound product needs.
//
// Each lane reads the weight and the activations in 16-byte pieces straight from global
// memory (the activations are small and stay in L1/L2).  The 8 consecutive k of a 16-byte
// piece are fed to two consecutive mma steps; since a dot product does not care in which
// order its terms are paired, the same assignment of k to fragment slots is used for both
// operands and no shuffle through shared memory is needed.
//
// The warps' partial sums are added in a fixed order (warp 0, 1, ...), so a token's result
// does not depend on what else is in the batch beyond which 16-row group it falls in (rows of
// other tokens never enter its dot products).
#include "epilogue.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int COLS = 8;          // output columns per block
constexpr int KCHUNK = 32;       // k covered by one 16-byte load of every lane
constexpr int UNROLL = 4;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// weights are read once: do not let them push the activations out of L1
__device__ __forceinline__ uint4 ldg16_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// MT: number of 16-row token tiles (M <= 16 * MT)
template <int MT, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, const bf16* __restrict__ bias,
                   const float* residual, TC* out, int M, int N, int K, int lda,
                   int ldw, int ldr, int ldc, int act) {
    __shared__ float partial[WARPS][MT * 16][COLS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * COLS;
    // this warp's contiguous slice of K, in whole chunks
    const int chunks = (K + KCHUNK - 1) / KCHUNK;
    const int per_warp = (chunks + WARPS - 1) / WARPS;
    const int c_begin = warp * per_warp, c_end = min(chunks, c_begin + per_warp);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    const int n = n0 + g;                       // the weight row this lane reads (as the B operand)
    const bool n_ok = n < N;
    const bf16* wrow = w + (size_t)(n_ok ? n : 0) * ldw;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // The weight pieces of the next round are requested before the current round is
    // multiplied, so a warp always has two rounds of loads in flight.
    uint4 wn[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
        const int k = (c_begin + u) * KCHUNK + t * 8;
        wn[u] = (n_ok && c_begin + u < c_end && k < K) ? ldg16_stream(wrow + k) : zero;
    }
    for (int c0 = c_begin; c0 < c_end; c0 += UNROLL) {
        uint4 wv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            wv[u] = wn[u];
            const int cn = c0 + UNROLL + u;
            const int k = cn * KCHUNK + t * 8;
            wn[u] = (n_ok && cn < c_end && k < K) ? ldg16_stream(wrow + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int k = (c0 + u) * KCHUNK + t * 8;
            const bool k_ok = c0 + u < c_end && k < K;
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const int r0 = mt * 16 + g, r1 = r0 + 8;
                const uint4 x0 = (k_ok && r0 < M) ? ldg16(a + (size_t)r0 * lda + k) : zero;
                const uint4 x1 = (k_ok && r1 < M) ? ldg16(a + (size_t)r1 * lda + k) : zero;
                // pieces .x .y feed the first mma step (slots 2t,2t+1 and 2t+8,2t+9), .z .w the second
                mma_bf16(acc[mt], x0.x, x1.x, x0.y, x1.y, wv[u].x, wv[u].y);
                mma_bf16(acc[mt], x0.z, x1.z, x0.w, x1.w, wv[u].z, wv[u].w);
            }
        }
    }
    // C fragment: c0,c1 = (token g, columns 2t, 2t+1); c2,c3 = (token g+8, same columns)
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        partial[warp][mt * 16 + g][2 * t] = acc[mt][0];
        partial[warp][mt * 16 + g][2 * t + 1] = acc[mt][1];
        partial[warp][mt * 16 + g + 8][2 * t] = acc[mt][2];
        partial[warp][mt * 16 + g + 8][2 * t + 1] = acc[mt][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < MT * 16 * COLS; idx += WARPS * 32) {
        const int m = idx / COLS, j = idx % COLS;
        const int col = n0 + j;
        if (m >= M || col >= N) continue;
        float v = partial[0][m][j];
#pragma unroll
        for (int wi = 1; wi < WARPS; wi++) v += partial[wi][m][j];
        if (bias) v += __bfloat162float(bias[col]);
        v = apply_act(v, act);
        if (residual) v += residual[(size_t)m * ldr + col];
        out[(size_t)m * ldc + col] = from_f32<TC>(v);
    }
}

template <int MT>
int launch(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
           int lda, int ldw, int ldr, int ldc, int act, int out_dtype, cudaStream_t stream) {
    const unsigned blocks = (unsigned)((N + COLS - 1) / COLS);
    if (out_dtype == SANDY_F32)
        gemm_skinny_kernel<MT, float><<<blocks, WARPS * 32, 0, stream>>>(
            (const bf16*)a, (const bf16*)w, (const bf16*)bias, residual, (float*)out, M, N, K, lda, ldw, ldr, ldc, act);
    else
        gemm_skinny_kernel<MT, bf16><<<blocks, WARPS * 32, 0, stream>>>(
            (const bf16*)a, (const bf16*)w, (const bf16*)bias, residual, (bf16*)out, M, N, K, lda, ldw, ldr, ldc, act);
    return sandy_launch_status();
}

}  // namespace

// Arguments as sandy_gemm_tc; M <= 64; K, lda, ldw multiples of 8; a and w 16-byte aligned.
SANDY_API int sandy_gemm_skinny(const void* a, const void* w, const void* bias, const float* residual, void* out,
                                int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype,
                                cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
    if (M > 64 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    if (M <= 16) return launch<1>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, stream);
    if (M <= 32) return launch<2>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, stream);
    return launch<4>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, stream);
}
