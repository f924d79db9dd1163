// bfloat16 matrix product for a few rows (a decode step: 1 to 64 tokens), shaped for
// reading the weight once at memory speed rather than for arithmetic, with the work that
// surrounds it in a decoder layer folded in:
//
//   a      = LayerNorm(x) (optional: the norm before the product runs inside this kernel)
//   out    = act( a @ w^T + bias ) + residual
//   cache  <- the key and value columns of out, written straight into the request's pages
//             (optional: the product is the fused q/k/v projection)
//
// a: [M, K] bfloat16 (M <= 64), or x: [M, K] float with gamma/beta when the norm is fused;
// w: [N, K] bfloat16 (K contiguous), as in gemm_tc.cu.  With so few rows the product is bound
// by streaming w from HBM, and a 128-row tensor-memory tile would leave most SMs idle; here
// every block owns just 8 output columns and its eight warps split K between them, so a
// 768 x 768 weight is read by 96 blocks of eight warps at once.  The arithmetic runs on the
// warp-level tensor-core instruction (mma.sync m16n8k16: 16 tokens x 8 columns), which is far
// more than this bandwidth-bound product needs.
//
// Three forms live in this file: the one described here (8 columns a block; every product of up to 16
// rows, and the narrow products beyond), one with 16 columns a block for 17 to 64 rows and 1,536 columns
// and more, and one whose warps walk the column groups of a vocabulary projection (both further down).
//
// Each lane reads the weight in 16-byte pieces straight from global memory.  The 8
// consecutive k of a piece are fed to two consecutive mma steps; since a dot product does not
// care in which order its terms are paired, the same assignment of k to fragment slots is
// used for both operands and no shuffle through shared memory is needed.  The first round of
// weight loads is issued before anything else, so it overlaps the norm.
//
// Fused norm (src/core/TensorCalc.cpp:2048-2072 of the reference: mean, biased variance in
// two passes, 1/sqrt(var + eps), gain and offset): every block normalises the M rows itself
// (warp per row, the row held in registers, statistics in float) into shared memory as
// bfloat16, the same rounding point as the stand-alone norm kernel.  This trades a launch for
// re-reading x (M x K floats, from L2) in every block, which pays while M is small.
//
// The warps' partial sums are added in a fixed order (warp 0, 1, ...), so a token's result
// does not depend on what else is in the batch (rows of other tokens never enter its dot
// products).
#include "epilogue.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int COLS = 8;          // output columns per block
constexpr int KCHUNK = 32;       // k covered by one 16-byte load of every lane
constexpr int XPAD = 32;         // elements of padding per shared-memory row (64 bytes: conflict-free 16-byte reads)
constexpr int MAX_ROW_VEC = 16;  // most float4 per lane a fused-norm row may take: K <= 2048

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
// weights are read once: do not let them push the activations out of L1
__device__ __forceinline__ uint4 ldg16_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Where the key/value columns of a fused q/k/v product go (see attention.cu for the layout).
struct KVWrite {
    bf16* k_cache;
    bf16* v_cache;
    long long page_stride;
    const int* block_table;
    const int* token_seq;
    const int* positions;
    int max_blocks, q_cols, kv_cols, head_dim, page_size, num_pages;
    int* status;
};

struct NormArgs {
    const float* x;          // [M, K] float, row stride ldx
    const bf16* gamma;       // [K]
    const bf16* beta;        // [K] or null
    int ldx;
    float eps;
};

// MT: number of 16-row token tiles (M <= 16 * MT).  UNROLL: 16-byte weight pieces a lane keeps in
// flight per round (chosen so that a warp's whole K slice is one or two rounds).  RV: float4 per
// lane that hold a row during the fused norm (K <= 128 * RV); sized to K so that registers,
// and with them the number of resident blocks, are not wasted on short rows.
// Blocks an SM: three for the one-tile form with short K slices; two for the multi-tile form with
// short K slices (left alone it takes 216 registers, one block an SM, and a product of 288 column
// groups runs in two waves); one otherwise (long K: few column groups, a block an SM at most).
template <int MT, typename TC, bool FUSE_LN, int UNROLL, int RV>
__global__ void __launch_bounds__(WARPS * 32, (UNROLL == 4 && RV <= 8 && MT == 1) ? 3 : ((MT > 1 && !FUSE_LN && UNROLL == 4) ? 2 : 1))
gemm_skinny_kernel(const bf16* __restrict__ a, NormArgs norm, const bf16* __restrict__ w,
                   const bf16* __restrict__ bias, const float* residual, TC* out, int M, int N, int K, int lda,
                   int ldw, int ldr, int ldc, int act, KVWrite kv) {
    __shared__ float partial[WARPS][MT * 16][COLS + 1];
    extern __shared__ __align__(16) uint8_t xs_raw[];
    bf16* xs = reinterpret_cast<bf16*>(xs_raw);          // [MT*16][K + XPAD], fused norm only
    const int xs_ld = K + XPAD;

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
    // multiplied, so a warp always has two rounds of loads in flight; the first round goes out
    // before the norm.
    uint4 wn[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
        const int k = (c_begin + u) * KCHUNK + t * 8;
        wn[u] = (n_ok && c_begin + u < c_end && k < K) ? ldg16_stream(wrow + k) : zero;
    }

    // The norm's gain and offset are weights too: they are copied into shared memory now, so that
    // they are not a trip to memory between a row's statistics and its normalised values.
    bf16* g_sm = xs + (size_t)MT * 16 * xs_ld;           // [K], then the offset [K]
    bf16* b_sm = g_sm + K;
    if (FUSE_LN) {
        for (int k = threadIdx.x * 8; k < K; k += WARPS * 32 * 8) {
            cp_async16(g_sm + k, norm.gamma + k);
            if (norm.beta) cp_async16(b_sm + k, norm.beta + k);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // The write-back at the end gives output (m, j) to thread m * COLS + j (further rows of a
    // multi-tile product to the same thread, 32 rows on): the bias of its column is asked for now ...
    const int my_col = n0 + (int)(threadIdx.x % COLS);
    const float my_bias = (bias && my_col < N) ? __bfloat162float(bias[my_col]) : 0.0f;

    // The page this thread's key/value element goes to: two dependent loads, needed only in the
    // write-back.  The index arrays are the step's input (written before the step, or by the sampler of
    // the step before in a burst; complete by now, see common.cuh), so the loads go out before the wait:
    // behind it they were a trip to memory between the wait and the norm.
    int kv_page = -1, kv_pos = 0;
    if (kv.k_cache && MT == 1 && threadIdx.x < 16 * COLS) {
        const int m = threadIdx.x / COLS;
        if (m < M && n0 + (int)(threadIdx.x % COLS) >= kv.q_cols) {
            kv_pos = kv.positions[m];
            const int b = kv_pos / kv.page_size;
            kv_page = (kv_pos >= 0 && b < kv.max_blocks) ? kv.block_table[(size_t)kv.token_seq[m] * kv.max_blocks + b] : -1;
        }
    }

    // Everything above touched only weights, which no kernel writes.  From here on the
    // activations are read: the kernels before this one must have finished.
    pdl_launch_dependents();
    pdl_wait();

    // ... and, for the one-tile product, the residual value it will add: neither is then a trip to
    // memory behind the sums.  (out may be the residual itself: each element is read and written by
    // one thread only.)
    float my_res = 0.0f;
    if (MT == 1 && residual && threadIdx.x < 16 * COLS && (int)(threadIdx.x / COLS) < M && my_col < N)
        my_res = residual[(size_t)(threadIdx.x / COLS) * ldr + my_col];


    if (FUSE_LN) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();            // gain and offset are in shared memory
        // warp per row; the row lives in registers between the passes
        for (int r = warp; r < MT * 16; r += WARPS) {
            bf16* dst = xs + (size_t)r * xs_ld;
            if (r >= M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = zero;
                continue;
            }
            const float* xr = norm.x + (size_t)r * norm.ldx;
            float4 v[RV];
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < RV; i++) {
                const int k = (i * 32 + lane) * 4;
                v[i] = k < K ? *reinterpret_cast<const float4*>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
            const float mean = warp_sum(s) / (float)K;
            float q = 0.0f;
#pragma unroll
            for (int i = 0; i < RV; i++) {
                const int k = (i * 32 + lane) * 4;
                if (k < K) {
                    const float cx = v[i].x - mean, cy = v[i].y - mean, cz = v[i].z - mean, cw = v[i].w - mean;
                    q += (cx * cx + cy * cy) + (cz * cz + cw * cw);
                }
            }
            const float inv = 1.0f / sqrtf(warp_sum(q) / (float)K + norm.eps);
#pragma unroll
            for (int i = 0; i < RV; i++) {
                const int k = (i * 32 + lane) * 4;
                if (k < K) {
                    const uint2 gm = *reinterpret_cast<const uint2*>(g_sm + k);
                    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gm);
                    const float2 g01 = __bfloat1622float2(gh[0]), g23 = __bfloat1622float2(gh[1]);
                    float y0 = (v[i].x - mean) * inv * g01.x, y1 = (v[i].y - mean) * inv * g01.y;
                    float y2 = (v[i].z - mean) * inv * g23.x, y3 = (v[i].w - mean) * inv * g23.y;
                    if (norm.beta) {
                        const uint2 bm = *reinterpret_cast<const uint2*>(b_sm + k);
                        const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bm);
                        const float2 b01 = __bfloat1622float2(bh[0]), b23 = __bfloat1622float2(bh[1]);
                        y0 += b01.x; y1 += b01.y; y2 += b23.x; y3 += b23.y;
                    }
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(y0, y1), p1 = __floats2bfloat162_rn(y2, y3);
                    uint2 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&p0);
                    pk.y = *reinterpret_cast<uint32_t*>(&p1);
                    *reinterpret_cast<uint2*>(dst + k) = pk;
                }
            }
        }
        __syncthreads();
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
                uint4 x0, x1;
                if (FUSE_LN) {
                    x0 = k_ok ? *reinterpret_cast<const uint4*>(xs + (size_t)r0 * xs_ld + k) : zero;
                    x1 = k_ok ? *reinterpret_cast<const uint4*>(xs + (size_t)r1 * xs_ld + k) : zero;
                } else {
                    x0 = (k_ok && r0 < M) ? ldg16(a + (size_t)r0 * lda + k) : zero;
                    x1 = (k_ok && r1 < M) ? ldg16(a + (size_t)r1 * lda + k) : zero;
                }
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
        v += my_bias;
        v = apply_act(v, act);
        if (residual) v += MT == 1 ? my_res : residual[(size_t)m * ldr + col];
        out[(size_t)m * ldc + col] = from_f32<TC>(v);
        if (kv.k_cache && col >= kv.q_cols) {
            // a key or value element: straight into the request's page
            const int c = col - kv.q_cols;
            const bool is_v = c >= kv.kv_cols;
            const int c2 = is_v ? c - kv.kv_cols : c;
            const int head = c2 / kv.head_dim, d = c2 % kv.head_dim;
            int pos = kv_pos, page = kv_page;
            if (MT != 1) {
                pos = kv.positions[m];
                const int b = pos / kv.page_size;
                page = (pos >= 0 && b < kv.max_blocks) ? kv.block_table[(size_t)kv.token_seq[m] * kv.max_blocks + b] : -1;
            }
            if (page < 0 || page >= kv.num_pages) {
                if (kv.status) atomicOr(kv.status, 8);
            } else {
                const size_t dst = (size_t)page * kv.page_stride +
                                   ((size_t)head * kv.page_size + (pos % kv.page_size)) * kv.head_dim + d;
                (is_v ? kv.v_cache : kv.k_cache)[dst] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int MT, bool FUSE_LN, int UNROLL, int RV>
int launch2(const void* a, const NormArgs& norm, const void* w, const void* bias, const float* residual, void* out,
            int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype, const KVWrite& kv,
            cudaStream_t stream) {
    const unsigned blocks = (unsigned)((N + COLS - 1) / COLS);
    const size_t smem = FUSE_LN ? ((size_t)MT * 16 * (K + XPAD) + 2 * (size_t)K) * sizeof(bf16) : 0;   // rows, gain, offset
    if (out_dtype == SANDY_F32) {
        auto kern = gemm_skinny_kernel<MT, float, FUSE_LN, UNROLL, RV>;
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return sandy_launch(kern, dim3(blocks), dim3(WARPS * 32), smem, stream, (const bf16*)a, norm, (const bf16*)w,
                            (const bf16*)bias, residual, (float*)out, M, N, K, lda, ldw, ldr, ldc, act, kv);
    } else {
        auto kern = gemm_skinny_kernel<MT, bf16, FUSE_LN, UNROLL, RV>;
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return sandy_launch(kern, dim3(blocks), dim3(WARPS * 32), smem, stream, (const bf16*)a, norm, (const bf16*)w,
                            (const bf16*)bias, residual, (bf16*)out, M, N, K, lda, ldw, ldr, ldc, act, kv);
    }
}

template <int MT, bool FUSE_LN, int RV>
int launch1(const void* a, const NormArgs& norm, const void* w, const void* bias, const float* residual, void* out,
            int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype, const KVWrite& kv,
            cudaStream_t stream) {
    // 16-byte pieces of one warp's K slice
    const int per_warp = ((K + KCHUNK - 1) / KCHUNK + WARPS - 1) / WARPS;
    // More blocks than SMs: what counts is how many blocks an SM holds, and the short rounds' 80 registers
    // allow three where the long rounds' 166 to 255 allow one (an 8 x 4800 x 1600 product: 13.7 us with one
    // round of eight pieces, 7.7 with two rounds of four; GPT-2 xl decode steps of 1 / 8 requests 2.80 / 3.11 ->
    // 1.89 / 2.23 ms).
    const bool crowded = MT == 1 && (N + COLS - 1) / COLS > sandy_sm_count();
    if (per_warp <= 4 || crowded)
        return launch2<MT, FUSE_LN, 4, RV>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    if (per_warp <= 8 || MT > 1)
        return launch2<MT, FUSE_LN, 8, RV>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    return launch2<MT, FUSE_LN, 16, RV>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
}

template <int MT, bool FUSE_LN>
int launch(const void* a, const NormArgs& norm, const void* w, const void* bias, const float* residual, void* out,
           int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype, const KVWrite& kv,
           cudaStream_t stream) {
    if (!FUSE_LN || K <= 512)
        return launch1<MT, FUSE_LN, 4>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    if (K <= 1024)
        return launch1<MT, FUSE_LN, 8>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    return launch1<MT, FUSE_LN, 16>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
}

// ---- 17 to 64 rows and many columns: sixteen columns a block ------------------------------------
// With more than one tile of rows the kernel above is bound by what it reads beside the weight: every
// block fetches all M rows of the activations (64 rows x 768: 98 KB from L2, against 12 KB of weight
// for its 8 columns), and with four row tiles it needs 216 registers, one block an SM, so that the 288
// blocks of a 2,304-column product run in two rounds.  Here a block owns 16 columns (two column
// tiles of the instruction): every activation fragment feeds four products instead of two, half as
// many blocks fetch the rows, and with two 16-byte weight pieces a lane in flight per column tile the
// kernel stays under 128 registers, two blocks an SM.  The sums are formed exactly as above (a warp's
// k slice in ascending order, then the warps in order), so the two kernels give the same bits.
// (Copying each warp's k slice of the rows into shared memory first, one trip for all of them, was
// tried and is slower: decode steps of 17 / 64 requests 0.399 / 0.735 ms against 0.359 / 0.655; the
// copies stand between the wait for the kernel before and the first product, and 106 KB of shared
// memory a block leave no room for the next kernel's blocks to start early.)
constexpr int COLS2 = 16;

template <int MT, typename TC>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_skinny_wide_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, const bf16* __restrict__ bias,
                        const float* residual, TC* out, int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act,
                        KVWrite kv) {
    constexpr int UNROLL = 2;
    __shared__ float partial[WARPS][MT * 16][COLS2 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * COLS2;
    const int chunks = (K + KCHUNK - 1) / KCHUNK;
    const int per_warp = (chunks + WARPS - 1) / WARPS;
    const int c_begin = warp * per_warp, c_end = min(chunks, c_begin + per_warp);

    float acc[MT][2][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][h][j] = 0.0f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bf16* wrow[2];
    bool n_ok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int n = n0 + 8 * h + g;               // the weight row this lane reads for column tile h
        n_ok[h] = n < N;
        wrow[h] = w + (size_t)(n_ok[h] ? n : 0) * ldw;
    }
    uint4 wn[2][UNROLL];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int k = (c_begin + u) * KCHUNK + t * 8;
            wn[h][u] = (n_ok[h] && c_begin + u < c_end && k < K) ? ldg16_stream(wrow[h] + k) : zero;
        }
    // thread i writes outputs i, i + 256, ...: always column i % 16 of the block, rows i / 16 + 16 j
    const int my_col = n0 + (int)(threadIdx.x % COLS2);
    const float my_bias = (bias && my_col < N) ? __bfloat162float(bias[my_col]) : 0.0f;
    // The pages its key/value elements go to: two dependent loads a row, asked for now (the index arrays are
    // the step's input, complete by now) and not in the write-back, where they were MT pairs of trips to
    // memory one after the other (ncu: the q/k/v product of 64 rows 14.2 us against 11.2 for the wider
    // up-projection).
    int kv_pos[MT], kv_page[MT];
#pragma unroll
    for (int j = 0; j < MT; j++) {
        kv_pos[j] = 0;
        kv_page[j] = -1;
        const int m = (int)(threadIdx.x / COLS2) + 16 * j;
        if (kv.k_cache && m < M && my_col >= kv.q_cols && my_col < N) {
            kv_pos[j] = kv.positions[m];
            const int b = kv_pos[j] / kv.page_size;
            kv_page[j] = (kv_pos[j] >= 0 && b < kv.max_blocks) ? kv.block_table[(size_t)kv.token_seq[m] * kv.max_blocks + b] : -1;
        }
    }

    pdl_launch_dependents();
    pdl_wait();

    for (int c0 = c_begin; c0 < c_end; c0 += UNROLL) {
        uint4 wv[2][UNROLL];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                wv[h][u] = wn[h][u];
                const int cn = c0 + UNROLL + u;
                const int k = cn * KCHUNK + t * 8;
                wn[h][u] = (n_ok[h] && cn < c_end && k < K) ? ldg16_stream(wrow[h] + k) : zero;
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
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    mma_bf16(acc[mt][h], x0.x, x1.x, x0.y, x1.y, wv[h][u].x, wv[h][u].y);
                    mma_bf16(acc[mt][h], x0.z, x1.z, x0.w, x1.w, wv[h][u].z, wv[h][u].w);
                }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            partial[warp][mt * 16 + g][8 * h + 2 * t] = acc[mt][h][0];
            partial[warp][mt * 16 + g][8 * h + 2 * t + 1] = acc[mt][h][1];
            partial[warp][mt * 16 + g + 8][8 * h + 2 * t] = acc[mt][h][2];
            partial[warp][mt * 16 + g + 8][8 * h + 2 * t + 1] = acc[mt][h][3];
        }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < MT; it++) {
        const int m = (int)(threadIdx.x / COLS2) + 16 * it, j = (int)(threadIdx.x % COLS2);
        const int col = n0 + j;
        if (m >= M || col >= N) continue;
        float v = partial[0][m][j];
#pragma unroll
        for (int wi = 1; wi < WARPS; wi++) v += partial[wi][m][j];
        v += my_bias;
        v = apply_act(v, act);
        if (residual) v += residual[(size_t)m * ldr + col];
        out[(size_t)m * ldc + col] = from_f32<TC>(v);
        if (kv.k_cache && col >= kv.q_cols) {
            // a key or value element: straight into the request's page
            const int c = col - kv.q_cols;
            const bool is_v = c >= kv.kv_cols;
            const int c2 = is_v ? c - kv.kv_cols : c;
            const int head = c2 / kv.head_dim, d = c2 % kv.head_dim;
            const int pos = kv_pos[it], page = kv_page[it];
            if (page < 0 || page >= kv.num_pages) {
                if (kv.status) atomicOr(kv.status, 8);
            } else {
                const size_t dst = (size_t)page * kv.page_stride +
                                   ((size_t)head * kv.page_size + (pos % kv.page_size)) * kv.head_dim + d;
                (is_v ? kv.v_cache : kv.k_cache)[dst] = __float2bfloat16_rn(v);
            }
        }
    }
}

constexpr int WIDE_MIN_COLS = 1536;     // from here on half the blocks still fill the GPU

template <int MT>
int launch_wide(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K, int lda,
                int ldw, int ldr, int ldc, int act, int out_dtype, const KVWrite& kv, cudaStream_t stream) {
    const unsigned blocks = (unsigned)((N + COLS2 - 1) / COLS2);
    if (out_dtype == SANDY_F32)
        return sandy_launch(gemm_skinny_wide_kernel<MT, float>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const bf16*)a,
                            (const bf16*)w, (const bf16*)bias, residual, (float*)out, M, N, K, lda, ldw, ldr, ldc, act, kv);
    return sandy_launch(gemm_skinny_wide_kernel<MT, bf16>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const bf16*)a,
                        (const bf16*)w, (const bf16*)bias, residual, (bf16*)out, M, N, K, lda, ldw, ldr, ldc, act, kv);
}

// ---- a vocabulary projection: up to 16 rows, very many columns, nothing fused -------------------
// The kernel above gives every 8 columns a block of eight warps that split K: for 50,257 columns
// that is 6,283 short-lived blocks, three of them on an SM at a time, each with 12 KB of weights in
// flight, and the product runs at half the memory's speed.  Here a WARP owns a group of 8 columns
// with all of K (no sums across warps, no barrier per group) and walks on to further groups; the
// rows are staged in shared memory once per block, and a warp always has the next eight 16-byte
// pieces of its weight rows (of this group or already of the next) on their way.  Same operand
// pairing as above; a row's result does not depend on the other rows.
constexpr int WALK_ROUND = 8;            // 16-byte weight pieces a lane keeps in flight
constexpr int WALK_MIN_GROUPS = 2048;    // from this many column groups on
constexpr int WALK_MAX_K = 2048;

template <typename TC>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_skinny_walk_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, TC* __restrict__ out, int M, int N,
                        int K, int lda, int ldw, int ldc) {
    extern __shared__ __align__(16) uint8_t xs_raw[];
    bf16* xs = reinterpret_cast<bf16*>(xs_raw);          // [16][K + XPAD]
    const int xs_ld = K + XPAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int chunks = (K + KCHUNK - 1) / KCHUNK;
    const int groups = (N + COLS - 1) / COLS;
    const int stride = (int)gridDim.x * WARPS;
    int grp = (int)blockIdx.x * WARPS + warp;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 wn[WALK_ROUND];
    auto load_round = [&](int grp_, int c0) {
        const int n = grp_ * COLS + g;
        const bool n_ok = grp_ < groups && n < N;
        const bf16* wrow = w + (size_t)(n_ok ? n : 0) * ldw;
#pragma unroll
        for (int u = 0; u < WALK_ROUND; u++) {
            const int k = (c0 + u) * KCHUNK + t * 8;
            wn[u] = (n_ok && c0 + u < chunks && k < K) ? ldg16_stream(wrow + k) : zero;
        }
    };
    load_round(grp, 0);          // weights: no kernel writes them

    pdl_launch_dependents();
    pdl_wait();
    const int pieces = K / 8;
    for (int idx = threadIdx.x; idx < 16 * pieces; idx += WARPS * 32) {
        const int r = idx / pieces, c8 = idx % pieces;
        *reinterpret_cast<uint4*>(xs + (size_t)r * xs_ld + c8 * 8) = r < M ? ldg16(a + (size_t)r * lda + c8 * 8) : zero;
    }
    __syncthreads();

    for (; grp < groups; grp += stride) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int c0 = 0; c0 < chunks; c0 += WALK_ROUND) {
            uint4 wv[WALK_ROUND];
#pragma unroll
            for (int u = 0; u < WALK_ROUND; u++) wv[u] = wn[u];
            if (c0 + WALK_ROUND < chunks) load_round(grp, c0 + WALK_ROUND);
            else load_round(grp + stride, 0);
#pragma unroll
            for (int u = 0; u < WALK_ROUND; u++) {
                if (c0 + u >= chunks) break;          // the same for every lane: the warp multiplies together
                const int k = (c0 + u) * KCHUNK + t * 8;
                const bool k_ok = k < K;               // a lane past K (a last, shorter chunk) feeds zeros
                const uint4 x0 = k_ok ? *reinterpret_cast<const uint4*>(xs + (size_t)g * xs_ld + k) : zero;
                const uint4 x1 = k_ok ? *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * xs_ld + k) : zero;
                mma_bf16(acc, x0.x, x1.x, x0.y, x1.y, wv[u].x, wv[u].y);
                mma_bf16(acc, x0.z, x1.z, x0.w, x1.w, wv[u].z, wv[u].w);
            }
        }
        // C fragment: c0,c1 = (row g, columns 2t, 2t+1); c2,c3 = (row g+8, same columns)
        const int col = grp * COLS + 2 * t;
        if (g < M) {
            if (col < N) out[(size_t)g * ldc + col] = from_f32<TC>(acc[0]);
            if (col + 1 < N) out[(size_t)g * ldc + col + 1] = from_f32<TC>(acc[1]);
        }
        if (g + 8 < M) {
            if (col < N) out[(size_t)(g + 8) * ldc + col] = from_f32<TC>(acc[2]);
            if (col + 1 < N) out[(size_t)(g + 8) * ldc + col + 1] = from_f32<TC>(acc[3]);
        }
    }
}

template <typename TC>
int launch_walk(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldc,
                cudaStream_t stream) {
    static int blocks_cap = 0;
    auto kern = gemm_skinny_walk_kernel<TC>;
    const size_t smem = (size_t)16 * (K + XPAD) * sizeof(bf16);
    if (blocks_cap == 0) {
        const int sms = sandy_sm_count();
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)((size_t)16 * (WALK_MAX_K + XPAD) * sizeof(bf16)));
        if (e != cudaSuccess) return (int)e;
        blocks_cap = 2 * sms;
    }
    const int groups = (N + COLS - 1) / COLS;
    const int want = (groups + WARPS - 1) / WARPS;
    const unsigned blocks = (unsigned)(want < blocks_cap ? want : blocks_cap);
    return sandy_launch(kern, dim3(blocks), dim3(WARPS * 32), smem, stream, (const bf16*)a, (const bf16*)w, (TC*)out, M, N,
                        K, lda, ldw, ldc);
}

}  // namespace

// Largest M and K the fused norm takes (the row is held in registers; the normalised rows
// in shared memory).
SANDY_API int sandy_gemm_skinny_norm_limits(int* max_rows, int* max_k) {
    *max_rows = 16;
    *max_k = MAX_ROW_VEC * 128;
    return SANDY_OK;
}

// Arguments as sandy_gemm_tc; M <= 64; K, lda, ldw multiples of 8; a and w 16-byte aligned.
//
// Fused norm: pass a = null and x (float [M, K], row stride ldx, 16-byte aligned, ldx % 4 == 0),
// gamma, beta (bfloat16 [K], beta may be null), eps; M <= 16 and K <= 2048.
// Key/value write: pass k_cache != null with the cache description of attention.cu; columns
// [q_cols, q_cols + kv_cols) of the product are keys, the next kv_cols are values, and row m
// belongs to position positions[m] of request token_seq[m].  out must be bfloat16 then.
SANDY_API int sandy_gemm_skinny(const void* a, const float* x, int ldx, const void* gamma, const void* beta,
                                float eps, const void* w, const void* bias, const float* residual, void* out,
                                int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype,
                                void* k_cache, void* v_cache, long long page_stride, const int* block_table,
                                int max_blocks, const int* token_seq, const int* positions, int q_cols,
                                int kv_cols, int head_dim, int page_size, int num_pages, int* status,
                                cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    const bool fuse = a == nullptr;
    if ((!a && !x) || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
    if (M > 64 || K % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) & 15) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    NormArgs norm{x, (const bf16*)gamma, (const bf16*)beta, ldx, eps};
    if (fuse) {
        if (!gamma || M > 16 || K > MAX_ROW_VEC * 128 || ldx % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) ||
            (reinterpret_cast<uintptr_t>(gamma) & 15) || (beta && (reinterpret_cast<uintptr_t>(beta) & 15)))
            return SANDY_ERR_UNSUPPORTED;
    } else {
        if (lda % 8 != 0 || (reinterpret_cast<uintptr_t>(a) & 15)) return SANDY_ERR_UNSUPPORTED;
    }
    KVWrite kv{(bf16*)k_cache, (bf16*)v_cache, page_stride, block_table, token_seq, positions,
               max_blocks, q_cols, kv_cols, head_dim, page_size, num_pages, status};
    if (k_cache) {
        if (!v_cache || !block_table || !token_seq || !positions || out_dtype != SANDY_BF16 || head_dim <= 0 ||
            kv_cols % head_dim != 0 || q_cols + 2 * kv_cols != N || page_size <= 0)
            return SANDY_ERR_ARGUMENT;
    }
    if (!fuse && !k_cache && !bias && !residual && act == SANDY_ACT_NONE && M <= 16 && K <= WALK_MAX_K &&
        (N + COLS - 1) / COLS >= WALK_MIN_GROUPS) {
        if (out_dtype == SANDY_F32) return launch_walk<float>(a, w, out, M, N, K, lda, ldw, ldc, stream);
        return launch_walk<bf16>(a, w, out, M, N, K, lda, ldw, ldc, stream);
    }
    if (fuse) return launch<1, true>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    if (M <= 16) return launch<1, false>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    if (N >= WIDE_MIN_COLS) {
        if (M <= 32) return launch_wide<2>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
        if (M <= 48) return launch_wide<3>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
        return launch_wide<4>(a, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    }
    if (M <= 32) return launch<2, false>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
    return launch<4, false>(a, norm, w, bias, residual, out, M, N, K, lda, ldw, ldr, ldc, act, out_dtype, kv, stream);
}
