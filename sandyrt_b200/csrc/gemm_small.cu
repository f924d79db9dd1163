// bfloat16 matrix product for 17 to 64 rows (a decode step of that many requests) on the tcgen05
// tensor cores, with the operands' roles swapped and K split over the blocks of a cluster.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) + residual[m, n],      M <= 64
//
// With so few rows a 128-row accumulator tile of `a` is mostly padding and a product has only
// N / 128 tiles (6 for a 768-column matrix: 6 of 148 SMs).  Here the WEIGHT is the 128-row operand
// of the instruction and the tokens are its narrow side: a block computes a [128 columns of w] x
// [64 tokens] accumulator, transposed, in 64 columns of tensor memory, so nothing is padding (rows
// of `a` past M come in as zeros from TMA).  K is cut into `splits` ranges, one block each, so a
// matrix of 6 tiles still runs on 48 SMs; every block streams its [128 x K/splits] piece of the
// weight through a ring of TMA stages exactly as gemm_tc.cu does.
//
// Partial sums.  The blocks that share an output tile are one thread-block cluster.  Each leaves
// its accumulator (float) in its own shared memory; after one cluster barrier block r of the
// cluster finishes the tokens r, r + splits, ...: it adds the blocks' accumulators through
// distributed shared memory IN THE ORDER OF THE BLOCKS, so an output element's sum is formed in one
// fixed order, and runs the write-back.  No scratch in global memory, no counters, no second
// kernel.  The number of splits is a rule of the shape and the SM count alone
// (sandy_gemm_small_splits), never a timing.
//
// Write-back: a thread owns one output column (its tensor-memory lane) and walks the tokens, so the
// 32 lanes of a warp store 32 consecutive columns of a row at a time.  Bias, activation, residual
// and the key/value write into the cache pages are folded in as in the other product kernels.
// The skinny kernel (gemm_skinny.cu, mma.sync) remains for up to 16 rows and for the fused norm.
//
// Every wait on an mbarrier is bounded: on expiry the kernel raises `*status`, stops issuing, still
// meets its cluster's barriers, frees its tensor memory and returns.  The reference's counterpart
// is one cuBLAS call per product (src/device/cuda/CudaMatMulKernels.cu:173-217).
#include "tcgen05.cuh"

namespace {

constexpr int NUM_THREADS = 192;
constexpr int W_BYTES = BM * BK * 2;   // 128 weight rows x 64 k
constexpr int MAX_SPLITS = 8;                     // the portable cluster size
constexpr int MAX_TOKENS = 256;                   // the instruction's narrow side at its widest

// TOKENS: the instruction's narrow side, tokens per tile: 64 (a decode step), 128 or 256 (a short prompt
// step, whose products of few row tiles the tile kernels run on a handful of CTAs).
template <int STAGES, int TOKENS>
struct Layout {
    static constexpr int A_BYTES = TOKENS * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int PART_BYTES = TOKENS * BM * 4;       // a block's accumulator as floats, [token][column]
    static_assert(STAGES * STAGE_BYTES >= PART_BYTES, "the accumulator is parked in the ring's memory");
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The float at `addr` (an address in this block's shared memory) in block `rank` of the cluster.
__device__ __forceinline__ float ld_peer(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// What the write-back needs of the epilogue arguments, read once into registers.  (Handing the kernel's
// parameter struct itself to the per-element function made every element's field reads slow: a 64 x 16384
// product took 16 us with it and 4.3 with these scalars.)
struct Finish {
    const float* residual;
    void* out;
    int ldr, ldc, act, out_f32;
    bf16* k_cache;
    bf16* v_cache;
    long long page_stride;
    int q_cols, kv_cols, head_dim, page_size, num_pages;
};

__device__ __forceinline__ Finish make_finish(const EpilogueArgs& ep) {
    Finish f;
    f.residual = ep.residual; f.out = ep.out; f.ldr = ep.ldr; f.ldc = ep.ldc; f.act = ep.act; f.out_f32 = ep.out_f32;
    f.k_cache = ep.kv.k_cache; f.v_cache = ep.kv.v_cache; f.page_stride = ep.kv.page_stride;
    f.q_cols = ep.kv.q_cols; f.kv_cols = ep.kv.kv_cols; f.head_dim = ep.kv.head_dim; f.page_size = ep.kv.page_size;
    f.num_pages = ep.kv.num_pages;
    return f;
}

// One output element: bias, activation, cache write, residual, store.  What the product has of these is a
// template argument: chosen per element at run time, the compiler computed every activation and the cache
// address with its divisions for every element and then picked (a 64 x 16384 product with none of them:
// 16 us, of which 12 went there).
template <int ACT, bool KV, bool RES, bool F32>
__device__ __forceinline__ void finish(float acc, int m, int n, float bias, const Finish& f, int N, const int* kv_page,
                                       const int* kv_slot, int* status) {
    if (n >= N) return;
    float v = acc + bias;
    if (ACT == SANDY_ACT_GELU_TANH) v = gelu_tanh_fast(v);
    if (ACT == SANDY_ACT_GELU_ERF) v = gelu_erf(v);
    if (KV) {
        if (n >= f.q_cols) {
            const int page = kv_page[m];
            if (page < 0 || page >= f.num_pages) {
                if (status) atomicOr(status, 8);                 // a key/value write with no page behind it
            } else {
                const int c = n - f.q_cols;
                const bool is_v = c >= f.kv_cols;
                const int c2 = is_v ? c - f.kv_cols : c;
                const int head = c2 / f.head_dim, d = c2 % f.head_dim;
                (is_v ? f.v_cache : f.k_cache)[(size_t)page * f.page_stride + ((size_t)head * f.page_size + kv_slot[m]) * f.head_dim + d] =
                    __float2bfloat16_rn(v);
            }
        }
    }
    if (RES) v += f.residual[(size_t)m * f.ldr + n];
    if (F32) reinterpret_cast<float*>(f.out)[(size_t)m * f.ldc + n] = v;
    else reinterpret_cast<bf16*>(f.out)[(size_t)m * f.ldc + n] = __float2bfloat16_rn(v);
}

// The write-back of one thread's column: `count` tokens from token m0 in steps of `step`, their sums given by
// value(i).  One instance per combination of epilogue features that occurs; the choice is made once, out here.
// FIXED > 0: the loop is unrolled FIXED times with `count` as a predicate (value(i) may then index registers).
template <int ACT, bool KV, bool RES, bool F32, int FIXED, typename Value>
__device__ __forceinline__ void finish_column(int m0, int step, int count, int n, float bias, const Finish& f, int N,
                                              const int* kv_page, const int* kv_slot, int* status, Value value) {
    if (FIXED > 0) {
#pragma unroll
        for (int i = 0; i < FIXED; i++)
            if (i < count) finish<ACT, KV, RES, F32>(value(i), m0 + i * step, n, bias, f, N, kv_page, kv_slot, status);
    } else {
#pragma unroll 2
        for (int i = 0; i < count; i++) finish<ACT, KV, RES, F32>(value(i), m0 + i * step, n, bias, f, N, kv_page, kv_slot, status);
    }
}

template <int FIXED, typename Value>
__device__ __forceinline__ void finish_dispatch(int m0, int step, int count, int n, float bias, const Finish& f, int N,
                                                const int* kv_page, const int* kv_slot, int* status, Value value) {
#define SANDY_FINISH(ACT, KV, RES, F32) finish_column<ACT, KV, RES, F32, FIXED>(m0, step, count, n, bias, f, N, kv_page, kv_slot, status, value)
    if (f.k_cache) SANDY_FINISH(SANDY_ACT_NONE, true, false, false);                 // the fused q/k/v product: bfloat16, nothing else
    else if (f.residual) {
        if (f.out_f32) SANDY_FINISH(SANDY_ACT_NONE, false, true, true);              // x += ...
        else SANDY_FINISH(SANDY_ACT_NONE, false, true, false);
    } else if (f.act == SANDY_ACT_GELU_TANH) {
        if (f.out_f32) SANDY_FINISH(SANDY_ACT_GELU_TANH, false, false, true);
        else SANDY_FINISH(SANDY_ACT_GELU_TANH, false, false, false);
    } else if (f.act == SANDY_ACT_GELU_ERF) {
        if (f.out_f32) SANDY_FINISH(SANDY_ACT_GELU_ERF, false, false, true);
        else SANDY_FINISH(SANDY_ACT_GELU_ERF, false, false, false);
    } else {
        if (f.out_f32) SANDY_FINISH(SANDY_ACT_NONE, false, false, true);
        else SANDY_FINISH(SANDY_ACT_NONE, false, false, false);
    }
#undef SANDY_FINISH
}

// grid (splits, tiles), clusters of (splits, 1, 1): blockIdx.x is the block's rank in its cluster.
template <int STAGES, int TOKENS>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_small_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, EpilogueArgs ep,
                  int M, int N, int K, int steps_per_split, int* __restrict__ status) {
    constexpr int STAGE_BYTES = Layout<STAGES, TOKENS>::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    __shared__ int kv_page[TOKENS], kv_slot[TOKENS];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, splits = gridDim.x, tile = blockIdx.y;
    const int n0 = tile * BM;
    const int k_tiles = (K + BK - 1) / BK;
    const int kt_begin = min(k_tiles, split * steps_per_split), kt_end = min(k_tiles, kt_begin + steps_per_split);
    constexpr uint32_t TMEM_COLS = TOKENS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            // the weight is nobody's output: its first stages are asked for before the kernel before has ended
            int ahead = 0;
            for (int kt = kt_begin; kt < kt_end && ahead < STAGES; kt++, ahead++) {
                mbar_expect_tx(&full_bar[ahead], STAGE_BYTES);
                tma_load_2d(smem + ahead * STAGE_BYTES, &map_w, kt * BK, n0, &full_bar[ahead]);
            }
            pdl_wait();          // a may be the output of the kernel before
            int issued = 0;
            for (int kt = kt_begin; kt < kt_end; kt++, issued++) {
                const int s = issued % STAGES;
                const uint32_t round = issued / STAGES;
                uint8_t* sw = smem + s * STAGE_BYTES;
                if (round > 0) {
                    if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1)) {
                        if (status) atomicOr(status, 1);
                        break;
                    }
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    tma_load_2d(sw, &map_w, kt * BK, n0, &full_bar[s]);
                }
                tma_load_2d(sw + W_BYTES, &map_a, kt * BK, 0, &full_bar[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: D[128 weight rows, 64 tokens] += W[128, 16] . A[64, 16]^T ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_instr_desc(TOKENS);
            int issued = 0;
            for (int kt = kt_begin; kt < kt_end; kt++, issued++) {
                const int s = issued % STAGES;
                const uint32_t round = issued / STAGES;
                if (!mbar_wait(&full_bar[s], round & 1)) {
                    if (status) atomicOr(status, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t w_addr = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t dw = make_smem_desc(w_addr), da = make_smem_desc(w_addr + W_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++)
                    umma_bf16(tmem_base, dw + (uint64_t)(2 * k), da + (uint64_t)(2 * k), idesc, (issued > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            umma_commit(accum_bar);
        }
        __syncwarp();
    }

    // ---------------- write-back: warps 2..5, a thread per output column ----------------
    const int quarter = warp & 3;                 // the tensor-memory lanes this warp may read
    const int col = quarter * 32 + lane;          // column inside the tile
    const int n = n0 + col;
    const int e = threadIdx.x - 64;               // 0..127 among the write-back threads
    float bias = 0.0f;
    const Finish fin = make_finish(ep);
    float* part = reinterpret_cast<float*>(smem);     // the ring is idle once the accumulator is complete
    if (warp >= 2) {
        if (ep.bias && n < N) bias = __bfloat162float(ep.bias[n]);     // a weight-like input: before the wait
        pdl_wait();              // out, residual and positions may still be in use by kernels before
        if (ep.kv.k_cache)
            for (int tok = e; tok < TOKENS; tok += 128) kv_row_target(ep.kv, tok, M, kv_page[tok], kv_slot[tok]);
        epilogue_sync();
        const bool has_work = kt_end > kt_begin;
        const bool ready = has_work ? mbar_wait(accum_bar, 0) : true;
        if (!ready && lane == 0 && status) atomicOr(status, 4);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < TOKENS / 32; c++) {
            if (c * 32 >= M) break;
            uint32_t r[32];
            if (has_work && ready) {
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) r[j] = 0u;              // a block without k-steps adds zeros
            }
            if (splits == 1) {
                const int count = min(32, M - c * 32);
                finish_dispatch<32>(c * 32, 1, count, n, bias, fin, N, kv_page, kv_slot, status,
                                    [&](int i) { return __uint_as_float(r[i]); });
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) part[(c * 32 + j) * BM + col] = __uint_as_float(r[j]);
            }
        }
    }
    if (splits > 1) {
        cluster_sync_all();                       // every block's accumulator is in its shared memory
        if (warp >= 2) {
            const uint32_t part_addr = smem_u32(part);
            const int count = M > split ? (M - split + splits - 1) / splits : 0;      // tokens split, split + splits, ...
            finish_dispatch<0>(split, splits, count, n, bias, fin, N, kv_page, kv_slot, status, [&](int i) {
                const uint32_t at = part_addr + (uint32_t)((((split + i * splits) * BM) + col) * 4);
                float v[MAX_SPLITS];
#pragma unroll
                for (int s = 0; s < MAX_SPLITS; s++) v[s] = s < splits ? ld_peer(at, (uint32_t)s) : 0.0f;
                float sum = v[0];
#pragma unroll
                for (int s = 1; s < MAX_SPLITS; s++) sum += v[s];                  // the blocks in order
                return sum;
            });
        }
        cluster_sync_all();                       // nobody leaves while a peer may still read its memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

int choose_splits(int N, int K) {
    const int tiles = (N + BM - 1) / BM, k_tiles = (K + BK - 1) / BK;
    int want = sandy_sm_count() / tiles;
    if (want > MAX_SPLITS) want = MAX_SPLITS;
    if (want > (k_tiles + 1) / 2) want = (k_tiles + 1) / 2;       // at least two k-steps a block
    if (want < 1) want = 1;
    const int steps = (k_tiles + want - 1) / want;
    return (k_tiles + steps - 1) / steps;
}

template <int STAGES, int TOKENS>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const EpilogueArgs& ep, int M, int N, int K, int tiles, int splits,
           int steps, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemm_small_kernel<STAGES, TOKENS>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<STAGES, TOKENS>::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, tiles);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Layout<STAGES, TOKENS>::TOTAL;
    cfg.stream = stream;
    // (a product that is not split is launched as an ordinary grid, not as clusters of one block)
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (splits > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = splits;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    if (sandy_pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_small_kernel<STAGES, TOKENS>, mw, ma, ep, M, N, K, steps, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// How many ranges K is cut into for an [*, K] x [N, K] product: enough blocks to spread a matrix of few
// column tiles over the GPU, at least two k-steps (128 k) a block, at most 8 (a cluster).  A rule of N, K
// and the device's SM count.
SANDY_API int sandy_gemm_small_splits(int N, int K) { return choose_splits(N, K); }

// a: bfloat16 [M, K] (M <= 256), row stride lda; w: bfloat16 [N, K], row stride ldw; bias: bfloat16 [N] or null;
// residual: float [M, N] or null (may be `out`); out: [M, N] bfloat16 (out_dtype 1) or float (0).
// The key/value arguments as in sandy_gemm_tc.
// status: bits 0-2 a barrier wait ran out, bit 3 a key/value write had no page behind it.
SANDY_API int sandy_gemm_small(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N,
                               int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype, void* k_cache,
                               void* v_cache, long long page_stride, const int* block_table, int max_blocks,
                               const int* token_seq, const int* positions, int q_cols, int kv_cols, int head_dim,
                               int page_size, int num_pages, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
    if (M > MAX_TOKENS || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    const int tokens = M <= 64 ? 64 : (M <= 128 ? 128 : 256);
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    const int tiles = (N + BM - 1) / BM, k_tiles = (K + BK - 1) / BK;
    if (tiles > 65535) return SANDY_ERR_UNSUPPORTED;
    const int splits = choose_splits(N, K);
    CUtensorMap mw, ma;
    if (!get_map(w, N, K, ldw, BM, &mw)) return SANDY_ERR_UNSUPPORTED;
    if (!get_map(a, M, K, lda, tokens, &ma)) return SANDY_ERR_UNSUPPORTED;
    KVWrite kv{(bf16*)k_cache, (bf16*)v_cache, page_stride, block_table, token_seq, positions,
               max_blocks, q_cols, kv_cols, head_dim, page_size, num_pages};
    if (k_cache) {
        if (!v_cache || !block_table || !token_seq || !positions || head_dim <= 0 || kv_cols % head_dim != 0 ||
            q_cols + 2 * kv_cols != N || page_size <= 0 || out_dtype != SANDY_BF16)
            return SANDY_ERR_ARGUMENT;
    }
    EpilogueArgs ep{(const bf16*)bias, residual, out, ldr, ldc, act, out_dtype == SANDY_F32 ? 1 : 0, kv};
    const int steps = (k_tiles + splits - 1) / splits;
    // many tiles and no split (a vocabulary projection): three stages, so that three blocks share an SM and
    // the tiles run as one wave; else a deeper ring for the one block an SM gets
    if (tokens == 128) return launch<6, 128>(mw, ma, ep, M, N, K, tiles, splits, steps, status, stream);
    if (tokens == 256) return launch<4, 256>(mw, ma, ep, M, N, K, tiles, splits, steps, status, stream);
    if (splits == 1) return launch<3, 64>(mw, ma, ep, M, N, K, tiles, splits, steps, status, stream);
    return launch<6, 64>(mw, ma, ep, M, N, K, tiles, splits, steps, status, stream);
}
