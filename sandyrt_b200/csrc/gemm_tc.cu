// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), operands staged by TMA,
// accumulator in tensor memory, bias / activation / residual folded into the write-back.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) + residual[m, n]
//
// a: [M, K] bfloat16, K contiguous.  w: [N, K] bfloat16, K contiguous (a Linear weight as
// stored, the token table used as the output head, or a Conv1D weight transposed once at
// load).  Sums are carried in float in tensor memory; out is bfloat16 or float.
// The reference hands this product to cuBLAS (cublasGemmEx with CUBLAS_COMPUTE_32F,
// src/device/cuda/CudaMatMulKernels.cu:173-217) and runs bias, gelu and the residual add as
// separate elementwise kernels (src/ir/BuiltinLowering.cpp:116-140).
//
// One CTA computes one 128 x BN tile of the output:
//   warp 0      one elected lane issues TMA loads of the A tile (128 x 64) and the W tile
//               (BN x 64) of each k-step into a ring of shared-memory stages (128-byte swizzle)
//   warp 1      allocates BN columns of tensor memory; one elected lane issues four
//               tcgen05.mma (128 x BN x 16) per stage and commits each stage back to the ring
//   warps 2..5  when the last commit lands, read the accumulator with tcgen05.ld (each warp its
//               32 lanes = 32 rows), apply the epilogue and write back: above one tile of rows
//               through tiles in shared memory (the ring, idle by then) that TMA stores, or
//               reduce-adds where the residual is the output itself; else from the registers
//               (write_back_warp in tcgen05.cuh)
// Rows and columns past M, N, K are zero-filled by TMA on the way in and masked on the way
// out, so any M and N are taken; K must be a multiple of 8 (TMA wants 16-byte row pitches).
// For a given output element the k-steps are always added in ascending order, so a row's
// result does not depend on M or on what else is in the batch.
//
// Every wait on an mbarrier is bounded: on expiry the kernel raises `*status`, stops issuing,
// frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace {

constexpr int NUM_THREADS = 192;

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static_assert(STAGES * STAGE_BYTES >= 8 * EPI_WARP_BYTES, "the one-tile kernel stages its write-back in the ring");
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, EpilogueArgs ep, int M, int N, int K, int* __restrict__ status) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int k_tiles = (K + BK - 1) / BK;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;   // power of two >= 32 for the BN values used

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up (barriers, tensor memory) ran while the kernel before was still finishing; the kernel
    // after this one may start its own set-up now.
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            pdl_wait();          // a may be the output of the kernel before
            for (int kt = 0; kt < k_tiles; kt++) {
                const int s = kt % STAGES;
                const uint32_t round = kt / STAGES;
                if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1)) {
                    if (status) atomicOr(status, 1);
                    break;
                }
                uint8_t* sa = stage_base + s * L::STAGE_BYTES;
                uint8_t* sb = sa + L::A_BYTES;
                mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                tma_load_2d(sa, &map_a, kt * BK, m0, &full_bar[s]);
                tma_load_2d(sb, &map_w, kt * BK, n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_instr_desc(BN);
            bool ok = true;
            for (int kt = 0; kt < k_tiles && ok; kt++) {
                const int s = kt % STAGES;
                const uint32_t round = kt / STAGES;
                if (!mbar_wait(&full_bar[s], round & 1)) {
                    if (status) atomicOr(status, 2);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(stage_base + s * L::STAGE_BYTES);
                const uint32_t b_addr = a_addr + L::A_BYTES;
                const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    // advance 16 elements = 32 bytes inside the swizzle row: +2 in 16-byte units
                    umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                              (kt > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
            }
            umma_commit(accum_bar);           // arrives when every MMA issued so far is complete
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int quarter = warp & 3;         // the TMEM lanes this warp may read: 32*quarter ..
        float bias[BN / 32];
        load_bias(bias, ep, n0, N);
        pdl_wait();              // out and residual may still be in use by the kernel before
        const bool ready = mbar_wait(accum_bar, 0);
        if (!ready && lane == 0 && status) atomicOr(status, 4);
        tc_fence_after();
        const int row = m0 + quarter * 32 + lane;
        int kv_page, kv_slot;
        kv_row_target(ep.kv, row, M, kv_page, kv_slot);
        if (ready) {
            // every MMA has completed, so nothing reads the ring any more: the warps stage their tiles in it
            write_back_warp<BN / 32, 2>(tmem_base + ((uint32_t)(quarter * 32) << 16), stage_base + quarter * 2 * EPI_WARP_BYTES,
                                     m0 + quarter * 32, n0, ep, &map_out, M, N, kv_page, kv_slot, status, bias, [] {});
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---- the persistent form -------------------------------------------------------------------------
// One CTA per SM walks the output tiles (tile = blockIdx.x, + gridDim.x, ...).  What the
// one-tile-per-CTA kernel above pays per tile -- barrier and tensor-memory set-up, a cold TMA
// ring, and above all an MMA pipe that idles while the accumulator is written back -- is paid
// once, or overlapped: tensor memory holds TWO accumulators, so the MMA warp starts the next
// tile while eight epilogue warps (two per 32-lane quarter of tensor memory, half of the tile's
// columns each) drain the last one, and the TMA warp runs ahead across tile boundaries.
//   warp 0      TMA producer            full[s] / empty[s] ring over all k-steps of all tiles
//   warp 1      MMA issuer              acc_empty[b] -> k-steps -> commit acc_full[b]
//   warps 2..9  epilogue                acc_full[b] -> tcgen05.ld, write-back -> acc_empty[b]
// Tiles are numbered m-fastest, so CTAs that run side by side share a W tile in L2.
constexpr int P_THREADS = 320;
constexpr int P_EPI_WARPS = 8;
// Shared memory of the persistent form: its ring never rests, so the write-back warps get staging tiles
// of their own between the ring and the barriers.
template <int BN, int STAGES>
constexpr int persistent_smem() { return SmemLayout<BN, STAGES>::TOTAL + P_EPI_WARPS * EPI_WARP_BYTES; }

template <int BN, int STAGES>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_out, EpilogueArgs ep, int M, int N, int K,
                          int* __restrict__ status) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* epi_tiles = smem + STAGES * L::STAGE_BYTES;          // 1024-byte aligned, a tile per write-back warp
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_tiles + P_EPI_WARPS * EPI_WARP_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (K + BK - 1) / BK;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;     // two accumulators; a power of two for BN = 64, 128, 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], P_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up (barriers, tensor memory) ran while the kernel before was still finishing; the kernel
    // after this one may start its own set-up now.
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            pdl_wait();             // a may be the output of the kernel before
            uint32_t it = 0;        // k-steps issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kt = 0; kt < k_tiles; kt++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1)) {
                        if (status) atomicOr(status, 1);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = stage_base + s * L::STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                    tma_load_2d(sa, &map_a, kt * BK, m0, &full_bar[s]);
                    tma_load_2d(sa + L::A_BYTES, &map_w, kt * BK, n0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_instr_desc(BN);
            uint32_t it = 0;
            bool ok = true;
            int ti = 0;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ti++) {
                const int b = ti & 1;
                // the accumulator must have been drained by the epilogue of two tiles ago
                if (!mbar_wait(&acc_empty[b], ((ti >> 1) & 1) ^ 1)) {
                    if (status) atomicOr(status, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(b * BN);
                for (int kt = 0; kt < k_tiles; kt++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
                        if (status) atomicOr(status, 2);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stage_base + s * L::STAGE_BYTES);
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_bf16(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9 ----------------
        const int quarter = warp & 3;                  // the TMEM lanes this warp may read
        // The tile's columns are halved between the two warps of a quarter.  (Half of a 64-column tile is a
        // single chunk: narrower than a bfloat16 staging tile, so it is written back from the registers, which
        // for the few rows this width is chosen for is the quicker way anyhow.)
        const int half = (warp - 2) >> 2;              // which half of the tile's columns
        constexpr int CHUNKS = BN / 32 / 2;            // 32-column chunks per warp
        uint8_t* tile_mem = epi_tiles + (warp - 2) * EPI_WARP_BYTES;
        bool dead = false;
        int ti = 0;
        pdl_wait();                 // out and residual may still be in use by the kernel before
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ti++) {
            const int b = ti & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            int kv_page, kv_slot;
            kv_row_target(ep.kv, row, M, kv_page, kv_slot);
            float bias[CHUNKS];
            load_bias(bias, ep, n0 + half * CHUNKS * 32, N);
            // A warp whose wait ran out keeps walking the tiles but touches nothing any more.
            if (!dead && !mbar_wait(&acc_full[b], (ti >> 1) & 1)) {
                if (lane == 0 && status) atomicOr(status, 4);
                dead = true;
            }
            if (dead) continue;
            tc_fence_after();
            write_back_warp<CHUNKS, 1>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * BN + half * CHUNKS * 32), tile_mem,
                                    m0 + quarter * 32, n0 + half * CHUNKS * 32, ep, &map_out, M, N, kv_page, kv_slot, status, bias, [&] {
                                        // everything this warp needs of the accumulator is in registers: hand it back
                                        tc_fence_before();
                                        __syncwarp();
                                        if (lane == 0) mbar_arrive(&acc_empty[b]);
                                    });
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const EpilogueArgs& ep, int M, int N, int K,
           int* status, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return sandy_launch(gemm_tc_kernel<BN, STAGES>, grid, dim3(NUM_THREADS), L::TOTAL, stream, ma, mw, mo, ep, M, N, K, status);
}

// Which kernel and tile width for a product.  Both kernels are bound by how fast an SM can pull
// operand tiles out of L2 (measured here: about 70 GB/s per SM, about 9 TB/s over all SMs), not
// by the tensor pipe, so the estimate is bytes over bandwidth plus what is not overlapped:
//   one tile per CTA, c CTAs resident per SM:  rounds(tiles / (SMs * c)) x c x tile bytes / rate + one epilogue
//   persistent:                                rounds(tiles / SMs) x tile bytes / rate + one epilogue
// The constants come from `python -m sandyrt_b200.csrc.microbench gemm` (2048 rows, GPT-2 small).
int choose_tile(int M, int N, int K) {
    const int sms = sandy_sm_count();
    const double rate = 70e3, all_rate = 9e6;        // bytes per microsecond: one SM, all SMs
    const int k_tiles = (K + BK - 1) / BK, m_tiles = (M + BM - 1) / BM;
    double best = 1e30;
    int best_tile = -64;
    const int widths[3] = {64, 128, 256};
    for (int persistent = 0; persistent < 2; persistent++) {
        for (int wi = 0; wi < 3; wi++) {
            const int bn = widths[wi];
            const double tile_bytes = (double)k_tiles * (BM + bn) * BK * 2;
            const long long tiles = (long long)m_tiles * ((N + bn - 1) / bn);
            const int resident = persistent ? 1 : (bn == 256 ? 1 : 2);
            const long long rounds = (tiles + (long long)sms * resident - 1) / ((long long)sms * resident);
            const long long busy = tiles < (long long)sms * resident ? tiles : (long long)sms * resident;
            const double per_sm = (double)rounds * (double)((busy + sms - 1) / sms < resident ? (busy + sms - 1) / sms : resident)
                                  * tile_bytes / rate;
            const double all = (double)tiles * tile_bytes / all_rate;
            const double epilogue = (persistent ? 3.0 : 2.0) + bn / 64.0 * (persistent ? 0.6 : 1.0);
            const double t = (per_sm > all ? per_sm : all) + epilogue;
            if (t < best) {
                best = t;
                best_tile = persistent ? bn : -bn;
            }
        }
    }
    return best_tile;
}

template <int BN, int STAGES>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const EpilogueArgs& ep, int M,
                      int N, int K, int* status, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static int sms = 0;
    if (sms == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, persistent_smem<BN, STAGES>());
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        sms = n;
    }
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = (int)(tiles < sms ? tiles : sms);
    return sandy_launch(gemm_tc_persistent_kernel<BN, STAGES>, dim3(grid), dim3(P_THREADS), persistent_smem<BN, STAGES>(), stream, ma, mw, mo, ep, M,
                        N, K, status);
}

}  // namespace

// a: bfloat16 [M, K], row stride lda; w: bfloat16 [N, K], row stride ldw; bias: bfloat16 [N] or
// null; residual: float [M, N] row stride ldr or null; out: [M, N] row stride ldc, bfloat16
// (out_dtype 1) or float (out_dtype 0).  Strides in elements; lda, ldw multiples of 8; a and w
// 16-byte aligned.  tile_n: 0 = choose (choose_tile), else 64, 128 or 256 (the persistent kernel),
// or -64, -128, -256 (one tile per CTA).
SANDY_API int sandy_gemm_tc(const void* a, const void* w, const void* bias, const float* residual, void* out,
                            int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype,
                            int tile_n, void* k_cache, void* v_cache, long long page_stride, const int* block_table,
                            int max_blocks, const int* token_seq, const int* positions, int q_cols, int kv_cols,
                            int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    if (tile_n == 0) tile_n = choose_tile(M, N, K);
    const int box_n = tile_n < 0 ? -tile_n : tile_n;
    CUtensorMap ma, mw;
    if (!get_map(a, M, K, lda, BM, &ma)) return SANDY_ERR_UNSUPPORTED;
    if (!get_map(w, N, K, ldw, box_n, &mw)) return SANDY_ERR_UNSUPPORTED;
    KVWrite kv{(bf16*)k_cache, (bf16*)v_cache, page_stride, block_table, token_seq, positions,
               max_blocks, q_cols, kv_cols, head_dim, page_size, num_pages};
    if (k_cache) {
        // the key/value write needs whole heads of a multiple of 16 and the three column ranges
        if (!v_cache || !block_table || !token_seq || !positions || head_dim <= 0 || head_dim % 16 != 0 ||
            kv_cols % head_dim != 0 || q_cols % 8 != 0 || q_cols + 2 * kv_cols != N || page_size <= 0 ||
            (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
            page_stride % 8 != 0 || act != SANDY_ACT_NONE)          // (the write-back has no form with both)
            return SANDY_ERR_ARGUMENT;
    }
    EpilogueArgs ep{(const bf16*)bias, residual, out, ldr, ldc, act, out_dtype == SANDY_F32 ? 1 : 0, kv, 0};
    CUtensorMap mo;
    get_out_map(ep, M, N, &mo);
    switch (tile_n) {
        case -64: return launch<64, 4>(ma, mw, mo, ep, M, N, K, status, stream);
        case -128: return launch<128, 3>(ma, mw, mo, ep, M, N, K, status, stream);
        case -256: return launch<256, 4>(ma, mw, mo, ep, M, N, K, status, stream);
        case 64: return launch_persistent<64, 7>(ma, mw, mo, ep, M, N, K, status, stream);
        case 128: return launch_persistent<128, 6>(ma, mw, mo, ep, M, N, K, status, stream);
        case 256: return launch_persistent<256, 4>(ma, mw, mo, ep, M, N, K, status, stream);
        default: return SANDY_ERR_UNSUPPORTED;
    }
}
