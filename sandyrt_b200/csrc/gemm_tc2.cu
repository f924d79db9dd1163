// bfloat16 matrix product on tcgen05 with TWO SMs on one tile (cta_group::2), persistent.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) + residual[m, n]      (as gemm_tc.cu)
//
// Why.  gemm_tc.cu is not bound by the tensor pipe but by how fast an SM pulls operand tiles out
// of L2 (measured: about 70 GB/s per SM): a 128 x 128 tile needs 32 KB per 64-wide k-step for
// 2 MFLOP.  Here a pair of CTAs (a cluster of two) computes a 256 x BN tile with one MMA
// instruction stream: each CTA loads its own 128 rows of A and only HALF of the BN rows of W
// (the pair's MMA reads both halves, each from the shared memory of the CTA that loaded it), so
// with BN = 256 a CTA loads the same 32 KB per k-step for twice the arithmetic.
//
// Roles (both CTAs run the same code; rank 0 of the pair is the leader):
//   warp 0      TMA producer, both CTAs: own A rows and own half of W into own shared memory,
//               completion counted on the LEADER's full[s]; the leader expects both CTAs' bytes
//   warp 1      leader only: tcgen05.mma.cta_group::2 (256 x BN x 16), commits multicast to both
//               CTAs' empty[s] (stage free) and acc_full[b] (accumulator ready)
//   warps 2..9  epilogue, both CTAs: own 128 rows from own tensor memory; when an accumulator
//               has been read, an arrive on the LEADER's acc_empty[b]
// Tensor memory holds two accumulators (2 x BN columns), so the next tile's products overlap
// the write-back of the last.  The pair is a thread-block cluster; no load is multicast.
//
// Every mbarrier wait is bounded (status bits 1, 2, 4 as in gemm_tc.cu); the cluster barriers at
// the start and the end are reached by every thread whatever the waits returned.
#include "tcgen05.cuh"

namespace {

constexpr int T2_THREADS = 320;
constexpr int T2_EPI_WARPS = 8;
constexpr int PAIR_M = 2 * BM;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of `smem_addr` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c_inner, int c_outer,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c_inner), "r"(c_outer)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    const uint32_t z = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z)
        : "memory");
}

// Arrives, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__host__ __device__ constexpr uint32_t make_instr_desc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PAIR_M >> 4) << 24);
}

template <int BN, int STAGES>
struct PairLayout {
    static constexpr int A_BYTES = BM * BK * 2;             // this CTA's 128 rows of A
    static constexpr int B_BYTES = (BN / 2) * BK * 2;       // this CTA's half of the W rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // the ring, a staging tile for each write-back warp, the barriers
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 8 * EPI_WARP_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_out, EpilogueArgs ep, int M, int N, int K, int* __restrict__ status) {
    using L = PairLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* epi_tiles = smem + STAGES * L::STAGE_BYTES;          // 1024-byte aligned, a tile per write-back warp
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_tiles + 8 * EPI_WARP_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_tiles = (K + BK - 1) / BK;
    const int m_tiles = (M + PAIR_M - 1) / PAIR_M, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    constexpr int TMEM_COLS = 2 * BN;              // two accumulators; BN = 128 or 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 2 * T2_EPI_WARPS);      // the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything of ours can reach them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();     // the kernel after this one may start its set-up

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (elect_one()) {
            pdl_wait();          // a may be the output of the kernel before
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += n_pairs) {
                const int m0 = (tile % m_tiles) * PAIR_M + (int)rank * BM;
                const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
                for (int kt = 0; kt < k_tiles; kt++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1)) {
                        if (status) atomicOr(status, 1);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = stage_base + s * L::STAGE_BYTES;
                    if (leader) mbar_expect_tx(&full_bar[s], 2 * L::STAGE_BYTES);
                    const uint32_t leader_full = in_cta(smem_u32(&full_bar[s]), 0);
                    tma_load_2d_pair(sa, &map_a, kt * BK, m0, leader_full);
                    tma_load_2d_pair(sa + L::A_BYTES, &map_w, kt * BK, n0, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (leader && elect_one()) {
            constexpr uint32_t idesc = make_instr_desc_pair(BN);
            uint32_t it = 0;
            bool ok = true;
            int ti = 0;
            for (int tile = pair; tile < tiles && ok; tile += n_pairs, ti++) {
                const int b = ti & 1;
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
                        umma_bf16_pair(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[s]);
                }
                if (ok) umma_commit_pair(&acc_full[b]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9 (both CTAs) ----------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int CHUNKS = BN / 32 / 2;
        uint8_t* tile_mem = epi_tiles + (warp - 2) * EPI_WARP_BYTES;
        bool dead = false;
        int ti = 0;
        pdl_wait();              // out and residual may still be in use by the kernel before
        for (int tile = pair; tile < tiles; tile += n_pairs, ti++) {
            const int b = ti & 1;
            const int m0 = (tile % m_tiles) * PAIR_M + (int)rank * BM, n0 = (tile / m_tiles) * BN;
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
                                        if (lane == 0) mbar_arrive_cluster(in_cta(smem_u32(&acc_empty[b]), 0));
                                    });
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

template <int BN, int STAGES>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const EpilogueArgs& ep, int M, int N, int K, int* status,
                cudaStream_t stream) {
    using L = PairLayout<BN, STAGES>;
    auto kern = gemm_tc2_kernel<BN, STAGES>;
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        max_pairs = n / 2 > 0 ? n / 2 : 1;
    }
    const long long tiles = (long long)((M + PAIR_M - 1) / PAIR_M) * ((N + BN - 1) / BN);
    const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(T2_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sandy_pdl_enabled() ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mw, mo, ep, M, N, K, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// Arguments as sandy_gemm_tc; tile_n: 128 or 256 (0 = 256).
SANDY_API int sandy_gemm_tc2(const void* a, const void* w, const void* bias, const float* residual, void* out,
                             int M, int N, int K, int lda, int ldw, int ldr, int ldc, int act, int out_dtype,
                             int tile_n, void* k_cache, void* v_cache, long long page_stride, const int* block_table,
                             int max_blocks, const int* token_seq, const int* positions, int q_cols, int kv_cols,
                             int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || K <= 0) return SANDY_ERR_ARGUMENT;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    if (tile_n == 0) tile_n = 256;
    if (tile_n != 128 && tile_n != 256) return SANDY_ERR_UNSUPPORTED;
    CUtensorMap ma, mw;
    if (!get_map(a, M, K, lda, BM, &ma)) return SANDY_ERR_UNSUPPORTED;
    if (!get_map(w, N, K, ldw, tile_n / 2, &mw)) return SANDY_ERR_UNSUPPORTED;
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
    if (tile_n == 128) return launch_pair<128, 8>(ma, mw, mo, ep, M, N, K, status, stream);
    return launch_pair<256, 6>(ma, mw, mo, ep, M, N, K, status, stream);
}
