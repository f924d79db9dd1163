// Causal attention of prompt portions over the paged cache on the tcgen05 tensor cores
// (bfloat16, heads of 64).
//
// Formula as in attention.cu (src/core/TensorCalc.cpp:1241-1311 of the reference; the
// reference's prefill kernel, flash_attention_prefill_kernel in
// src/device/cuda/CudaAttentionKernels.cu:91-244, forms every score with a warp-shuffle
// reduction on the ordinary pipes).  Here a block owns 128 consecutive new tokens of one
// (request, head) and walks the keys in tiles of 128:
//
//   S = Q K^T     one tcgen05.mma chain (M 128, N 128, four k-steps of 16), Q and the key tile
//                 in shared memory as K-major operands in the 128-byte swizzle, S in tensor
//                 memory (128 columns of float);
//   softmax       eight warps; two threads share query row r (tensor-memory lane r), one for each
//                 half of the tile's keys: each reads its 64 scores with tcgen05.ld, the two
//                 exchange their maxima through shared memory, then exp2, row sum, rounding to
//                 bfloat16, and each writes its half row of P back into tensor memory (64
//                 columns of bfloat16 pairs) with tcgen05.st;
//   O += P V      a second chain (M 128, N 64, eight k-steps of 16 keys) that takes P from
//                 tensor memory as its A operand and the value tile as an MN-major B operand
//                 (the values lie in shared memory as they lie in the cache, one key a row)
//                 and accumulates into 64 further columns of tensor memory over all tiles.
//
// The accumulator is rescaled where it lies, and only when it has to be: a row keeps the
// maximum its exponentials refer to until a tile's maximum exceeds it by more than 8 in the
// exponent (P then stays below 256, harmless for bfloat16 and the float sums); then the row's
// two threads multiply their columns of O and the row sum by exp2(old - new).  After the
// first tiles of a row this hardly happens.
//
// A ninth warp issues the products and the TMA copies, so that no softmax warp waits for the
// tensor pipe to take an instruction (a chain of dependent products of this size takes about
// 120 cycles an instruction): Q.K^T of tile j+1 as soon as every thread has read S of tile j,
// P.V of tile j when P is written; each has its own mbarrier (tcgen05.commit), and the warps
// tell each other with named barriers (bar.arrive / bar.sync).  A tile's softmax thus waits
// for neither product: S is ready before it starts, P.V runs beside the next tile's.
//
// Three key tiles and two value tiles are kept; keys are asked for three tiles ahead, into the
// tile S just left, values one tile ahead, into the tile the last P.V left.  How they come
// depends on where the request's pages lie.  A tile whose pages follow one another in the cache
// (page ids p, p+1, ...: what a pool hands out to a prompt unless it is fragmented) and that lies
// wholly inside the request is fetched by one TMA copy: a 3-D tensor map sees the cache as
// [page][head x slot][64], a box takes one head's rows of all the tile's pages, and the 128-byte
// swizzle the copy applies is the layout the operands need.  Any other tile (scattered pages;
// the request's last, partly filled tile) comes by 16-byte cp.async copies of the softmax
// threads, with zero fill for keys past the request's last position, so that a poisoned slot
// never meets a zero of P.  These hold the warps up (each copy instruction of a warp takes
// about 300 cycles to be taken up, however few are in flight); one TMA copy per page was tried
// too and is slower still (about 100 ns a copy, sixteen a tile).  Two blocks fit an SM (106 KB
// of shared memory, 256 columns of tensor memory, 288 threads of 96 registers each).
//
// Like every attention kernel here it reads all keys from the cache (the step's own keys are
// appended first): query i of a portion sits at position kv_before + i and sees keys
// max(0, pos+1-window) .. pos.  Softmax statistics and the accumulator are float; P is rounded
// to bfloat16 for the product (the row sum is taken before rounding).
//
// Every wait on an mbarrier is bounded; a wait that runs out raises bit 8 of the status word
// and the block runs to its end without waiting again (its output is then not valid).
#include <cstring>
#include <utility>
#include <vector>

#include "tcgen05.cuh"

namespace {

constexpr int HD = 64;                  // head size
constexpr int BN = 128;                 // keys per tile
constexpr int SOFTMAX_THREADS = 256;    // eight warps
constexpr int THREADS = 288;            // ... and one that issues the products and the TMA copies
constexpr int ISSUE_THREAD = 256;
// named barriers (0 is __syncthreads)
constexpr int BAR_MAX = 1;              // the softmax threads: maxima (at the end: sums) are in shared memory
constexpr int BAR_S_READ = 2;           // softmax threads arrive, the issuing warp waits: S has been read
constexpr int BAR_P_READY = 3;          // softmax threads arrive, the issuing warp waits: P is written
constexpr float RESCALE_LOG2 = 8.0f;    // how far (in the exponent) a row's maximum may run ahead of its reference
constexpr int TABLE_SMEM = 1024;        // block-table entries kept in shared memory
constexpr int RUNS_SMEM = 128;          // key tiles whose first page (if their pages are a run) is kept
constexpr uint32_t TMEM_COLS = 256;     // S: columns 0..127, O: 128..191, P (bfloat16 pairs): 192..255
constexpr uint32_t O_COL = 128, P_COL = 192;
constexpr uint32_t TILE_BYTES = 128 * 128;       // 128 rows of 128 bytes
constexpr int K_TILES = 3, V_TILES = 2;
constexpr uint32_t OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = (1 + K_TILES) * TILE_BYTES;
constexpr uint32_t SMEM_BYTES = (1 + K_TILES + V_TILES) * TILE_BYTES + 1024;   // + room to align to 1024 bytes

constexpr uint32_t IDESC_S = make_instr_desc(BN);
constexpr uint32_t IDESC_PV = make_instr_desc(HD) | (1u << 16);      // B operand MN-major

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_two() { asm volatile("cp.async.wait_group 2;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// tensor-core product with the A operand in tensor memory
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One head's rows of `pages` consecutive pages, starting at page `page`: box [pages][page_size][64].
__device__ __forceinline__ void tma_pages(uint32_t dst, const CUtensorMap* map, int head_row, int page, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(0), "r"(head_row), "r"(page)
        : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ k_cache,
                            const bf16* __restrict__ v_cache, long long page_stride,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ q_start,
                            const int* __restrict__ kv_before, bf16* __restrict__ out, int ld_out, int n_heads,
                            int n_kv_heads, int page_size, float scale, int window, int num_pages,
                            int use_tma, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_table[TABLE_SMEM];
    __shared__ int s_run[RUNS_SMEM];    // per key tile: its first page if TMA fetches it, else -1
    __shared__ uint64_t bar_s, bar_pv, bar_k[K_TILES], bar_v[V_TILES];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_failed;
    __shared__ float s_max[2][2][BM];   // the maxima a row's two threads tell each other (two copies, used in turn)
    __shared__ float s_sum[2][BM];      // ... and at the end their sums

    // Which tokens and pages a block works on is written by the host before the step; only q and the
    // caches are the predecessor's output.  So the set-up below (barriers, tensor memory, the
    // request's block table, the run marks) runs while the kernel before is still finishing.
    const int s = blockIdx.z, h = blockIdx.y;
    const int qs = q_start[s];
    const int q_len = q_start[s + 1] - qs;
    const int n_tiles = (q_len + BM - 1) / BM;
    if ((int)blockIdx.x >= n_tiles) return;
    const int tile = n_tiles - 1 - blockIdx.x;         // the tiles with the most keys start first
    const int t0 = tile * BM;
    const int rows_valid = min(BM, q_len - t0);
    const int before = kv_before[s];
    const int pos_first = before + t0;
    const int pos_last = pos_first + rows_valid - 1;
    const int key_lo = window > 0 ? max(0, pos_first + 1 - window) : 0;
    const int kt_begin = key_lo / BN, kt_end = pos_last / BN;
    const int n_it = kt_end - kt_begin + 1;
    const int kvh = h / (n_heads / n_kv_heads);
    const int* table = block_table + (size_t)s * max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5;
    const bool softmax = tid < SOFTMAX_THREADS;
    const int page_shift = __ffs(page_size) - 1, page_mask = page_size - 1;      // a power of two
    const int blocks_used = min(max_blocks, (pos_last >> page_shift) + 1);
    const bool table_staged = blocks_used <= TABLE_SMEM;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V;

    if (tid == 0) {
        mbar_init(&bar_s, 1);
        mbar_init(&bar_pv, 1);
        for (int i = 0; i < K_TILES; i++) mbar_init(&bar_k[i], 1);
        for (int i = 0; i < V_TILES; i++) mbar_init(&bar_v[i], 1);
        s_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (table_staged)
        for (int i = tid; i < blocks_used; i += THREADS) s_table[i] = table[i];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Which key tiles TMA fetches: all keys inside the request, all pages there and one after another.
    const int pages_per_tile = BN >> page_shift;
    const bool runs_known = table_staged && n_it <= RUNS_SMEM && use_tma;
    if (runs_known) {
        for (int t = tid; t < n_it; t += THREADS) {
            const int kt = kt_begin + t;
            const int b0 = kt * pages_per_tile;
            int first = -1;
            if (kt * BN + BN - 1 <= pos_last && b0 + pages_per_tile <= max_blocks) {
                first = s_table[b0];
                for (int i = 1; i < pages_per_tile; i++)
                    if (s_table[b0 + i] != first + i) first = -1;
                if (first < 0 || first + pages_per_tile > num_pages) first = -1;
            }
            s_run[t] = first;
        }
        __syncthreads();
    }
    const uint32_t tmem_base = tmem_slot;
    pdl_wait();             // from here on q and the caches are read

    // ---- copies ---------------------------------------------------------------------------
    // A tile row is 128 bytes (64 bfloat16); 16-byte piece c of row r lies at piece c ^ (r & 7).
    // Eight consecutive softmax threads copy one row; a thread copies piece cc of rows i * 32 + tid / 8.
    const int cc = tid & 7;
    if (softmax) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = i * 32 + (tid >> 3);
            const bool ok = r < rows_valid;
            const bf16* src = q + (size_t)(qs + t0 + (ok ? r : 0)) * ld_q + h * HD + cc * 8;
            cp_async16(sQ + r * 128 + ((cc ^ (r & 7)) << 4), src, ok ? 16 : 0);
        }
    }
    // this thread's i-th piece of tile kt of the keys or of the values
    auto load_piece = [&](const bf16* cache, uint32_t dst, int kt, int i) {
        const int r = i * 32 + (tid >> 3);
        const int j = kt * BN + r;
        bool ok = j <= pos_last;
        size_t off = 0;
        if (ok) {
            const int b = j >> page_shift;
            const int page = b < max_blocks ? (table_staged ? s_table[b] : table[b]) : -1;
            if (page < 0 || page >= num_pages) {
                // a key with no page behind it; inside the visible range this is a fault
                if (j >= key_lo && status && cc == 0) atomicOr(status, 16);
                ok = false;
            } else {
                off = (size_t)page * page_stride + ((size_t)kvh * page_size + (j & page_mask)) * HD + cc * 8;
            }
        }
        cp_async16(dst + r * 128 + ((cc ^ (r & 7)) << 4), cache + off, ok ? 16 : 0);
    };
    auto k_tile = [&](int t) { return sK + (uint32_t)(t % K_TILES) * TILE_BYTES; };
    auto v_tile = [&](int t) { return sV + (uint32_t)(t % V_TILES) * TILE_BYTES; };
    // Tile number t of the keys / of the values.  Every thread calls this, each when it knows the
    // tile's place in shared memory to be free: if the tile's pages are a run, the issuing thread
    // starts one TMA copy; else the softmax threads copy their pieces and the issuing thread
    // lets the tile's mbarrier pass at once (what the threads copy is waited for as cp.async
    // groups; every call closes one group of a softmax thread).
    auto load_k = [&](int t) {
        const int first = runs_known ? s_run[t] : -1;
        if (tid == ISSUE_THREAD) {
            if (first >= 0) {
                mbar_expect_tx(&bar_k[t % K_TILES], TILE_BYTES);
                tma_pages(k_tile(t), &map_k, kvh * page_size, first, &bar_k[t % K_TILES]);
            } else {
                mbar_arrive(&bar_k[t % K_TILES]);
            }
        } else if (softmax) {
            if (first < 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) load_piece(k_cache, k_tile(t), kt_begin + t, i);
            }
            cp_async_commit();
        }
    };
    auto load_v = [&](int t) {
        const int first = runs_known ? s_run[t] : -1;
        if (tid == ISSUE_THREAD) {
            if (first >= 0) {
                mbar_expect_tx(&bar_v[t % V_TILES], TILE_BYTES);
                tma_pages(v_tile(t), &map_v, kvh * page_size, first, &bar_v[t % V_TILES]);
            } else {
                mbar_arrive(&bar_v[t % V_TILES]);
            }
        } else if (softmax) {
            if (first < 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) load_piece(v_cache, v_tile(t), kt_begin + t, i);
            }
            cp_async_commit();
        }
    };
    auto wait_for = [&](uint64_t* bar, uint32_t parity) {
        if (s_failed) return;
        if (!mbar_wait(bar, parity)) {
            if (status) atomicOr(status, 256);
            s_failed = 1;
        }
    };

    // the first tiles: keys 0..2, values 0
    load_k(0);
    load_v(0);
    for (int t = 1; t < K_TILES && t < n_it; t++) load_k(t);
    cp_async_commit();
    cp_async_wait_all();
    fence_async_proxy();
    __syncthreads();

    if (!softmax) {
        // ---- the issuing warp --------------------------------------------------------------------
        const bool me = tid == ISSUE_THREAD;
        auto issue_s = [&](uint32_t k) {
#pragma unroll
            for (int ks = 0; ks < HD / UMMA_K; ks++)
                umma_bf16(tmem_base, make_smem_desc(sQ + ks * 32), make_smem_desc(k + ks * 32), IDESC_S, ks > 0);
        };
        auto issue_pv = [&](uint32_t v, bool first_tile) {
#pragma unroll
            for (int ks = 0; ks < BN / UMMA_K; ks++)
                umma_bf16_ta(tmem_base + O_COL, tmem_base + P_COL + ks * (UMMA_K / 2),
                             make_smem_desc(v + ks * (UMMA_K * 128)), IDESC_PV, !first_tile || ks > 0);
        };
        if (me) {
            wait_for(&bar_k[0], 0);
            tc_fence_after();
            issue_s(k_tile(0));
            umma_commit(&bar_s);
        }
        for (int it = 0; it < n_it; it++) {
            bar_sync(BAR_S_READ, THREADS);          // every thread has read S of this tile
            if (me) {
                tc_fence_after();
                if (it + 1 < n_it) {
                    wait_for(&bar_k[(it + 1) % K_TILES], ((it + 1) / K_TILES) & 1);      // landed a tile ago
                    tc_fence_after();
                    issue_s(k_tile(it + 1));
                    umma_commit(&bar_s);
                }
                if (it + K_TILES < n_it) load_k(it + K_TILES);      // into the tile S just left
                if (it + 1 < n_it) {
                    if (it > 0) wait_for(&bar_pv, (it - 1) & 1);    // into the tile the last P.V left
                    load_v(it + 1);
                }
            }
            __syncwarp();
            bar_sync(BAR_P_READY, THREADS);         // P of this tile is written
            if (me) {
                wait_for(&bar_v[it % V_TILES], (it / V_TILES) & 1);
                tc_fence_after();
                issue_pv(v_tile(it), it == 0);
                umma_commit(&bar_pv);
            }
            __syncwarp();
        }
        pdl_launch_dependents();
    } else {
        // ---- the softmax warps -------------------------------------------------------------------
        const int row = tid & 127;              // the query row (and tensor-memory lane) of this thread
        const int half = tid >> 7;              // which 64 keys of a tile, which 32 columns of the output
        const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);      // this warp's 32 lanes
        float m_ref = -INFINITY, l_run = 0.0f;  // the maximum the row's exponentials refer to; the row's sum
        const float scale_log2 = scale * 1.4426950408889634f;
        const int pos = pos_first + row;
        const int lo = window > 0 ? max(0, pos + 1 - window) : 0;

        for (int it = 0; it < n_it; it++) {
            const int kt = kt_begin + it;
            wait_for(&bar_s, it & 1);       // S of this tile is complete
            tc_fence_after();
            if (it + K_TILES < n_it) load_k(it + K_TILES); else cp_async_commit();      // into the tile S just left
            uint32_t sa[32], sb[32];        // this thread's 64 scores; later its 64 values of P, as pairs, in sa
            tmem_ld_32x32(t_row + half * 64, sa);
            tmem_ld_32x32(t_row + half * 64 + 32, sb);
            tmem_wait_ld();
            tc_fence_before();
            bar_arrive(BAR_S_READ, THREADS);

            // a tile every row of the block sees whole needs no mask
            const bool whole = kt * BN + BN - 1 <= pos_first && (window == 0 || kt * BN >= pos_last + 1 - window);
            const int j0 = kt * BN + half * 64;
            if (!whole) {
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    if (j0 + e > pos || j0 + e < lo) sa[e] = __float_as_uint(-INFINITY);
                    if (j0 + 32 + e > pos || j0 + 32 + e < lo) sb[e] = __float_as_uint(-INFINITY);
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < 32; e++) {
                mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(sa[e]));
                mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(sb[e]));
            }
            const float mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            s_max[it & 1][half][row] = mine;
            bar_sync(BAR_MAX, SOFTMAX_THREADS);
            const float m_new = fmaxf(m_ref, fmaxf(mine, s_max[it & 1][half ^ 1][row]));
            // The row's reference moves only when the maximum has run far ahead of it (always on the
            // row's first keys: -inf).  Then O and the sum are brought to the new reference; a warp
            // does this together, rows that need not move multiply by one.
            const bool move = (m_new - m_ref) * scale_log2 > RESCALE_LOG2;
            if (__any_sync(0xffffffffu, move)) {
                const float alpha = move ? ex2((m_ref - m_new) * scale_log2) : 1.0f;      // 0 on the row's first keys
                if (it > 0) {
                    wait_for(&bar_pv, (it - 1) & 1);      // O is at rest: the last P.V is complete, the next not issued
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t r[16];
                        tmem_ld_32x16(t_row + O_COL + half * 32 + c * 16, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 16; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                        tmem_st_32x16(t_row + O_COL + half * 32 + c * 16, r);
                    }
                    tmem_wait_st();
                }
                l_run *= alpha;
                if (move) m_ref = m_new;
            }
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;      // a row that has seen no key yet
            const float m_scaled = m_use * scale_log2;
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int g = 0; g < 8; g++) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const uint32_t bits = g < 4 ? sa[8 * g + e] : sb[8 * (g - 4) + e];
                    p[e] = ex2(fmaf(__uint_as_float(bits), scale_log2, -m_scaled));      // exp2(-inf) = 0: masked keys
                    sum[e & 3] += p[e];
                }
                sa[4 * g] = pack_bf16(p[0], p[1]);
                sa[4 * g + 1] = pack_bf16(p[2], p[3]);
                sa[4 * g + 2] = pack_bf16(p[4], p[5]);
                sa[4 * g + 3] = pack_bf16(p[6], p[7]);
            }
            l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            // P and the other value tile are free once P.V of the tile before is complete
            if (it > 0) {
                wait_for(&bar_pv, (it - 1) & 1);
                tc_fence_after();
            }
            if (it + 1 < n_it) load_v(it + 1); else cp_async_commit();
            tmem_st_32x32(t_row + P_COL + half * 32, sa);
            tmem_wait_st();
            cp_async_wait_but_two();        // what the threads copied a tile ago has landed: this tile's values
            fence_async_proxy();            // ... and is visible to the tensor cores
            tc_fence_before();
            bar_arrive(BAR_P_READY, THREADS);
        }
        wait_for(&bar_pv, (n_it - 1) & 1);
        tc_fence_after();
        cp_async_wait_all();
        pdl_launch_dependents();

        // ---- write back ----------------------------------------------------------------------------
        s_sum[half][row] = l_run;           // the row's sum is the two halves' together
        uint32_t r[32];
        tmem_ld_32x32(t_row + O_COL + half * 32, r);
        tmem_wait_ld();
        bar_sync(BAR_MAX, SOFTMAX_THREADS);
        if (row < rows_valid) {
            const float l = l_run + s_sum[half ^ 1][row];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = out + (size_t)(qs + t0 + row) * ld_out + h * HD + half * 32;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                uint4 pk;
                pk.x = pack_bf16(__uint_as_float(r[8 * g]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
                pk.y = pack_bf16(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
                pk.z = pack_bf16(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
                pk.w = pack_bf16(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
                *reinterpret_cast<uint4*>(dst + 8 * g) = pk;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// The cache as a 3-D tensor [page][head x slot][64] for boxes of one head's rows of the pages of a key
// tile.  Encoded maps are kept: the caches of a model stay where they are.
struct PageMapKey {
    const void* ptr;
    long long page_stride;
    int num_pages, n_kv_heads, page_size;
    bool operator==(const PageMapKey& o) const {
        return ptr == o.ptr && page_stride == o.page_stride && num_pages == o.num_pages &&
               n_kv_heads == o.n_kv_heads && page_size == o.page_size;
    }
};

bool get_page_map(const void* cache, long long page_stride, int num_pages, int n_kv_heads, int page_size,
                  CUtensorMap* out) {
    static std::vector<std::pair<PageMapKey, CUtensorMap>> cache_maps;
    static std::mutex mu;
    const PageMapKey key{cache, page_stride, num_pages, n_kv_heads, page_size};
    std::lock_guard<std::mutex> g(mu);
    for (const auto& e : cache_maps)
        if (e.first == key) {
            *out = e.second;
            return true;
        }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)n_kv_heads * page_size, (cuuint64_t)num_pages};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[3] = {(cuuint32_t)HD, (cuuint32_t)page_size, (cuuint32_t)(BN / page_size)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache_maps.size() > 256) cache_maps.clear();
    cache_maps.emplace_back(key, m);
    *out = m;
    return true;
}

}  // namespace

// Arguments as sandy_prefill_attention (attention_prefill.cu).  Heads of 64 only; out and q rows
// must be 16-byte aligned.  SANDY_ERR_UNSUPPORTED for everything else: the caller then takes the
// mma.sync kernel.
SANDY_API int sandy_prefill_attention_tc(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                         long long page_stride, const int* block_table, int max_blocks,
                                         const int* q_start, const int* kv_before, void* out, int ld_out, int n_seqs,
                                         int max_q_len, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                         float scale, int window, int num_pages, int* status, cudaStream_t stream) {
    if (n_seqs == 0 || max_q_len == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !q_start || !kv_before || !out) return SANDY_ERR_ARGUMENT;
    if (head_dim != HD) return SANDY_ERR_UNSUPPORTED;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (page_size & (page_size - 1)) return SANDY_ERR_UNSUPPORTED;      // pages are a power of two long
    if (n_heads > 65535 || n_seqs > 65535) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return SANDY_ERR_UNSUPPORTED;
    if (ld_q % 8 != 0 || page_stride % 8 != 0 || ld_out % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    // TMA fetches whole key tiles where it can: pages of 8 to 128 positions (a box row group of the
    // 128-byte swizzle is 8 rows; a tile is 128 keys)
    CUtensorMap mk, mv;
    int use_tma = page_size >= 8 && page_size <= BN && num_pages > 0 && (long long)n_kv_heads * page_size < (1ll << 31) &&
                  get_page_map(k_cache, page_stride, num_pages, n_kv_heads, page_size, &mk) &&
                  get_page_map(v_cache, page_stride, num_pages, n_kv_heads, page_size, &mv);
    if (!use_tma) {
        memset(&mk, 0, sizeof(mk));
        memset(&mv, 0, sizeof(mv));
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_q_len + BM - 1) / BM, n_heads, n_seqs);
    return sandy_launch(prefill_attention_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mk, mv, (const bf16*)q, ld_q,
                        (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table, max_blocks, q_start,
                        kv_before, (bf16*)out, ld_out, n_heads, n_kv_heads, page_size, scale, window, num_pages, use_tma,
                        status);
}
