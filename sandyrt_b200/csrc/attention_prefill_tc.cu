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
//   softmax       two threads share query row r (tensor-memory lane r), one for each half of the
//                 tile's keys: each reads its 64 scores with tcgen05.ld, the two exchange
//                 their maxima through shared memory, then exp2, row sum, rounding to bfloat16,
//                 and each writes its half row of P into shared memory in the swizzled K-major
//                 layout an A operand has (eight warps instead of four halve the chain of
//                 dependent steps a tile costs, which is what bounds a causal block);
//   P V           a second chain (M 128, N 64, eight k-steps of 16 keys) with the value tile
//                 as an MN-major B operand: the values lie in shared memory as they lie in
//                 the cache, one key a row.  Its result goes to 64 further columns of tensor
//                 memory and is folded into the threads' float accumulators one tile later
//                 (o = o * exp2(m_old - m_new) + P V; each of a row's two threads keeps 32 of
//                 the 64 columns), so nothing in tensor memory is ever rescaled.
//
// The chains of a tile are issued by one thread, P.V of tile j followed at once by Q.K^T of
// tile j+1; one mbarrier (tcgen05.commit) tells all threads that both are done.  Keys and
// values come from the request's pages with 16-byte cp.async copies (zero fill for keys past
// the request's last position, so a poisoned page never meets a zero of P), one key tile and
// two value tiles deep: the next tile's copies are issued as soon as S of this tile is
// complete and overlap its softmax.  Two blocks fit an SM (97 KB of shared memory, 256
// columns of tensor memory each), so one block's softmax runs beside the other's products.
//
// Like every attention kernel here it reads all keys from the cache (the step's own keys are
// appended first): query i of a portion sits at position kv_before + i and sees keys
// max(0, pos+1-window) .. pos.  Softmax statistics and the output accumulators are float; P is
// rounded to bfloat16 for the product (the row sum is taken before rounding).
//
// Every wait on the mbarrier is bounded; a wait that runs out raises bit 8 of the status word
// and the block runs to its end without waiting again (its output is then not valid).
#include "tcgen05.cuh"

namespace {

constexpr int HD = 64;                  // head size
constexpr int BN = 128;                 // keys per tile
constexpr int THREADS = 256;
constexpr int TABLE_SMEM = 512;         // block-table entries kept in shared memory
constexpr uint32_t TMEM_COLS = 256;     // S: columns 0..127, P.V: columns 128..191
constexpr uint32_t TILE_BYTES = 128 * 128;       // 128 rows of 128 bytes
constexpr uint32_t OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = 2 * TILE_BYTES, OFF_P = 4 * TILE_BYTES;
constexpr uint32_t SMEM_BYTES = 6 * TILE_BYTES + 1024;   // + room to align to 1024 bytes

constexpr uint32_t IDESC_S = make_instr_desc(BN);
constexpr uint32_t IDESC_PV = make_instr_desc(HD) | (1u << 16);      // B operand MN-major

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

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
prefill_attention_tc_kernel(const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ k_cache,
                            const bf16* __restrict__ v_cache, long long page_stride,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ q_start,
                            const int* __restrict__ kv_before, bf16* __restrict__ out, int ld_out, int n_heads,
                            int n_kv_heads, int page_size, float scale, int window, int num_pages,
                            int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_table[TABLE_SMEM];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_failed;
    __shared__ float s_max[2][BM];      // what a row's two threads tell each other: maxima, at the end sums

    pdl_wait();
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
    const int kvh = h / (n_heads / n_kv_heads);
    const int* table = block_table + (size_t)s * max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int page_shift = __ffs(page_size) - 1, page_mask = page_size - 1;      // a power of two
    const int blocks_used = min(max_blocks, (pos_last >> page_shift) + 1);
    const bool table_staged = blocks_used <= TABLE_SMEM;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* const p_tile = smem_raw + (base - raw) + OFF_P;      // the P tile through an ordinary pointer
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V, sP = base + OFF_P;

    if (tid == 0) {
        mbar_init(&bar, 1);
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
    const uint32_t tmem_base = tmem_slot;
    const int row = tid & 127;              // the query row (and tensor-memory lane) of this thread
    const int half = tid >> 7;              // which 64 keys of a tile, which 32 columns of the output
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);      // this warp's 32 lanes

    // ---- copies ---------------------------------------------------------------------------
    // A tile row is 128 bytes (64 bfloat16); 16-byte piece c of row r lies at piece c ^ (r & 7).
    // Eight consecutive threads copy one row.
    const int cc = tid & 7;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = i * 32 + (tid >> 3);
        const bool ok = r < rows_valid;
        const bf16* src = q + (size_t)(qs + t0 + (ok ? r : 0)) * ld_q + h * HD + cc * 8;
        cp_async16(sQ + r * 128 + ((cc ^ (r & 7)) << 4), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int kt, uint32_t dst_v) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
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
            const uint32_t o = r * 128 + ((cc ^ (r & 7)) << 4);
            cp_async16(sK + o, k_cache + off, ok ? 16 : 0);
            cp_async16(dst_v + o, v_cache + off, ok ? 16 : 0);
        }
    };
    // ---- products (one thread issues them) ----------------------------------------------------
    auto issue_s = [&]() {
#pragma unroll
        for (int ks = 0; ks < HD / UMMA_K; ks++)
            umma_bf16(tmem_base, make_smem_desc(sQ + ks * 32), make_smem_desc(sK + ks * 32), IDESC_S, ks > 0);
    };
    auto issue_pv = [&](uint32_t v) {
#pragma unroll
        for (int ks = 0; ks < BN / UMMA_K; ks++)
            umma_bf16(tmem_base + BN, make_smem_desc(sP + (ks >> 2) * TILE_BYTES + (ks & 3) * 32),
                      make_smem_desc(v + ks * (UMMA_K * 128)), IDESC_PV, ks > 0);
    };
    auto wait_products = [&](uint32_t parity) {
        if (s_failed) return;
        if (!mbar_wait(&bar, parity)) {
            if (status) atomicOr(status, 256);
            s_failed = 1;
        }
    };

    load_kv(kt_begin, sV);
    cp_async_commit();
    cp_async_wait_all();
    fence_async_proxy();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        issue_s();
        umma_commit(&bar);
    }

    float o[HD / 2];
#pragma unroll
    for (int i = 0; i < HD / 2; i++) o[i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f, alpha = 0.0f;
    const float scale_log2 = scale * 1.4426950408889634f;
    const int pos = pos_first + row;
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;

    // o = o * alpha + (P V of the tile before), alpha being the factor that tile's maximum brought
    auto fold = [&]() {
        uint32_t r[32];
        tmem_ld_32x32(t_row + BN + half * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e++) o[e] = fmaf(o[e], alpha, __uint_as_float(r[e]));
    };

    for (int kt = kt_begin; kt <= kt_end; kt++) {
        const int it = kt - kt_begin;
        wait_products(it & 1);          // S of this tile, and P.V of the tile before, are complete
        tc_fence_after();
        uint32_t sa[32], sb[32];        // this thread's 64 scores
        tmem_ld_32x32(t_row + half * 64, sa);
        tmem_ld_32x32(t_row + half * 64 + 32, sb);
        if (kt < kt_end) load_kv(kt + 1, sV + ((it + 1) & 1) * TILE_BYTES);
        cp_async_commit();
        tmem_wait_ld();

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
        s_max[half][row] = mine;
        if (it > 0) fold();              // while the other half's maximum is on its way
        asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
        const float m_new = fmaxf(m_run, fmaxf(mine, s_max[half ^ 1][row]));
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;      // a row that has seen no key yet
        alpha = ex2((m_run - m_use) * scale_log2);                   // 0 on the row's first keys
        const float m_scaled = m_use * scale_log2;
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint8_t* blk = p_tile + half * TILE_BYTES + row * 128;
#pragma unroll
        for (int g = 0; g < 8; g++) {
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const uint32_t bits = g < 4 ? sa[8 * g + e] : sb[8 * (g - 4) + e];
                p[e] = ex2(fmaf(__uint_as_float(bits), scale_log2, -m_scaled));      // exp2(-inf) = 0: masked keys
                sum[e & 3] += p[e];
            }
            uint4 pk;
            pk.x = pack_bf16(p[0], p[1]);
            pk.y = pack_bf16(p[2], p[3]);
            pk.z = pack_bf16(p[4], p[5]);
            pk.w = pack_bf16(p[6], p[7]);
            *reinterpret_cast<uint4*>(blk + ((g ^ (row & 7)) << 4)) = pk;
        }
        l_run = l_run * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
        m_run = m_new;

        cp_async_wait_all();            // the next tile's keys and values have landed
        fence_async_proxy();            // ... and they and P are visible to the tensor cores
        tc_fence_before();
        __syncthreads();                // everyone has read S and the last P.V, and written P
        if (tid == 0) {
            tc_fence_after();
            issue_pv(sV + (it & 1) * TILE_BYTES);
            if (kt < kt_end) issue_s();
            umma_commit(&bar);
        }
    }
    wait_products((kt_end - kt_begin + 1) & 1);
    tc_fence_after();
    fold();
    pdl_launch_dependents();

    // ---- write back ----------------------------------------------------------------------------
    s_max[half][row] = l_run;           // the row's sum is the two halves' together
    tc_fence_before();
    __syncthreads();
    if (row < rows_valid) {
        const float l = l_run + s_max[half ^ 1][row];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        bf16* dst = out + (size_t)(qs + t0 + row) * ld_out + h * HD + half * 32;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            uint4 pk;
            pk.x = pack_bf16(o[8 * g] * inv, o[8 * g + 1] * inv);
            pk.y = pack_bf16(o[8 * g + 2] * inv, o[8 * g + 3] * inv);
            pk.z = pack_bf16(o[8 * g + 4] * inv, o[8 * g + 5] * inv);
            pk.w = pack_bf16(o[8 * g + 6] * inv, o[8 * g + 7] * inv);
            *reinterpret_cast<uint4*>(dst + 8 * g) = pk;
        }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
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
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_q_len + BM - 1) / BM, n_heads, n_seqs);
    return sandy_launch(prefill_attention_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, (const bf16*)q, ld_q,
                        (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table, max_blocks, q_start,
                        kv_before, (bf16*)out, ld_out, n_heads, n_kv_heads, page_size, scale, window, num_pages, status);
}
