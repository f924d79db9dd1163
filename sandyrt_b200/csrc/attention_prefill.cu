// Causal attention of prompt portions over the paged cache on tensor cores (bfloat16).
//
// Formula as in attention.cu (src/core/TensorCalc.cpp:1241-1311 of the reference).  The
// reference's prefill kernel gives each query its own warp and forms every score with a
// warp-shuffle reduction on the ordinary pipes (flash_attention_prefill_kernel,
// src/device/cuda/CudaAttentionKernels.cu:91-244).  Here a block owns 64 consecutive new
// tokens of one (request, head); Q.K^T and P.V run as warp-level matrix instructions
// (mma.sync m16n8k16, bfloat16 in, float accumulate), the softmax is the online form carried
// in float registers, and key/value tiles of 64 positions stream from the request's pages
// into shared memory with cp.async through a ring of three buffers (one block-wide barrier per
// tile).  The request's row of the block table is copied to shared memory once, so finding a
// key's page costs no trip to global memory inside the loop.
//
// Like every attention kernel here it reads all keys from the cache (the step's own keys are
// appended first), the prefix a request already had and the portion it brings alike, so a
// portion that starts in the middle of a prompt needs nothing special: query i of the
// portion sits at position kv_before + i and sees keys max(0, pos+1-window) .. pos.
// A request that brings a single token is just a tile with one live row.
//
// A block has eight warps: four row groups of 16 queries, each served by two warps that take
// one half of every key tile (32 keys) and keep their own running (max, sum, output); the two
// halves are merged through shared memory at the end.  This doubles the warps that work on a
// tile's chain of dependent steps, which is what bounds a causal block with many key tiles.
//
// P is rounded to bfloat16 for the P.V product (the row sum is taken before rounding).
// Head sizes: multiples of 16 up to 128.  Larger heads, and float32, use the general kernel.
#include "common.cuh"

namespace {

constexpr int BM = 64;          // queries per block (16 per warp)
constexpr int BN = 64;          // keys per tile
constexpr int KSPLIT = 2;        // warp groups that share a query tile and split each key tile between them
constexpr int BNW = BN / KSPLIT; // keys of a tile one warp works on
constexpr int THREADS = 128 * KSPLIT;
constexpr int STAGES = 3;       // key/value tiles in flight
constexpr int TABLE_SMEM = 1024; // block-table entries kept in shared memory (longer rows are read from global)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy; with src_bytes == 0 the destination is filled with zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(p)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(THREADS)
prefill_attention_kernel(const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, long long page_stride,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ q_start,
                         const int* __restrict__ kv_before, bf16* __restrict__ out, int ld_out, int n_heads,
                         int n_kv_heads, int page_size, float scale, int window, int num_pages,
                         int* __restrict__ status) {
    constexpr int LDS = D + 8;               // row pitch in elements: 16 bytes of padding
    constexpr int CHUNKS = D / 8;            // 16-byte pieces per row
    constexpr int KSTEPS = D / 16;           // k-steps of Q.K^T
    constexpr int DTILES = D / 8;            // 8-wide column tiles of the output
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + BM * LDS;                // [STAGES][BN][LDS]
    bf16* sV = sK + STAGES * BN * LDS;       // [STAGES][BN][LDS]
    __shared__ int s_table[TABLE_SMEM];

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
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int page_shift = __ffs(page_size) - 1, page_mask = page_size - 1;      // a power of two
    const int blocks_used = min(max_blocks, (pos_last >> page_shift) + 1);
    const bool table_staged = blocks_used <= TABLE_SMEM;
    if (table_staged) {
        for (int i = tid; i < blocks_used; i += THREADS) s_table[i] = table[i];
        __syncthreads();
    }

    // ---- Q tile -------------------------------------------------------------------------
    for (int idx = tid; idx < BM * CHUNKS; idx += THREADS) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        const bool ok = r < rows_valid;
        const bf16* src = q + (size_t)(qs + t0 + (ok ? r : 0)) * ld_q + h * D + c * 8;
        cp_async16(sQ + r * LDS + c * 8, src, ok ? 16 : 0);
    }
    auto load_kv = [&](int kt, int buf) {
        bf16* dk = sK + buf * BN * LDS;
        bf16* dv = sV + buf * BN * LDS;
        for (int idx = tid; idx < BN * CHUNKS; idx += THREADS) {
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            const int j = kt * BN + r;
            bool ok = j <= pos_last;
            size_t off = 0;
            if (ok) {
                const int b = j >> page_shift;
                const int page = b < max_blocks ? (table_staged ? s_table[b] : table[b]) : -1;
                if (page < 0 || page >= num_pages) {
                    // a key with no page behind it; inside the visible range this is a fault
                    if (j >= key_lo && status && c == 0) atomicOr(status, 16);
                    ok = false;
                } else {
                    off = (size_t)page * page_stride + ((size_t)kvh * page_size + (j & page_mask)) * D + c * 8;
                }
            }
            cp_async16(dk + r * LDS + c * 8, k_cache + off, ok ? 16 : 0);
            cp_async16(dv + r * LDS + c * 8, v_cache + off, ok ? 16 : 0);
        }
    };
    load_kv(kt_begin, 0);
    cp_async_commit();
    if (kt_begin < kt_end) load_kv(kt_begin + 1, 1);
    cp_async_commit();

    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float scale_log2 = scale * 1.4426950408889634f;
    // positions of this thread's two rows (g and g+8 of the warp's 16)
    const int rgroup = warp & 3, khalf = warp >> 2;          // which 16 rows, which half of each key tile
    const int row0 = rgroup * 16 + g, row1 = row0 + 8;
    const int pos0 = pos_first + row0, pos1 = pos_first + row1;
    const int lo0 = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int lo1 = window > 0 ? max(0, pos1 + 1 - window) : 0;

    uint32_t qa[KSTEPS][4];
    bool q_loaded = false;

    for (int kt = kt_begin; kt <= kt_end; kt++) {
        const int buf = (kt - kt_begin) % STAGES;
        cp_async_wait<1>();          // tile kt has landed (tile kt+1 may still be on its way)
        __syncthreads();             // ... for everyone; and everyone is done with tile kt-1
        if (kt + 2 <= kt_end) load_kv(kt + 2, (kt + 2 - kt_begin) % STAGES);     // into tile kt-1's buffer
        cp_async_commit();
        if (!q_loaded) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; kk++)
                ldmatrix_x4(qa[kk], sQ + (rgroup * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 16 + (lane >> 4) * 8);
            q_loaded = true;
        }
        const bf16* tk = sK + (buf * BN + khalf * BNW) * LDS;      // this warp's half of the tile
        const bf16* tv = sV + (buf * BN + khalf * BNW) * LDS;

        // ---- S = Q K^T : 16 x 32 per warp ------------------------------------------------
        float sc[BNW / 8][4];
#pragma unroll
        for (int i = 0; i < BNW / 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) sc[i][j] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++) {
#pragma unroll
            for (int nt = 0; nt < BNW / 8; nt += 2) {
                uint32_t kb[4];
                ldmatrix_x4(kb, tk + (nt * 8 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(sc[nt], qa[kk], kb[0], kb[1]);
                mma_bf16(sc[nt + 1], qa[kk], kb[2], kb[3]);
            }
        }
        // ---- mask, online softmax --------------------------------------------------------
        float m_new[2] = {m_run[0], m_run[1]};
        // a tile every row of the block sees whole needs no mask (all tiles but the last one
        // or two of a causal block, when there is no window)
        const bool whole = kt * BN + BN - 1 <= pos_first && (window == 0 || kt * BN >= pos_last + 1 - window);
#pragma unroll
        for (int nt = 0; nt < BNW / 8; nt++) {
            if (whole) {
#pragma unroll
                for (int e = 0; e < 4; e++) sc[nt][e] *= scale_log2;
            } else {
                const int j0 = kt * BN + khalf * BNW + nt * 8 + 2 * t;
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int j = j0 + e;
                    sc[nt][e] = (j <= pos0 && j >= lo0) ? sc[nt][e] * scale_log2 : -INFINITY;
                    sc[nt][2 + e] = (j <= pos1 && j >= lo1) ? sc[nt][2 + e] * scale_log2 : -INFINITY;
                }
            }
            m_new[0] = fmaxf(m_new[0], fmaxf(sc[nt][0], sc[nt][1]));
            m_new[1] = fmaxf(m_new[1], fmaxf(sc[nt][2], sc[nt][3]));
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            msafe[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];   // a row that has seen no key yet
            corr[r] = exp2f(m_run[r] - msafe[r]);                 // exp2(-inf) = 0 on the first tile
            m_run[r] = m_new[r];
        }
        float l_add[2] = {0.0f, 0.0f};
        uint32_t pa[BNW / 16][4];
#pragma unroll
        for (int nt = 0; nt < BNW / 8; nt++) {
            const float p0 = exp2f(sc[nt][0] - msafe[0]), p1 = exp2f(sc[nt][1] - msafe[0]);
            const float p2 = exp2f(sc[nt][2] - msafe[1]), p3 = exp2f(sc[nt][3] - msafe[1]);
            l_add[0] += p0 + p1;
            l_add[1] += p2 + p3;
            // C layout of two neighbouring 8-wide tiles is the A layout of one 16-wide k-step
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            l_add[r] += __shfl_xor_sync(0xffffffffu, l_add[r], 1);
            l_add[r] += __shfl_xor_sync(0xffffffffu, l_add[r], 2);
            l_run[r] = l_run[r] * corr[r] + l_add[r];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; dt++) {
            o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
            o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
        }
        // ---- O += P V --------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < BNW / 16; kk++) {
#pragma unroll
            for (int dt = 0; dt < DTILES; dt += 2) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, tv + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + dt * 8 + (lane >> 4) * 8);
                mma_bf16(o[dt], pa[kk], vb[0], vb[1]);
                mma_bf16(o[dt + 1], pa[kk], vb[2], vb[3]);
            }
        }
    }
    cp_async_wait<0>();

    // ---- merge the two key halves of every row group (the tile buffers are free now) ------
    __syncthreads();
    float* mrg = reinterpret_cast<float*>(sK);               // [4 row groups][32 lanes][DTILES*4 + 4]
    constexpr int MRG = DTILES * 4 + 4;
    if (khalf == 1) {
        float* dst = mrg + (size_t)(rgroup * 32 + lane) * MRG;
#pragma unroll
        for (int dt = 0; dt < DTILES; dt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dst[dt * 4 + e] = o[dt][e];
        dst[DTILES * 4 + 0] = m_run[0]; dst[DTILES * 4 + 1] = m_run[1];
        dst[DTILES * 4 + 2] = l_run[0]; dst[DTILES * 4 + 3] = l_run[1];
    }
    __syncthreads();
    if (khalf == 1) return;
    {
        const float* src = mrg + (size_t)(rgroup * 32 + lane) * MRG;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float m_o = src[DTILES * 4 + r], l_o = src[DTILES * 4 + 2 + r];
            const float m_all = fmaxf(m_run[r], m_o);
            const float msafe = m_all == -INFINITY ? 0.0f : m_all;
            const float wa = exp2f(m_run[r] - msafe), wb = exp2f(m_o - msafe);
            l_run[r] = l_run[r] * wa + l_o * wb;
#pragma unroll
            for (int dt = 0; dt < DTILES; dt++) {
                o[dt][2 * r] = o[dt][2 * r] * wa + src[dt * 4 + 2 * r] * wb;
                o[dt][2 * r + 1] = o[dt][2 * r + 1] * wa + src[dt * 4 + 2 * r + 1] * wb;
            }
        }
    }

    // ---- write back ----------------------------------------------------------------------
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f;
    const float inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
#pragma unroll
    for (int dt = 0; dt < DTILES; dt++) {
        const int col = h * D + dt * 8 + 2 * t;
        if (row0 < rows_valid)
            *reinterpret_cast<uint32_t*>(out + (size_t)(qs + t0 + row0) * ld_out + col) =
                pack_bf16(o[dt][0] * inv0, o[dt][1] * inv0);
        if (row1 < rows_valid)
            *reinterpret_cast<uint32_t*>(out + (size_t)(qs + t0 + row1) * ld_out + col) =
                pack_bf16(o[dt][2] * inv1, o[dt][3] * inv1);
    }
}

template <int D>
int launch(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
           const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out, int ld_out,
           int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int page_size, float scale, int window,
           int num_pages, int* status, cudaStream_t stream) {
    constexpr int LDS = D + 8;
    const int smem = (BM + 2 * STAGES * BN) * LDS * (int)sizeof(bf16);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_q_len + BM - 1) / BM, n_heads, n_seqs);
    prefill_attention_kernel<D><<<grid, THREADS, smem, stream>>>(
        (const bf16*)q, ld_q, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table, max_blocks, q_start,
        kv_before, (bf16*)out, ld_out, n_heads, n_kv_heads, page_size, scale, window, num_pages, status);
    return sandy_launch_status();
}

}  // namespace

// q, out: bfloat16 [n_tokens, H*D]; q_start: int32 [n_seqs + 1], first new token of each request;
// kv_before: int32 [n_seqs], tokens each request had in the cache before the step;
// max_q_len: the longest portion (sizes the grid).  Caches as in attention.cu.
SANDY_API int sandy_prefill_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                      long long page_stride, const int* block_table, int max_blocks,
                                      const int* q_start, const int* kv_before, void* out, int ld_out, int n_seqs,
                                      int max_q_len, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                      float scale, int window, int num_pages, int* status, cudaStream_t stream) {
    if (n_seqs == 0 || max_q_len == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !q_start || !kv_before || !out) return SANDY_ERR_ARGUMENT;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (page_size & (page_size - 1)) return SANDY_ERR_UNSUPPORTED;      // pages are a power of two long
    if (n_heads > 65535 || n_seqs > 65535) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 3))
        return SANDY_ERR_UNSUPPORTED;
    if (ld_q % 8 != 0 || page_stride % 8 != 0 || ld_out % 2 != 0) return SANDY_ERR_UNSUPPORTED;
#define CASE(DD)                                                                                                \
    if (head_dim == DD)                                                                                         \
        return launch<DD>(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, q_start, kv_before,  \
                          out, ld_out, n_seqs, max_q_len, n_heads, n_kv_heads, page_size, scale, window,        \
                          num_pages, status, stream)
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}
