// Attention of single tokens over the paged cache on the warp-level tensor-core instruction
// (bfloat16, heads of 64): the split-KV computation of attention_decode.cu with the dot products
// and the weighted sums as mma.sync m16n8k16 products.
//
// Why.  In attention_decode.cu and attention_decode_bulk.cu every score is eight to sixteen FMAs and
// a few shuffles on the ordinary pipes, every weighted sum as many FMAs again, and each 16-byte
// piece of a key is first turned into floats.  With hundreds of (token, head) pairs that arithmetic,
// not memory, bounds the kernel (64 requests x 400 keys x 12 heads: 17 us whether the cache comes
// from HBM or from L2, against 12 us for the bytes at the measured copy rate).  A query is one row;
// the instruction wants sixteen, so fifteen rows of every product are zeros -- the tensor cores have
// that to spare, and the instruction count per key falls to a quarter.
//
// Formula as in attention.cu (src/core/TensorCalc.cpp:1241-1311 of the reference).  Block (split,
// head, token): keys [begin, end) of the token's visible range in groups of 16; each of the four
// warps takes every fourth group and walks its groups at its own pace: it copies a group into a
// stage of its own in shared memory (16-byte cp.async copies in the 128-byte swizzle: piece c of
// key row r lies at piece c ^ (r % 8), so that ldmatrix reads without bank conflicts), two groups
// ahead of the one it multiplies, with no barrier of the block in the loop:
//   S = q K^T     A: the query in row 0 (lanes 0..3 hold it as bfloat16 pairs), B: ldmatrix of the
//                 keys' rows; 2 column tiles x 4 k-steps;
//   softmax       base 2, running maximum and sum per warp, in the four lanes that hold row 0;
//   O += P V      A: P rounded to bfloat16 in row 0 (the score registers are the A fragment),
//                 B: ldmatrix.trans of the values' rows; 8 column tiles.
// Rows of keys outside the range (or without a page) are zero-filled in shared memory, so that a
// poisoned slot never meets a zero of P.  As in attention_decode.cu the first groups -- all positions but the token's own, which
// the kernel before is still writing -- are asked for BEFORE the wait on that kernel, and up to 8
// splits of a pair merge as one thread-block cluster through distributed shared memory.
// Softmax statistics and the accumulator are float; P is rounded to bfloat16 for the product (the
// row sum is taken before rounding).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int D = 64;                      // head size
constexpr int WARPS = 4;
constexpr int GROUP = 16;                  // keys a warp multiplies at a time
constexpr int STAGES = 2;                  // groups a warp has in shared memory: one being multiplied, one on its way
constexpr int GROUP_BYTES = GROUP * D * 2; // 2 KB of keys (and as much of values)
constexpr int MAX_PAGES = 160;             // block-table entries of a block's range kept in shared memory
constexpr int MAX_CLUSTER_SPLITS = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void copy16_async(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(WARPS * 32)
decode_attention_mma_kernel(const bf16* __restrict__ q, int ld_q, const bf16* __restrict__ k_cache,
                            const bf16* __restrict__ v_cache, long long page_stride, const int* __restrict__ block_table,
                            int max_blocks, const int* __restrict__ token_seq, const int* __restrict__ positions,
                            bf16* __restrict__ out, int ld_out, int n_heads, int n_kv_heads, int page_size, float scale,
                            int window, int num_splits, int num_pages, int* __restrict__ status) {
    // a warp's own stages: [stage][keys | values][16 rows of 128 bytes]
    __shared__ __align__(128) uint8_t st[WARPS][STAGES][2][GROUP_BYTES];
    __shared__ int s_pages[MAX_PAGES];
    __shared__ float sm_m[WARPS], sm_l[WARPS];
    __shared__ float sm_o[WARPS][D];
    __shared__ float cl_all[MAX_CLUSTER_SPLITS][D + 2];   // in the cluster's first block: every split's (output, max, sum)

    pdl_launch_dependents();
    const bool in_cluster = num_splits > 1;
    // A block may write into another block's shared memory only once that block is running: every
    // block says so here, and waits for the others only when it has its partial state to hand over.
    if (in_cluster) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int split = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int s = token_seq[t];
    const int pos = positions[t];
    const int kvh = h / (n_heads / n_kv_heads);
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    const int n_keys = pos - lo + 1;
    int chunk = (n_keys + num_splits - 1) / num_splits;
    chunk = (chunk + GROUP - 1) / GROUP * GROUP;
    const int begin = lo + split * chunk;
    const int end = min(pos + 1, begin + chunk);
    const int n_groups = end > begin ? (end - begin + GROUP - 1) / GROUP : 0;          // groups of 16 keys
    const int my_groups = n_groups > warp ? (n_groups - warp + WARPS - 1) / WARPS : 0;  // this warp takes groups warp, warp + 4, ..
    const int* table = block_table + (size_t)s * max_blocks;

    // the pages of the block's range, once
    const int p0 = begin / page_size;
    const int n_pages = end > begin ? (end - 1) / page_size - p0 + 1 : 0;
    for (int i = tid; i < n_pages && i < MAX_PAGES; i += WARPS * 32) s_pages[i] = p0 + i < max_blocks ? table[p0 + i] : -1;
    __syncthreads();

    // Copies this warp's k-th group of keys into its stage k % STAGES.  Keys at or past `end`, the key `skip`
    // and keys without a page become rows of zeros.  A lane copies piece lane % 8 of the rows lane / 8 + 4 i
    // (i = 0..3), of the keys and of the values: one page lookup and one address a row, shared by both copies.
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;       // -1: no power of two
    auto stage_group = [&](int k, int skip) {
        const int first = begin + (warp + k * WARPS) * GROUP;
        const uint32_t kb = smem_u32(st[warp][k % STAGES][0]), vb = smem_u32(st[warp][k % STAGES][1]);
        const int c = lane & 7;
#pragma unroll
        for (int i = 0; i < GROUP / 4; i++) {
            const int row = (lane >> 3) + 4 * i;
            const int j = first + row;
            const uint32_t at = row * 128 + ((c ^ (row & 7)) << 4);
            bool ok = j < end && j != skip;
            size_t off = 0;
            if (ok) {
                const int blk = page_shift >= 0 ? j >> page_shift : j / page_size;
                const int slot = page_shift >= 0 ? j & (page_size - 1) : j % page_size;
                const int pi = blk - p0;
                const int page = pi < MAX_PAGES ? s_pages[pi] : -1;
                if (page < 0 || page >= num_pages) {
                    if (status && c == 0) atomicOr(status, 16);     // a visible key with no page behind it
                    ok = false;
                } else {
                    off = (size_t)page * page_stride + ((size_t)kvh * page_size + slot) * D + c * 8;
                }
            }
            if (ok) {
                copy16_async(kb + at, k_cache + off);
                copy16_async(vb + at, v_cache + off);
            } else {
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(kb + at), "r"(0u) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vb + at), "r"(0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Before the wait: everything but the token's own key and value (see attention_decode.cu).
    const int pre = min(my_groups, STAGES);
    for (int k = 0; k < pre; k++) stage_group(k, pos);
    pdl_wait();

    // the query: row 0 of the A operand, in the lanes that hold row 0 (g == 0); four k-steps of 16
    uint32_t qa[4][2];
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
        qa[ks][0] = qa[ks][1] = 0u;
        if (g == 0) {
            const bf16* qp = q + (size_t)t * ld_q + h * D + ks * 16 + 2 * tq;
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
        }
    }
    // the token's own key, if it lies in a group this warp staged without it
    if (pos >= begin && pos < end) {
        const int gi = (pos - begin) / GROUP;                 // its group in the block; this warp's k-th if gi = warp + 4 k
        if (gi % WARPS == warp && gi / WARPS < pre && lane < 16) {
            const int k = gi / WARPS, row = (pos - begin) % GROUP, is_v = lane / 8, c = lane % 8;
            const int pi = pos / page_size - p0;
            const int page = pi < MAX_PAGES ? s_pages[pi] : -1;
            if (page >= 0 && page < num_pages) {
                const uint32_t dst = smem_u32(st[warp][k % STAGES][is_v]) + row * 128 + ((c ^ (row & 7)) << 4);
                const size_t off = (size_t)page * page_stride + ((size_t)kvh * page_size + (pos % page_size)) * D + c * 8;
                copy16_async(dst, (is_v ? v_cache : k_cache) + off);
            } else if (status && lane == 0) {
                atomicOr(status, 16);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    const float sl2 = scale * 1.4426950408889634f;      // scores in units of log2
    float m = -INFINITY, l = 0.0f;
    float o[8][4];
#pragma unroll
    for (int jn = 0; jn < 8; jn++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[jn][e] = 0.0f;

    // Each warp walks its own groups at its own pace: its copies, its stages, no barrier of the block.
    for (int k = 0; k < my_groups; k++) {
        // Group k must have landed.  A lane's copies were committed in the order: groups 0 and 1, the token's own
        // key, then group k + 2 at the end of every round; so from the second round on all but the newest (group
        // k + 1, if there is one) must be complete, and in the first round everything asked for before the loop.
        if (k >= 1 && k + 1 < my_groups) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        const uint32_t kb = smem_u32(st[warp][k % STAGES][0]), vb = smem_u32(st[warp][k % STAGES][1]);
        const int first = begin + (warp + k * WARPS) * GROUP;
        // S = q K^T: two column tiles of 8 keys
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) sc[j][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            // matrices: (keys 0-7, piece 2ks), (keys 0-7, piece 2ks+1), (keys 8-15, piece 2ks), (keys 8-15, piece 2ks+1)
            const int mat = lane >> 3, row = (mat >> 1) * 8 + (lane & 7), c = 2 * ks + (mat & 1);
            uint32_t kf[4];
            ldmatrix_x4(kf, kb + row * 128 + ((c ^ (row & 7)) << 4));
            mma_bf16(sc[0], qa[ks][0], 0u, qa[ks][1], 0u, kf[0], kf[1]);
            mma_bf16(sc[1], qa[ks][0], 0u, qa[ks][1], 0u, kf[2], kf[3]);
        }
        // row 0 lives in lanes 0..3: sc[j][0], sc[j][1] are keys first + 8 j + 2 tq, + 1
        float sv[4];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int key = first + 8 * j + 2 * tq + e;
                sv[2 * j + e] = key < end ? sc[j][e] * sl2 : -INFINITY;
            }
        float group_max = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        group_max = fmaxf(group_max, __shfl_xor_sync(0xffffffffu, group_max, 1));
        group_max = fmaxf(group_max, __shfl_xor_sync(0xffffffffu, group_max, 2));
        const float m_new = fmaxf(m, group_max);         // finite: the group has at least one key in range
        const float corr = exp2f(m - m_new);             // exp2(-inf) = 0 on the first group
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; e++) p[e] = exp2f(sv[e] - m_new);
        l = l * corr + (p[0] + p[1]) + (p[2] + p[3]);
        m = m_new;
#pragma unroll
        for (int jn = 0; jn < 8; jn++) {
            o[jn][0] *= corr;
            o[jn][1] *= corr;
        }
        // O += P V: P in row 0 of the A operand (keys 2 tq, 2 tq + 1 and 8 + 2 tq, 9 + 2 tq of the group)
        const uint32_t pa0 = g == 0 ? pack_bf16(p[0], p[1]) : 0u, pa2 = g == 0 ? pack_bf16(p[2], p[3]) : 0u;
#pragma unroll
        for (int jp = 0; jp < 4; jp++) {
            // matrices: (keys 0-7, piece 2jp), (keys 8-15, piece 2jp), (keys 0-7, piece 2jp+1), (keys 8-15, piece 2jp+1)
            const int mat = lane >> 3, row = (mat & 1) * 8 + (lane & 7), c = 2 * jp + (mat >> 1);
            uint32_t vf[4];
            ldmatrix_x4_trans(vf, vb + row * 128 + ((c ^ (row & 7)) << 4));
            mma_bf16(o[2 * jp], pa0, 0u, pa2, 0u, vf[0], vf[1]);
            mma_bf16(o[2 * jp + 1], pa0, 0u, pa2, 0u, vf[2], vf[3]);
        }
        __syncwarp();                                     // the stage may be overwritten
        if (k + STAGES < my_groups) stage_group(k + STAGES, -1);
    }

    // the warp's state: row 0 is in lanes 0..3 (dims 8 jn + 2 tq, + 1); the sum is spread over them
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
    if (g == 0) {
#pragma unroll
        for (int jn = 0; jn < 8; jn++) {
            sm_o[warp][8 * jn + 2 * tq] = o[jn][0];
            sm_o[warp][8 * jn + 2 * tq + 1] = o[jn][1];
        }
    }
    __syncthreads();

    // merge the warps, one thread per output dimension, fixed order
    float* first_all = nullptr;                 // cl_all of the cluster's first block
    if (in_cluster) {
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // everyone arrived long ago
        first_all = cg::this_cluster().map_shared_rank(&cl_all[0][0], 0);
    }
    for (int d = tid; d < D; d += WARPS * 32) {
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < WARPS; i++) M = fmaxf(M, sm_m[i]);
        float L = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int i = 0; i < WARPS; i++) {
                const float w = exp2f(sm_m[i] - M);     // exp2(-inf) = 0 for warps that saw no key
                L = fmaf(sm_l[i], w, L);
                O = fmaf(sm_o[i][d], w, O);
            }
        }
        if (!in_cluster) {
            out[(size_t)t * ld_out + h * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
        } else {
            first_all[split * (D + 2) + d] = O;
            if (d == 0) {
                first_all[split * (D + 2) + D] = M;
                first_all[split * (D + 2) + D + 1] = L;
            }
        }
    }
    if (in_cluster) {
        // One barrier makes the partial states visible; the first block then merges them out of
        // its own shared memory (fixed order: split 0, 1, ..) and nobody else has anything left to do.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            float M = -INFINITY;
            for (int r = 0; r < num_splits; r++) M = fmaxf(M, cl_all[r][D]);
            for (int d = tid; d < D; d += WARPS * 32) {
                float L = 0.0f, O = 0.0f;
                if (M > -INFINITY) {
                    for (int r = 0; r < num_splits; r++) {
                        const float w = exp2f(cl_all[r][D] - M);
                        L = fmaf(cl_all[r][D + 1], w, L);
                        O = fmaf(cl_all[r][d], w, O);
                    }
                }
                out[(size_t)t * ld_out + h * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
            }
        }
    }
}

}  // namespace

// Most keys a (token, head) pair may have with this many splits: a block keeps the page numbers of its range.
SANDY_API int sandy_decode_attention_mma_max_keys(int num_splits, int page_size) {
    if (num_splits < 1 || page_size < 1) return 0;
    const long long keys = (long long)(MAX_PAGES - 2) * page_size * num_splits;
    return keys > 0x3fffffff ? 0x3fffffff : (int)keys;
}

// Arguments as sandy_decode_attention_cluster (attention_decode.cu); bfloat16, heads of 64, 1 <= num_splits <= 8;
// max_keys: the longest visible range of any token of the launch (checked against the block's table of pages).
SANDY_API int sandy_decode_attention_mma(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                         long long page_stride, const int* block_table, int max_blocks,
                                         const int* token_seq, const int* positions, void* out, int ld_out, int n_tokens,
                                         int n_heads, int n_kv_heads, int head_dim, int page_size, float scale, int window,
                                         int num_splits, int num_pages, int max_keys, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out) return SANDY_ERR_ARGUMENT;
    if (head_dim != D || num_splits < 1 || num_splits > MAX_CLUSTER_SPLITS) return SANDY_ERR_UNSUPPORTED;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_tokens > 65535) return SANDY_ERR_UNSUPPORTED;
    if (max_keys > sandy_decode_attention_mma_max_keys(num_splits, page_size)) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15) || ld_q % 2 != 0 || page_stride % 8 != 0)
        return SANDY_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_splits, n_heads, n_tokens);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (num_splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = num_splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    if (sandy_pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attention_mma_kernel, (const bf16*)q, ld_q, (const bf16*)k_cache,
                                             (const bf16*)v_cache, page_stride, block_table, max_blocks, token_seq, positions,
                                             (bf16*)out, ld_out, n_heads, n_kv_heads, page_size, scale, window, num_splits,
                                             num_pages, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
