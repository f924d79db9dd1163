// Attention of single tokens over long cached contexts, with the keys of one (token, head)
// pair split over several thread blocks ("split-KV"), then merged.
//
// Formula as in attention.cu (src/core/TensorCalc.cpp:1241-1311 of the reference); the
// reference's decode pair of kernels does the same split and merge
// (flash_attention_decode_partial/reduce, src/device/cuda/CudaAttentionKernels.cu:246-404:
// one warp per split, a scratch of (D + 2) floats per split that it allocates on every
// call, :496-503).  Differences here: the scratch is the caller's (allocated once, reused by
// every layer and step); a block is four warps that read keys and values in 16-byte pieces,
// several lanes per key, so that every load instruction of a warp covers whole rows; the
// block table of the token's request is walked directly; and the number of splits is fixed
// by the caller per launch shape, so the launch can be recorded in a CUDA graph; and the keys
// and values of older positions (all but the token's own, which the kernel before this one is
// still writing) are asked for BEFORE the wait on that kernel, into shared memory, so that their
// trip to memory runs under its tail (a decode step of 8 requests: 0.347 -> 0.329 ms).
//
// Block (split, head, token): keys [lo + split*chunk, ...) of the token's visible range
// [lo, pos].  Each group of LPK lanes owns one key per round and keeps its own running
// (max, sum, weighted values); the groups are merged in shared memory in a fixed order, and
// the block writes either the final output (one split) or its partial state
// (max, sum, unnormalised output) to the scratch.  A second kernel merges the splits.
// Scores, softmax and sums are float.
//
// Head sizes: D * sizeof(T) / 16 must divide 32 (D = 16, 32, 64, 128, and 256 in bfloat16).
// Other head sizes are served by the general kernel in attention.cu.
//
// Merging the splits.  With up to 8 splits the blocks of one (token, head) pair are launched
// as one thread-block cluster and merge through distributed shared memory: every block writes
// its partial state into the first block's shared memory, one cluster barrier, the first
// block merges; no scratch, no second kernel (sandy_decode_attention_cluster).  The scratch form with its merge kernel
// remains for more splits and for callers that want it (sandy_decode_attention).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int WARPS = 4;
constexpr int UNROLL = 4;
constexpr int MAX_CLUSTER_SPLITS = 8;      // the portable cluster size

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[VEC]);

template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float (&f)[4]) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

template <>
__device__ __forceinline__ void load_vec<bf16, 8>(const bf16* p, float (&f)[8]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// The same 16-byte piece out of shared memory (a staged key or value).
template <typename T, int VEC>
__device__ __forceinline__ void load_vec_staged(const uint8_t* p, float (&f)[VEC]);

template <>
__device__ __forceinline__ void load_vec_staged<float, 4>(const uint8_t* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

template <>
__device__ __forceinline__ void load_vec_staged<bf16, 8>(const uint8_t* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// 16 bytes from global to shared memory, asynchronously, past L1.
__device__ __forceinline__ void copy16_async(uint8_t* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <typename T, int D>
__global__ void __launch_bounds__(WARPS * 32)
decode_attention_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, long long page_stride,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ token_seq, const int* __restrict__ positions,
                        T* __restrict__ out, int ld_out, float* __restrict__ partial_o,
                        float* __restrict__ partial_ml, int n_heads, int n_kv_heads, int page_size,
                        float scale, int window, int num_splits, int num_pages, int* __restrict__ status) {
    constexpr int VEC = 16 / sizeof(T);         // elements per 16-byte piece
    constexpr int LPK = D / VEC;                // lanes per key
    constexpr int KPW = 32 / LPK;               // keys per warp per round
    constexpr int GROUPS = WARPS * KPW;
    static_assert(LPK >= 1 && LPK <= 32 && (32 % LPK) == 0, "head size not supported by this kernel");

    // Keys and values asked for before the wait (see below): up to STAGE_KEYS of the block's range.
    constexpr int ROW_BYTES = D * (int)sizeof(T);
    constexpr int STAGE_KEYS = (16 * 1024 / ROW_BYTES) / GROUPS * GROUPS;
    static_assert(STAGE_KEYS >= GROUPS, "the staging area holds at least one round of keys");

    __shared__ float sm_m[GROUPS], sm_l[GROUPS];
    __shared__ float sm_o[GROUPS][D];
    __shared__ float cl_all[MAX_CLUSTER_SPLITS][D + 2];   // in the cluster's first block: every split's (output, max, sum)
    __shared__ __align__(16) uint8_t st_k[STAGE_KEYS * ROW_BYTES], st_v[STAGE_KEYS * ROW_BYTES];
    __shared__ uint8_t st_ok[STAGE_KEYS];       // whether a staged key had a page behind it

    pdl_launch_dependents();
    const bool in_cluster = num_splits > 1 && partial_o == nullptr;
    // A block may write into another block's shared memory only once that block is running: every
    // block says so here, and waits for the others only when it has its partial state to hand over.
    if (in_cluster) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int split = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane / LPK, sub = lane % LPK;
    const int group = warp * KPW + g;
    const int s = token_seq[t];
    const int pos = positions[t];
    const int kvh = h / (n_heads / n_kv_heads);
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    const int n_keys = pos - lo + 1;
    int chunk = (n_keys + num_splits - 1) / num_splits;
    chunk = (chunk + GROUPS - 1) / GROUPS * GROUPS;
    const int begin = lo + split * chunk;
    const int end = min(pos + 1, begin + chunk);
    const int* table = block_table + (size_t)s * max_blocks;

    // Before the wait: the kernel before this one writes the query and the token's own key and value,
    // nothing else this block reads.  The index arrays and the keys of older positions were written by
    // earlier steps (complete by now, see common.cuh), so their pieces are asked for at once, into shared
    // memory, each by the thread that will use it: the trip to memory runs under the tail of the kernel
    // before.  The token's own key, and what does not fit the staging area, is read after the wait.
    const int stage_end = min(min(end, pos), begin + STAGE_KEYS);
    for (int j = begin + group; j < stage_end; j += GROUPS) {
        const int b = j / page_size;
        const int page = b < max_blocks ? table[b] : -1;
        const bool ok = page >= 0 && page < num_pages;
        if (ok) {
            const size_t off = (size_t)page * page_stride + ((size_t)kvh * page_size + (j % page_size)) * D + sub * VEC;
            copy16_async(st_k + (j - begin) * ROW_BYTES + sub * 16, k_cache + off);
            copy16_async(st_v + (j - begin) * ROW_BYTES + sub * 16, v_cache + off);
        }
        if (sub == 0) st_ok[j - begin] = ok ? 1 : 0;     // read back by this group's lanes only
    }
    __syncwarp();                                          // ... which are lanes of this warp
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the page of the token's own position too: its table entry is the step's input like the others
    const int own_b = pos / page_size;
    const int own_page = (pos >= begin && pos < end && own_b < max_blocks) ? table[own_b] : -1;
    pdl_wait();

    float qf[VEC];
    load_vec<T, VEC>(q + (size_t)t * ld_q + h * D + sub * VEC, qf);
    asm volatile("cp.async.wait_group 0;" ::: "memory");       // my own pieces: no other thread reads them

    float m = -INFINITY, l = 0.0f;
    float o[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) o[i] = 0.0f;

    // The trip count is the same for every lane of a warp (the shuffles below need the whole
    // warp): `base` is warp-uniform, and a group whose key lies past `end` just sits the round out.
    for (int base = begin + warp * KPW; base < end; base += GROUPS * UNROLL) {
        float kf[UNROLL][VEC], vf[UNROLL][VEC];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int j = base + g + u * GROUPS;
            ok[u] = j < end;
            if (ok[u]) {
                // staged keys carry their answer; the token's own page was looked up before the wait; only a
                // range too long for the staging area walks the table here
                int page;
                if (j < stage_end) page = st_ok[j - begin] ? 0 : -1;
                else if (j == pos) page = own_page;
                else {
                    const int b = j / page_size;
                    page = b < max_blocks ? table[b] : -1;
                }
                if (page < 0 || page >= num_pages) {
                    if (status && sub == 0) atomicOr(status, 16);   // a visible key with no page behind it
                    ok[u] = false;
                } else {
                    if (j < stage_end) {
                        load_vec_staged<T, VEC>(st_k + (j - begin) * ROW_BYTES + sub * 16, kf[u]);
                        load_vec_staged<T, VEC>(st_v + (j - begin) * ROW_BYTES + sub * 16, vf[u]);
                    } else {
                        const size_t off = (size_t)page * page_stride +
                                           ((size_t)kvh * page_size + (j % page_size)) * D + sub * VEC;
                        load_vec<T, VEC>(k_cache + off, kf[u]);
                        load_vec<T, VEC>(v_cache + off, vf[u]);
                    }
                }
            }
        }
        // The round's scores first (independent of one another), then ONE new maximum and one correction for
        // the round, then the round's exponentials: a key's update no longer waits for the key before it.
        float sc[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            float d = 0.0f;
            if (ok[u]) {
#pragma unroll
                for (int i = 0; i < VEC; i++) d = fmaf(qf[i], kf[u][i], d);
            }
#pragma unroll
            for (int w = LPK / 2; w > 0; w >>= 1) d += __shfl_xor_sync(0xffffffffu, d, w);
            sc[u] = ok[u] ? d * scale : -INFINITY;          // ok[u] is uniform across the LPK lanes of the group
        }
        float m_new = m;
#pragma unroll
        for (int u = 0; u < UNROLL; u++) m_new = fmaxf(m_new, sc[u]);
        if (m_new > -INFINITY) {
            const float corr = expf(m - m_new);              // exp(-inf) = 0 while nothing has been seen yet
            l *= corr;
#pragma unroll
            for (int i = 0; i < VEC; i++) o[i] *= corr;
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                if (ok[u]) {
                    const float p = expf(sc[u] - m_new);
                    l += p;
#pragma unroll
                    for (int i = 0; i < VEC; i++) o[i] = fmaf(p, vf[u][i], o[i]);
                }
            }
            m = m_new;
        }
    }

    if (sub == 0) {
        sm_m[group] = m;
        sm_l[group] = l;
    }
#pragma unroll
    for (int i = 0; i < VEC; i++) sm_o[group][sub * VEC + i] = o[i];
    __syncthreads();

    // merge the groups, one thread per output dimension, fixed order
    float* first_all = nullptr;                 // cl_all of the cluster's first block
    if (in_cluster) {
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // everyone arrived long ago
        first_all = cg::this_cluster().map_shared_rank(&cl_all[0][0], 0);
    }
    for (int d = threadIdx.x; d < D; d += WARPS * 32) {
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < GROUPS; i++) M = fmaxf(M, sm_m[i]);
        float L = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int i = 0; i < GROUPS; i++) {
                const float w = expf(sm_m[i] - M);     // exp(-inf) = 0 for groups that saw no key
                L = fmaf(sm_l[i], w, L);
                O = fmaf(sm_o[i][d], w, O);
            }
        }
        if (num_splits == 1) {
            out[(size_t)t * ld_out + h * D + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
        } else if (partial_o == nullptr) {
            // cluster mode: the splits of this (token, head) are the blocks of one cluster, and each
            // hands its partial state to the first block's shared memory
            first_all[split * (D + 2) + d] = O;
            if (d == 0) {
                first_all[split * (D + 2) + D] = M;
                first_all[split * (D + 2) + D + 1] = L;
            }
        } else {
            const size_t slot = ((size_t)t * n_heads + h) * num_splits + split;
            partial_o[slot * D + d] = O;
            if (d == 0) {
                partial_ml[slot * 2] = M;
                partial_ml[slot * 2 + 1] = L;
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
            for (int d = threadIdx.x; d < D; d += WARPS * 32) {
                float L = 0.0f, O = 0.0f;
                if (M > -INFINITY) {
                    for (int r = 0; r < num_splits; r++) {
                        const float w = expf(cl_all[r][D] - M);
                        L = fmaf(cl_all[r][D + 1], w, L);
                        O = fmaf(cl_all[r][d], w, O);
                    }
                }
                out[(size_t)t * ld_out + h * D + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
            }
        }
    }
}

template <typename T, int D>
__global__ void merge_splits_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                    T* __restrict__ out, int ld_out, int n_heads, int num_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, t = blockIdx.y;
    const size_t base = ((size_t)t * n_heads + h) * num_splits;
    float M = -INFINITY;
    for (int i = 0; i < num_splits; i++) M = fmaxf(M, partial_ml[(base + i) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
            for (int i = 0; i < num_splits; i++) {
                const float w = expf(partial_ml[(base + i) * 2] - M);
                L = fmaf(partial_ml[(base + i) * 2 + 1], w, L);
                O = fmaf(partial_o[(base + i) * D + d], w, O);
            }
        }
        out[(size_t)t * ld_out + h * D + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
    }
}

template <typename T, int D>
int launch(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
           const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
           int ld_out, float* scratch, int n_tokens, int n_heads, int n_kv_heads, int page_size, float scale,
           int window, int num_splits, int num_pages, int* status, cudaStream_t stream) {
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)n_tokens * n_heads * num_splits * D : nullptr;
    dim3 grid(num_splits, n_heads, n_tokens);
    int code = sandy_launch(decode_attention_kernel<T, D>, grid, dim3(WARPS * 32), 0, stream, (const T*)q, ld_q,
                            (const T*)k_cache, (const T*)v_cache, page_stride, block_table, max_blocks, token_seq,
                            positions, (T*)out, ld_out, partial_o, partial_ml, n_heads, n_kv_heads, page_size, scale,
                            window, num_splits, num_pages, status);
    if (code != 0 || num_splits == 1) return code;
    return sandy_launch(merge_splits_kernel<T, D>, dim3(n_heads, n_tokens), dim3(D < 32 ? 32 : (D > 256 ? 256 : D)), 0,
                        stream, (const float*)partial_o, (const float*)partial_ml, (T*)out, ld_out, n_heads, num_splits);
}

// Cluster form: grid (splits, heads, tokens), clusters of (splits, 1, 1).
template <typename T, int D>
int launch_cluster(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                   const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                   int ld_out, int n_tokens, int n_heads, int n_kv_heads, int page_size, float scale, int window,
                   int num_splits, int num_pages, int* status, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_splits, n_heads, n_tokens);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = num_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sandy_pdl_enabled() ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(
        &cfg, decode_attention_kernel<T, D>, (const T*)q, ld_q, (const T*)k_cache, (const T*)v_cache, page_stride,
        block_table, max_blocks, token_seq, positions, (T*)out, ld_out, (float*)nullptr, (float*)nullptr, n_heads,
        n_kv_heads, page_size, scale, window, num_splits, num_pages, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// The cluster form: 2 <= num_splits <= 8, no scratch.  Other arguments as sandy_decode_attention.
SANDY_API int sandy_decode_attention_cluster(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                             long long page_stride, const int* block_table, int max_blocks,
                                             const int* token_seq, const int* positions, void* out, int ld_out,
                                             int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                             float scale, int window, int num_splits, int num_pages, int dtype,
                                             int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out) return SANDY_ERR_ARGUMENT;
    if (num_splits < 2 || num_splits > MAX_CLUSTER_SPLITS) return SANDY_ERR_UNSUPPORTED;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_tokens > 65535) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15))
        return SANDY_ERR_UNSUPPORTED;
    const int esz = dtype == SANDY_F32 ? 4 : 2;
    if ((ld_q * esz) % 16 != 0 || (page_stride * esz) % 16 != 0) return SANDY_ERR_UNSUPPORTED;
#define CASE(DT, TT, DD)                                                                                        \
    if (dtype == DT && head_dim == DD)                                                                          \
        return launch_cluster<TT, DD>(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq, \
                                      positions, out, ld_out, n_tokens, n_heads, n_kv_heads, page_size, scale,  \
                                      window, num_splits, num_pages, status, stream)
    CASE(SANDY_BF16, bf16, 16); CASE(SANDY_BF16, bf16, 32); CASE(SANDY_BF16, bf16, 64);
    CASE(SANDY_BF16, bf16, 128); CASE(SANDY_BF16, bf16, 256);
    CASE(SANDY_F32, float, 16); CASE(SANDY_F32, float, 32); CASE(SANDY_F32, float, 64); CASE(SANDY_F32, float, 128);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

// Floats of scratch the split kernel needs for this shape (0 when num_splits == 1).
SANDY_API long long sandy_decode_attention_scratch_floats(int n_tokens, int n_heads, int head_dim, int num_splits) {
    if (num_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * num_splits * (head_dim + 2);
}

// q, out: [n_tokens, H*D] (row strides ld_q, ld_out); caches as in attention.cu; scratch: float
// array of sandy_decode_attention_scratch_floats(...) elements (may be null for one split).
SANDY_API int sandy_decode_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                     long long page_stride, const int* block_table, int max_blocks,
                                     const int* token_seq, const int* positions, void* out, int ld_out,
                                     float* scratch, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     int page_size, float scale, int window, int num_splits, int num_pages,
                                     int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out) return SANDY_ERR_ARGUMENT;
    if (num_splits < 1 || (num_splits > 1 && !scratch)) return SANDY_ERR_ARGUMENT;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_tokens > 65535) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15))
        return SANDY_ERR_UNSUPPORTED;
    const int esz = dtype == SANDY_F32 ? 4 : 2;
    if ((ld_q * esz) % 16 != 0 || (page_stride * esz) % 16 != 0) return SANDY_ERR_UNSUPPORTED;
#define CASE(DT, TT, DD)                                                                                    \
    if (dtype == DT && head_dim == DD)                                                                      \
        return launch<TT, DD>(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq,   \
                              positions, out, ld_out, scratch, n_tokens, n_heads, n_kv_heads, page_size,    \
                              scale, window, num_splits, num_pages, status, stream)
    CASE(SANDY_BF16, bf16, 16); CASE(SANDY_BF16, bf16, 32); CASE(SANDY_BF16, bf16, 64);
    CASE(SANDY_BF16, bf16, 128); CASE(SANDY_BF16, bf16, 256);
    CASE(SANDY_F32, float, 16); CASE(SANDY_F32, float, 32); CASE(SANDY_F32, float, 64); CASE(SANDY_F32, float, 128);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

// ---- the entry point that allocates nothing ------------------------------------------------
// See attention_decode_static.h for who needs it, its limit and its rules.
#include "attention_decode_static.h"

namespace {

// The scratch of sandy_decode_attention_static().  In host code this name is only a handle
// for cudaGetSymbolAddress: it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) float g_decode_static_scratch[SANDY_DECODE_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;

// Device address of the array on the current device, looked up once per device.
float* static_scratch_address(int* error) {
    static float* address[MAX_DEVICES] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        *error = SANDY_ERR_STATIC_SETUP;
        return nullptr;
    }
    if (address[dev] == nullptr) {
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            *error = SANDY_ERR_STATIC_SETUP;
            return nullptr;
        }
        address[dev] = p;
    }
    return address[dev];
}

}  // namespace

SANDY_API long long sandy_decode_attention_static_capacity(void) {
    return (long long)SANDY_DECODE_STATIC_SCRATCH_FLOATS;
}

SANDY_API const char* sandy_decode_attention_static_strerror(int code) {
    switch (code) {
        case SANDY_OK: return "ok";
        case SANDY_ERR_UNSUPPORTED: return "sizes or dtypes this kernel does not take";
        case SANDY_ERR_ARGUMENT: return "a null pointer or an impossible size";
        case SANDY_ERR_STATIC_SCRATCH:
            return "the shape needs more scratch than the static array holds "
                   "(n_tokens * n_heads * num_splits * (head_dim + 2) floats > 1048576): "
                   "use fewer splits or sandy_decode_attention() with a buffer of your own";
        case SANDY_ERR_STATIC_SETUP: return "the device address of the static scratch array could not be obtained";
        default: return code > 0 ? "a CUDA error (the value is a cudaError_t)" : "unknown code";
    }
}

SANDY_API int sandy_decode_attention_static(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                            long long page_stride, const int* block_table, int max_blocks,
                                            const int* token_seq, const int* positions, void* out, int ld_out,
                                            int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                            float scale, int window, int num_splits, int num_pages, int dtype,
                                            int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (n_tokens < 0 || n_heads <= 0 || head_dim <= 0 || num_splits < 1) return SANDY_ERR_ARGUMENT;
    // Bound every factor before multiplying, so that the product below cannot wrap around and
    // slip under the capacity: no factor alone may exceed what the whole array holds.
    const long long cap = (long long)SANDY_DECODE_STATIC_SCRATCH_FLOATS;
    if (head_dim > 256) return SANDY_ERR_UNSUPPORTED;
    if (n_tokens > cap || n_heads > cap || num_splits > cap) return SANDY_ERR_STATIC_SCRATCH;
    long long need = 0;
    if (num_splits > 1) {
        need = (long long)n_tokens * n_heads;                 // <= 2^40
        if (need > cap) return SANDY_ERR_STATIC_SCRATCH;
        need *= num_splits;                                   // <= 2^40
        if (need > cap) return SANDY_ERR_STATIC_SCRATCH;
        need *= head_dim + 2;                                 // <= 2^29
    }
    if (need > cap) return SANDY_ERR_STATIC_SCRATCH;
    int error = SANDY_OK;
    float* scratch = static_scratch_address(&error);     // first call on a device: the one-time look-up
    if (scratch == nullptr) return error;
    return sandy_decode_attention(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq,
                                  positions, out, ld_out, scratch, n_tokens, n_heads, n_kv_heads, head_dim,
                                  page_size, scale, window, num_splits, num_pages, dtype, status, stream);
}
