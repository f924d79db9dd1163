// Causal attention over a paged key/value cache, and the kernel that appends to it.
//
// Formula, as the reference computes it (src/core/TensorCalc.cpp:1241-1311):
//   s[j] = (q . k_j) * scale            for  max(0, pos+1-window) <= j <= pos   (window 0: all)
//   p[j] = exp(s[j] - max s) / sum exp(s - max s);   o = sum_j p[j] * v_j
// with query head h reading key/value head h / (H / Hkv) (:1246).  Scores, the softmax and
// the weighted sum are carried in 32-bit; the reference's CUDA kernels do the same with an
// online softmax (src/device/cuda/CudaAttentionKernels.cu:171-243).
//
// Unlike the reference, which hands each kernel one request's K and V through a table of
// page pointers per tensor (src/device/cuda/CudaKernelUtils.cuh:82-108), a launch here
// covers every token of a step: prompt portions of some requests beside single decoded
// tokens of others.  A token finds its request through `token_seq`, its position through
// `positions`, and that request's pages through one row of `block_table`.  Keys and
// values of the step's own tokens are appended to the pages first (sandy_kv_append), so
// attention reads everything from the cache, in the same format, however the tokens were
// cut into steps; a query walks its keys in blocks of 32 counted from its first visible
// key, so its result does not depend on the batch it is in or on which pages hold the keys.
//
// Cache layout of one layer: K and V each [num_pages][Hkv][page_size][D], page stride
// given in elements (K and V of a page may be interleaved in one arena).
//
// This is the general kernel: any head size that is a multiple of 16 up to 256, any
// number of heads and groups, both storage types.  One warp owns one (token, head) pair.
#include "common.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS_PER_BLOCK = 4;

template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int ld_src,
                                 T* __restrict__ k_cache, T* __restrict__ v_cache, long long page_stride,
                                 const int* __restrict__ block_table, int max_blocks,
                                 const int* __restrict__ token_seq, const int* __restrict__ positions,
                                 int n_kv_heads, int head_dim, int page_size, int num_pages,
                                 int* __restrict__ status) {
    const int t = blockIdx.x;
    const int s = token_seq[t];
    const int pos = positions[t];
    if (pos < 0 || pos / page_size >= max_blocks) {   // a position the block table does not cover
        if (threadIdx.x == 0 && status) atomicOr(status, 8);
        return;
    }
    const int page = block_table[(size_t)s * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) {              // no page behind this position: nothing may be written
        if (threadIdx.x == 0 && status) atomicOr(status, 8);
        return;
    }
    const int slot = pos % page_size;
    const int n = n_kv_heads * head_dim;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int h = i / head_dim, d = i % head_dim;
        const size_t dst = (size_t)page * page_stride + ((size_t)h * page_size + slot) * head_dim + d;
        k_cache[dst] = k_src[(size_t)t * ld_src + i];
        v_cache[dst] = v_src[(size_t)t * ld_src + i];
    }
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ row, const float* __restrict__ q, int head_dim);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ row, const float* __restrict__ q, int head_dim) {
    float acc = 0.0f;
    for (int d = 0; d < head_dim; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(row + d);
        acc = fmaf(q[d + 0], kv.x, acc);
        acc = fmaf(q[d + 1], kv.y, acc);
        acc = fmaf(q[d + 2], kv.z, acc);
        acc = fmaf(q[d + 3], kv.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ row, const float* __restrict__ q, int head_dim) {
    float acc = 0.0f;
    for (int d = 0; d < head_dim; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __bfloat1622float2(p[i]);
            acc = fmaf(q[d + 2 * i], f.x, acc);
            acc = fmaf(q[d + 2 * i + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32)
paged_attention_kernel(const T* __restrict__ q, int ld_q,
                       const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride,
                       const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ token_seq, const int* __restrict__ positions,
                       T* __restrict__ out, int ld_out,
                       int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                       float scale, int window, int num_pages, int* __restrict__ status) {
    __shared__ float q_smem[WARPS_PER_BLOCK][MAX_HEAD_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * WARPS_PER_BLOCK + warp;
    if (pair >= (long long)n_tokens * n_heads) return;
    const int t = (int)(pair / n_heads), h = (int)(pair % n_heads);
    const int s = token_seq[t];
    const int pos = positions[t];
    const int kvh = h / (n_heads / n_kv_heads);
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = block_table + (size_t)s * max_blocks;
    const long long rows_per_page = page_stride / head_dim;  // page stride in rows of D

    float* qs = q_smem[warp];
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_f32(q[(size_t)t * ld_q + h * head_dim + d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < MAX_HEAD_DIM / 32; i++) acc[i] = 0.0f;

    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j <= pos;
        long long row = 0;  // row index (units of D elements) of key j inside the layer's cache
        float sc = -INFINITY;
        if (valid) {
            const int page = (j / page_size < max_blocks) ? table[j / page_size] : -1;
            if (page < 0 || page >= num_pages) {
                // a visible key with no page behind it: report it, read nothing
                if (status) atomicOr(status, 16);
            } else {
                row = (long long)page * rows_per_page + (long long)kvh * page_size + (j % page_size);
                sc = dot_row<T>(k_cache + row * head_dim, qs, head_dim) * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float corr = expf(m - m_new);   // first block: exp(-inf) = 0
        const float p = (valid && sc > -INFINITY) ? expf(sc - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_HEAD_DIM / 32; i++) acc[i] *= corr;
        const int count = min(32, pos - base + 1);
        for (int jj = 0; jj < count; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vrow = v_cache + rj * head_dim;
#pragma unroll
            for (int i = 0; i < MAX_HEAD_DIM / 32; i++) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_HEAD_DIM / 32; i++) {
        const int d = lane + 32 * i;
        if (d < head_dim) out[(size_t)t * ld_out + h * head_dim + d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

// Append the step's keys and values to the pages.  k_src, v_src: [n_tokens, Hkv*D] with
// row stride ld_src (elements); token t goes to position positions[t] of request
// token_seq[t], i.e. page block_table[seq][pos / page_size], slot pos % page_size.
SANDY_API int sandy_kv_append(const void* k_src, const void* v_src, int ld_src,
                              void* k_cache, void* v_cache, long long page_stride,
                              const int* block_table, int max_blocks,
                              const int* token_seq, const int* positions,
                              int n_tokens, int n_kv_heads, int head_dim, int page_size, int num_pages,
                              int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!k_src || !v_src || !k_cache || !v_cache || !block_table || !token_seq || !positions)
        return SANDY_ERR_ARGUMENT;
    const int n = n_kv_heads * head_dim;
    const int threads = n >= 512 ? 256 : 128;
    if (dtype == SANDY_F32)
        kv_append_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (const float*)k_src, (const float*)v_src, ld_src, (float*)k_cache, (float*)v_cache, page_stride,
            block_table, max_blocks, token_seq, positions, n_kv_heads, head_dim, page_size, num_pages, status);
    else if (dtype == SANDY_BF16)
        kv_append_kernel<bf16><<<n_tokens, threads, 0, stream>>>(
            (const bf16*)k_src, (const bf16*)v_src, ld_src, (bf16*)k_cache, (bf16*)v_cache, page_stride,
            block_table, max_blocks, token_seq, positions, n_kv_heads, head_dim, page_size, num_pages, status);
    else
        return SANDY_ERR_UNSUPPORTED;
    return sandy_launch_status();
}

// q: [n_tokens, H*D] with row stride ld_q; out: [n_tokens, H*D] with row stride ld_out.
// window 0 = every earlier key is visible.
SANDY_API int sandy_paged_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                    long long page_stride, const int* block_table, int max_blocks,
                                    const int* token_seq, const int* positions, void* out, int ld_out,
                                    int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                    float scale, int window, int num_pages, int dtype, int* status,
                                    cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out)
        return SANDY_ERR_ARGUMENT;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > MAX_HEAD_DIM) return SANDY_ERR_UNSUPPORTED;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (page_stride % head_dim != 0) return SANDY_ERR_UNSUPPORTED;
    const long long pairs = (long long)n_tokens * n_heads;
    const unsigned blocks = (unsigned)((pairs + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK);
#define LAUNCH(T)                                                                                     \
    paged_attention_kernel<T><<<blocks, WARPS_PER_BLOCK * 32, 0, stream>>>(                           \
        (const T*)q, ld_q, (const T*)k_cache, (const T*)v_cache, page_stride, block_table, max_blocks, \
        token_seq, positions, (T*)out, ld_out, n_tokens, n_heads, n_kv_heads, head_dim, page_size,    \
        scale, window, num_pages, status)
    if (dtype == SANDY_F32) LAUNCH(float);
    else if (dtype == SANDY_BF16) LAUNCH(bf16);
    else return SANDY_ERR_UNSUPPORTED;
#undef LAUNCH
    return sandy_launch_status();
}
