// Attention of single tokens over the paged cache for LARGE batches: the same split-KV
// computation as attention_decode.cu, fed by bulk asynchronous copies.
//
// Why a second kernel.  In attention_decode.cu every lane fetches its keys and values into
// registers, so the bytes a block has in flight are bounded by its registers, and a block
// walks its keys in rounds that each wait for memory.  With few (token, head) pairs that is
// the right shape (shortest path for one pair).  With hundreds of pairs the step is bound by
// streaming the cache from HBM (64 requests x 384 positions of GPT-2 small: 75 MB per layer),
// and what matters is bytes in flight per SM.  Here a producer warp asks for whole
// (page, head) blocks of K and V -- which are contiguous in the cache, [page_size][D] each --
// with cp.async.bulk into a ring of shared-memory stages, completion on mbarriers; four consumer
// warps work on the stages as they land.  Registers hold no cache data, several blocks fit on
// an SM, and tens of KB per SM are always on their way.
//
// Arithmetic.  A key's D numbers are 16-byte pieces; a group of LPK lanes shares a key, each
// lane taking one or two pieces (two from 4 pieces on, which halves the shuffles and the
// softmax bookkeeping per byte).  Scores, running maximum, sum and output are float; the
// exponentials are base 2 (the query is multiplied by scale * log2(e) once), and the running
// output is rescaled only when the maximum rises.  Lane groups merge in a fixed order, then
// the splits of a (token, head) pair -- the blocks of one thread-block cluster -- merge through
// distributed shared memory; 1 <= splits <= 8.  Every wait on an mbarrier is bounded.
//
// Head sizes as attention_decode.cu.  Pages must be a power of two long.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int WARPS = 4;                    // consumer warps; one more warp produces
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int MAX_STAGES = 16;
// A wait sleeps in hardware until its barrier's phase ends or about SUSPEND_NS have passed, and
// gives up after WAIT_LIMIT such sleeps (seconds; the kernel itself runs for microseconds).
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr uint32_t SUSPEND_NS = 2000;
int g_ring_bytes = 0;                       // shared memory of one block's ring of stages; 0: by grid size

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(SUSPEND_NS)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// one 16-byte piece -> floats
__device__ __forceinline__ void piece_to_f32(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void piece_to_f32(const bf16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T, int D>
struct Shape {
    static constexpr int VEC = 16 / sizeof(T);       // elements of a 16-byte piece
    static constexpr int NP = D / VEC;               // pieces of a key
    static constexpr int PPL = NP >= 4 ? 2 : 1;      // pieces per lane
    static constexpr int LPK = NP / PPL;             // lanes per key
    static constexpr int KPW = 32 / LPK;             // keys per warp and round
    static constexpr int GROUPS = WARPS * KPW;       // keys per block and round
    static constexpr int EPL = PPL * VEC;            // elements per lane
    static_assert(NP >= 1 && LPK >= 1 && LPK <= 32 && (32 % LPK) == 0, "head size not supported by this kernel");
};

template <typename T, int D>
__global__ void __launch_bounds__(THREADS)
decode_attention_bulk_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_cache,
                             const T* __restrict__ v_cache, long long page_stride,
                             const int* __restrict__ block_table, int max_blocks,
                             const int* __restrict__ token_seq, const int* __restrict__ positions,
                             T* __restrict__ out, int ld_out, int n_heads, int n_kv_heads, int page_size,
                             float scale, int window, int num_splits, int num_pages, int n_stages,
                             int* __restrict__ status) {
    using S = Shape<T, D>;
    constexpr int VEC = S::VEC, PPL = S::PPL, LPK = S::LPK, KPW = S::KPW, GROUPS = S::GROUPS, EPL = S::EPL;

    extern __shared__ __align__(128) uint8_t smem_raw[];       // n_stages x { K [page_size][D], V [page_size][D] }
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
    __shared__ int stage_ok[MAX_STAGES];
    __shared__ float sm_m[GROUPS], sm_l[GROUPS];
    __shared__ float sm_o[GROUPS][D];
    __shared__ float cl_o[D], cl_ml[2];

    // The kernel before this one writes the query and the token's own key and value; the index arrays and
    // the pages of older positions were written by earlier steps (complete by now, see common.cuh).  So the
    // producer starts filling the ring at once and waits for that kernel only in front of the page that
    // holds the token's own position; the consumers wait before they read the query.
    pdl_launch_dependents();
    const int split = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = token_seq[t];
    const int pos = positions[t];
    const int kvh = h / (n_heads / n_kv_heads);
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    const int n_keys = pos - lo + 1;
    int chunk = (n_keys + num_splits - 1) / num_splits;
    const int grain = max(GROUPS, page_size);          // both powers of two: splits meet at page edges
    chunk = (chunk + grain - 1) / grain * grain;
    const int begin = lo + split * chunk;
    const int end = min(pos + 1, begin + chunk);
    const int page_shift = __ffs(page_size) - 1;
    const int p0 = begin >> page_shift;
    const int n_pages = end > begin ? ((end - 1) >> page_shift) - p0 + 1 : 0;
    const int* table = block_table + (size_t)s * max_blocks;
    const uint32_t block_bytes = (uint32_t)page_size * D * sizeof(T);     // one head's K (or V) of one page
    const size_t stage_bytes = 2 * (size_t)block_bytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < n_stages; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[i])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---------------- producer ----------------
        // The warp reads 32 block-table entries at a time (one coalesced load, the next 32
        // already on their way); lane 0 then feeds the ring.
        auto entry = [&](int i) { return (i < n_pages && p0 + i < max_blocks) ? __ldg(table + p0 + i) : -1; };
        bool failed = false;
        const int own_page = (pos >> page_shift) - p0;       // the page the kernel before is still writing to
        bool waited = false;
        int mine = entry(lane);
        for (int c = 0; c < n_pages; c += 32) {
            const int ahead = entry(c + 32 + lane);
            const int cnt = min(32, n_pages - c);
            for (int jj = 0; jj < cnt; jj++) {
                const int page = __shfl_sync(0xffffffffu, mine, jj);
                if (lane != 0 || failed) continue;
                const int i = c + jj;
                if (i >= own_page && !waited) {
                    pdl_wait();
                    waited = true;
                }
                const int st = i % n_stages;
                if (i >= n_stages && !mbar_wait(&empty_bar[st], ((i / n_stages) - 1) & 1)) {
                    if (status) atomicOr(status, 32);
                    failed = true;
                    continue;
                }
                if (page < 0 || page >= num_pages) {
                    // a visible key with no page behind it: report it, hand over an empty stage
                    if (status) atomicOr(status, 16);
                    stage_ok[st] = 0;
                    mbar_arrive(&full_bar[st]);
                    continue;
                }
                stage_ok[st] = 1;
                const size_t src = (size_t)page * page_stride + (size_t)kvh * page_size * D;
                uint8_t* dst = smem_raw + st * stage_bytes;
                mbar_expect_tx(&full_bar[st], 2 * block_bytes);
                bulk_load(dst, k_cache + src, block_bytes, &full_bar[st]);
                bulk_load(dst + block_bytes, v_cache + src, block_bytes, &full_bar[st]);
            }
            mine = ahead;
        }
        pdl_wait();       // every thread has waited before the block writes its output (a second wait returns at once)
    } else {
        // ---------------- consumers ----------------
        pdl_wait();
        const int g = lane / LPK, sub = lane % LPK;
        const int group = warp * KPW + g;
        // Which pieces this lane takes.  Lane groups of odd index start with the upper half of
        // the key, so that with 128-byte keys two neighbouring groups read all 32 banks.
        int piece[PPL];
#pragma unroll
        for (int r = 0; r < PPL; r++) piece[r] = sub + LPK * ((r + g) % PPL);

        float qf[EPL];
        const float qscale = scale * 1.4426950408889634f;
#pragma unroll
        for (int r = 0; r < PPL; r++) {
            const T* qp = q + (size_t)t * ld_q + h * D + piece[r] * VEC;
            if (sizeof(T) == 2) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qp));
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    qf[r * VEC + 2 * i] = __uint_as_float(w[i] << 16);
                    qf[r * VEC + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                }
            } else {
                const float4 v4 = __ldg(reinterpret_cast<const float4*>(qp));
                qf[r * VEC] = v4.x; qf[r * VEC + 1] = v4.y; qf[r * VEC + 2] = v4.z; qf[r * VEC + 3] = v4.w;
            }
        }
#pragma unroll
        for (int e = 0; e < EPL; e++) qf[e] *= qscale;

        float m = -INFINITY, l = 0.0f;          // m in units of log2
        float o[EPL];
#pragma unroll
        for (int e = 0; e < EPL; e++) o[e] = 0.0f;

        // Each warp takes whole pages (its own, every WARPS-th): one wait and one release per
        // page and warp, and no warp runs in step with another.
        for (int i = warp; i < n_pages; i += WARPS) {
            const int st = i % n_stages;
            // the warp decides together: lanes must not part ways before the shuffles below
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[st], (i / n_stages) & 1))) {
                if (status && lane == 0) atomicOr(status, 64);
                break;
            }
            if (stage_ok[st]) {
                const T* ks = reinterpret_cast<const T*>(smem_raw + st * stage_bytes);
                const T* vs = reinterpret_cast<const T*>(smem_raw + st * stage_bytes + block_bytes);
                const int page_first = (p0 + i) << page_shift;
                // keys of this page, KPW at a time; the trip count is the same for the whole warp
                for (int base = 0; base < page_size; base += KPW) {
                    const int slot = base + g;
                    const int j = page_first + slot;
                    const bool ok = slot < page_size && j >= begin && j < end;
                    float sc = 0.0f, vf[EPL];
                    if (ok) {
                        float kf[EPL];
#pragma unroll
                        for (int r = 0; r < PPL; r++) {
                            piece_to_f32(ks + (size_t)slot * D + piece[r] * VEC, kf + r * VEC);
                            piece_to_f32(vs + (size_t)slot * D + piece[r] * VEC, vf + r * VEC);
                        }
#pragma unroll
                        for (int e = 0; e < EPL; e++) sc = fmaf(qf[e], kf[e], sc);
                    }
#pragma unroll
                    for (int w = LPK / 2; w > 0; w >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, w);
                    if (ok) {
                        if (sc > m) {          // rare after the first keys
                            const float corr = exp2f(m - sc);
                            l *= corr;
#pragma unroll
                            for (int e = 0; e < EPL; e++) o[e] *= corr;
                            m = sc;
                        }
                        const float p = exp2f(sc - m);
                        l += p;
#pragma unroll
                        for (int e = 0; e < EPL; e++) o[e] = fmaf(p, vf[e], o[e]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);
        }
        if (sub == 0) {
            sm_m[group] = m;
            sm_l[group] = l;
        }
#pragma unroll
        for (int r = 0; r < PPL; r++)
#pragma unroll
            for (int e = 0; e < VEC; e++) sm_o[group][piece[r] * VEC + e] = o[r * VEC + e];
    }
    __syncthreads();

    // merge the groups, one thread per output dimension, fixed order
    for (int d = threadIdx.x; d < D; d += THREADS) {
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < GROUPS; i++) M = fmaxf(M, sm_m[i]);
        float L = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
#pragma unroll 8
            for (int i = 0; i < GROUPS; i++) {
                const float w = exp2f(sm_m[i] - M);
                L = fmaf(sm_l[i], w, L);
                O = fmaf(sm_o[i][d], w, O);
            }
        }
        if (num_splits == 1) {
            out[(size_t)t * ld_out + h * D + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
        } else {
            cl_o[d] = O;
            if (d == 0) {
                cl_ml[0] = M;
                cl_ml[1] = L;
            }
        }
    }
    if (num_splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            float M = -INFINITY;
            for (int r = 0; r < num_splits; r++) M = fmaxf(M, cluster.map_shared_rank(cl_ml, r)[0]);
            for (int d = threadIdx.x; d < D; d += THREADS) {
                float L = 0.0f, O = 0.0f;
                if (M > -INFINITY) {
                    for (int r = 0; r < num_splits; r++) {
                        const float* rml = cluster.map_shared_rank(cl_ml, r);
                        const float w = exp2f(rml[0] - M);
                        L = fmaf(rml[1], w, L);
                        O = fmaf(cluster.map_shared_rank(cl_o, r)[d], w, O);
                    }
                }
                out[(size_t)t * ld_out + h * D + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
            }
        }
        cluster.sync();
    }
}

template <typename T, int D>
int launch(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
           const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
           int ld_out, int n_tokens, int n_heads, int n_kv_heads, int page_size, float scale, int window,
           int num_splits, int num_pages, int* status, cudaStream_t stream) {
    const size_t stage_bytes = 2 * (size_t)page_size * D * sizeof(T);
    // Many blocks: a short ring each, so that more blocks share an SM (measured on 64 x 12 pairs of
    // 384 keys: 18.8 us with 16 KB, 25.6 us with 32 KB); few blocks: a longer ring each.
    const long long blocks = (long long)num_splits * n_heads * n_tokens;
    const int ring = g_ring_bytes > 0 ? g_ring_bytes : (blocks >= 3LL * sandy_sm_count() ? 16 * 1024 : 32 * 1024);
    int n_stages = (int)(ring / stage_bytes);
    // A multiple of WARPS, so that a stage always serves the same warp: a warp that skipped a
    // phase of a stage's barrier could not tell the phases apart by their parity.
    n_stages = n_stages / WARPS * WARPS;
    n_stages = n_stages < WARPS ? WARPS : (n_stages > MAX_STAGES ? MAX_STAGES : n_stages);
    const size_t smem = n_stages * stage_bytes;
    if (smem > 160 * 1024) return SANDY_ERR_UNSUPPORTED;
    auto kern = decode_attention_bulk_kernel<T, D>;
    static size_t configured = 0;
    if (smem > 40 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_splits, n_heads, n_tokens);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, (const T*)q, ld_q, (const T*)k_cache, (const T*)v_cache,
                                             page_stride, block_table, max_blocks, token_seq, positions, (T*)out,
                                             ld_out, n_heads, n_kv_heads, page_size, scale, window, num_splits,
                                             num_pages, n_stages, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// Tuning: how much shared memory a block's ring may take (more bytes in flight per block, fewer
// blocks per SM); 0 lets the launch choose by the size of the grid.  Returns the value in force.
SANDY_API int sandy_decode_attention_bulk_ring_bytes(int bytes) {
    if (bytes == 0 || (bytes >= 1024 && bytes <= 160 * 1024)) g_ring_bytes = bytes;
    return g_ring_bytes;
}

// Arguments as sandy_decode_attention_cluster (attention_decode.cu); 1 <= num_splits <= 8.
SANDY_API int sandy_decode_attention_bulk(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                          long long page_stride, const int* block_table, int max_blocks,
                                          const int* token_seq, const int* positions, void* out, int ld_out,
                                          int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                          float scale, int window, int num_splits, int num_pages, int dtype,
                                          int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!q || !k_cache || !v_cache || !block_table || !token_seq || !positions || !out) return SANDY_ERR_ARGUMENT;
    if (num_splits < 1 || num_splits > 8) return SANDY_ERR_UNSUPPORTED;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0 || window < 0) return SANDY_ERR_UNSUPPORTED;
    if (page_size & (page_size - 1)) return SANDY_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_tokens > 65535) return SANDY_ERR_UNSUPPORTED;
    const int esz = dtype == SANDY_F32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15) || (ld_q * esz) % 16 != 0 || (page_stride * esz) % 16 != 0 ||
        ((long long)page_size * head_dim * esz) % 16 != 0)
        return SANDY_ERR_UNSUPPORTED;
#define CASE(DT, TT, DD)                                                                                        \
    if (dtype == DT && head_dim == DD)                                                                          \
        return launch<TT, DD>(q, ld_q, k_cache, v_cache, page_stride, block_table, max_blocks, token_seq,       \
                              positions, out, ld_out, n_tokens, n_heads, n_kv_heads, page_size, scale, window,  \
                              num_splits, num_pages, status, stream)
    CASE(SANDY_BF16, bf16, 16); CASE(SANDY_BF16, bf16, 32); CASE(SANDY_BF16, bf16, 64);
    CASE(SANDY_BF16, bf16, 128); CASE(SANDY_BF16, bf16, 256);
    CASE(SANDY_F32, float, 16); CASE(SANDY_F32, float, 32); CASE(SANDY_F32, float, 64); CASE(SANDY_F32, float, 128);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}
