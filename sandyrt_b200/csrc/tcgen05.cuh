// Pieces shared by the tcgen05 matrix-product kernels: mbarrier and TMA wrappers, shared-memory
// and instruction descriptors, tensor-memory loads, the write-back of one accumulator chunk, and
// the host-side cache of TMA tensor maps.
#pragma once

#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "epilogue.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait; false means the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c_inner, int c_outer,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c_inner), "r"(c_outer)
        : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// 128-byte mode: 8-row groups are 1024 bytes apart (stride byte offset); the leading byte
// offset is unused for swizzled K-major layouts (set to 1); version 1; layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: float accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr uint32_t make_instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Where the key and value columns of a fused q/k/v product go (the cache layout of attention.cu):
// columns [q_cols, q_cols + kv_cols) are keys, the next kv_cols values; row m belongs to
// position positions[m] of request token_seq[m].  k_cache null: no cache write.
struct KVWrite {
    bf16* k_cache;
    bf16* v_cache;
    long long page_stride;
    const int* block_table;
    const int* token_seq;
    const int* positions;
    int max_blocks, q_cols, kv_cols, head_dim, page_size, num_pages;
};

struct EpilogueArgs {
    const bf16* bias;        // [N] or null
    const float* residual;   // [M, N] row stride ldr, or null
    void* out;               // [M, N] row stride ldc
    int ldr, ldc;
    int act;
    int out_f32;             // 1: float out, 0: bfloat16 out
    KVWrite kv;
};

// The page (or -1) and the slot inside it where row `row`'s key and value belong.
__device__ __forceinline__ void kv_row_target(const KVWrite& kv, int row, int M, int& page, int& slot) {
    page = -1;
    slot = 0;
    if (!kv.k_cache || row >= M) return;
    const int pos = kv.positions[row];
    const int b = pos / kv.page_size;
    slot = pos % kv.page_size;
    if (pos >= 0 && b < kv.max_blocks) page = kv.block_table[(size_t)kv.token_seq[row] * kv.max_blocks + b];
}

// The residual values of 32 consecutive columns of one row, asked for before the accumulator is
// read so that the trip to memory overlaps the tensor-memory load.  False (nothing loaded) if
// there is no residual or it cannot be fetched as eight aligned float4; store_chunk then reads
// what it needs itself.
__device__ __forceinline__ bool load_residual(float4 (&res)[8], int row, int col0, const EpilogueArgs& ep, int M, int N) {
    if (!ep.residual || row >= M || col0 + 32 > N) return false;
    const float* rr = ep.residual + (size_t)row * ep.ldr + col0;
    if (reinterpret_cast<uintptr_t>(rr) & 15) return false;
#pragma unroll
    for (int j = 0; j < 8; j++) res[j] = *reinterpret_cast<const float4*>(rr + 4 * j);
    return true;
}

// Write-back of 32 consecutive columns of one row: bias, activation, residual, rounding, store.
// kv_page, kv_slot: from kv_row_target, used when the chunk holds key or value columns.
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], int row, int col0, const EpilogueArgs& ep, int M,
                                            int N, const float4 (&res)[8], bool have_res, int kv_page, int kv_slot,
                                            int* status) {
    // the chunk's 32 bias values: one load per lane, handed round by shuffles (32 scalar loads per
    // thread were a trip to memory in front of every chunk's arithmetic)
    const int lane = threadIdx.x & 31;
    float my_bias = 0.0f;
    if (ep.bias && col0 + lane < N) my_bias = __bfloat162float(ep.bias[col0 + lane]);
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = apply_act_fast(__uint_as_float(r[j]) + __shfl_sync(0xffffffffu, my_bias, j), ep.act);
    if (ep.kv.k_cache && row < M && col0 + 32 > ep.kv.q_cols) {
        // key / value columns also go straight into the request's page, eight at a time (a head's
        // size is a multiple of 16, so eight consecutive columns never straddle two heads)
        if (kv_page < 0 || kv_page >= ep.kv.num_pages) {
            if (status) atomicOr(status, 8);
        } else {
#pragma unroll
            for (int g8 = 0; g8 < 4; g8++) {
                const int col = col0 + 8 * g8;
                if (col >= ep.kv.q_cols && col + 8 <= N) {
                    const int c = col - ep.kv.q_cols;
                    const bool is_v = c >= ep.kv.kv_cols;
                    const int c2 = is_v ? c - ep.kv.kv_cols : c;
                    const int head = c2 / ep.kv.head_dim, d = c2 % ep.kv.head_dim;
                    bf16* dst = (is_v ? ep.kv.v_cache : ep.kv.k_cache) + (size_t)kv_page * ep.kv.page_stride +
                                ((size_t)head * ep.kv.page_size + kv_slot) * ep.kv.head_dim + d;
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * g8], v[8 * g8 + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * g8 + 2], v[8 * g8 + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * g8 + 4], v[8 * g8 + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * g8 + 6], v[8 * g8 + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2);
                    pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(dst) = pk;
                }
            }
        }
    }
    if (row < M && col0 < N) {
        const bool full = col0 + 32 <= N;
        if (have_res) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                v[4 * j] += res[j].x; v[4 * j + 1] += res[j].y; v[4 * j + 2] += res[j].z; v[4 * j + 3] += res[j].w;
            }
        } else if (ep.residual) {
            const float* rr = ep.residual + (size_t)row * ep.ldr + col0;
            if (full && ((reinterpret_cast<uintptr_t>(rr) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(rr + j);
                    v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < N) v[j] += rr[j];
            }
        }
        if (ep.out_f32) {
            float* o = reinterpret_cast<float*>(ep.out) + (size_t)row * ep.ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < N) o[j] = v[j];
            }
        } else {
            bf16* o = reinterpret_cast<bf16*>(ep.out) + (size_t)row * ep.ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2);
                    pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(o + j) = pk;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < N) o[j] = __float2bfloat16_rn(v[j]);
            }
        }
    }
}


// ---- host side: tensor maps ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<long long>()(k.rows * 1000003 + k.cols) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= std::hash<long long>()(k.ld * 31 + k.box_rows) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

// A 2-D bfloat16 tensor [rows, cols] with row pitch ld, cut into boxes of box_rows x 64 with
// 128-byte swizzle.  Encoded maps are kept: a model's operands come back every step.
bool get_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

}  // namespace
