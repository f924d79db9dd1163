// Pieces shared by the tcgen05 matrix-product kernels: mbarrier and TMA wrappers, shared-memory
// and instruction descriptors, tensor-memory loads, the write-back of one accumulator chunk, and
// the host-side cache of TMA tensor maps.
#pragma once

#include <cuda.h>

#include <cstring>
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
    int tma_out;             // 1: the kernel's output tensor map is valid and the write-back goes through it
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

// The activation as a template argument.  Chosen per element at run time (apply_act_fast with the kernel's
// `act`), the compiler computed every activation for every element and picked one; the same went for the cache
// address of the key/value write with its divisions.  So what a product has of these is decided once per
// warp, outside the element loops (write_back_warp), and the loops are instantiated for each case.
template <int ACT>
__device__ __forceinline__ float act_of(float v) {
    if (ACT == SANDY_ACT_GELU_TANH) return gelu_tanh_fast(v);
    if (ACT == SANDY_ACT_GELU_ERF) return gelu_erf(v);
    return v;
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
// my_bias: the bias of column col0 + lane (load_bias), handed round by shuffles.
template <int ACT, bool KV>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], int row, int col0, const EpilogueArgs& ep, int M,
                                            int N, const float4 (&res)[8], bool have_res, int kv_page, int kv_slot,
                                            int* status, float my_bias) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = act_of<ACT>(__uint_as_float(r[j]) + __shfl_sync(0xffffffffu, my_bias, j));
    if (KV && row < M && col0 + 32 > ep.kv.q_cols) {
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


// ---- write-back through TMA stores -----------------------------------------------------------------
// tcgen05.ld hands a thread 32 consecutive columns of ONE row (its tensor-memory lane).  Stored
// straight from those registers (store_chunk above) a warp writes 32 pieces of 16 bytes in 32
// different rows per instruction and the kernel sits in its write-back for longer than in its main
// loop (measured on a 2048 x 2304 x 768 product: 13.6 us with register stores, 10.7 through the copy
// engine; turning the chunk round in shared memory and storing whole row pieces was no faster than
// the register stores).  So each warp builds its 32 rows x 128 bytes (64 bfloat16 or 32 float
// columns) in a shared-memory tile in the 128-byte swizzle and one lane hands the tile to TMA:
//   - rows past M and columns past N are clipped by the tensor map, so every M and N is taken;
//   - a residual that is the output itself (x += ...) becomes a TMA reduce-add into x: the SM never
//     reads the old value, and every element still receives exactly one addition;
//   - key and value columns go into their cache pages from the registers, as in store_chunk.
// A tensor map wants a 16-byte aligned base and row pitch, and the store clips rows in pieces of 16
// bytes; products whose output does not fit that, or whose residual is another tensor than the output,
// are written back by store_chunk.
constexpr int EPI_WARP_BYTES = 32 * 128;                   // a warp's staging tile; 1024-byte aligned

__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// This lane's 32 accumulator values of the chunk at global column col0 (its row: `row`): bias,
// activation, rounding, into the warp's tile; `h` is the chunk's place in the tile (bfloat16: 0 or 1,
// float: 0).  Key and value columns also go to the cache.
// my_bias: the bias of column col0 + lane (load_bias).
template <int ACT, bool KV>
__device__ __forceinline__ void stage_chunk(const uint32_t (&r)[32], uint8_t* tile, int h, int row, int col0,
                                            const EpilogueArgs& ep, int M, int N, int kv_page, int kv_slot, int* status,
                                            float my_bias) {
    const int lane = threadIdx.x & 31;
    uint8_t* my_row = tile + lane * 128;
    const int twist = lane & 7;                 // the 128-byte swizzle: 16-byte piece j of row l lies at piece j ^ (l % 8)
    if (ep.out_f32) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++)
                v[e] = act_of<ACT>(__uint_as_float(r[4 * j + e]) + __shfl_sync(0xffffffffu, my_bias, 4 * j + e));
            *reinterpret_cast<float4*>(my_row + ((j ^ twist) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        }
    } else {
        const bool to_cache = KV && row < M && col0 + 32 > ep.kv.q_cols;
        const bool page_ok = kv_page >= 0 && kv_page < ep.kv.num_pages;
        if (to_cache && !page_ok && status) atomicOr(status, 8);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; e++)
                v[e] = act_of<ACT>(__uint_as_float(r[8 * q + e]) + __shfl_sync(0xffffffffu, my_bias, 8 * q + e));
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
            uint4 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&h0);
            pk.y = *reinterpret_cast<const uint32_t*>(&h1);
            pk.z = *reinterpret_cast<const uint32_t*>(&h2);
            pk.w = *reinterpret_cast<const uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(my_row + (((4 * h + q) ^ twist) << 4)) = pk;
            // eight columns from a multiple of eight never straddle the query / key / value ranges or two
            // heads (the host checks q_cols % 8 == 0 and head_dim % 16 == 0)
            const int col = col0 + 8 * q;
            if (KV && to_cache && page_ok && col >= ep.kv.q_cols && col + 8 <= N) {
                const int c = col - ep.kv.q_cols;
                const bool is_v = c >= ep.kv.kv_cols;
                const int c2 = is_v ? c - ep.kv.kv_cols : c;
                const int head = c2 / ep.kv.head_dim, d = c2 % ep.kv.head_dim;
                bf16* dst = (is_v ? ep.kv.v_cache : ep.kv.k_cache) + (size_t)kv_page * ep.kv.page_stride +
                            ((size_t)head * ep.kv.page_size + kv_slot) * ep.kv.head_dim + d;
                *reinterpret_cast<uint4*>(dst) = pk;
            }
        }
    }
}

// One lane hands the warp's tile to TMA: output columns from col0, rows from row0.
__device__ __forceinline__ void store_tile(const CUtensorMap* map_out, const uint8_t* tile, int col0, int row0, bool add) {
    if (add)
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_out),
                     "r"(smem_u32(tile)), "r"(col0), "r"(row0)
                     : "memory");
    else
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_out),
                     "r"(smem_u32(tile)), "r"(col0), "r"(row0)
                     : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// The bias values a lane needs in write_back_warp: of column col_first + 32 c + lane for each chunk c.
// A trip to memory each, so the kernels ask for them before they wait for the accumulator (the bias is a
// weight: no kernel writes it).
template <int NCHUNKS>
__device__ __forceinline__ void load_bias(float (&b)[NCHUNKS], const EpilogueArgs& ep, int col_first, int N) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int c = 0; c < NCHUNKS; c++) {
        const int col = col_first + c * 32 + lane;
        b[c] = (ep.bias && col < N) ? __bfloat162float(ep.bias[col]) : 0.0f;
    }
}

template <int NCHUNKS>
__device__ __forceinline__ float bias_of(const float (&b)[NCHUNKS], int c) {
    float v = b[0];
#pragma unroll
    for (int k = 1; k < NCHUNKS; k++)
        if (c == k) v = b[k];           // selects, so that b stays in registers under a rolled loop
    return v;
}

// A warp's whole write-back: NCHUNKS chunks of 32 columns from tensor-memory address taddr (its lane
// quarter, the first chunk's column); output rows row0 .. row0 + 31 (this lane: row0 + lane), first
// column col_first.  tiles: the warp's NTILES staging tiles of EPI_WARP_BYTES each; with two, a tile is
// filled while the copy engine still reads the other.  Chunks leave tensor memory two at a time (one
// wait for both loads).  after_loads() runs once the last chunk has left tensor memory (the persistent
// kernels hand the accumulator back there).
template <int NCHUNKS, int NTILES, int ACT, bool KV, typename AfterLoads>
__device__ __forceinline__ void write_back_warp_as(uint32_t taddr, uint8_t* tiles, int row0, int col_first, const EpilogueArgs& ep,
                                                const CUtensorMap* map_out, int M, int N, int kv_page, int kv_slot, int* status,
                                                const float (&bias)[NCHUNKS], AfterLoads after_loads) {
    static_assert(NTILES == 1 || NTILES == 2, "one or two staging tiles");
    const int lane = threadIdx.x & 31;
    const int row = row0 + lane;
    if (!ep.tma_out) {
#pragma unroll 1
        for (int c = 0; c < NCHUNKS; c++) {
            float4 res[8];
            const bool have_res = load_residual(res, row, col_first + c * 32, ep, M, N);
            uint32_t r[32];
            tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
            tmem_wait_ld();
            if (c == NCHUNKS - 1) after_loads();
            store_chunk<ACT, KV>(r, row, col_first + c * 32, ep, M, N, res, have_res, kv_page, kv_slot, status, bias_of(bias, c));
        }
        return;
    }
    int stores = 0;                 // TMA stores issued so far: store i uses tile i % NTILES
    // before tile `stores % NTILES` is written again, the store that last read it must have done so
    auto tile_free = [&] {
        if (stores >= NTILES) {
            if (lane == 0) {
                if (NTILES == 1) bulk_wait_read();
                else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            __syncwarp();
        }
    };
    auto send = [&](uint8_t* tile, int col0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // my writes, before the copy engine reads them
        __syncwarp();
        if (lane == 0 && col0 < N && row0 < M) store_tile(map_out, tile, col0, row0, ep.residual != nullptr);
        else if (lane == 0) asm volatile("cp.async.bulk.commit_group;" ::: "memory");     // keeps the groups counted alike
        stores++;
    };
#pragma unroll 1
    for (int c0 = 0; c0 < NCHUNKS; c0 += 2) {
        const int col0 = col_first + c0 * 32;
        const bool two = c0 + 1 < NCHUNKS;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(taddr + (uint32_t)(c0 * 32), ra);
        if (two) tmem_ld_32x32(taddr + (uint32_t)(c0 * 32 + 32), rb);
        tmem_wait_ld();
        if (c0 + 2 >= NCHUNKS) after_loads();
        if (ep.out_f32) {
            // a float tile is one chunk wide
            tile_free();
            uint8_t* tile = tiles + (stores % NTILES) * EPI_WARP_BYTES;
            stage_chunk<ACT, KV>(ra, tile, 0, row, col0, ep, M, N, kv_page, kv_slot, status, bias_of(bias, c0));
            send(tile, col0);
            if (two) {
                tile_free();
                tile = tiles + (stores % NTILES) * EPI_WARP_BYTES;
                stage_chunk<ACT, KV>(rb, tile, 0, row, col0 + 32, ep, M, N, kv_page, kv_slot, status, bias_of(bias, c0 + 1));
                send(tile, col0 + 32);
            }
        } else if (two) {
            // a bfloat16 tile is two chunks wide
            tile_free();
            uint8_t* tile = tiles + (stores % NTILES) * EPI_WARP_BYTES;
            stage_chunk<ACT, KV>(ra, tile, 0, row, col0, ep, M, N, kv_page, kv_slot, status, bias_of(bias, c0));
            stage_chunk<ACT, KV>(rb, tile, 1, row, col0 + 32, ep, M, N, kv_page, kv_slot, status, bias_of(bias, c0 + 1));
            send(tile, col0);
        } else {
            // a last bfloat16 chunk that fills only half of a tile's rows: the store would write the other
            // half too, so this chunk goes out of the registers
            float4 res[8];
            store_chunk<ACT, KV>(ra, row, col0, ep, M, N, res, false, kv_page, kv_slot, status, bias_of(bias, c0));
        }
    }
    if (lane == 0) bulk_wait_read();       // the staging memory may be reused (or die) after this
    __syncwarp();
}

// The write-back of a warp, instantiated for what the product has: the key/value write (never with an
// activation: the host refuses that), one of the activations, or neither.
template <int NCHUNKS, int NTILES, typename AfterLoads>
__device__ __forceinline__ void write_back_warp(uint32_t taddr, uint8_t* tiles, int row0, int col_first, const EpilogueArgs& ep,
                                                const CUtensorMap* map_out, int M, int N, int kv_page, int kv_slot, int* status,
                                                const float (&bias)[NCHUNKS], AfterLoads after_loads) {
    if (ep.kv.k_cache)
        write_back_warp_as<NCHUNKS, NTILES, SANDY_ACT_NONE, true>(taddr, tiles, row0, col_first, ep, map_out, M, N, kv_page, kv_slot,
                                                                  status, bias, after_loads);
    else if (ep.act == SANDY_ACT_GELU_TANH)
        write_back_warp_as<NCHUNKS, NTILES, SANDY_ACT_GELU_TANH, false>(taddr, tiles, row0, col_first, ep, map_out, M, N, kv_page,
                                                                        kv_slot, status, bias, after_loads);
    else if (ep.act == SANDY_ACT_GELU_ERF)
        write_back_warp_as<NCHUNKS, NTILES, SANDY_ACT_GELU_ERF, false>(taddr, tiles, row0, col_first, ep, map_out, M, N, kv_page,
                                                                       kv_slot, status, bias, after_loads);
    else
        write_back_warp_as<NCHUNKS, NTILES, SANDY_ACT_NONE, false>(taddr, tiles, row0, col_first, ep, map_out, M, N, kv_page, kv_slot,
                                                                   status, bias, after_loads);
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
    int box_rows, elem;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && elem == o.elem;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<long long>()(k.rows * 1000003 + k.cols) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= std::hash<long long>()(k.ld * 31 + k.box_rows + 1000 * k.elem) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

// A 2-D tensor [rows, cols] with row pitch ld (in elements) of bfloat16 (elem 2) or float (elem 4), cut
// into boxes of box_rows x 128 bytes (64 or 32 columns) with 128-byte swizzle.  Encoded maps are kept: a
// model's operands come back every step.
bool get_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out, int elem = 2) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows, elem};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem), (cuuint32_t)box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem_strides,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// The tensor map of a product's output for the write-back through TMA, if the output allows one: a
// 16-byte aligned base and row pitch, and no residual other than the (float) output itself.  Up to one
// tile of rows the registers are the quicker way (a store through TMA has the longer latency, and so few
// rows are written in no time either way: at 64 rows 5.4 us against 6.1 for a 2304 x 768 product).
bool get_out_map(EpilogueArgs& ep, int M, int N, CUtensorMap* out) {
    const int elem = ep.out_f32 ? 4 : 2;
    ep.tma_out = 0;
    memset(out, 0, sizeof(*out));
    if (M <= BM) return false;
    if ((reinterpret_cast<uintptr_t>(ep.out) & 15) || ((long long)ep.ldc * elem) % 16 != 0) return false;
    // a row's end too: the store clips a row in pieces of 16 bytes (a 777-column bfloat16 output with room
    // behind its rows had columns 777 .. 783 overwritten)
    if (((long long)N * elem) % 16 != 0) return false;
    if (ep.residual && (ep.residual != ep.out || ep.ldr != ep.ldc || !ep.out_f32)) return false;
    if (!get_map(ep.out, M, N, ep.ldc, 32, out, elem)) return false;
    ep.tma_out = 1;
    return true;
}

}  // namespace
