// A decode step as ONE kernel: a resident grid (one block per SM) that walks a list of
// operations, with a grid-wide barrier between one operation and the next.
//
// Why.  A decode step of a few tokens is a chain of some seventy small operations, each of
// which reads a weight matrix once.  As seventy kernels, each costs about five microseconds
// however little it does (launch, first trip to memory, tail), five to ten times what
// streaming its weights takes.  Here the chain is data: an array of `Op` records that the
// host fills once per step shape (the model's parts describe their products, norms and
// attention calls instead of launching them) and that every block interprets.
//
// State.  The kernel is correct (tested against the plain implementation and against the chain of
// kernels) and OFF by default: measured on GPT-2 small with 8 requests it takes 0.66 ms a step
// where the chain of kernels under a CUDA graph takes 0.40 ms.  Its timeline (block 0's clock
// inside every operation, see `timeline`) says why: a barrier over 148 blocks costs 1.6 to 3 us,
// a trip to L2 for data that every block reads at once 1.5 to 2.5 us, and with nine warps on an
// SM nothing hides the latency between dependent instructions, so a product that does 0.3 us of
// arithmetic takes 3 us and attention over 170 keys 9 us.  Five operations a layer leave a floor
// near 18 us a layer, against 27 us for the chain of kernels, which was not worth the rest of
// the work; the file stays as a measured experiment and a tool (the timeline).
//
// What was done for speed, each measured on this kernel:
//  (1) Trips to memory that depend on one another inside an operation.  What does not depend on
//      the operation before is fetched ahead: the weights, and with them each product's bias and
//      the gain and offset of a fused norm, by a producer warp that runs through the whole list on
//      its own (bulk asynchronous copies into a ring of shared-memory stages, across the
//      barriers); the step's index arrays (positions, request of each token, block tables), once,
//      into shared memory; the record of the next operation while the current one runs.
//  (2) The number of bulk copies.  A copy costs the SM's copy engine about 60 ns whatever its
//      size (1 KB rows gave 12 GB/s per SM), so a stage is ONE copy wherever the weight allows
//      it: a block owns a contiguous range of output columns, and the rows of up to 16 units
//      (8 columns each) of a dense [N, K] weight are one run of bytes.  Only a K too long for a
//      stage falls back to one copy per row and k piece.
//  (3) The size of the code (148 KB at first, 100 KB now): loops stay rolled where registers
//      allow, and every operation has one code path.
//
// Operations (all bfloat16 storage, float arithmetic):
//   EMBED  x[t] = wte[id[t]] + wpe[pos[t]]                              (embed.cu)
//   NORM   y[r] = LayerNorm(x[rows[r]])                                 (norm.cu)
//   GEMM   out = act(A w^T + bias) + residual, A = a or LayerNorm(x); key/value columns go to
//          the paged cache                                               (gemm_skinny.cu)
//   ATTN   attention of single tokens over the paged cache, keys split over blocks, the last
//          block of a (token, head) pair to finish merges the splits    (attention_decode.cu)
// Rows M <= 16.  Sums are float; a dot product's k slices are added in a fixed order.
//
// Memory ordering.  Data written by one operation and read by a later one crosses blocks:
// writers arrive on the barrier with release semantics, readers load with ld.global.cg (L2,
// never a stale L1 line: the residual stream is rewritten at the same address by every layer).
//
// Every wait (mbarrier, grid barrier) is bounded.  When one expires the block raises a status
// bit and an abort flag that makes every other wait return at once; nobody leaves on the spot
// (the warps of a block must keep meeting at the same block barriers), the block leaves
// together at the next grid barrier.
#include "epilogue.cuh"

namespace {

constexpr int CWARPS = 8;                      // compute warps
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = CTHREADS + 32;         // and the producer warp
constexpr int COLS = 8;                        // output columns of a GEMM unit
constexpr int STAGE_DATA = 24 * 1024;          // weight bytes of a dense stage
constexpr int KPIECE_MAX = 1536;               // k per stage when rows are copied one by one
constexpr int ROW_PAD = 64;                    // bytes of padding per row then: 16-byte slots = 4 mod 8
constexpr int MAX_STAGE_UNITS = 16;
constexpr int BIAS_OFF = COLS * (KPIECE_MAX * 2 + ROW_PAD);       // 25088 >= STAGE_DATA
constexpr int STAGE_BYTES = BIAS_OFF + MAX_STAGE_UNITS * 16;
constexpr int NSTAGE = 4;
constexpr int A_BYTES = 100 * 1024;            // activation rows of the running GEMM / attention scratch
constexpr int TABLE_INTS = 2048;               // block tables of the step, cached
constexpr int MAX_TABLES = 4;
constexpr int XPAD = 32;                       // elements of padding per activation row (as gemm_skinny.cu)
constexpr int SMEM_BYTES = A_BYTES + NSTAGE * STAGE_BYTES + TABLE_INTS * 4;
constexpr int MAX_ROWS = 16;
constexpr int MAX_NORM_WIDTH = 2048;           // gain and offset of a fused norm share one stage
constexpr int BATCH_FROM = 4;                  // more units per block than this: sums are exchanged per 8 units
constexpr int UB = 8;                          // units of such a batch
constexpr uint32_t WAIT_LIMIT = 1u << 20;      // sleeps of about SUSPEND_NS each
constexpr uint32_t SUSPEND_NS = 2000;
constexpr uint32_t SPIN_LIMIT = 1u << 22;      // polls of the grid barrier's counter
constexpr int ATT_UNROLL = 4;
static_assert(BIAS_OFF >= STAGE_DATA && 2 * MAX_NORM_WIDTH * 2 <= STAGE_BYTES, "stage layout");

enum OpKind : int { OP_EMBED = 0, OP_NORM = 1, OP_GEMM = 2, OP_ATTN = 3 };
enum StatusBits : int { ST_BAD_ID = 1, ST_BAD_POS = 2, ST_KV_PAGE = 8, ST_ATT_PAGE = 16, ST_WAIT = 128 };

// One operation.  Field use by kind is given in the Python mirror of this struct (program.py).
struct Op {
    int kind, M, N, K;
    int lda, ldw, ldr, ldc;
    int act, out_dtype, ldx, max_blocks;
    int q_cols, kv_cols, head_dim, page_size;
    int num_pages, n_heads, n_kv_heads, window;
    int num_splits, vocab, n_pos, ld_q;
    int table_slot, flags;
    float eps, scale;
    long long page_stride;
    const bf16* a;  const float* x;  const bf16* gamma;  const bf16* beta;
    const bf16* w;  const bf16* bias;  const float* residual;  void* out;
    bf16* k_cache;  bf16* v_cache;  const int* block_table;  const int* token_seq;
    const int* positions;  const int* rows;  const int* ids;  const bf16* wpe;
    float* partial;  int* counters;  int* status;  void* reserved;
};

// The step's index arrays, the same for every operation of a program.
struct StepArrays {
    const int* positions;          // [n_tokens]
    const int* token_seq;          // [n_tokens]
    const int* tables[MAX_TABLES]; // block tables [n_seqs, max_blocks[i]]
    int max_blocks[MAX_TABLES];
    int n_tokens, n_seqs, n_tables, pad;
};

struct Sync {
    unsigned long long count;     // arrivals at grid barriers since the buffer was zeroed
    unsigned long long base;      // value of `count` when the running launch began
    int abort;
    int pad;
};

struct Shared {
    uint64_t full_bar[NSTAGE], empty_bar[NSTAGE];
    float partial[CWARPS][16][COLS + 1];       // the warps' sums of one unit
    float bias[UB * COLS];
    Op op[2];              // the running operation and the next one
    int pos[MAX_ROWS], seq[MAX_ROWS];
    int table_off[MAX_TABLES];
    int flag;
    int stop;              // written by thread 0 between two block barriers: everyone reads the same value
    volatile int abort;
    unsigned long long* mark;   // where block 0's thread 0 notes the time inside the running operation, or null
};

// How a block walks a GEMM: its units and the shape of its weight stages.  The producer and the
// compute warps both derive it from the record, so they agree on the order of the stages.
struct GemmPlan {
    int u_begin, n_units;      // this block's units: [u_begin, u_begin + n_units)
    bool dense;                // a stage is one run of bytes: the whole K of `per_stage` units
    int per_stage;             // units in a dense stage
    int npieces, kpiece;       // otherwise: k pieces of a unit, one stage each, rows copied one by one
    int pitch;                 // bytes between weight rows in a stage
};

__device__ __forceinline__ GemmPlan gemm_plan(int N, int K, int ldw) {
    GemmPlan p;
    const int units = (N + COLS - 1) / COLS;
    const int upb = (units + gridDim.x - 1) / gridDim.x;
    p.u_begin = min(units, (int)blockIdx.x * upb);
    p.n_units = min(units, p.u_begin + upb) - p.u_begin;
    p.dense = ldw == K && COLS * K * 2 <= STAGE_DATA;
    if (p.dense) {
        p.per_stage = min(MAX_STAGE_UNITS, STAGE_DATA / (COLS * K * 2));
        p.npieces = 1;
        p.kpiece = K;
        p.pitch = K * 2;
    } else {
        p.per_stage = 1;
        p.npieces = (K + KPIECE_MAX - 1) / KPIECE_MAX;
        p.kpiece = ((K + p.npieces - 1) / p.npieces + 31) / 32 * 32;
        p.pitch = p.kpiece * 2 + ROW_PAD;
    }
    return p;
}

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Optional time marks inside an operation (slot 0: its activations are staged / its first keys
// are asked for; slot 1: its work is done, before the barrier).
__device__ __forceinline__ void mark(Shared& sh, int slot) {
    if (sh.mark && threadIdx.x == 0) sh.mark[slot] = now_ns();
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }

__device__ __noinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* s_abort) {
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
        if (*s_abort) return false;
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
__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned long long* p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A wait has expired: tell this block and the grid.
__device__ __noinline__ void give_up(Shared& sh, Sync* sync, int* status) {
    if (!sh.abort) {
        sh.abort = 1;
        atomicExch(&sync->abort, 1);
        if (status) atomicOr(status, ST_WAIT);
    }
}

// ---- the barrier over the grid ---------------------------------------------------------------
// All compute threads of all blocks; `target` is the value the counter has once every block has
// arrived.  The block barrier before the release-add makes every thread's writes part of what
// the add releases; the acquire poll and the block barrier after it order every thread's later
// reads behind the other blocks' arrivals.  Returns false if the launch is being abandoned.
__device__ __noinline__ bool grid_barrier(Sync* sync, unsigned long long target, Shared& sh, int* status) {
    compute_sync();
    if (threadIdx.x == 0) {
        red_release_add(&sync->count, 1ULL);
        bool ok = false;
        for (uint32_t it = 0; it < SPIN_LIMIT && !sh.abort; it++) {
            if (ld_acquire(&sync->count) >= target) {
                ok = true;
                break;
            }
            if ((it & 63) == 63 && *reinterpret_cast<volatile int*>(&sync->abort)) break;
        }
        if (!ok) give_up(sh, sync, status);
        sh.stop = sh.abort;
    }
    compute_sync();
    return sh.stop == 0;
}

// ---- LayerNorm of one row by one warp ----------------------------------------------------------
// Mean, biased variance in two passes, 1/sqrt(var + eps), gain and offset, rounded to bfloat16
// (src/core/TensorCalc.cpp:2048-2072 of the reference).  Up to 1024 wide the row is held in
// registers; wider rows are read again from L2 for each pass (rolled loops, four loads in flight).
// gamma, beta: global or shared memory.  One body for every caller keeps the code small.
__device__ __forceinline__ void ln_store4(const float4& v, float mean, float inv, const bf16* gamma, const bf16* beta,
                                          bf16* dst, int k) {
    const uint2 gm = *reinterpret_cast<const uint2*>(gamma + k);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gm);
    const float2 g01 = __bfloat1622float2(gh[0]), g23 = __bfloat1622float2(gh[1]);
    float y0 = (v.x - mean) * inv * g01.x, y1 = (v.y - mean) * inv * g01.y;
    float y2 = (v.z - mean) * inv * g23.x, y3 = (v.w - mean) * inv * g23.y;
    if (beta) {
        const uint2 bm = *reinterpret_cast<const uint2*>(beta + k);
        const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bm);
        const float2 b01 = __bfloat1622float2(bh[0]), b23 = __bfloat1622float2(bh[1]);
        y0 += b01.x; y1 += b01.y; y2 += b23.x; y3 += b23.y;
    }
    __nv_bfloat162 p0 = __floats2bfloat162_rn(y0, y1), p1 = __floats2bfloat162_rn(y2, y3);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&p0);
    pk.y = *reinterpret_cast<uint32_t*>(&p1);
    *reinterpret_cast<uint2*>(dst + k) = pk;
}

__device__ __noinline__ void ln_row(const float* xr, const bf16* gamma, const bf16* beta, float eps, int K,
                                    bf16* dst, int lane) {
    constexpr int RV = 8;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (K <= RV * 128) {
        float4 v[RV];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < RV; i++) {
            const int k = (i * 32 + lane) * 4;
            v[i] = k < K ? __ldcg(reinterpret_cast<const float4*>(xr + k)) : zero4;
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        const float mean = warp_sum(s) / (float)K;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < RV; i++) {
            const int k = (i * 32 + lane) * 4;
            if (k < K) {
                const float cx = v[i].x - mean, cy = v[i].y - mean, cz = v[i].z - mean, cw = v[i].w - mean;
                q += (cx * cx + cy * cy) + (cz * cz + cw * cw);
            }
        }
        const float inv = 1.0f / sqrtf(warp_sum(q) / (float)K + eps);
#pragma unroll
        for (int i = 0; i < RV; i++) {
            const int k = (i * 32 + lane) * 4;
            if (k < K) ln_store4(v[i], mean, inv, gamma, beta, dst, k);
        }
        return;
    }
    float s = 0.0f;
    for (int k0 = lane * 4; k0 < K; k0 += 512) {
        float4 v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = k0 + e * 128 < K ? __ldcg(reinterpret_cast<const float4*>(xr + k0 + e * 128)) : zero4;
#pragma unroll
        for (int e = 0; e < 4; e++) s += (v[e].x + v[e].y) + (v[e].z + v[e].w);
    }
    const float mean = warp_sum(s) / (float)K;
    float q = 0.0f;
    for (int k0 = lane * 4; k0 < K; k0 += 512) {
        float4 v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = k0 + e * 128 < K ? __ldcg(reinterpret_cast<const float4*>(xr + k0 + e * 128)) : zero4;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (k0 + e * 128 < K) {
                const float cx = v[e].x - mean, cy = v[e].y - mean, cz = v[e].z - mean, cw = v[e].w - mean;
                q += (cx * cx + cy * cy) + (cz * cz + cw * cw);
            }
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(q) / (float)K + eps);
    for (int k0 = lane * 4; k0 < K; k0 += 512) {
        float4 v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = k0 + e * 128 < K ? __ldcg(reinterpret_cast<const float4*>(xr + k0 + e * 128)) : zero4;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (k0 + e * 128 < K) ln_store4(v[e], mean, inv, gamma, beta, dst, k0 + e * 128);
        }
    }
}

// ---- EMBED ---------------------------------------------------------------------------------------
__device__ void run_embed(const Op& op) {
    float* out = reinterpret_cast<float*>(op.out);
    for (int t = blockIdx.x; t < op.M; t += gridDim.x) {
        const int id = __ldg(op.ids + t);
        const int p = op.wpe ? __ldg(op.positions + t) : 0;
        const bool ok = id >= 0 && id < op.vocab && (!op.wpe || (p >= 0 && p < op.n_pos));
        if (!ok && threadIdx.x == 0 && op.status) atomicOr(op.status, (id >= 0 && id < op.vocab) ? ST_BAD_POS : ST_BAD_ID);
        const bf16* trow = op.w + (size_t)(ok ? id : 0) * op.N;
        const bf16* prow = op.wpe ? op.wpe + (size_t)(ok ? p : 0) * op.N : nullptr;
        for (int e = threadIdx.x; e < op.N; e += CTHREADS) {
            float v = 0.0f;
            if (ok) {
                v = __bfloat162float(trow[e]);
                if (prow) v += __bfloat162float(prow[e]);
            }
            out[(size_t)t * op.ldc + e] = v;
        }
    }
}

// ---- NORM ----------------------------------------------------------------------------------------
__device__ void run_norm(const Op& op) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bf16* out = reinterpret_cast<bf16*>(op.out);
    for (int r = blockIdx.x + gridDim.x * warp; r < op.M; r += gridDim.x * CWARPS) {
        const int src = op.rows ? __ldg(op.rows + r) : r;
        ln_row(op.x + (size_t)src * op.ldx, op.gamma, op.beta, op.eps, op.K, out + (size_t)r * op.ldc, lane);
    }
}

// ---- GEMM ----------------------------------------------------------------------------------------
// The page of row m's key/value (from the cached index arrays when the operation's table is cached).
__device__ __forceinline__ int kv_page_of(const Op& op, const Shared& sh, const int* tables, int m, int& pos) {
    if (op.table_slot >= 0) {
        pos = sh.pos[m];
        const int b = pos / op.page_size;
        return (pos >= 0 && b < op.max_blocks) ? tables[sh.table_off[op.table_slot] + sh.seq[m] * op.max_blocks + b] : -1;
    }
    pos = __ldg(op.positions + m);
    const int b = pos / op.page_size;
    return (pos >= 0 && b < op.max_blocks)
        ? __ldg(op.block_table + (size_t)__ldg(op.token_seq + m) * op.max_blocks + b) : -1;
}

// v = the finished dot product of row m, column col, bias included: activation, residual, store,
// and the cache write if col is a key or value column.
__device__ __forceinline__ void finish_element(const Op& op, const Shared& sh, const int* tables, int m, int col,
                                               float v, float res) {
    v = apply_act(v, op.act) + res;
    if (op.out_dtype == SANDY_F32) reinterpret_cast<float*>(op.out)[(size_t)m * op.ldc + col] = v;
    else reinterpret_cast<bf16*>(op.out)[(size_t)m * op.ldc + col] = __float2bfloat16_rn(v);
    if (op.k_cache && col >= op.q_cols) {
        const int c = col - op.q_cols;
        const bool is_v = c >= op.kv_cols;
        const int c2 = is_v ? c - op.kv_cols : c;
        const int head = c2 / op.head_dim, d = c2 % op.head_dim;
        int pos;
        const int page = kv_page_of(op, sh, tables, m, pos);
        if (page < 0 || page >= op.num_pages) {
            if (op.status) atomicOr(op.status, ST_KV_PAGE);
        } else {
            const size_t dst = (size_t)page * op.page_stride +
                               ((size_t)head * op.page_size + (pos % op.page_size)) * op.head_dim + d;
            (is_v ? op.v_cache : op.k_cache)[dst] = __float2bfloat16_rn(v);
        }
    }
}

__device__ void run_gemm(const Op& op, uint32_t& wcount, uint8_t* a_region, uint8_t* w_ring, const int* tables,
                         Shared& sh, Sync* sync) {
    const int M = op.M, N = op.N, K = op.K;
    const GemmPlan plan = gemm_plan(N, K, op.ldw);
    if (plan.n_units <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int apitch = K + XPAD;
    bf16* as = reinterpret_cast<bf16*>(a_region);

    // the activation rows, in shared memory for all of this block's units
    if (op.x) {
        // gain and offset arrive through the ring, one stage ahead of the weights
        const int st = wcount % NSTAGE;
        if (!mbar_wait(&sh.full_bar[st], (wcount / NSTAGE) & 1, &sh.abort)) give_up(sh, sync, op.status);
        const bf16* gamma = reinterpret_cast<const bf16*>(w_ring + (size_t)st * STAGE_BYTES);
        const bf16* beta = op.beta ? gamma + K : nullptr;
        for (int r = warp; r < M; r += CWARPS)
            ln_row(op.x + (size_t)r * op.ldx, gamma, beta, op.eps, K, as + (size_t)r * apitch, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty_bar[st]);
        wcount++;
    } else {
        // four loads in flight per thread before the first store
        const int per_row = K / 8;
        const int total = M * per_row;
        for (int i0 = threadIdx.x; i0 < total; i0 += 4 * CTHREADS) {
            uint4 v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * CTHREADS;
                if (i < total) v[e] = __ldcg(reinterpret_cast<const uint4*>(op.a + (size_t)(i / per_row) * op.lda + (i % per_row) * 8));
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * CTHREADS;
                if (i < total) *reinterpret_cast<uint4*>(as + (size_t)(i / per_row) * apitch + (i % per_row) * 8) = v[e];
            }
        }
    }
    compute_sync();
    mark(sh, 0);

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bool r0_ok = g < M, r1_ok = g + 8 < M;
    const bf16* a0 = as + (size_t)g * apitch;
    const bf16* a1 = as + (size_t)(g + 8) * apitch;

    // The warps' sums are exchanged once per batch of units: one unit when the block has few, eight
    // when it has many (the vocabulary projection) and the activation rows leave room for it.
    const size_t a_used = ((size_t)M * apitch * 2 + 15) / 16 * 16;
    const bool batched = plan.n_units > BATCH_FROM && a_used + (size_t)CWARPS * 16 * (UB * COLS + 1) * 4 <= (size_t)A_BYTES;
    const int ub = batched ? UB : 1;
    const int bp = ub * COLS + 1;                                        // floats per row of the sums
    float* part = batched ? reinterpret_cast<float*>(a_region + a_used) : &sh.partial[0][0][0];   // [CWARPS][16][bp]
    float* mine = part + (size_t)warp * 16 * bp;

    const uint8_t* stage = nullptr;
    for (int i0 = 0; i0 < plan.n_units; i0 += ub) {
        const int nb = min(ub, plan.n_units - i0);
        // this thread's first output element of the batch: its residual is asked for now
        float res0 = 0.0f;
        {
            const int m = threadIdx.x / (nb * COLS), jc = threadIdx.x % (nb * COLS);
            const int col = (plan.u_begin + i0 + jc / COLS) * COLS + jc % COLS;
            if (op.residual && m < M && col < N) res0 = __ldcg(op.residual + (size_t)m * op.ldr + col);
        }
        for (int jb = 0; jb < nb; jb++) {
            const int i = i0 + jb, u = plan.u_begin + i;
            const int slot = plan.dense ? i % plan.per_stage : 0;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int p = 0; p < plan.npieces; p++) {
                const int st = wcount % NSTAGE;
                if (slot == 0) {
                    if (!mbar_wait(&sh.full_bar[st], (wcount / NSTAGE) & 1, &sh.abort)) give_up(sh, sync, op.status);
                    stage = w_ring + (size_t)st * STAGE_BYTES;
                }
                const int k0 = p * plan.kpiece;
                const int kw = min(plan.kpiece, K - k0);
                const int chunks = (kw + 31) / 32;
                const uint8_t* wst = stage + (size_t)(slot * COLS + g) * plan.pitch;
                if (p == 0 && warp == 0 && lane < COLS && op.bias) {
                    const int c = u * COLS + lane;
                    sh.bias[jb * COLS + lane] = (u * COLS + COLS <= N)
                        ? __bfloat162float(reinterpret_cast<const bf16*>(stage + BIAS_OFF)[slot * COLS + lane])
                        : (c < N ? __bfloat162float(__ldg(op.bias + c)) : 0.0f);
                }
                for (int c = warp; c < chunks; c += CWARPS) {
                    const int kk = c * 32 + t * 8;
                    const bool k_ok = kk < kw;
                    // one 16-byte piece of 8 consecutive k feeds two mma steps; both operands use the
                    // same assignment of k to fragment slots (see gemm_skinny.cu)
                    const uint4 wv = k_ok ? *reinterpret_cast<const uint4*>(wst + kk * 2) : zero;
                    const uint4 x0 = (k_ok && r0_ok) ? *reinterpret_cast<const uint4*>(a0 + k0 + kk) : zero;
                    const uint4 x1 = (k_ok && r1_ok) ? *reinterpret_cast<const uint4*>(a1 + k0 + kk) : zero;
                    mma_bf16(acc, x0.x, x1.x, x0.y, x1.y, wv.x, wv.y);
                    mma_bf16(acc, x0.z, x1.z, x0.w, x1.w, wv.z, wv.w);
                }
                // the stage goes back when its last unit is done with it
                if (!plan.dense || slot == plan.per_stage - 1 || i == plan.n_units - 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.empty_bar[st]);
                    wcount++;
                }
            }
            // C fragment: c0,c1 = (row g, columns 2t, 2t+1); c2,c3 = (row g+8, same columns)
            mine[g * bp + jb * COLS + 2 * t] = acc[0];
            mine[g * bp + jb * COLS + 2 * t + 1] = acc[1];
            mine[(g + 8) * bp + jb * COLS + 2 * t] = acc[2];
            mine[(g + 8) * bp + jb * COLS + 2 * t + 1] = acc[3];
        }
        compute_sync();
        for (int idx = threadIdx.x; idx < 16 * nb * COLS; idx += CTHREADS) {
            const int m = idx / (nb * COLS), jc = idx % (nb * COLS);
            const int col = (plan.u_begin + i0 + jc / COLS) * COLS + jc % COLS;
            if (m < M && col < N) {
                float v = part[m * bp + jc];
#pragma unroll
                for (int wi = 1; wi < CWARPS; wi++) v += part[((size_t)wi * 16 + m) * bp + jc];
                if (op.bias) v += sh.bias[jc];
                const float res = !op.residual ? 0.0f
                    : (idx == (int)threadIdx.x ? res0 : __ldcg(op.residual + (size_t)m * op.ldr + col));
                finish_element(op, sh, tables, m, col, v, res);
            }
        }
        compute_sync();      // the sums and the bias slots are reused by the next batch
    }
}

// The producer's view of the same walk: which stages this block will ask for, in order.
__device__ void run_producer(const Op* ops, int n_ops, uint8_t* w_ring, Shared& sh, Sync* sync, int* status) {
    const int lane = threadIdx.x & 31;
    uint32_t wcount = 0;
    auto acquire = [&](int st) -> bool {
        if (wcount < NSTAGE) return true;
        const bool got = mbar_wait(&sh.empty_bar[st], ((wcount / NSTAGE) - 1) & 1, &sh.abort);
        if (!__all_sync(0xffffffffu, got)) {      // the producer warp stands alone: it may leave
            give_up(sh, sync, status);
            return false;
        }
        return true;
    };
    for (int i = 0; i < n_ops; i++) {
        const Op& op = ops[i];
        if (op.kind != OP_GEMM) continue;
        const int N = op.N, K = op.K, ldw = op.ldw;
        const GemmPlan plan = gemm_plan(N, K, ldw);
        if (plan.n_units <= 0) continue;
        const bf16* w = op.w;
        const bf16* bias = op.bias;
        if (op.x) {
            const int st = wcount % NSTAGE;
            if (!acquire(st)) return;
            const bf16* gamma = op.gamma;
            const bf16* beta = op.beta;
            uint8_t* dst = w_ring + (size_t)st * STAGE_BYTES;
            if (lane == 0) {
                mbar_expect_tx(&sh.full_bar[st], (uint32_t)K * 2u * (beta ? 2u : 1u));
                bulk_load(dst, gamma, (uint32_t)K * 2u, &sh.full_bar[st]);
                if (beta) bulk_load(dst + (size_t)K * 2, beta, (uint32_t)K * 2u, &sh.full_bar[st]);
            }
            __syncwarp();
            wcount++;
        }
        if (plan.dense) {
            for (int i0 = 0; i0 < plan.n_units; i0 += plan.per_stage) {
                const int st = wcount % NSTAGE;
                if (!acquire(st)) return;
                const int u0 = plan.u_begin + i0;
                const int cnt = min(plan.per_stage, plan.n_units - i0);
                const int rows = min(N, (u0 + cnt) * COLS) - u0 * COLS;
                const uint32_t bytes = (uint32_t)rows * (uint32_t)K * 2u;
                const uint32_t bias_bytes = bias ? (uint32_t)(rows / COLS) * 16u : 0u;     // whole units only
                uint8_t* dst = w_ring + (size_t)st * STAGE_BYTES;
                if (lane == 0) {
                    mbar_expect_tx(&sh.full_bar[st], bytes + bias_bytes);
                    bulk_load(dst, w + (size_t)u0 * COLS * ldw, bytes, &sh.full_bar[st]);
                    if (bias_bytes) bulk_load(dst + BIAS_OFF, bias + (size_t)u0 * COLS, bias_bytes, &sh.full_bar[st]);
                }
                __syncwarp();
                wcount++;
            }
        } else {
            for (int i0 = 0; i0 < plan.n_units; i0++) {
                const int u = plan.u_begin + i0;
                const int rows = min(COLS, N - u * COLS);
                for (int p = 0; p < plan.npieces; p++) {
                    const int st = wcount % NSTAGE;
                    if (!acquire(st)) return;
                    const int k0 = p * plan.kpiece;
                    const uint32_t bytes = (uint32_t)min(plan.kpiece, K - k0) * 2u;
                    const bool with_bias = p == 0 && bias != nullptr && rows == COLS;
                    uint8_t* dst = w_ring + (size_t)st * STAGE_BYTES;
                    if (lane == 0) mbar_expect_tx(&sh.full_bar[st], bytes * rows + (with_bias ? 16u : 0u));
                    __syncwarp();
                    if (lane < rows)
                        bulk_load(dst + (size_t)lane * plan.pitch, w + (size_t)(u * COLS + lane) * ldw + k0, bytes, &sh.full_bar[st]);
                    if (lane == 31 && with_bias) bulk_load(dst + BIAS_OFF, bias + (size_t)u * COLS, 16u, &sh.full_bar[st]);
                    wcount++;
                }
            }
        }
    }
}

// ---- ATTN ----------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// The head size is a run-time value here (16, 32, 64, 128 or 256): one body for all of them.
// Scores are kept in units of log2 (the query is multiplied by scale * log2(e) once) and the
// running output is rescaled only when the maximum rises, as in attention_decode_bulk.cu.
__device__ void run_attn(const Op& op, uint8_t* scratch, const int* tables, Shared& sh) {
    constexpr int VEC = 8;
    const int D = op.head_dim;
    const int LPK = D / VEC;                    // lanes per key
    const int lpk_shift = __ffs(LPK) - 1;
    const int KPW = 32 >> lpk_shift;            // keys per warp per round
    const int GROUPS = CWARPS * KPW;
    float* sm_m = reinterpret_cast<float*>(scratch);
    float* sm_l = sm_m + GROUPS;
    float* sm_o = sm_l + GROUPS;                // [GROUPS][D]
    float* sm_w = sm_o + GROUPS * D;            // [GROUPS + 1]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> lpk_shift, sub = lane & (LPK - 1);
    const int group = warp * KPW + g;
    const int H = op.n_heads, splits = op.num_splits;
    const int units = op.M * H * splits;
    const int page_shift = __ffs(op.page_size) - 1, page_mask = op.page_size - 1;
    const int max_blocks = op.max_blocks, num_pages = op.num_pages;
    const long long page_stride = op.page_stride;
    const bf16* kbase = op.k_cache;
    const bf16* vbase = op.v_cache;
    bf16* out = reinterpret_cast<bf16*>(op.out);
    float* partial_o = op.partial;
    float* partial_ml = op.partial + (size_t)op.M * H * splits * D;
    const bool cached = op.table_slot >= 0;
    const float qscale = op.scale * 1.4426950408889634f;

    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int split = u % splits, pair = u / splits;
        const int h = pair % H, t = pair / H;
        const int s = cached ? sh.seq[t] : __ldg(op.token_seq + t);
        const int pos = cached ? sh.pos[t] : __ldg(op.positions + t);
        const int kvh = h / (H / op.n_kv_heads);
        const int lo = op.window > 0 ? max(0, pos + 1 - op.window) : 0;
        const int n_keys = pos - lo + 1;
        int chunk = (n_keys + splits - 1) / splits;
        chunk = (chunk + GROUPS - 1) / GROUPS * GROUPS;
        const int begin = lo + split * chunk;
        const int end = min(pos + 1, begin + chunk);
        const int* table = cached ? tables + sh.table_off[op.table_slot] + s * max_blocks
                                  : op.block_table + (size_t)s * max_blocks;
        const size_t head_off = (size_t)kvh * op.page_size * D + sub * VEC;

        const uint4 qraw = __ldcg(reinterpret_cast<const uint4*>(op.a + (size_t)t * op.ld_q + h * D + sub * VEC));
        float qf[VEC];
        float m = -INFINITY, l = 0.0f;
        float o[VEC];
#pragma unroll
        for (int i = 0; i < VEC; i++) o[i] = 0.0f;

        // Rounds of ATT_UNROLL keys per lane group, 16 bytes of each per lane.  One loop body asks
        // for round r + 1 and then works on round r (the first pass only asks), so the loads of a
        // round travel while the round before is multiplied and the code exists once.  The loads
        // are unconditional (a key past the end reads the first page instead): straight-line code,
        // all eight in flight together.  The trip count is the same for every lane of a warp.
        uint4 kraw[ATT_UNROLL], vraw[ATT_UNROLL], kc[ATT_UNROLL], vc[ATT_UNROLL];
        bool ok[ATT_UNROLL], okc[ATT_UNROLL];
        const int first = begin + warp * KPW, step = GROUPS * ATT_UNROLL;
        for (int base = first - step; base < end; base += step) {
            const bool work = base >= first;
            if (work) {
#pragma unroll
                for (int uu = 0; uu < ATT_UNROLL; uu++) {
                    kc[uu] = kraw[uu];
                    vc[uu] = vraw[uu];
                    okc[uu] = ok[uu];
                }
            } else {
                unpack8(qraw, qf);
#pragma unroll
                for (int i = 0; i < VEC; i++) qf[i] *= qscale;
            }
            if (base + step < end) {
#pragma unroll
                for (int uu = 0; uu < ATT_UNROLL; uu++) {
                    const int j = base + step + g + uu * GROUPS;
                    const bool in = j < end;
                    const int b = in ? (j >> page_shift) : 0;
                    const int page = b < max_blocks ? (cached ? table[b] : __ldg(table + b)) : -1;
                    const bool page_ok = page >= 0 && page < num_pages;
                    if (in && !page_ok && op.status && sub == 0) atomicOr(op.status, ST_ATT_PAGE);
                    ok[uu] = in && page_ok;
                    const size_t off = (size_t)(page_ok ? page : 0) * page_stride + head_off + (size_t)(j & page_mask) * D;
                    kraw[uu] = __ldcg(reinterpret_cast<const uint4*>(kbase + off));
                    vraw[uu] = __ldcg(reinterpret_cast<const uint4*>(vbase + off));
                }
            }
            if (!work) {
                if (u == (int)blockIdx.x) mark(sh, 0);
                continue;
            }
#pragma unroll
            for (int uu = 0; uu < ATT_UNROLL; uu++) {
                float sc = 0.0f;
                float kf[VEC];
                unpack8(kc[uu], kf);
#pragma unroll
                for (int i = 0; i < VEC; i++) sc = fmaf(qf[i], kf[i], sc);
                for (int w = LPK >> 1; w > 0; w >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, w);
                if (okc[uu]) {
                    if (sc > m) {          // rare after the first keys
                        const float corr = exp2f(m - sc);
                        l *= corr;
#pragma unroll
                        for (int i = 0; i < VEC; i++) o[i] *= corr;
                        m = sc;
                    }
                    const float pr = exp2f(sc - m);
                    l += pr;
                    float vf[VEC];
                    unpack8(vc[uu], vf);
#pragma unroll
                    for (int i = 0; i < VEC; i++) o[i] = fmaf(pr, vf[i], o[i]);
                }
            }
        }
        if (sub == 0) {
            sm_m[group] = m;
            sm_l[group] = l;
        }
#pragma unroll
        for (int i = 0; i < VEC; i++) sm_o[group * D + sub * VEC + i] = o[i];
        compute_sync();

        // merge the groups, fixed order: each group's weight once, then one thread per output dimension
        if (threadIdx.x < GROUPS) {
            float Mx = -INFINITY;
            for (int i = 0; i < GROUPS; i++) Mx = fmaxf(Mx, sm_m[i]);
            sm_w[threadIdx.x] = Mx > -INFINITY ? exp2f(sm_m[threadIdx.x] - Mx) : 0.0f;
            if (threadIdx.x == 0) sm_w[GROUPS] = Mx;
        }
        compute_sync();
        for (int d = threadIdx.x; d < D; d += CTHREADS) {
            const float Mx = sm_w[GROUPS];
            float L = 0.0f, O = 0.0f;
#pragma unroll 4
            for (int i = 0; i < GROUPS; i++) {
                const float w = sm_w[i];
                L = fmaf(sm_l[i], w, L);
                O = fmaf(sm_o[i * D + d], w, O);
            }
            if (splits == 1) {
                out[(size_t)t * op.ldc + h * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
            } else {
                const size_t slot = (size_t)pair * splits + split;
                partial_o[slot * D + d] = O;
                if (d == 0) {
                    partial_ml[slot * 2] = Mx;
                    partial_ml[slot * 2 + 1] = L;
                }
                __threadfence();
            }
        }
        if (splits > 1) {
            // The block that finds the other splits of this (token, head) already counted merges
            // them (fixed order: split 0, 1, ...) and leaves the counter at zero for the next use.
            compute_sync();
            if (threadIdx.x == 0) sh.flag = atomicAdd(op.counters + pair, 1) == splits - 1;
            compute_sync();
            if (sh.flag) {
                __threadfence();
                const size_t base = (size_t)pair * splits;
                float Mx = -INFINITY;
                for (int i = 0; i < splits; i++) Mx = fmaxf(Mx, __ldcg(partial_ml + (base + i) * 2));
                for (int d = threadIdx.x; d < D; d += CTHREADS) {
                    float L = 0.0f, O = 0.0f;
                    if (Mx > -INFINITY) {
                        for (int i = 0; i < splits; i++) {
                            const float w = exp2f(__ldcg(partial_ml + (base + i) * 2) - Mx);
                            L = fmaf(__ldcg(partial_ml + (base + i) * 2 + 1), w, L);
                            O = fmaf(__ldcg(partial_o + (base + i) * D + d), w, O);
                        }
                    }
                    out[(size_t)t * op.ldc + h * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
                }
                if (threadIdx.x == 0) op.counters[pair] = 0;
            }
        }
        compute_sync();      // the scratch and the flag are reused by the next unit
    }
}

__device__ __forceinline__ void load_record(Op* dst, const Op* src) {
    static_assert(sizeof(Op) % 4 == 0, "Op is copied in words");
    for (int wd = threadIdx.x; wd < (int)(sizeof(Op) / 4); wd += CTHREADS)
        reinterpret_cast<uint32_t*>(dst)[wd] = __ldg(reinterpret_cast<const uint32_t*>(src) + wd);
}

__global__ void __launch_bounds__(THREADS, 1)
decode_program_kernel(const Op* __restrict__ ops, int n_ops, Sync* sync, int* status,
                      unsigned long long* __restrict__ timeline, const StepArrays sa) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ Shared sh;
    uint8_t* a_region = smem;
    uint8_t* w_ring = smem + A_BYTES;
    int* tables = reinterpret_cast<int*>(smem + A_BYTES + NSTAGE * STAGE_BYTES);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sh.full_bar[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&sh.empty_bar[i])), "r"(CWARPS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        sh.abort = 0;
        sh.flag = 0;
        sh.stop = 0;
        sh.mark = nullptr;
        int off = 0;
        for (int i = 0; i < MAX_TABLES; i++) {
            sh.table_off[i] = off;
            if (i < sa.n_tables) off += sa.n_seqs * sa.max_blocks[i];
        }
    }
    __syncthreads();
    if (threadIdx.x >= CTHREADS) {
        run_producer(ops, n_ops, w_ring, sh, sync, status);
        return;
    }

    // the step's index arrays and the first record
    if (threadIdx.x < sa.n_tokens) {
        sh.pos[threadIdx.x] = __ldg(sa.positions + threadIdx.x);
        sh.seq[threadIdx.x] = __ldg(sa.token_seq + threadIdx.x);
    }
    for (int i = 0; i < sa.n_tables; i++) {
        const int n = sa.n_seqs * sa.max_blocks[i];
        for (int e = threadIdx.x; e < n; e += CTHREADS) tables[sh.table_off[i] + e] = __ldg(sa.tables[i] + e);
    }
    load_record(&sh.op[0], ops);
    const unsigned long long base = ld_acquire(&sync->base);
    uint32_t wcount = 0;
    // timeline (optional, 3 * n_ops + 1 entries): the nanosecond clock as block 0 starts; then per
    // operation two marks inside it (see mark()) and the time it leaves the barrier after it
    const bool timed = timeline != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    if (timed) timeline[0] = now_ns();
    compute_sync();

    for (int i = 0; i < n_ops; i++) {
        const Op& op = sh.op[i & 1];
        // the next record travels while this operation runs (its slot was last read two operations
        // ago, with a grid barrier since)
        if (i + 1 < n_ops) load_record(&sh.op[(i + 1) & 1], ops + i + 1);
        if (timed) {
            sh.mark = timeline + 1 + 3 * i;
            sh.mark[0] = sh.mark[1] = 0;
        }
        switch (op.kind) {
            case OP_EMBED: run_embed(op); break;
            case OP_NORM: run_norm(op); break;
            case OP_GEMM: run_gemm(op, wcount, a_region, w_ring, tables, sh, sync); break;
            case OP_ATTN: run_attn(op, a_region, tables, sh); break;
            default: break;
        }
        mark(sh, 1);
        if (i + 1 < n_ops) {
            if (!grid_barrier(sync, base + (unsigned long long)(i + 1) * gridDim.x, sh, status)) return;
        }
        if (timed) timeline[3 + 3 * i] = now_ns();
    }
    // Every block has read `base` before it arrived at the first barrier, and block 0 is past
    // the last one: the counter stands at its final value, which the next launch starts from.
    if (blockIdx.x == 0 && threadIdx.x == 0 && n_ops > 1)
        sync->base = base + (unsigned long long)(n_ops - 1) * gridDim.x;
}

}  // namespace

// Sizes the program interpreter takes, for the host's checks.
SANDY_API int sandy_decode_program_limits(int* max_rows, int* a_bytes, int* op_bytes, int* sync_bytes, int* row_pad,
                                          int* max_norm_width, int* table_ints, int* max_tables, int* arrays_bytes) {
    *max_rows = MAX_ROWS;
    *max_norm_width = MAX_NORM_WIDTH;
    *a_bytes = A_BYTES;
    *op_bytes = (int)sizeof(Op);
    *sync_bytes = (int)sizeof(Sync);
    *row_pad = XPAD;
    *table_ints = TABLE_INTS;
    *max_tables = MAX_TABLES;
    *arrays_bytes = (int)sizeof(StepArrays);
    return SANDY_OK;
}

// How many blocks a launch uses on the current device (one per SM).
SANDY_API int sandy_decode_program_grid(int* grid) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    *grid = sms;
    return SANDY_OK;
}

// ops: device array of n_ops records; sync: device Sync, zeroed once by the caller and then left
// to the kernel (zero it again after a launch that reported ST_WAIT).  arrays: host pointer to a
// StepArrays (copied into the launch).  timeline: null, or 3 * n_ops + 1 64-bit slots that receive
// block 0's nanosecond clock: [0] at the start, then per operation two marks inside it and the
// time after its barrier.  The launch is cooperative: all blocks are resident together or the
// launch fails.
SANDY_API int sandy_decode_program_run(const void* ops, int n_ops, void* sync, int* status, void* timeline,
                                       const void* arrays, cudaStream_t stream) {
    if (n_ops == 0) return SANDY_OK;
    if (!ops || !sync || !arrays) return SANDY_ERR_ARGUMENT;
    const StepArrays sa = *reinterpret_cast<const StepArrays*>(arrays);
    if (sa.n_tokens < 0 || sa.n_tokens > MAX_ROWS || sa.n_tables < 0 || sa.n_tables > MAX_TABLES) return SANDY_ERR_ARGUMENT;
    long long ints = 0;
    for (int i = 0; i < sa.n_tables; i++) ints += (long long)sa.n_seqs * sa.max_blocks[i];
    if (ints > TABLE_INTS) return SANDY_ERR_UNSUPPORTED;
    static int grid = 0;
    if (grid == 0) {
        int g = 0;
        const int rc = sandy_decode_program_grid(&g);
        if (rc != SANDY_OK) return rc;
        cudaError_t e = cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel, THREADS, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return SANDY_ERR_UNSUPPORTED;
        grid = g;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_program_kernel, (const Op*)ops, n_ops, (Sync*)sync, status,
                                             (unsigned long long*)timeline, sa);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
