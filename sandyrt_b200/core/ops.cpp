#include "ops.h"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <tuple>

#include "kernels.h"

namespace sandy {
namespace ops {

namespace {

int code_of(DType d) {
    if (d == DType::F32) return 0;
    if (d == DType::BF16) return 1;
    throw UnsupportedShape("kernels take float32 or bfloat16 tensors");
}

void check(int code, const std::string& what) {
    g_launches++;
    if (code == 0) return;
    if (code == -1) throw UnsupportedShape(what + ": sizes or dtypes not supported by this kernel");
    if (code == -2) throw KernelError(what + ": bad argument (null pointer or impossible size)");
    throw KernelError(what + ": CUDA error " + std::to_string(code) + " (" + cudaGetErrorString((cudaError_t)code) + ")");
}

bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) return false;
    return st != cudaStreamCaptureStatusNone;
}

int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : fallback;
}

// ---- per-class timing ---------------------------------------------------------------------------
struct OpRecord {
    const char* op_class;
    cudaEvent_t e0, e1;
    double bytes, flops;
};
bool g_profile = false;
std::vector<OpRecord> g_records;

class OpTimer {
public:
    OpTimer(const Launch& l, const char* op_class, double bytes, double flops) : stream_(l.stream) {
        if (!g_profile || capturing(l.stream)) return;
        rec_.op_class = op_class;
        rec_.bytes = bytes;
        rec_.flops = flops;
        if (cudaEventCreate(&rec_.e0) != cudaSuccess || cudaEventCreate(&rec_.e1) != cudaSuccess) return;
        cudaEventRecord(rec_.e0, stream_);
        on_ = true;
    }
    ~OpTimer() {
        if (!on_) return;
        cudaEventRecord(rec_.e1, stream_);
        g_records.push_back(rec_);
    }
private:
    cudaStream_t stream_;
    OpRecord rec_{};
    bool on_ = false;
};

// ---- leaving launches out -------------------------------------------------------------------------
// What a kernel costs inside a step -- where its set-up runs under the tail of the kernel before and the
// next one's under its own -- is not what it takes when timed alone.  For that figure a step is timed with
// a family of launches left out (its results are then garbage; only the time is read) and the difference
// to the whole step taken: families "layernorm", "attention", "kv_append", and "product" or
// "product <N>x<K>" for the products of one shape.  Set through the control plane (leave_out); graphs
// recorded before a change still hold the launches, so a fresh engine is made for every setting.
std::vector<std::string> g_left_out;

bool left_out(const char* family, int64_t N = 0, int64_t K = 0) {
    if (g_left_out.empty()) return false;
    const std::string f = family;
    const std::string shaped = N ? f + " " + std::to_string(N) + "x" + std::to_string(K) : f;
    for (const std::string& x : g_left_out)
        if (x == f || x == shaped) return true;
    return false;
}

double tensor_bytes(const Tensor* t) { return t ? (double)t->numel() * (double)t->elem_size() : 0.0; }

std::string dims(const Tensor& t) { return "[" + std::to_string(t.rows) + ", " + std::to_string(t.cols) + "]"; }

}  // namespace

Act act_from_name(const std::string& name) {
    if (name.empty() || name == "none") return Act::None;
    if (name == "gelu_new" || name == "gelu_tanh") return Act::GeluNew;
    if (name == "gelu" || name == "gelu_erf") return Act::Gelu;
    throw ValueError("unknown activation '" + name + "'");
}

const char* kernel_status_text() {
    return "bits 0-2 a barrier wait ran out in the tensor-core product, bit 3 a key/value write and bit 4 a key read had "
           "no page behind it, bits 5-6 a wait ran out in the bulk decode attention, bit 8 in the tcgen05 prefill attention";
}

void profile_enable(bool on) { g_profile = on; }

void leave_out(const std::vector<std::string>& families) { g_left_out = families; }

std::vector<ProfileRow> profile_report() {
    std::map<std::string, ProfileRow> by_class;
    for (OpRecord& r : g_records) {
        float ms = 0;
        if (cudaEventSynchronize(r.e1) == cudaSuccess) cudaEventElapsedTime(&ms, r.e0, r.e1);
        ProfileRow& row = by_class[r.op_class];
        row.op_class = r.op_class;
        row.calls++;
        row.us += 1e3 * ms;
        row.bytes += r.bytes;
        row.flops += r.flops;
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    g_records.clear();
    std::vector<ProfileRow> out;
    for (auto& kv : by_class) out.push_back(kv.second);
    return out;
}

int sm_count() {
    static int n = 0;
    if (n == 0) n = SANDY_KERNEL(embed, sandy_device_sm_count)();
    return n;
}

void spin(cudaStream_t stream, long long nanoseconds) {
    static auto fn = SANDY_KERNEL(embed, sandy_spin);
    const int code = fn(nanoseconds, stream);
    if (code) throw KernelError("spin: CUDA error " + std::to_string(code));
}

void embed_positions(const Launch& l, const int* ids, const int* positions, const Tensor& wte, const Tensor* wpe, Tensor& out,
                     int n_tokens) {
    if (wpe && (wpe->dtype != wte.dtype || wpe->cols != out.cols))
        throw KernelError("position table must match the token table in dtype and width");
    if (wte.cols != out.cols || !wte.contiguous() || !out.contiguous() || out.rows < n_tokens)
        throw KernelError("embed_positions: tables and output must be contiguous and of one width");
    static auto fn = SANDY_KERNEL(embed, sandy_embed_pos);
    OpTimer timer(l, "embedding", (double)n_tokens * out.cols * ((wpe ? 2.0 : 1.0) * wte.elem_size() + out.elem_size()), 0);
    check(fn(ids, positions, wte.data, wpe ? wpe->data : nullptr, out.data, n_tokens, (int)out.cols, (int)wte.rows,
             wpe ? (int)wpe->rows : 0, code_of(wte.dtype), code_of(out.dtype), l.status, l.stream),
          "embed_positions");
}

void layernorm(const Launch& l, const Tensor& x, const Tensor& gamma, const Tensor* beta, float eps, Tensor& out,
               const int* rows, int n_rows) {
    const int64_t width = x.cols;
    if (!rows && x.rows < n_rows) throw KernelError("layernorm: x and out disagree");
    if (!x.contiguous() || !out.contiguous() || out.cols != width || gamma.numel() != width || out.rows < n_rows)
        throw KernelError("layernorm: contiguous [rows, width] tensors expected");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(norm, sandy_layernorm);
    OpTimer timer(l, "layernorm", (double)n_rows * width * (x.elem_size() + out.elem_size()), 0);
    check(fn(x.data, gamma.data, beta ? beta->data : nullptr, out.data, rows, n_rows, (int)width, eps, code_of(x.dtype),
             code_of(gamma.dtype), code_of(out.dtype), l.stream),
          "layernorm(width=" + std::to_string(width) + ")");
}

void gemm_simt(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, bool w_out_in, Act act,
               const Tensor* residual) {
    const int64_t M = a.rows, K = a.cols, N = out.cols;
    const int64_t wk = w_out_in ? w.cols : w.rows, wn = w_out_in ? w.rows : w.cols;
    if (wk != K || wn != N || out.rows != M)
        throw KernelError("gemm: shapes disagree: a " + dims(a) + ", w " + dims(w) + (w_out_in ? " (out_in)" : " (in_out)") +
                          ", out " + dims(out));
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm: residual must be float32 [M, N]");
    if (bias && (bias->dtype != w.dtype || bias->numel() != N)) throw KernelError("gemm: bias must have the weight's dtype and N elements");
    static auto fn = SANDY_KERNEL(gemm_simt, sandy_gemm_simt);
    OpTimer timer(l, "product, FFMA (float32)", tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual),
                  2.0 * M * N * K);
    check(fn(a.data, w.data, bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M,
             (int)N, (int)K, (int)a.ld, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, w_out_in ? 1 : 0, (int)act,
             code_of(a.dtype), code_of(w.dtype), code_of(out.dtype), l.stream),
          "gemm_simt(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
}

bool tensor_core_gemm_supported(int64_t K, int64_t N) {
    (void)N;
    return K % 8 == 0 && K >= 8;       // operand rows must start on 16-byte boundaries for TMA
}

// ---- the tcgen05 product and its variants -----------------------------------------------------------
// Which of the tcgen05 variants (three tile widths, one tile per CTA or persistent; two CTAs on a
// 256-row tile, two widths) is fastest depends on how the tiles of a product fall on the SMs, and a
// model of it was off by 20 % on half the shapes tried.  So the first product of a shape (rows in
// steps of 128) with at least 256 rows times each variant on a scratch output and remembers the
// winner.  All variants add the k-steps of an output element in the same order, so the choice never
// changes a result.  Not done while a CUDA graph is being captured (the kernel's own default stands
// then).  Tile codes: n < 0 one tile of 128 x |n| per CTA, n > 0 the persistent kernel with tiles of
// 128 x n, kPairTile + n two CTAs on a 256 x n tile.
constexpr int kPairTile = 2000;
constexpr int kGemmTuneMinRows = 256;
constexpr int kTuneLaunches = 8;
const int kGemmVariants[] = {-64, -128, -256, 64, 128, 256, kPairTile + 128, kPairTile + 256};

namespace {
using TileKey = std::tuple<int64_t, int64_t, int64_t, int, bool, int>;
std::map<TileKey, int> g_tiles;
std::map<std::pair<int64_t, int64_t>, int> g_forced_tiles;      // (N, K) -> variant, for comparisons (force_tile)

struct TcArgs {
    const Tensor* a; const Tensor* w; const Tensor* bias; Act act; int64_t M, N, K;
};

void launch_tc(const Launch& l, const TcArgs& g, int tile, Tensor& dst, const Tensor* res, const KVTarget* kv) {
    static auto fn1 = SANDY_KERNEL(gemm_tc, sandy_gemm_tc);
    auto fn = fn1;
    if (tile >= kPairTile) {
        static auto fn2 = SANDY_KERNEL(gemm_tc2, sandy_gemm_tc2);
        fn = fn2;
        tile -= kPairTile;
    }
    const KVView* c = kv ? &kv->cache : nullptr;
    check(fn(g.a->data, g.w->data, g.bias ? g.bias->data : nullptr, res ? (const float*)res->data : nullptr, dst.data, (int)g.M,
             (int)g.N, (int)g.K, (int)g.a->ld, (int)g.w->ld, res ? (int)res->ld : 0, (int)dst.ld, (int)g.act, code_of(dst.dtype),
             tile, c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr,
             kv ? kv->max_blocks : 0, kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0,
             kv ? kv->kv_cols : 0, c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_tc(M=" + std::to_string(g.M) + ",N=" + std::to_string(g.N) + ",K=" + std::to_string(g.K) +
              ",tile=" + std::to_string(tile) + ")");
}
}  // namespace

void gemm_tc(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
             const Tensor* residual, int tile_n, KVTarget* kv) {
    const int64_t M = a.rows, K = a.cols, N = w.rows;
    if (a.dtype != DType::BF16 || w.dtype != DType::BF16) throw UnsupportedShape("gemm_tc takes bfloat16 operands");
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_tc: shapes disagree: a " + dims(a) + ", w " + dims(w) + ", out " + dims(out));
    if (K % 8 || a.ld % 8 || w.ld % 8 || ((uintptr_t)a.data & 15) || ((uintptr_t)w.data & 15))
        throw UnsupportedShape("gemm_tc: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_tc: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_tc: bias must be bfloat16 [N]");
    if (kv) {
        const KVView& c = kv->cache;
        if (c.dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c.n_kv_heads * c.head_dim ||
            kv->q_cols + 2 * kv->kv_cols != N)
            throw KernelError("gemm_tc: the key/value target does not match the product");
    }
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    OpTimer timer(l, kv ? "product, tcgen05 (+ cache write)" : "product, tcgen05",
                  tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual), 2.0 * M * N * K);
    const TcArgs g{&a, &w, bias, act, M, N, K};
    const TileKey key{(M + 127) / 128, N, K, (int)act, residual != nullptr, (int)out.dtype};
    if (tile_n == 0 && !g_forced_tiles.empty() && M >= kGemmTuneMinRows) {
        auto forced = g_forced_tiles.find({N, K});
        if (forced != g_forced_tiles.end()) tile_n = forced->second;
    }
    if (tile_n == 0) {
        auto hit = g_tiles.find(key);
        if (hit != g_tiles.end()) tile_n = hit->second;
        else if (M >= kGemmTuneMinRows && !capturing(l.stream)) {
            // timed without the cache write: the scratch runs must not touch pages.  A product that adds
            // into its own output (x += ...) is timed adding into the scratch, the way it will run.
            DeviceBuffer scratch((size_t)M * (size_t)N * out.elem_size());
            cuda_check(cudaMemsetAsync(scratch.get(), 0, (size_t)M * (size_t)N * out.elem_size(), l.stream), "clearing the tuner's scratch");
            Tensor dst = out;
            dst.data = scratch.get();
            dst.ld = N;
            const bool in_place = residual && residual->data == out.data;
            const Tensor* tune_res = in_place ? &dst : residual;
            cudaEvent_t e0, e1;
            cuda_check(cudaEventCreate(&e0), "creating an event");
            cuda_check(cudaEventCreate(&e1), "creating an event");
            float best_ms = 1e30f;
            int best = 0;
            static const bool tune_log = std::getenv("SANDYRT_TUNE_LOG") != nullptr;      // what the tuner saw, on stderr
            for (int tile : kGemmVariants) {
                launch_tc(l, g, tile, dst, tune_res, nullptr);
                // A launch costs the host about as long as one of these kernels takes the GPU, so timed
                // naively the host's pace is what is measured; here the GPU is kept busy with a spin kernel
                // while the launches queue up behind it.
                spin(l.stream, 300000);
                cudaEventRecord(e0, l.stream);
                for (int i = 0; i < kTuneLaunches; i++) launch_tc(l, g, tile, dst, tune_res, nullptr);
                cudaEventRecord(e1, l.stream);
                cuda_check(cudaEventSynchronize(e1), "timing a product");
                float ms = 0;
                cudaEventElapsedTime(&ms, e0, e1);
                if (ms < best_ms) { best_ms = ms; best = tile; }
                if (tune_log) fprintf(stderr, "[sandyrt_b200] product %lld x %lld x %lld, tile %d: %.2f us\n", (long long)M, (long long)N, (long long)K, tile, ms * 1e3f / kTuneLaunches);
            }
            if (tune_log) fprintf(stderr, "[sandyrt_b200] product %lld x %lld x %lld: tile %d\n", (long long)M, (long long)N, (long long)K, best);
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            g_tiles[key] = best;
            tile_n = best;
        }
    }
    launch_tc(l, g, tile_n, out, residual, kv);
    if (kv) kv->written = true;
}

// The variant that products of W [N, K] with at least 256 rows take from now on, whatever the tuner
// found (0: the tuner's choice again).  For comparing variants inside a whole step; steps already
// recorded as graphs keep what they were recorded with.
void force_tile(int64_t N, int64_t K, int tile) {
    if (tile == 0) g_forced_tiles.erase({N, K});
    else g_forced_tiles[{N, K}] = tile;
}

// ---- the weight-streaming product ---------------------------------------------------------------------
constexpr int kSkinnyNormMaxRows = 16;
constexpr int kSkinnyNormMaxK = 2048;
bool skinny_norm_fusable(const FusedNorm& n, int64_t K, DType out_dtype) {
    return n.gamma.dtype == DType::BF16 && out_dtype == DType::BF16 && n.x.dtype == DType::F32 &&
           n.x.rows <= kSkinnyNormMaxRows && K <= kSkinnyNormMaxK && n.x.ld % 4 == 0 && !((uintptr_t)n.x.data & 15) &&
           !((uintptr_t)n.gamma.data & 15) && (!n.beta || !((uintptr_t)n.beta->data & 15));
}

void gemm_skinny(const Launch& l, const Tensor* a, const FusedNorm* norm, const Tensor& w, const Tensor* bias, Tensor& out,
                 Act act, const Tensor* residual, KVTarget* kv) {
    const int64_t M = norm ? norm->x.rows : a->rows, K = norm ? norm->x.cols : a->cols, N = w.rows;
    if (norm && !skinny_norm_fusable(*norm, K, DType::BF16)) throw UnsupportedShape("gemm_skinny: this norm cannot be fused");
    if ((!norm && a->dtype != DType::BF16) || w.dtype != DType::BF16) throw UnsupportedShape("gemm_skinny takes bfloat16 operands");
    if (M > kSkinnyMaxRows) throw UnsupportedShape("gemm_skinny takes at most 64 rows, got " + std::to_string(M));
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_skinny: shapes disagree: a [" + std::to_string(M) + ", " + std::to_string(K) + "], w " + dims(w) +
                          ", out " + dims(out));
    if (K % 8 || w.ld % 8 || ((uintptr_t)w.data & 15) || (a && (a->ld % 8 || ((uintptr_t)a->data & 15))))
        throw UnsupportedShape("gemm_skinny: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_skinny: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_skinny: bias must be bfloat16 [N]");
    const KVView* c = kv ? &kv->cache : nullptr;
    if (kv && (c->dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c->n_kv_heads * c->head_dim ||
               kv->q_cols + 2 * kv->kv_cols != N))
        throw KernelError("gemm_skinny: the key/value target does not match the product");
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    static auto fn = SANDY_KERNEL(gemm_skinny, sandy_gemm_skinny);
    OpTimer timer(l, norm ? (kv ? "product, streaming (+ norm, cache write)" : "product, streaming (+ norm)") : "product, streaming",
                  (norm ? tensor_bytes(&norm->x) : tensor_bytes(a)) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual),
                  2.0 * M * N * K);
    check(fn(a ? a->data : nullptr, norm ? (const float*)norm->x.data : nullptr, norm ? (int)norm->x.ld : 0,
             norm ? norm->gamma.data : nullptr, (norm && norm->beta) ? norm->beta->data : nullptr, norm ? norm->eps : 0.0f, w.data,
             bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M, (int)N, (int)K,
             a ? (int)a->ld : 0, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, (int)act, code_of(out.dtype),
             c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr, kv ? kv->max_blocks : 0,
             kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0, kv ? kv->kv_cols : 0,
             c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_skinny(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
    if (kv) kv->written = true;
}

// ---- 17 to 64 rows on the tensor cores -----------------------------------------------------------------
// Which kernel a product of 17 to 64 rows gets.  Timed one kernel after itself the tcgen05 kernel with
// 64-wide tiles wins the up-projection (3072 x 768 at 64 rows: 6.8 us against 9.8 streaming) and split-K
// the down-projection (768 x 3072: 8.2 against 11.2) and the vocabulary (50257 x 768: 26 against 98).
// Inside a decode step of 64 requests, where a kernel's set-up and first loads run under the tail of the
// kernel before it if its blocks find room beside that kernel's, the streaming kernel with its small blocks
// beats the tiled one on the up-projection (step 0.723 ms against 0.756), split-K keeps its lead on the
// down-projection (0.756 against 0.820) and is level on the vocabulary.  So: split-K for a long K or very
// many columns, streaming otherwise.  The kernels add in different orders, so the choice is a fixed rule
// of the shape and never a timing: the same batch gives the same bfloat16 tokens in every process.
constexpr int kSmallMinRows = 17;
constexpr int kSplitKMinK = 2048;
constexpr int kSplitKMinCols = 16384;
// Below 17 rows the streaming kernel keeps the products up to K = 4,096 (8 rows, us alone, streaming / split-K:
// 768 x 3072 4.7 / 4.7 and a decode step 0.296 / 0.304 ms; 1024 x 4096 5.0 / 5.1; 1280 x 5120 8.1 / 6.2;
// 1600 x 6400 10.1 / 7.6).
constexpr int kSplitKMinKFewRows = 5120;
constexpr int kSplitKMinKManyRows = 1280;

SmallGemm small_gemm_kernel(int64_t M, int64_t N, int64_t K) {
    if (M < kSmallMinRows) return K >= kSplitKMinKFewRows ? SmallGemm::SplitK : SmallGemm::Skinny;
    if (K >= kSplitKMinK || N >= kSplitKMinCols) return SmallGemm::SplitK;
    // more than two row tiles of wide rows: the streaming kernel's blocks each fetch all rows (64 x 1,600: 205 KB)
    // (64 rows, us alone, streaming / split-K: 4800 x 1600 18.7 / 10.4, 1600 x 1600 10.0 / 7.7, 6400 x 1600 20.3 /
    // 14.5; at 32 rows level; at K = 1,024 the streaming kernel leads: 3072 x 1024 7.2 / 11.9)
    if (M > 32 && K >= kSplitKMinKManyRows) return SmallGemm::SplitK;
    return SmallGemm::Skinny;
}

void gemm_small(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
                const Tensor* residual, KVTarget* kv) {
    const int64_t M = a.rows, K = a.cols, N = w.rows;
    if (a.dtype != DType::BF16 || w.dtype != DType::BF16) throw UnsupportedShape("gemm_small takes bfloat16 operands");
    if (M > kSmallMaxRows) throw UnsupportedShape("gemm_small takes at most 256 rows, got " + std::to_string(M));
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_small: shapes disagree: a " + dims(a) + ", w " + dims(w) + ", out " + dims(out));
    if (K % 8 || w.ld % 8 || a.ld % 8 || ((uintptr_t)w.data & 15) || ((uintptr_t)a.data & 15))
        throw UnsupportedShape("gemm_small: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_small: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_small: bias must be bfloat16 [N]");
    const KVView* c = kv ? &kv->cache : nullptr;
    if (kv && (c->dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c->n_kv_heads * c->head_dim ||
               kv->q_cols + 2 * kv->kv_cols != N))
        throw KernelError("gemm_small: the key/value target does not match the product");
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    static auto fn = SANDY_KERNEL(gemm_small, sandy_gemm_small);
    OpTimer timer(l, kv ? "product, tcgen05 split-K (+ cache write)" : "product, tcgen05 split-K",
                  tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual), 2.0 * M * N * K);
    check(fn(a.data, w.data, bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M,
             (int)N, (int)K, (int)a.ld, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, (int)act, code_of(out.dtype),
             c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr, kv ? kv->max_blocks : 0,
             kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0, kv ? kv->kv_cols : 0,
             c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_small(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
    if (kv) kv->written = true;
}

// ---- the cache and attention ------------------------------------------------------------------------------
void kv_append(const Launch& l, const Tensor& k_src, const Tensor& v_src, const KVView& c, const int* block_table,
               int max_blocks, const int* token_seq, const int* positions) {
    if (k_src.rows != v_src.rows || k_src.cols != v_src.cols || k_src.cols != (int64_t)c.n_kv_heads * c.head_dim ||
        k_src.ld != v_src.ld || k_src.dtype != c.dtype || v_src.dtype != c.dtype)
        throw KernelError("kv_append: sources must be [T, Hkv*D] of the cache's dtype with one stride");
    if (left_out("kv_append")) return;
    static auto fn = SANDY_KERNEL(attention, sandy_kv_append);
    OpTimer timer(l, "key/value append", 2 * (tensor_bytes(&k_src) + tensor_bytes(&v_src)), 0);
    check(fn(k_src.data, v_src.data, (int)k_src.ld, c.k, c.v, c.page_stride, block_table, max_blocks, token_seq, positions,
             (int)k_src.rows, c.n_kv_heads, c.head_dim, c.page_size, c.num_pages, code_of(c.dtype), l.kernel_status, l.stream),
          "kv_append");
}

int decode_splits(int n_tokens, int n_heads, int max_kv, int sms) {
    static const int forced = env_int("SANDYRT_DECODE_SPLITS", 0);       // > 0: this many splits, for comparisons
    if (forced > 0) return forced;
    if (sms <= 0) sms = sm_count();
    // About four blocks an SM in all, to the nearest number of splits.  (Rounded up, as it was for the
    // register kernel, 12 / 16 / 24 requests of 12 heads got 5 / 4 / 3 splits; whole decode steps with the
    // mma.sync kernel, GPT-2 small, context ~400, ms by splits 1 / 2 / 3 / 4 / 5: 12 requests .340 / .334 /
    // .323 / .311 / .342; 16: .361 / .350 / .341 / .361 / .374; 24: .490 / .409 / .455 / .437 / .473; 32:
    // .509 / .494 / .484 / .512 / .508; 48: .627 / .626 / .664 / .685 / .731; 8: .330 / .323 / .310 / .303 / .306.)
    // Long ranges: a block that walks more than some 256 keys alone is the step's longest chain, so a pair is
    // cut further as long as no more than eight blocks an SM come of it (32 requests at context 965, ms by
    // splits 1 / 2 / 3 / 4: .741 / .655 / .596 / .633; GPT-2 medium, 32 requests of mixed lengths, tokens a
    // second with 1 / 2 / 3 splits: 17-19 k / 21-23 k / 21 k).
    const int pairs = std::max(1, n_tokens * n_heads);
    const int by_blocks = (4 * sms + pairs / 2) / pairs;
    const int by_length = std::min((max_kv + 255) / 256, (8 * sms) / pairs);
    const int want = std::max(by_blocks, by_length);
    const int cap = std::max(1, max_kv / 64);
    const int n = std::max(1, std::min({want, cap, 32}));
    // The splits of a pair are one thread-block cluster.  Clusters of 6 and 7 blocks pack badly into
    // the GPU's groups of SMs: a whole decode step of 8 x 12 pairs took 0.439 / 0.441 ms with them
    // against 0.376 ms with 5 (0.383 with 4, 0.420 with 8).
    return (n == 6 || n == 7) ? 5 : n;
}

namespace {
constexpr int kClusterMaxSplits = 8;
// From this many (token, head) pairs on, a decode step's attention streams pages through shared
// memory with bulk copies (attention_decode_bulk.cu) instead of through registers.  Measured on
// GPT-2 small's shape: 64 x 12 pairs of 384 keys, cache read from HBM, 18.8 against 45.5 us a layer;
// but a whole decode step of 8 x 12 pairs (its cache fits in L2) took 414 against 400 us and one of
// 1 x 12 pairs 356 against 333 us, the register kernel starting sooner.
constexpr int kBulkMinPairs = 256;

bool decode_head_dim(DType dt, int d) {
    if (d == 16 || d == 32 || d == 64 || d == 128) return true;
    return d == 256 && dt == DType::BF16;
}
}  // namespace

void attention(const Launch& l, const AttentionStep& s, const Tensor& q, const KVView& c, Tensor& out, int n_heads,
               float scale, int window, Workspace& ws) {
    (void)ws;
    const int d = c.head_dim, hkv = c.n_kv_heads;
    if (d % 16 != 0 || d > 256) throw UnsupportedShape("attention: head size " + std::to_string(d) + " must be a multiple of 16, at most 256");
    if (hkv <= 0 || n_heads % hkv != 0)
        throw UnsupportedShape("attention: " + std::to_string(n_heads) + " heads do not divide into " + std::to_string(hkv) + " key/value heads");
    if (q.cols != (int64_t)n_heads * d || out.rows != q.rows || out.cols != q.cols || q.dtype != c.dtype || out.dtype != q.dtype)
        throw KernelError("attention: q and out must be [T, H*D] of the cache's dtype");
    const int T = (int)q.rows;
    if (left_out("attention")) return;
    const double attn_bytes = 2.0 * s.kv_tokens * hkv * d * q.elem_size() + 2 * tensor_bytes(&q);
    const double attn_flops = 4.0 * s.pairs * n_heads * d;
    const std::string shape = "(H=" + std::to_string(n_heads) + ",Hkv=" + std::to_string(hkv) + ",D=" + std::to_string(d) + ")";
    if (s.max_q_len > 1 && q.dtype == DType::BF16 && d <= 128) {
        static const bool use_tc = env_int("SANDYRT_PREFILL_TC", 1) != 0;     // 0 keeps every head size on the mma.sync kernel
        if (use_tc && d == 64) {
            static auto fn = SANDY_KERNEL(attention_prefill_tc, sandy_prefill_attention_tc);
            OpTimer timer(l, "attention, prompt (tcgen05)", attn_bytes, attn_flops);
            const int code = fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.q_start, s.kv_before,
                                out.data, (int)out.ld, s.n_seqs, s.max_q_len, n_heads, hkv, d, c.page_size, scale, window,
                                c.num_pages, l.kernel_status, l.stream);
            if (code != -1) { check(code, "prefill_attention_tc" + shape); return; }
        }
        static auto fn = SANDY_KERNEL(attention_prefill, sandy_prefill_attention);
        OpTimer timer(l, "attention, prompt (mma.sync)", attn_bytes, attn_flops);
        check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.q_start, s.kv_before, out.data,
                 (int)out.ld, s.n_seqs, s.max_q_len, n_heads, hkv, d, c.page_size, scale, window, c.num_pages, l.kernel_status,
                 l.stream),
              "prefill_attention" + shape);
        return;
    }
    if (s.max_q_len == 1 && decode_head_dim(q.dtype, d)) {
        const int max_kv = s.max_blocks * c.page_size;
        const int splits = std::min(decode_splits(T, n_heads, max_kv), kClusterMaxSplits);
        const size_t stage = 2 * (size_t)c.page_size * (size_t)d * q.elem_size();
        const bool fits = stage * 4 <= 160 * 1024;           // the ring holds at least four stages
        static const int bulk_mode = env_int("SANDYRT_DECODE_BULK", -1);      // 0 / 1 force one kernel, for comparisons
        const bool bulk = fits && (bulk_mode < 0 ? T * n_heads >= kBulkMinPairs : bulk_mode == 1);
        // bfloat16 heads of 64: the products on mma.sync (attention_decode_mma.cu).  Timed alone on caches from
        // HBM, 12 heads, 400 keys (us; register / bulk / mma.sync kernel): 1 token 4.5 / 5.2 / 3.4; 8 tokens 6.0 /
        // 7.5 / 5.1; 24 tokens 15.9 / 17.4 / 11.7; 48 tokens 25.9 / 23.2 / 16.0; 64 tokens 45 / 17.5 / 19.9; and
        // 8 tokens of 1,000 keys 12.9 / 12.5 / 7.8.  So it takes every launch but those with so many pairs that
        // a pair is one block (one split), where the bulk kernel's deeper ring of pages keeps its small lead.
        static const int mma_mode = env_int("SANDYRT_DECODE_MMA", 1);          // 0 keeps the two kernels below, for comparisons
        if (mma_mode != 0 && q.dtype == DType::BF16 && d == 64 && !(bulk && splits == 1)) {
            static auto max_keys_fn = SANDY_KERNEL(attention_decode_mma, sandy_decode_attention_mma_max_keys);
            if (max_kv <= max_keys_fn(splits, c.page_size)) {
                static auto fn = SANDY_KERNEL(attention_decode_mma, sandy_decode_attention_mma);
                OpTimer timer(l, "attention, decode (mma.sync)", attn_bytes, attn_flops);
                check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                         (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, max_kv, l.kernel_status,
                         l.stream),
                      "decode_attention_mma" + shape);
                return;
            }
        }
        if (bulk) {
            static auto fn = SANDY_KERNEL(attention_decode_bulk, sandy_decode_attention_bulk);
            OpTimer timer(l, "attention, decode (bulk copies)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, code_of(q.dtype),
                     l.kernel_status, l.stream),
                  "decode_attention_bulk" + shape);
        } else if (splits > 1) {
            static auto fn = SANDY_KERNEL(attention_decode, sandy_decode_attention_cluster);
            OpTimer timer(l, "attention, decode (cluster)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, code_of(q.dtype),
                     l.kernel_status, l.stream),
                  "decode_attention_cluster" + shape);
        } else {
            static auto fn = SANDY_KERNEL(attention_decode, sandy_decode_attention);
            OpTimer timer(l, "attention, decode (one block)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, nullptr, T, n_heads, hkv, d, c.page_size, scale, window, 1, c.num_pages, code_of(q.dtype),
                     l.kernel_status, l.stream),
                  "decode_attention" + shape);
        }
        return;
    }
    static auto fn = SANDY_KERNEL(attention, sandy_paged_attention);
    OpTimer timer(l, "attention, general", attn_bytes, attn_flops);
    check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
             (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, c.num_pages, code_of(q.dtype), l.kernel_status, l.stream),
          "paged_attention" + shape);
}

void sample(const Launch& l, const Tensor& logits, int* out_tokens, const float* temperature, const int* top_k,
            const float* top_p, const float* uniform, const SampleFeedback* fb) {
    if (logits.dtype != DType::F32) throw KernelError("sample: logits must be float32");
    if (temperature && !uniform) throw KernelError("sample: temperature sampling needs a uniform number per row");
    static auto fn = SANDY_KERNEL(sampling, sandy_sample);
    OpTimer timer(l, "sampling", tensor_bytes(&logits), 0);
    check(fn((const float*)logits.data, (int)logits.ld, (int)logits.rows, (int)logits.cols, temperature, top_k, top_p, uniform,
             out_tokens, l.status, fb ? fb->token_ids : nullptr, fb ? fb->logit_rows : nullptr, fb ? fb->positions : nullptr,
             fb ? fb->burst_tokens : nullptr, fb ? fb->row_step : nullptr, l.stream),
          "sample");
}

}  // namespace ops
}  // namespace sandy
