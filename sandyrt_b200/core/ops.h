// The kernels as the host side calls them: argument checks, the choice among kernels that serve
// the same operation, then one launch.
//
// Every function works on device views, launches on the given stream (so a launch can be captured
// in a CUDA graph) and returns nothing; outputs are written into tensors the caller passes.  Sizes
// a kernel does not take are refused with UnsupportedShape before anything runs.  There is no other
// implementation behind these functions: if a kernel library cannot be loaded, the call throws.
#pragma once

#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "cache.h"
#include "device.h"

namespace sandy {
namespace ops {

enum class Act : int { None = 0, GeluNew = 1, Gelu = 2 };
Act act_from_name(const std::string& name);          // "gelu_new" / "gelu_tanh" / "gelu" / "gelu_erf" / "none"

// Where the launches of one step go and where kernels report trouble.
struct Launch {
    cudaStream_t stream = nullptr;
    int* status = nullptr;             // device int: bit 0 bad token id or NaN logits, bit 1 bad position
    int* kernel_status = nullptr;      // device int: expired waits, pages that do not exist (see kernel_status_text)
};
const char* kernel_status_text();

// Device time per kernel class, behind a switch (the reference times every op the same way through
// EngineRunOptions::profileKernel, src/engine/Engine.h:56-60, src/engine/Engine.cpp:887-921).  While
// it is on, every launch outside a graph capture gets a pair of CUDA events; `profile_report` waits
// for them and returns per class the launches, microseconds, bytes that had to move and operations.
struct ProfileRow {
    std::string op_class;
    long long calls = 0;
    double us = 0, bytes = 0, flops = 0;
};
void profile_enable(bool on);
// Families of launches that are skipped from now on ("layernorm", "attention", "kv_append", "product",
// "product <N>x<K>"): for timing what a family costs inside a step; results are garbage meanwhile.
void leave_out(const std::vector<std::string>& families);
void force_tile(int64_t N, int64_t K, int tile);      // tcgen05 variant for products of W [N, K]; 0: the tuner's
std::vector<ProfileRow> profile_report();              // also clears what was gathered

int sm_count();                                        // streaming multiprocessors of the current device
void spin(cudaStream_t stream, long long nanoseconds); // keeps the stream busy (timing loops queue launches behind it)

void embed_positions(const Launch& l, const int* ids, const int* positions, const Tensor& wte, const Tensor* wpe,
                     Tensor& out, int n_tokens);
void layernorm(const Launch& l, const Tensor& x, const Tensor& gamma, const Tensor* beta, float eps, Tensor& out,
               const int* rows, int n_rows);

// Where the key/value columns of a fused q/k/v product belong: the layer's cache view and the
// step's index arrays.  `written` is set by the product if its kernel did the write.
struct KVTarget {
    KVView cache;
    const int* block_table = nullptr;
    int max_blocks = 0;
    const int* token_seq = nullptr;
    const int* positions = nullptr;
    int q_cols = 0, kv_cols = 0;
    bool written = false;
};

// A LayerNorm that the product's kernel runs itself on the float32 rows `x` (decode steps).
struct FusedNorm {
    Tensor x;
    Tensor gamma;
    const Tensor* beta = nullptr;
    float eps = 0.0f;
};

// out = act(a @ W + bias) + residual.  W is [K, N], or [N, K] with w_out_in.
void gemm_simt(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, bool w_out_in, Act act,
               const Tensor* residual);
// tcgen05 tensor cores: a bfloat16 [M, K], w bfloat16 [N, K].  tile_n 0 lets the tuner (256 rows and more) or the
// kernel choose; see GEMM_VARIANTS in ops.cpp for the codes.
bool tensor_core_gemm_supported(int64_t K, int64_t N);
void gemm_tc(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
             const Tensor* residual, int tile_n = 0, KVTarget* kv = nullptr);
// Weight streaming for up to 64 rows (a decode step); optional LayerNorm prologue and key/value write.
bool skinny_norm_fusable(const FusedNorm& n, int64_t K, DType out_dtype);
// Up to how many rows running the norm inside the product pays.  Every block of the product norms all
// rows itself, so that traffic grows with rows x blocks, while the norm as a launch of its own costs a
// fixed 1.5 us or so behind programmatic dependent launch.  Whole decode steps of GPT-2 small (ms, norm
// inside / norm apart): 1 request .244 / .250, 2: .255 / .262, 4: .267 / .270, 6: .290 / .285, 7: .297 /
// .288, 8: .303 / .294, 12: .381 / .341, 16: .409 / .361.
constexpr int kSkinnyNormPaysRows = 4;
// ... and up to which K: the blocks' norms also grow with the row's width.  One request, ms a decode step, norm
// inside / apart: GPT-2 small (K 768) .244 / .250, medium (1,024) .572 / .573, xl (1,600) 3.45 / 2.80.
constexpr int kSkinnyNormPaysK = 1024;
void gemm_skinny(const Launch& l, const Tensor* a, const FusedNorm* norm, const Tensor& w, const Tensor* bias, Tensor& out,
                 Act act, const Tensor* residual, KVTarget* kv = nullptr);
constexpr int kSkinnyMaxRows = 64;
// tcgen05 with the weight as the wide operand and K split over a cluster, for 17 to 64 rows (gemm_small.cu).
// small_gemm_kernel: which kernel a bfloat16 product of 17 to 64 rows gets, from its shape alone.
// The split-K kernel also takes 65 to 256 rows (a short prompt step, or a portion of one): products with a
// long K and few row tiles, which the tile kernels run on a handful of CTAs (128 x 768 x 3072: six CTAs of 48
// k-steps each, 18 us inside the step).
// Prompt steps of one request, us, tile kernels / split-K for the down-projection: 65 tokens 642 / 556, 128: 686 /
// 595, 129: 680 / 640, 192: 673 / 683, 256: 692 / 697: it pays up to 128 rows (one 128-wide side); the kernel
// itself takes up to 256.
constexpr int kSmallMaxRows = 256;
constexpr int kSmallPaysRows = 128;
constexpr int kSmallManyRowsMinK = 2048;
enum class SmallGemm { Skinny, SplitK };
SmallGemm small_gemm_kernel(int64_t M, int64_t N, int64_t K);
void gemm_small(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
                const Tensor* residual, KVTarget* kv = nullptr);

void kv_append(const Launch& l, const Tensor& k_src, const Tensor& v_src, const KVView& cache, const int* block_table,
               int max_blocks, const int* token_seq, const int* positions);

// What an attention launch needs to know about the step.
struct AttentionStep {
    int n_tokens = 0, n_seqs = 0, max_q_len = 0;
    const int* token_seq = nullptr;
    const int* positions = nullptr;
    const int* q_start = nullptr;
    const int* kv_before = nullptr;
    const int* block_table = nullptr;
    int max_blocks = 0;
    // from the step's host-side lists, for the profile's figures only: keys the step's requests hold
    // after it, and (query, key) pairs the causal attention looks at
    double kv_tokens = 0, pairs = 0;
};
// Attention of a step's tokens over the cache: picks the kernel for the step's shape.
void attention(const Launch& l, const AttentionStep& s, const Tensor& q, const KVView& cache, Tensor& out, int n_heads,
               float scale, int window, Workspace& ws);
int decode_splits(int n_tokens, int n_heads, int max_kv, int sms = 0);

// Choose one token per row of float32 `logits`; per-row option arrays may be null.  With `feedback`
// the drawn token also replaces the row's input token, its position moves on, and the token is
// recorded in burst_tokens[row_step[r], r]; `uniform` then holds [steps, rows] numbers.
struct SampleFeedback {
    int* token_ids = nullptr;
    const int* logit_rows = nullptr;
    int* positions = nullptr;
    int* burst_tokens = nullptr;
    int* row_step = nullptr;
};
void sample(const Launch& l, const Tensor& logits, int* out_tokens, const float* temperature, const int* top_k,
            const float* top_p, const float* uniform, const SampleFeedback* feedback);

}  // namespace ops
}  // namespace sandy
