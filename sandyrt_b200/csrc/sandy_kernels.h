// C declarations of every kernel launcher of this folder.  Each `<name>.cu` builds into one
// shared library that exports the functions listed under its name; all take raw device pointers
// and a stream, launch on that stream (so a launch can be captured in a CUDA graph) and return 0,
// SANDY_ERR_UNSUPPORTED (-1: sizes or dtypes the kernel refuses), SANDY_ERR_ARGUMENT (-2) or a
// cudaError_t.  dtype codes: 0 = float32, 1 = bfloat16.  `status` arguments are device ints in
// which kernels raise bits instead of faulting (bad token ids, pages that do not exist, waits
// that ran out).
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* embed.cu */
int sandy_embed_pos(const int* ids, const int* pos, const void* wte, const void* wpe, void* out, int n_tokens, int width,
                    int vocab, int n_pos, int table_dtype, int out_dtype, int* status, cudaStream_t stream);
int sandy_device_sm_count(void);
int sandy_spin(long long nanoseconds, cudaStream_t stream);

/* norm.cu */
int sandy_layernorm(const void* x, const void* gamma, const void* beta, void* out, const int* rows, int n_rows, int width,
                    float eps, int in_dtype, int w_dtype, int out_dtype, cudaStream_t stream);

/* gemm_simt.cu */
int sandy_gemm_simt(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                    int lda, int ldw, int ldr, int ldc, int w_out_in, int act, int a_dtype, int w_dtype, int out_dtype,
                    cudaStream_t stream);

/* gemm_tc.cu, gemm_tc2.cu */
int sandy_gemm_tc(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                  int lda, int ldw, int ldr, int ldc, int act, int out_dtype, int tile_n, void* k_cache, void* v_cache,
                  long long page_stride, const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                  int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);
int sandy_gemm_tc2(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                   int lda, int ldw, int ldr, int ldc, int act, int out_dtype, int tile_n, void* k_cache, void* v_cache,
                   long long page_stride, const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                   int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);

/* gemm_skinny.cu */
int sandy_gemm_skinny_norm_limits(int* max_rows, int* max_k);
int sandy_gemm_skinny(const void* a, const float* x, int ldx, const void* gamma, const void* beta, float eps, const void* w,
                      const void* bias, const float* residual, void* out, int M, int N, int K, int lda, int ldw, int ldr,
                      int ldc, int act, int out_dtype, void* k_cache, void* v_cache, long long page_stride,
                      const int* block_table, int max_blocks, const int* token_seq, const int* positions, int q_cols,
                      int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);

/* gemm_small.cu */
int sandy_gemm_small_splits(int N, int K);
int sandy_gemm_small(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                     int lda, int ldw, int ldr, int ldc, int act, int out_dtype, void* k_cache, void* v_cache,
                     long long page_stride, const int* block_table, int max_blocks, const int* token_seq,
                     const int* positions, int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status,
                     cudaStream_t stream);

/* attention.cu */
int sandy_kv_append(const void* k_src, const void* v_src, int ld_src, void* k_cache, void* v_cache, long long page_stride,
                    const int* block_table, int max_blocks, const int* token_seq, const int* positions, int n_tokens,
                    int n_kv_heads, int head_dim, int page_size, int num_pages, int dtype, int* status, cudaStream_t stream);
int sandy_paged_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                          const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                          int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                          int window, int num_pages, int dtype, int* status, cudaStream_t stream);

/* attention_decode.cu */
int sandy_decode_attention_cluster(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                   void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                   int* status, cudaStream_t stream);
long long sandy_decode_attention_scratch_floats(int n_tokens, int n_heads, int head_dim, int num_splits);
int sandy_decode_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                           const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                           int ld_out, float* scratch, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                           int page_size, float scale, int window, int num_splits, int num_pages, int dtype, int* status,
                           cudaStream_t stream);

/* attention_decode_mma.cu */
int sandy_decode_attention_mma_max_keys(int num_splits, int page_size);
int sandy_decode_attention_mma(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                               int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                               int window, int num_splits, int num_pages, int max_keys, int* status, cudaStream_t stream);

/* attention_decode_bulk.cu */
int sandy_decode_attention_bulk(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                int* status, cudaStream_t stream);

/* attention_prefill.cu, attention_prefill_tc.cu */
int sandy_prefill_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                            const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                            int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                            int page_size, float scale, int window, int num_pages, int* status, cudaStream_t stream);
int sandy_prefill_attention_tc(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                               int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                               int page_size, float scale, int window, int num_pages, int* status, cudaStream_t stream);

/* sampling.cu */
int sandy_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature, const int* top_k,
                 const float* top_p, const float* uniform, int* out_token, int* status, int* token_ids,
                 const int* logit_rows, int* positions, int* out_tokens, int* row_step, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
