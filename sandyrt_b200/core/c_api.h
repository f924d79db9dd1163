/* The C interface of the engine's host library (libsandy_core.so).
 *
 * Two kinds of calls.  The hot path (adding requests, stepping, reading tokens and logits) has typed
 * functions that take plain arrays.  Everything else (configuration, model descriptions, the cache
 * allocator and the scheduler on their own, counters, random model folders) goes through one
 * function, sandy_call(object, handle, method, args_json) -> result_json.
 *
 * Errors: a function that fails returns NULL, a negative count or a non-zero code, and the calling
 * thread's last error is set: its kind (the name of the C++ error class: "ConfigError",
 * "WeightBindingError", "OutOfPages", ...), its message, and for some kinds its parts as JSON.
 * Strings returned by this library stay valid until the calling thread's next call into it.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

const char* sandy_last_error_kind(void);
const char* sandy_last_error_message(void);
const char* sandy_last_error_details(void);

/* ---- where the kernel libraries are, and who can build a missing one ---------------------------- */
void sandy_set_kernel_dir(const char* dir);
typedef int (*sandy_kernel_provider)(const char* name, char* dir, int dir_capacity);
void sandy_set_kernel_provider(sandy_kernel_provider provider);
long long sandy_kernel_launches(void);

/* ---- the structured control plane -------------------------------------------------------------------
 * object: "global", "pool", "allocator", "scheduler", "model", "engine", "llm", "weights", "harness".
 * Creating calls ("global" methods new_pool, new_allocator, new_scheduler, load_model, build_model, new_engine,
 * new_llm, open_weights, new_harness) return {"handle": <integer>}; pass that integer as `handle` afterwards and
 * give it back with sandy_release. */
const char* sandy_call(const char* object, void* handle, const char* method, const char* args_json);
void sandy_release(const char* object, void* handle);

/* ---- architectures and parts defined by the caller ---------------------------------------------------
 * An architecture: parse(raw config.json) -> normalised config JSON, describe(config JSON) -> model
 * description JSON (the form ModelSpec is written in).  Both return NULL on failure after calling
 * sandy_set_callback_error. */
typedef const char* (*sandy_json_fn)(void* user, const char* json);
int sandy_register_architecture(const char* name, sandy_json_fn parse, sandy_json_fn describe, void* user);
void sandy_set_callback_error(const char* kind, const char* message);

typedef struct SandyTensorView {
    void* data;
    int dtype;                 /* 0 float32, 1 bfloat16, 2 int32 */
    long long rows, cols, ld;  /* ld: row pitch in elements */
} SandyTensorView;

typedef struct SandyStepView {
    int n_tokens, n_seqs, n_rows, max_blocks, max_q_len, max_kv_len, compute_dtype, n_groups;
    int* token_ids;
    int* positions;
    const int* token_seq;
    const int* seq_slots;
    const int* q_start;
    const int* kv_before;
    const int* logit_rows;
    const int* const* block_tables;  /* [n_groups] device arrays [n_seqs, max_blocks] */
    const int* host_q_lens;          /* [n_seqs] host copies, for parts that plan on the host */
    const int* host_kv_before;
    const int* host_slots;
    void* stream;                    /* the cudaStream_t every launch of the step goes to */
    void* context;                   /* for sandy_step_state / sandy_step_kv */
} SandyStepView;

/* A part kind implemented by the caller (families "mixer", "feed_forward", "norm", "position").
 * create: an instance from the part's description (JSON: kind, params, tensors).
 * requests: JSON {"local name": {"shape": [...], "init": "weight|bias|gamma|beta|zeros", "integer": false, "keep_32bit": false}}.
 * info: JSON {"graph_safe": bool, "cache": null | {"kind": "paged", "n_kv_heads", "head_dim", "window"} |
 *       {"kind": "state", "shape": [...], "dtype": "float32"}, "max_positions": null | n, "rotates": bool, "weight_bytes": n}.
 * bind: one call per requested tensor, with the host data as stored (dtype name "F32", "BF16", ...).
 * forward: mixer (a = normed input h, b = residual stream x, cache, write_cache); feed_forward (a = h, b = x);
 *          norm (a = x, b = out, rows/n_rows); position (a = q, b = k or NULL): the rotation.
 * Callbacks return 0 / non-NULL on success; on failure they call sandy_set_callback_error first. */
typedef struct SandyForeignPart {
    void* (*create)(void* user, const char* spec_json);
    void (*destroy)(void* user, void* instance);
    const char* (*requests)(void* user, void* instance);
    const char* (*info)(void* user, void* instance);
    int (*bind)(void* user, void* instance, const char* name, const void* host_data, const char* store_dtype,
                const long long* shape, int rank, int compute_dtype);
    int (*forward)(void* user, void* instance, const SandyStepView* step, const SandyTensorView* a, const SandyTensorView* b,
                   int cache, int write_cache, const int* rows, int n_rows);
} SandyForeignPart;
int sandy_register_part(const char* family, const char* kind, const SandyForeignPart* vtable, void* user);
/* A step's cache entries, for foreign mixers: the fixed-size state [max_requests, elems] of a cache entry ... */
int sandy_step_state(const SandyStepView* step, int cache, SandyTensorView* out);
/* ... and the key / value pages [num_pages, Hkv, page_size, D] (views: data, dtype, rows = num_pages, ld = page stride). */
int sandy_step_kv(const SandyStepView* step, int cache, SandyTensorView* k, SandyTensorView* v, int* group, int* n_kv_heads,
                  int* page_size, int* head_dim);

/* ---- the entry point: requests in, tokens out -------------------------------------------------------- */
void* sandy_llm_load(const char* model_dir, const char* options_json);
void* sandy_llm_from_model(void* model, const char* options_json);      /* takes the model handle over */
long long sandy_llm_add_request(void* llm, const int* prompt_ids, int n_prompt, int max_tokens, float temperature, int top_k,
                                float top_p, int has_seed, unsigned long long seed, const int* stop_ids, int n_stop);
/* One step (or burst).  Writes up to `capacity` (request, token) pairs; returns how many were drawn (may exceed
 * capacity: call again with more room is not possible, so give max_live * 32), or -1. */
int sandy_llm_step(void* llm, long long* rids, int* tokens, int capacity);
int sandy_llm_drain(void* llm, long long* rids, int* tokens, int capacity);
int sandy_llm_has_work(void* llm);
int sandy_llm_finished(void* llm, long long rid);
/* Blocking generation of several prompts (ids back to back, lengths in prompt_lens).  Result: JSON list of
 * results with the reference's GenerateResult fields.  on_token may be NULL. */
typedef int (*sandy_token_fn)(void* user, int request_index, int token);
const char* sandy_llm_generate(void* llm, const int* prompt_ids, const int* prompt_lens, int n_prompts, const char* params_json,
                               sandy_token_fn on_token, void* user);
void* sandy_llm_engine(void* llm);            /* borrowed: do not release */

/* ---- the step function on its own --------------------------------------------------------------------- */
/* entries: rids[n], n_tokens[n], tokens (back to back), n_want[n], want (back to back).  sampling: NULL or
 * 4 floats per wanted row (temperature, top_k, top_p, uniform).  On success *logits points at float32
 * [rows, cols] on the device (valid until the next step; complete once sandy_engine_synchronize returns). */
int sandy_engine_step(void* engine, int n_entries, const long long* rids, const int* n_tokens, const int* tokens,
                      const int* n_want, const int* want, const float* sampling, void** logits, int* rows, int* cols);
int sandy_engine_read_sampled(void* engine, int n, int* out);
/* returns a burst handle (>= 0) or -1 */
int sandy_engine_decode_burst_async(void* engine, int n_requests, const long long* rids, const int* first_tokens,
                                    const float* sampling, const float* uniforms, int n_steps, int in_flight);
int sandy_engine_burst_tokens(void* engine, int burst, int* out);      /* out: [n_steps, n_requests] */
int sandy_engine_synchronize(void* engine);
void* sandy_engine_stream(void* engine);
/* device time in milliseconds between two marks on the engine's stream */
int sandy_engine_mark(void* engine, int which);
/* Keeps the engine's stream busy for so many microseconds (a kernel that only waits), so that what the
   host queues meanwhile runs back to back behind it: for timing the device's share of a step. */
int sandy_engine_hold(void* engine, int microseconds);
float sandy_engine_elapsed_ms(void* engine);

#ifdef __cplusplus
}
#endif
