// The parts a model is put together from, the per-step context they see, and their registry.
//
// A part is built from a PartSpec (its kind, its sizes and constants, the names of its tensors),
// says which tensors it needs (`requests`), receives them (`bind`) and then runs on the tokens of a
// step (`forward`).  It knows its own sizes and nothing of the model it sits in: layer indices,
// architecture names and config.json keys never reach it.
//
// Families and what each must provide:
//   Norm              forward(ctx, x, out, rows, n_rows)      out = norm(x[rows] or x)
//   PositionEncoding  table() -> tensor added at the embedding, or null
//                     rotate(ctx, q, k)  (in place), for encodings applied to queries and keys
//                     max_positions() -> limit or nullopt
//   Embedding         forward(ctx, x)                          x = the tokens' rows (+ position table)
//                     table() -> the bound token table
//   Head              forward(ctx, y, logits)                  float32 logits of the normed rows y
//   Mixer             cache_spec() -> pages, a fixed-size state, or nothing
//                     forward(ctx, h, x, call)                 x += mix(h), in place
//   FeedForward       forward(ctx, h, x)                       x += ff(h), in place
//   Block             forward(ctx, x, call)                    runs its norms, mixer, feed-forward
//
// `x` is the residual stream: float32 [tokens, width] in both compute dtypes, so the residual sum is
// always formed and kept in 32-bit.  `h` is a normed copy in the compute dtype, handed over as a
// NormedInput: a consumer either asks for the tensor (computed once) or, if its kernel can run the
// norm itself, takes the norm's parameters and never materialises it.
//
// A new kind is added with `register_part(family, kind, factory)`; no file of the engine changes.
// Kinds defined outside this library (the Python binding) register through the C interface and run
// as ForeignPart adapters around their callbacks.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "cache.h"
#include "device.h"
#include "ops.h"
#include "spec.h"
#include "weights.h"

namespace sandy {

class PositionEncoding;

// Everything a part may read about the running step.  Device arrays are int32.
struct StepContext {
    int n_tokens = 0, n_seqs = 0, n_rows = 0;
    int* token_ids = nullptr;            // [T] the step's tokens, requests back to back
    int* positions = nullptr;            // [T] position of each token in its request
    const int* token_seq = nullptr;      // [T] which of the step's requests a token belongs to
    const int* seq_slots = nullptr;      // [S] state slot of each request
    const int* q_start = nullptr;        // [S+1] first token of each request in the step
    const int* kv_before = nullptr;      // [S] tokens each request had before the step
    const int* logit_rows = nullptr;     // [R] tokens whose logits are wanted
    std::vector<const int*> block_tables;    // per cache group: [S, max_blocks]
    int max_blocks = 0;
    DType compute_dtype = DType::F32;
    Workspace* workspace = nullptr;
    DeviceCaches* caches = nullptr;
    PositionEncoding* position = nullptr;    // the model's position encoding
    // host copies, for parts that plan their launches on the host
    std::vector<int> host_q_lens, host_kv_before, host_slots;
    int max_q_len = 0, max_kv_len = 0;
    ops::Launch launch;                  // stream and status words

    ops::AttentionStep attention_step(int group) const;
};

class Part {
public:
    explicit Part(const PartSpec& spec) : spec_(spec) {}
    virtual ~Part() = default;
    const PartSpec& spec() const { return spec_; }
    virtual TensorRequests requests() const { return {}; }             // local tensor name -> what is expected of it
    virtual void bind(const TensorMap& tensors, DType dtype) { (void)tensors; (void)dtype; }
    // Bytes of weights one step reads from this part (for roofline figures); parts with matrices override it.
    virtual size_t weight_bytes() const { return 0; }
    // A part whose `forward` only launches kernels that read the step's device arrays may be recorded
    // in a CUDA graph and replayed.  A part that decides anything from the step's host-side lists
    // must say false; the engine then runs every step of a model that holds such a part without graphs.
    virtual bool graph_safe() const { return true; }
protected:
    PartSpec spec_;
};

struct LayerNormParams { Tensor gamma; const Tensor* beta = nullptr; float eps = 0.0f; };

class Norm : public Part {
public:
    using Part::Part;
    virtual void forward(StepContext& ctx, const Tensor& x, Tensor& out, const int* rows, int n_rows) = 0;
    // Kernels that can run a LayerNorm inside themselves ask for its parameters here.
    virtual bool layernorm_params(LayerNormParams& out) const { (void)out; return false; }
};

class PositionEncoding : public Part {
public:
    using Part::Part;
    virtual std::optional<int64_t> max_positions() const { return std::nullopt; }
    virtual const Tensor* table() const { return nullptr; }
    virtual bool rotates() const { return false; }                      // true for encodings that act on queries and keys
    virtual void rotate(StepContext& ctx, Tensor& q, Tensor* k) { (void)ctx; (void)q; (void)k; }
};

class Embedding : public Part {
public:
    using Part::Part;
    virtual const Tensor* table() const { return nullptr; }
    virtual void forward(StepContext& ctx, Tensor& x) = 0;
};

class Head : public Part {
public:
    using Part::Part;
    virtual bool tied() const { return false; }        // shares the embedding's table: `bind` then receives it
    virtual void bind_head(const TensorMap& tensors, DType dtype, const Tensor* tied_weight) = 0;
    virtual void forward(StepContext& ctx, const Tensor& y, Tensor& logits) = 0;
};

// A normed view of the residual stream that has not been computed yet.
class NormedInput {
public:
    NormedInput(StepContext& ctx, Norm& norm, const Tensor& x) : ctx_(ctx), norm_(norm), x_(x) {}
    int64_t rows() const { return x_.rows; }
    int64_t cols() const { return x_.cols; }
    const Tensor& tensor();                            // computed once and shared
    bool fusable(ops::FusedNorm& out) const;           // the norm's parameters, if it is a LayerNorm
private:
    StepContext& ctx_;
    Norm& norm_;
    Tensor x_;
    Tensor tensor_;
};

class Mixer : public Part {
public:
    using Part::Part;
    virtual CacheSpec cache_spec() const { return CacheSpec::none(); }
    virtual void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) = 0;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual void forward(StepContext& ctx, NormedInput& h, Tensor& x) = 0;
};

// An arrangement of norms, a mixer and a feed-forward (built from a LayerSpec).
class Block {
public:
    Block(std::unique_ptr<Mixer> mixer, std::unique_ptr<FeedForward> ff, std::map<std::string, std::unique_ptr<Norm>> norms,
          int64_t width)
        : mixer_(std::move(mixer)), ff_(std::move(ff)), norms_(std::move(norms)), width_(width) {}
    virtual ~Block() = default;
    virtual void forward(StepContext& ctx, Tensor& x, const LayerCall& call) = 0;
    Mixer& mixer() { return *mixer_; }
    FeedForward& feed_forward() { return *ff_; }
    std::map<std::string, std::unique_ptr<Norm>>& norms() { return norms_; }
protected:
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<FeedForward> ff_;
    std::map<std::string, std::unique_ptr<Norm>> norms_;
    int64_t width_;
};

// One weight matrix with its bias, and the choice of the kernel that multiplies by it.
//
// The weight file may store a matrix as [in, out] (GPT-2's Conv1D layout; the reference transposes
// these offline, scripts/run_gpt2.py:177-189) or as [out, in].  Both are read as they are: the
// 32-bit kernel takes either layout, and for the tensor-core kernels the matrix is brought into
// [out, in] once, when it is bound, which is the K-major operand layout those kernels read.
// Kernel choice per call, by dtype and row count: float32 -> the FFMA kernel; bfloat16 with up to 64
// rows (a decode step) -> the weight-streaming kernel, which can also run the norm before the
// product and write key/value columns into the cache; bfloat16 with more rows -> tcgen05.
class Linear {
public:
    Linear(int64_t in_features, int64_t out_features, bool bias, const std::string& layout, std::string name);
    TensorRequests requests() const;
    void bind(const TensorMap& tensors, DType dtype, const Tensor* shared_weight = nullptr);
    size_t weight_bytes() const;
    // out = act(a @ W + b) + residual.  `out` may be `residual` itself.  If `kv` is given and the
    // kernel used can write keys/values into the cache, it does and sets kv->written.
    void run(StepContext& ctx, NormedInput* lazy, const Tensor* a, Tensor& out, ops::Act act, const Tensor* residual,
             ops::KVTarget* kv = nullptr);
    const Tensor& weight() const { return weight_.view; }
private:
    int64_t in_, out_;
    bool has_bias_, w_out_in_, use_tc_ = false;
    std::string layout_, name_;
    DeviceWeight weight_, bias_;
};

// ---- registry of part kinds ---------------------------------------------------------------------------
struct BlockParts {
    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> feed_forward;
    std::map<std::string, std::unique_ptr<Norm>> norms;
    int64_t width = 0;
};
struct PartFactory {
    std::function<std::unique_ptr<Part>(const PartSpec&)> make;                // every family but "block"
    std::function<std::unique_ptr<Block>(BlockParts)> make_block;              // "block"
    std::vector<std::string> norm_names;                                       // "block": the norms it wants
};
// family: "mixer", "feed_forward", "norm", "position", "embedding", "head" or "block"
void register_part(const std::string& family, const std::string& kind, PartFactory factory);
const PartFactory& get_part(const std::string& family, const std::string& kind);    // unknown -> ConfigError listing the known kinds
std::vector<std::string> part_kinds(const std::string& family);

template <typename T>
std::unique_ptr<T> make_part(const std::string& family, const PartSpec& spec) {
    std::unique_ptr<Part> p = get_part(family, spec.kind).make(spec);
    T* typed = dynamic_cast<T*>(p.get());
    if (!typed) throw ConfigError("part kind '" + spec.kind + "' is not a " + family);
    p.release();
    return std::unique_ptr<T>(typed);
}

}  // namespace sandy
