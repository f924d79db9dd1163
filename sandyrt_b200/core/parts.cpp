#include "parts.h"

#include <mutex>

namespace sandy {

ops::AttentionStep StepContext::attention_step(int group) const {
    ops::AttentionStep s;
    s.n_tokens = n_tokens;
    s.n_seqs = n_seqs;
    s.max_q_len = max_q_len;
    s.token_seq = token_seq;
    s.positions = positions;
    s.q_start = q_start;
    s.kv_before = kv_before;
    s.block_table = block_tables.at((size_t)group);
    s.max_blocks = max_blocks;
    for (size_t i = 0; i < host_q_lens.size() && i < host_kv_before.size(); i++) {
        const double n = host_q_lens[i], before = host_kv_before[i];
        s.kv_tokens += before + n;
        s.pairs += n * before + n * (n + 1) / 2;
    }
    return s;
}

// ---- NormedInput ---------------------------------------------------------------------------------------
const Tensor& NormedInput::tensor() {
    if (!tensor_.defined()) {
        tensor_ = ctx_.workspace->get("normed", x_.rows, x_.cols, ctx_.compute_dtype);
        norm_.forward(ctx_, x_, tensor_, nullptr, (int)x_.rows);
    }
    return tensor_;
}

bool NormedInput::fusable(ops::FusedNorm& out) const {
    LayerNormParams p;
    if (!norm_.layernorm_params(p)) return false;
    out.x = x_;
    out.gamma = p.gamma;
    out.beta = p.beta;
    out.eps = p.eps;
    return true;
}

// ---- Linear ----------------------------------------------------------------------------------------------
Linear::Linear(int64_t in_features, int64_t out_features, bool bias, const std::string& layout, std::string name)
    : in_(in_features), out_(out_features), has_bias_(bias), w_out_in_(layout == "out_in"), layout_(layout), name_(std::move(name)) {
    if (layout != "in_out" && layout != "out_in") throw ConfigError("linear layout must be 'in_out' or 'out_in', got '" + layout + "'");
}

TensorRequests Linear::requests() const {
    TensorRequests req;
    TensorRequest w;
    w.shape = layout_ == "in_out" ? std::vector<int64_t>{in_, out_} : std::vector<int64_t>{out_, in_};
    w.init = "weight";
    req[name_ + ".weight"] = w;
    if (has_bias_) {
        TensorRequest b;
        b.shape = {out_};
        b.init = "bias";
        req[name_ + ".bias"] = b;
    }
    return req;
}

void Linear::bind(const TensorMap& tensors, DType dtype, const Tensor* shared_weight) {
    use_tc_ = dtype == DType::BF16 && ops::tensor_core_gemm_supported(in_, out_);
    if (shared_weight) {
        // a table bound elsewhere (a tied head): [out, in] as it is
        weight_.buffer.reset();
        weight_.view = *shared_weight;
        w_out_in_ = true;
    } else {
        // the tensor-core kernels read K-major operand rows: one-time repack to [out, in]
        const bool turn = use_tc_ && layout_ == "in_out";
        weight_ = to_device(tensors.at(name_ + ".weight"), dtype, false, turn);
        w_out_in_ = layout_ == "out_in" || turn;
    }
    if (has_bias_) bias_ = to_device(tensors.at(name_ + ".bias"), dtype);
}

size_t Linear::weight_bytes() const {
    return (size_t)weight_.view.numel() * weight_.view.elem_size() + (has_bias_ ? bias_.bytes() : 0);
}

void Linear::run(StepContext& ctx, NormedInput* lazy, const Tensor* a, Tensor& out, ops::Act act, const Tensor* residual,
                 ops::KVTarget* kv) {
    const int64_t rows = lazy ? lazy->rows() : a->rows;
    const Tensor* bias = has_bias_ ? &bias_.view : nullptr;
    const ops::Launch& l = ctx.launch;
    if (use_tc_ && rows <= ops::kSkinnyMaxRows) {
        ops::FusedNorm fused;
        const bool fuse = lazy && rows <= ops::kSkinnyNormPaysRows && in_ <= ops::kSkinnyNormPaysK && lazy->fusable(fused) && ops::skinny_norm_fusable(fused, in_, DType::BF16);
        if (!fuse && lazy) a = &lazy->tensor();
        if (!fuse && ops::small_gemm_kernel(rows, out_, in_) == ops::SmallGemm::SplitK) {
            ops::gemm_small(l, *a, weight_.view, bias, out, act, residual, kv);
            return;
        }
        ops::gemm_skinny(l, fuse ? nullptr : a, fuse ? &fused : nullptr, weight_.view, bias, out, act, residual, kv);
        return;
    }
    if (lazy) a = &lazy->tensor();
    if (use_tc_ && rows <= ops::kSmallPaysRows && in_ >= ops::kSmallManyRowsMinK && !kv) {
        ops::gemm_small(l, *a, weight_.view, bias, out, act, residual, nullptr);
        return;
    }
    if (use_tc_) {
        const bool fused_kv = kv && kv->cache.head_dim % 16 == 0 && kv->q_cols % 8 == 0;
        ops::gemm_tc(l, *a, weight_.view, bias, out, act, residual, 0, fused_kv ? kv : nullptr);
    } else {
        ops::gemm_simt(l, *a, weight_.view, bias, out, w_out_in_, act, residual);
    }
}

// ---- built-in parts -----------------------------------------------------------------------------------------
namespace {

// LayerNorm (kind "layernorm"): statistics in 32-bit, eps and width as parameters.  Formula:
// src/core/TensorCalc.cpp:2048-2072 of the reference (biased variance, two passes, 1/sqrt(var + eps),
// then gamma and beta).  Parameters: width, eps, bias (whether beta exists).  Tensors: "weight", "bias".
class LayerNorm : public Norm {
public:
    explicit LayerNorm(const PartSpec& s)
        : Norm(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), has_bias_(s.get_bool("bias", true)) {}
    TensorRequests requests() const override {
        TensorRequests r;
        TensorRequest g;
        g.shape = {width_};
        g.init = "gamma";
        r["weight"] = g;
        if (has_bias_) {
            TensorRequest b;
            b.shape = {width_};
            b.init = "beta";
            r["bias"] = b;
        }
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        gamma_ = to_device(t.at("weight"), dtype);
        if (has_bias_) beta_ = to_device(t.at("bias"), dtype);
    }
    size_t weight_bytes() const override { return gamma_.bytes() + (has_bias_ ? beta_.bytes() : 0); }
    void forward(StepContext& ctx, const Tensor& x, Tensor& out, const int* rows, int n_rows) override {
        ops::layernorm(ctx.launch, x, gamma_.view, has_bias_ ? &beta_.view : nullptr, eps_, out, rows, n_rows);
    }
    bool layernorm_params(LayerNormParams& p) const override {
        p.gamma = gamma_.view;
        p.beta = has_bias_ ? &beta_.view : nullptr;
        p.eps = eps_;
        return true;
    }
private:
    int64_t width_;
    float eps_;
    bool has_bias_;
    DeviceWeight gamma_, beta_;
};

// "learned_absolute": a table [max_positions, width] added to the token embedding
// (src/models/gpt2_small.sandy.go:49-50 of the reference: a second embedding lookup with position
// ids, then an add).  Positions are supplied by the step, not derived.  The table's length is a hard
// limit on a request's length.
class LearnedAbsolute : public PositionEncoding {
public:
    explicit LearnedAbsolute(const PartSpec& s) : PositionEncoding(s), width_(s.get_int("width")), max_(s.get_int("max_positions")) {}
    TensorRequests requests() const override {
        TensorRequest w;
        w.shape = {max_, width_};
        return {{"weight", w}};
    }
    void bind(const TensorMap& t, DType dtype) override { table_ = to_device(t.at("weight"), dtype); }
    std::optional<int64_t> max_positions() const override { return max_; }
    const Tensor* table() const override { return &table_.view; }
private:
    int64_t width_, max_;
    DeviceWeight table_;
};

// "none": no encoding at the embedding and no limit.
class NoPosition : public PositionEncoding {
public:
    using PositionEncoding::PositionEncoding;
};

// Token embedding: x[t] = table[id[t]] (+ position table[pos[t]] when the position encoding has one),
// one fused pass (src/models/gpt2_small.sandy.go:48-50 of the reference).
class TokenEmbedding : public Embedding {
public:
    explicit TokenEmbedding(const PartSpec& s) : Embedding(s), vocab_(s.get_int("vocab_size")), width_(s.get_int("width")) {}
    TensorRequests requests() const override {
        TensorRequest w;
        w.shape = {vocab_, width_};
        return {{"weight", w}};
    }
    void bind(const TensorMap& t, DType dtype) override { weight_ = to_device(t.at("weight"), dtype); }
    const Tensor* table() const override { return &weight_.view; }
    void forward(StepContext& ctx, Tensor& x) override {
        const Tensor* pos = ctx.position ? ctx.position->table() : nullptr;
        ops::embed_positions(ctx.launch, ctx.token_ids, ctx.positions, weight_.view, pos, x, ctx.n_tokens);
    }
private:
    int64_t vocab_, width_;
    DeviceWeight weight_;
};

// Output head: logits = y @ W^T in float32.  With `tied` the token table itself is the weight: the
// reference ties by naming `wte.weight` twice (:57, a transposed-operand matmul,
// src/ir/MidIRPass.cpp:30-69), and no second copy exists here either.
class OutputHead : public Head {
public:
    explicit OutputHead(const PartSpec& s)
        : Head(s), vocab_(s.get_int("vocab_size")), width_(s.get_int("width")), tied_(s.get_bool("tied", false)),
          linear_(width_, vocab_, false, "out_in", "head") {}
    TensorRequests requests() const override {
        if (tied_) return {};
        TensorRequest w;
        w.shape = {vocab_, width_};
        return {{"weight", w}};
    }
    bool tied() const override { return tied_; }
    void bind_head(const TensorMap& t, DType dtype, const Tensor* tied_weight) override {
        if (tied_) {
            if (!tied_weight) throw ConfigError("tied output head needs the token table");
            linear_.bind({}, dtype, tied_weight);
        } else {
            TensorMap m;
            m["head.weight"] = t.at("weight");
            linear_.bind(m, dtype);
        }
    }
    size_t weight_bytes() const override { return linear_.weight_bytes(); }
    void forward(StepContext& ctx, const Tensor& y, Tensor& logits) override {
        linear_.run(ctx, nullptr, &y, logits, ops::Act::None, nullptr);
    }
private:
    int64_t vocab_, width_;
    bool tied_;
    Linear linear_;
};

// Causal self-attention over the paged cache (kind "causal_attention").
//   qkv = h @ W_qkv + b_qkv;  q, k, v = column ranges [0, H*D), [H*D, (H+Hkv)*D), the rest
//   (k, v) of the step's tokens are appended to the request's pages
//   o = attention(q, all cached k, v up to each token's own position)
//   x += o @ W_out + b_out
// Formulas: src/models/gpt2_small.sandy.go:1-23 and src/core/TensorCalc.cpp:1241-1311 of the
// reference (which splits the fused matrix offline into q/k/v, scripts/run_gpt2.py:170-175; here the
// fused matrix is used as stored and the split is three column ranges).
// Parameters: width, n_heads, n_kv_heads, head_dim, scale (the factor on q.k, already including any
// per-layer factor the architecture wants), window (null = all positions), bias, weight_layout.
// Tensors: "qkv.weight", "qkv.bias", "out.weight", "out.bias".
class CausalSelfAttention : public Mixer {
public:
    explicit CausalSelfAttention(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), n_heads_((int)s.get_int("n_heads")),
          n_kv_heads_((int)s.get_int("n_kv_heads", s.get_int("n_heads"))), head_dim_((int)s.get_int("head_dim")),
          scale_((float)s.get_double("scale")), window_((int)s.get_optional_int("window").value_or(0)),
          q_cols_((int64_t)n_heads_ * head_dim_), kv_cols_((int64_t)n_kv_heads_ * head_dim_),
          qkv_(width_, q_cols_ + 2 * kv_cols_, s.get_bool("bias", true), s.get_string("weight_layout", "out_in"), "qkv"),
          out_(q_cols_, width_, s.get_bool("bias", true), s.get_string("weight_layout", "out_in"), "out") {
        if (n_kv_heads_ <= 0 || n_heads_ % n_kv_heads_ != 0)
            throw ConfigError("causal_attention: " + std::to_string(n_heads_) + " heads do not divide into " +
                              std::to_string(n_kv_heads_) + " key/value heads");
        if (head_dim_ % 16 != 0 || head_dim_ <= 0 || head_dim_ > 256)
            throw ConfigError("causal_attention: head size " + std::to_string(head_dim_) + " must be a multiple of 16, at most 256");
    }
    TensorRequests requests() const override {
        TensorRequests r = qkv_.requests();
        for (auto& kv : out_.requests()) r[kv.first] = kv.second;
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        qkv_.bind(t, dtype);
        out_.bind(t, dtype);
    }
    size_t weight_bytes() const override { return qkv_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override { return CacheSpec::paged(n_kv_heads_, head_dim_, window_); }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        Tensor qkv = ws.get("qkv", T, q_cols_ + 2 * kv_cols_, ctx.compute_dtype);
        const KVView cache = ctx.caches->kv(call.cache);
        const int* table = ctx.block_tables.at((size_t)cache.group);
        const bool rotates = ctx.position && ctx.position->rotates();
        // keys/values may go straight from the projection's write-back into the pages, unless a
        // position encoding still has to turn them first
        ops::KVTarget target;
        const bool fuse = call.write_cache && !rotates;
        if (fuse) {
            target.cache = cache;
            target.block_table = table;
            target.max_blocks = ctx.max_blocks;
            target.token_seq = ctx.token_seq;
            target.positions = ctx.positions;
            target.q_cols = (int)q_cols_;
            target.kv_cols = (int)kv_cols_;
        }
        qkv_.run(ctx, &h, nullptr, qkv, ops::Act::None, nullptr, fuse ? &target : nullptr);
        Tensor q = qkv.col_range(0, q_cols_);
        Tensor k = qkv.col_range(q_cols_, q_cols_ + kv_cols_);
        Tensor v = qkv.col_range(q_cols_ + kv_cols_, q_cols_ + 2 * kv_cols_);
        if (rotates) ctx.position->rotate(ctx, q, call.write_cache ? &k : nullptr);
        if (call.write_cache && !target.written)
            ops::kv_append(ctx.launch, k, v, cache, table, ctx.max_blocks, ctx.token_seq, ctx.positions);
        Tensor o = ws.get("attn_out", T, q_cols_, ctx.compute_dtype);
        ops::attention(ctx.launch, ctx.attention_step(cache.group), q, cache, o, n_heads_, scale_, window_, ws);
        out_.run(ctx, nullptr, &o, x, ops::Act::None, &x);
    }
private:
    int64_t width_;
    int n_heads_, n_kv_heads_, head_dim_;
    float scale_;
    int window_;
    int64_t q_cols_, kv_cols_;
    Linear qkv_, out_;
};

// Dense feed-forward (kind "dense_mlp"): u = h @ W_up + b_up;  g = act(u);  x += g @ W_down + b_down
// (src/models/gpt2_small.sandy.go:25-32,40-42 of the reference).  The activation runs in the
// up-projection's write-back and the residual sum in the down-projection's, both in 32-bit.
// Parameters: width, inner, activation ("gelu_new" | "gelu"), bias, weight_layout.
// Tensors: "up.weight", "up.bias", "down.weight", "down.bias".
class DenseMLP : public FeedForward {
public:
    explicit DenseMLP(const PartSpec& s)
        : FeedForward(s), width_(s.get_int("width")), inner_(s.get_int("inner")),
          up_(width_, inner_, s.get_bool("bias", true), s.get_string("weight_layout", "out_in"), "up"),
          down_(inner_, width_, s.get_bool("bias", true), s.get_string("weight_layout", "out_in"), "down") {
        const std::string name = s.get_string("activation");
        try {
            act_ = ops::act_from_name(name);
        } catch (const ValueError&) {
            act_ = ops::Act::None;
        }
        if (act_ == ops::Act::None) throw ConfigError("dense_mlp: unknown activation '" + name + "'");
    }
    TensorRequests requests() const override {
        TensorRequests r = up_.requests();
        for (auto& kv : down_.requests()) r[kv.first] = kv.second;
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        up_.bind(t, dtype);
        down_.bind(t, dtype);
    }
    size_t weight_bytes() const override { return up_.weight_bytes() + down_.weight_bytes(); }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x) override {
        Tensor g = ctx.workspace->get("ff_inner", h.rows(), inner_, ctx.compute_dtype);
        up_.run(ctx, &h, nullptr, g, act_, nullptr);
        down_.run(ctx, nullptr, &g, x, ops::Act::None, &x);
    }
private:
    int64_t width_, inner_;
    ops::Act act_ = ops::Act::None;
    Linear up_, down_;
};

// "pre_norm": x += mixer(norm_1(x)); x += feed_forward(norm_2(x))
// (src/models/gpt2_small.sandy.go:34-45 of the reference).  Norm names: "mixer", "feed_forward".
class PreNormBlock : public Block {
public:
    using Block::Block;
    void forward(StepContext& ctx, Tensor& x, const LayerCall& call) override {
        NormedInput h1(ctx, *norms_.at("mixer"), x);
        mixer_->forward(ctx, h1, x, call);
        NormedInput h2(ctx, *norms_.at("feed_forward"), x);
        ff_->forward(ctx, h2, x);
    }
};

template <typename T>
PartFactory simple() {
    PartFactory f;
    f.make = [](const PartSpec& s) { return std::unique_ptr<Part>(new T(s)); };
    return f;
}

using Table = std::map<std::string, std::map<std::string, PartFactory>>;

Table& table() {
    static Table t;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* fam : {"mixer", "feed_forward", "norm", "position", "embedding", "head", "block"}) t[fam];
        t["norm"]["layernorm"] = simple<LayerNorm>();
        t["position"]["learned_absolute"] = simple<LearnedAbsolute>();
        t["position"]["none"] = simple<NoPosition>();
        t["embedding"]["token_embedding"] = simple<TokenEmbedding>();
        t["head"]["output_head"] = simple<OutputHead>();
        t["mixer"]["causal_attention"] = simple<CausalSelfAttention>();
        t["feed_forward"]["dense_mlp"] = simple<DenseMLP>();
        PartFactory pre;
        pre.norm_names = {"mixer", "feed_forward"};
        pre.make_block = [](BlockParts p) {
            return std::unique_ptr<Block>(new PreNormBlock(std::move(p.mixer), std::move(p.feed_forward), std::move(p.norms), p.width));
        };
        t["block"]["pre_norm"] = std::move(pre);
    });
    return t;
}
std::mutex& table_lock() { static std::mutex m; return m; }

}  // namespace

void register_part(const std::string& family, const std::string& kind, PartFactory factory) {
    Table& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    auto it = t.find(family);
    if (it == t.end()) throw ConfigError("unknown part family '" + family + "'; one of mixer, feed_forward, norm, position, embedding, head, block");
    it->second[kind] = std::move(factory);
}

const PartFactory& get_part(const std::string& family, const std::string& kind) {
    Table& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    auto fam = t.find(family);
    if (fam == t.end()) throw ConfigError("unknown part family '" + family + "'");
    auto it = fam->second.find(kind);
    if (it == fam->second.end()) {
        std::string known;
        for (const auto& kv : fam->second) known += (known.empty() ? "'" : ", '") + kv.first + "'";
        throw ConfigError("unknown " + family + " kind '" + kind + "'; registered: [" + known + "]");
    }
    return it->second;
}

std::vector<std::string> part_kinds(const std::string& family) {
    Table& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    std::vector<std::string> out;
    auto fam = t.find(family);
    if (fam != t.end())
        for (const auto& kv : fam->second) out.push_back(kv.first);
    return out;
}

}  // namespace sandy
