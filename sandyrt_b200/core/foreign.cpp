#include "foreign.h"

#include "config.h"

namespace sandy {

namespace {
thread_local std::string t_cb_kind, t_cb_message;

SandyTensorView view_of(const Tensor& t) { return SandyTensorView{t.data, (int)t.dtype, t.rows, t.cols, t.ld}; }

struct Foreign {
    SandyForeignPart vt;
    void* user;
    std::string family, kind;
};

// What a foreign part says about itself (`info`), read once after it was made.
struct ForeignInfo {
    bool graph_safe = true;
    CacheSpec cache;
    std::optional<int64_t> max_positions;
    bool rotates = false;
    size_t weight_bytes = 0;
};

class Instance {
public:
    Instance(const Foreign& f, const PartSpec& spec) : f_(f) {
        inst_ = f.vt.create(f.user, to_json(spec).dump().c_str());
        if (!inst_) throw_callback_error(f.family + " '" + f.kind + "' could not be made");
        refresh();
    }
    ~Instance() {
        if (inst_ && f_.vt.destroy) f_.vt.destroy(f_.user, inst_);
    }
    void refresh() {
        if (!f_.vt.info) return;
        const char* text = f_.vt.info(f_.user, inst_);
        if (!text) throw_callback_error(f_.kind + ".info");
        const Json j = Json::parse(text);
        if (const Json* g = j.find("graph_safe")) info_.graph_safe = g->as_bool();
        if (const Json* r = j.find("rotates")) info_.rotates = r->as_bool();
        if (const Json* w = j.find("weight_bytes")) info_.weight_bytes = (size_t)w->as_int();
        if (const Json* m = j.find("max_positions"))
            if (!m->is_null()) info_.max_positions = m->as_int();
        if (const Json* c = j.find("cache"))
            if (c->is_object()) {
                const std::string kind = c->at("kind").as_string();
                if (kind == "paged") {
                    int window = 0;
                    if (const Json* w = c->find("window"))
                        if (!w->is_null()) window = (int)w->as_int();
                    info_.cache = CacheSpec::paged((int)c->at("n_kv_heads").as_int(), (int)c->at("head_dim").as_int(), window);
                } else if (kind == "state") {
                    std::vector<int64_t> shape;
                    for (const Json& d : c->at("shape").items()) shape.push_back(d.as_int());
                    DType dt = DType::F32;
                    if (const Json* d = c->find("dtype")) {
                        const std::string n = d->as_string();
                        dt = n == "bfloat16" ? DType::BF16 : (n == "int32" ? DType::I32 : DType::F32);
                    }
                    info_.cache = CacheSpec::state(shape, dt);
                }
            }
    }
    TensorRequests requests() const {
        TensorRequests out;
        if (!f_.vt.requests) return out;
        const char* text = f_.vt.requests(f_.user, inst_);
        if (!text) throw_callback_error(f_.kind + ".requests");
        const Json j = Json::parse(text);
        for (const auto& m : j.members()) {
            TensorRequest r;
            for (const Json& d : m.second.at("shape").items()) r.shape.push_back(d.as_int());
            if (const Json* v = m.second.find("init")) r.init = v->as_string();
            if (const Json* v = m.second.find("integer")) r.integer = v->as_bool();
            if (const Json* v = m.second.find("keep_32bit")) r.keep_32bit = v->as_bool();
            out[m.first] = r;
        }
        return out;
    }
    void bind(const TensorMap& tensors, DType dtype) {
        for (const auto& kv : tensors) {
            const HostTensor& t = kv.second;
            std::vector<long long> shape(t.shape.begin(), t.shape.end());
            if (!f_.vt.bind || f_.vt.bind(f_.user, inst_, kv.first.c_str(), t.data, store_dtype_name(t.dtype), shape.data(),
                                          (int)shape.size(), (int)dtype) != 0)
                throw_callback_error(f_.kind + ".bind('" + kv.first + "')");
        }
        refresh();
    }
    void forward(StepContext& ctx, const Tensor* a, const Tensor* b, int cache, bool write_cache, const int* rows, int n_rows) {
        StepViewHolder step(ctx);
        SandyTensorView va{}, vb{};
        if (a) va = view_of(*a);
        if (b) vb = view_of(*b);
        if (!f_.vt.forward || f_.vt.forward(f_.user, inst_, &step.view, a ? &va : nullptr, b ? &vb : nullptr, cache,
                                            write_cache ? 1 : 0, rows, n_rows) != 0)
            throw_callback_error(f_.kind + ".forward");
    }
    const ForeignInfo& info() const { return info_; }
private:
    Foreign f_;
    void* inst_ = nullptr;
    ForeignInfo info_;
};

class ForeignMixer : public Mixer {
public:
    ForeignMixer(const Foreign& f, const PartSpec& s) : Mixer(s), in_(f, s) {}
    TensorRequests requests() const override { return in_.requests(); }
    void bind(const TensorMap& t, DType d) override { in_.bind(t, d); }
    size_t weight_bytes() const override { return in_.info().weight_bytes; }
    bool graph_safe() const override { return in_.info().graph_safe; }
    CacheSpec cache_spec() const override { return in_.info().cache; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const Tensor& a = h.tensor();
        in_.forward(ctx, &a, &x, call.cache, call.write_cache, nullptr, 0);
    }
private:
    Instance in_;
};

class ForeignFeedForward : public FeedForward {
public:
    ForeignFeedForward(const Foreign& f, const PartSpec& s) : FeedForward(s), in_(f, s) {}
    TensorRequests requests() const override { return in_.requests(); }
    void bind(const TensorMap& t, DType d) override { in_.bind(t, d); }
    size_t weight_bytes() const override { return in_.info().weight_bytes; }
    bool graph_safe() const override { return in_.info().graph_safe; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x) override {
        const Tensor& a = h.tensor();
        in_.forward(ctx, &a, &x, -1, false, nullptr, 0);
    }
private:
    Instance in_;
};

class ForeignNorm : public Norm {
public:
    ForeignNorm(const Foreign& f, const PartSpec& s) : Norm(s), in_(f, s) {}
    TensorRequests requests() const override { return in_.requests(); }
    void bind(const TensorMap& t, DType d) override { in_.bind(t, d); }
    size_t weight_bytes() const override { return in_.info().weight_bytes; }
    bool graph_safe() const override { return in_.info().graph_safe; }
    void forward(StepContext& ctx, const Tensor& x, Tensor& out, const int* rows, int n_rows) override {
        in_.forward(ctx, &x, &out, -1, false, rows, n_rows);
    }
private:
    Instance in_;
};

class ForeignPosition : public PositionEncoding {
public:
    ForeignPosition(const Foreign& f, const PartSpec& s) : PositionEncoding(s), in_(f, s) {}
    TensorRequests requests() const override { return in_.requests(); }
    void bind(const TensorMap& t, DType d) override { in_.bind(t, d); }
    bool graph_safe() const override { return in_.info().graph_safe; }
    std::optional<int64_t> max_positions() const override { return in_.info().max_positions; }
    bool rotates() const override { return in_.info().rotates; }
    void rotate(StepContext& ctx, Tensor& q, Tensor* k) override { in_.forward(ctx, &q, k, -1, false, nullptr, 0); }
private:
    Instance in_;
};

}  // namespace

void set_callback_error(const std::string& kind, const std::string& message) {
    t_cb_kind = kind;
    t_cb_message = message;
}

void throw_callback_error(const std::string& where) {
    std::string kind = t_cb_kind.empty() ? "ForeignError" : t_cb_kind;
    std::string message = t_cb_message.empty() ? where + " failed" : t_cb_message;
    t_cb_kind.clear();
    t_cb_message.clear();
    throw Error(kind, message);
}

StepViewHolder::StepViewHolder(StepContext& ctx) : tables(ctx.block_tables) {
    view.n_tokens = ctx.n_tokens;
    view.n_seqs = ctx.n_seqs;
    view.n_rows = ctx.n_rows;
    view.max_blocks = ctx.max_blocks;
    view.max_q_len = ctx.max_q_len;
    view.max_kv_len = ctx.max_kv_len;
    view.compute_dtype = (int)ctx.compute_dtype;
    view.n_groups = (int)tables.size();
    view.token_ids = ctx.token_ids;
    view.positions = ctx.positions;
    view.token_seq = ctx.token_seq;
    view.seq_slots = ctx.seq_slots;
    view.q_start = ctx.q_start;
    view.kv_before = ctx.kv_before;
    view.logit_rows = ctx.logit_rows;
    view.block_tables = tables.data();
    view.host_q_lens = ctx.host_q_lens.data();
    view.host_kv_before = ctx.host_kv_before.data();
    view.host_slots = ctx.host_slots.data();
    view.stream = ctx.launch.stream;
    view.context = &ctx;
}

void register_foreign_part(const std::string& family, const std::string& kind, const SandyForeignPart& vtable, void* user) {
    const Foreign f{vtable, user, family, kind};
    PartFactory pf;
    if (family == "mixer") pf.make = [f](const PartSpec& s) { return std::unique_ptr<Part>(new ForeignMixer(f, s)); };
    else if (family == "feed_forward") pf.make = [f](const PartSpec& s) { return std::unique_ptr<Part>(new ForeignFeedForward(f, s)); };
    else if (family == "norm") pf.make = [f](const PartSpec& s) { return std::unique_ptr<Part>(new ForeignNorm(f, s)); };
    else if (family == "position") pf.make = [f](const PartSpec& s) { return std::unique_ptr<Part>(new ForeignPosition(f, s)); };
    else
        throw ConfigError("parts of family '" + family + "' cannot be defined through the C interface "
                          "(mixer, feed_forward, norm and position can; embeddings, heads and blocks are registered in C++)");
    register_part(family, kind, std::move(pf));
}

void register_foreign_architecture(const std::string& name, sandy_json_fn parse, sandy_json_fn describe_fn, void* user) {
    Architecture a;
    a.name = name;
    a.parse = [name, parse, user](const Json& raw) {
        const char* text = parse(user, raw.dump().c_str());
        if (!text) throw_callback_error("parsing the configuration of " + name);
        return std::unique_ptr<ModelConfig>(new ForeignConfig(name, Json::parse(text)));
    };
    a.describe = [name, describe_fn, user](const ModelConfig& c) {
        const char* text = describe_fn(user, c.to_json().dump().c_str());
        if (!text) throw_callback_error("describing " + name);
        return model_spec_from_json(Json::parse(text));
    };
    register_architecture(std::move(a));
}

}  // namespace sandy
