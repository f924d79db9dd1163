#include "model.h"

namespace sandy {

Model::Model(ModelSpec spec) : spec_(std::move(spec)) {
    embedding_ = make_part<Embedding>("embedding", spec_.embedding);
    position_ = make_part<PositionEncoding>("position", spec_.position);
    for (const LayerSpec& l : spec_.layers) {
        const PartFactory& bf = get_part("block", l.block);
        BlockParts p;
        p.mixer = make_part<Mixer>("mixer", l.mixer);
        p.feed_forward = make_part<FeedForward>("feed_forward", l.feed_forward);
        for (const auto& kv : l.norms) p.norms[kv.first] = make_part<Norm>("norm", kv.second);
        std::string missing;
        for (const auto& n : bf.norm_names)
            if (!p.norms.count(n)) missing += (missing.empty() ? "" : ", ") + n;
        if (!missing.empty()) throw ConfigError("block '" + l.block + "' needs norms " + missing);
        p.width = spec_.width;
        if (!bf.make_block) throw ConfigError("part kind '" + l.block + "' is not a block");
        blocks_.push_back(bf.make_block(std::move(p)));
    }
    final_norm_ = make_part<Norm>("norm", spec_.final_norm);
    head_ = make_part<Head>("head", spec_.head);
    for (const LayerCall& c : spec_.schedule)
        if (c.layer < 0 || c.layer >= (int)blocks_.size())
            throw ConfigError("run order names layer " + std::to_string(c.layer) + ", the model has " + std::to_string(blocks_.size()));
}

std::vector<Model::PartRef> Model::parts() const {
    std::vector<PartRef> out;
    out.push_back({embedding_.get(), &spec_.embedding});
    out.push_back({position_.get(), &spec_.position});
    for (size_t i = 0; i < blocks_.size(); i++) {
        const LayerSpec& l = spec_.layers[i];
        out.push_back({&blocks_[i]->mixer(), &l.mixer});
        out.push_back({&blocks_[i]->feed_forward(), &l.feed_forward});
        for (auto& kv : blocks_[i]->norms()) out.push_back({kv.second.get(), &l.norms.at(kv.first)});
    }
    out.push_back({final_norm_.get(), &spec_.final_norm});
    out.push_back({head_.get(), &spec_.head});
    return out;
}

TensorRequests Model::tensor_requests() const {
    TensorRequests out;
    for (const PartRef& p : parts())
        for (const auto& kv : p.part->requests()) {
            auto name = p.spec->tensors.find(kv.first);
            if (name == p.spec->tensors.end())
                throw ConfigError(p.spec->kind + ": the model description names no tensor for '" + kv.first + "'");
            auto hit = out.find(name->second);
            if (hit != out.end() && hit->second.shape != kv.second.shape)
                throw ConfigError("tensor '" + name->second + "' is requested with two shapes");
            out[name->second] = kv.second;
        }
    return out;
}

void Model::bind(const TensorMap& tensors, DType dtype) {
    if (dtype != DType::F32 && dtype != DType::BF16) throw ValueError("compute dtype must be float32 or bfloat16");
    dtype_ = dtype;
    for (const PartRef& p : parts()) {
        TensorMap local;
        for (const auto& kv : p.part->requests()) {
            auto it = tensors.find(p.spec->tensors.at(kv.first));
            if (it == tensors.end()) throw ConfigError("tensor '" + p.spec->tensors.at(kv.first) + "' was not loaded");
            local[kv.first] = it->second;
        }
        if (p.part == head_.get()) head_->bind_head(local, dtype, head_->tied() ? embedding_->table() : nullptr);
        else p.part->bind(local, dtype);
    }
    bound_ = true;
}

std::vector<CacheSpec> Model::cache_specs() const {
    std::vector<CacheSpec> specs((size_t)spec_.n_caches());
    std::vector<char> seen(specs.size(), 0);
    for (const LayerCall& c : spec_.schedule) {
        const CacheSpec s = blocks_[(size_t)c.layer]->mixer().cache_spec();
        if (seen[(size_t)c.cache] && specs[(size_t)c.cache] != s)
            throw ConfigError("cache entry " + std::to_string(c.cache) + " is used by layers with different needs");
        specs[(size_t)c.cache] = s;
        seen[(size_t)c.cache] = 1;
    }
    return specs;
}

bool Model::graph_safe() const {
    for (const PartRef& p : parts())
        if (!p.part->graph_safe()) return false;
    return true;
}

size_t Model::weight_bytes() const {
    size_t total = head_->weight_bytes() + final_norm_->weight_bytes();
    for (const LayerCall& c : spec_.schedule) {
        Block& b = *blocks_[(size_t)c.layer];
        total += b.mixer().weight_bytes() + b.feed_forward().weight_bytes();
        for (auto& kv : b.norms()) total += kv.second->weight_bytes();
    }
    return total;
}

Tensor Model::forward(StepContext& ctx) {
    Workspace& ws = *ctx.workspace;
    ctx.position = position_.get();
    Tensor x = ws.get("stream", ctx.n_tokens, spec_.width, DType::F32);
    embedding_->forward(ctx, x);
    for (const LayerCall& c : spec_.schedule) blocks_[(size_t)c.layer]->forward(ctx, x, c);
    Tensor logits = ws.get("logits", ctx.n_rows, spec_.vocab_size, DType::F32);
    if (ctx.n_rows) {
        Tensor y = ws.get("final_normed", ctx.n_rows, spec_.width, ctx.compute_dtype);
        final_norm_->forward(ctx, x, y, ctx.logit_rows, ctx.n_rows);
        head_->forward(ctx, y, logits);
    }
    return logits;
}

std::unique_ptr<Model> load_model(const std::string& model_dir, DType dtype) {
    std::shared_ptr<ModelConfig> config = load_config(model_dir);
    ModelSpec spec = describe(*config);
    std::unique_ptr<Model> model(new Model(std::move(spec)));
    const TensorMap tensors = load_weights(model_dir, model->tensor_requests(), model->spec().name_prefixes, model->spec().ignored_tensors);
    model->bind(tensors, dtype);
    model->set_config(std::move(config));
    return model;
}

std::string write_random_model(const ModelConfig& config, const std::string& out_dir, uint64_t seed, StoreDType store) {
    config.validate();
    Model model(describe(config));
    const TensorMap tensors = random_tensors(model.tensor_requests(), seed, store);
    save_config(config, out_dir);
    write_safetensors(out_dir + "/" + kWeightFile, tensors);
    return out_dir;
}

}  // namespace sandy
