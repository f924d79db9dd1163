// Model: the parts of a ModelSpec built, bound to weights, and run over a step's tokens.
//
// Building is three stages, each usable on its own:
//   Model(spec)                 part objects from the spec (no weights, no device)
//   model.tensor_requests()     every tensor the model wants, by name in the weight file
//   model.bind(tensors, dtype)  hand the loaded tensors to the parts and move them to the device
// `load_model(dir, dtype)` does all three from a model folder, choosing the architecture by the
// folder's config.json.
//
// `forward` runs the layer calls of the spec's schedule in order over the residual stream and
// returns float32 logits at the wanted rows only (the reference computes every row,
// src/models/gpt2_small.sandy.go:56-57; here the final norm and the head see just the rows that
// were asked for).
#pragma once

#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "config.h"
#include "parts.h"
#include "spec.h"

namespace sandy {

class Model {
public:
    explicit Model(ModelSpec spec);
    const ModelSpec& spec() const { return spec_; }
    TensorRequests tensor_requests() const;                // name in the weight file -> expected shape
    void bind(const TensorMap& tensors, DType dtype);      // the current CUDA device receives the weights
    bool bound() const { return bound_; }
    DType compute_dtype() const { return dtype_; }
    std::vector<CacheSpec> cache_specs() const;            // one per cache entry of the run order
    bool graph_safe() const;                               // whether every part may be recorded in a CUDA graph
    std::optional<int64_t> max_positions() const { return position_->max_positions(); }
    size_t weight_bytes() const;                           // bytes of weights a decode step reads once
    Tensor forward(StepContext& ctx);                      // float32 logits [wanted rows, vocab] (workspace memory)
    const ModelConfig* config() const { return config_.get(); }
    void set_config(std::shared_ptr<ModelConfig> c) { config_ = std::move(c); }

private:
    struct PartRef { Part* part; const PartSpec* spec; };
    std::vector<PartRef> parts() const;
    ModelSpec spec_;
    std::unique_ptr<Embedding> embedding_;
    std::unique_ptr<PositionEncoding> position_;
    std::vector<std::unique_ptr<Block>> blocks_;
    std::unique_ptr<Norm> final_norm_;
    std::unique_ptr<Head> head_;
    bool bound_ = false;
    DType dtype_ = DType::F32;
    std::shared_ptr<ModelConfig> config_;
};

std::unique_ptr<Model> load_model(const std::string& model_dir, DType dtype);

// Random-weights mode: create `out_dir` with config.json and a model.safetensors of seeded random
// weights stored as `store` (F32, BF16 or F16).
std::string write_random_model(const ModelConfig& config, const std::string& out_dir, uint64_t seed, StoreDType store);

}  // namespace sandy
