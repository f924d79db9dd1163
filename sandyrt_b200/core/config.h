// Typed model configuration and the architecture registry.
//
// A configuration is a typed object whose fields are the architecture's own config.json keys.
// Every size and constant the model code uses comes from one of these fields; the model code
// holds no literals of its own.  (The reference keeps every size as a literal in its model
// program, src/models/gpt2_small.sandy.go:7,18,36,52, and picks a model by an if/else chain over
// an `architecture` string, src/server/Model.cpp:100-160; here both are data and an open table.)
#pragma once

#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "json.h"
#include "spec.h"

namespace sandy {

// Base of every architecture's typed configuration.
class ModelConfig {
public:
    virtual ~ModelConfig() = default;
    virtual std::string architecture() const = 0;     // the registry key ("GPT2LMHeadModel", ...)
    virtual Json to_json() const = 0;                 // what config.json holds
    virtual void validate() const = 0;                // throws ConfigError
};

// GPT-2's config.json.  Keys and defaults follow the reference's artefact
// experiments/gpt2_small/config.json:1-30 (n_layer :16, n_embd :14, n_head :15, n_positions :17,
// vocab_size :30, layer_norm_epsilon :11, activation_function :2, architectures :3-5, bos/eos
// :7,9).  Keys that file does not carry get the architecture's usual defaults: n_inner (null ->
// 4 * n_embd), scale_attn_weights (true), scale_attn_by_inverse_layer_idx (false),
// tie_word_embeddings (true).
class GPT2Config : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "GPT2LMHeadModel";
    int64_t n_layer = 0, n_embd = 0, n_head = 0, n_positions = 0, vocab_size = 0;
    std::optional<int64_t> n_inner;
    double layer_norm_epsilon = 1e-5;
    std::string activation_function = "gelu_new";
    bool scale_attn_weights = true;
    bool scale_attn_by_inverse_layer_idx = false;
    bool tie_word_embeddings = true;
    std::optional<int64_t> bos_token_id, eos_token_id;

    int64_t head_dim() const { return n_embd / n_head; }
    int64_t inner_dim() const { return n_inner ? *n_inner : 4 * n_embd; }

    static GPT2Config from_json(const Json& raw);     // type checks only; call validate() for the sizes
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
};

// A configuration of an architecture defined outside this library: its normalised config.json
// as the architecture's own `parse` returned it.
class ForeignConfig : public ModelConfig {
public:
    ForeignConfig(std::string arch, Json normalised) : arch_(std::move(arch)), json_(std::move(normalised)) {}
    std::string architecture() const override { return arch_; }
    Json to_json() const override { return json_; }
    void validate() const override {}
private:
    std::string arch_;
    Json json_;
};

struct Architecture {
    std::string name;
    // raw config.json -> typed configuration (type checks; throws ConfigError)
    std::function<std::unique_ptr<ModelConfig>(const Json&)> parse;
    // the parts of every layer, the run order and the tensor names
    std::function<ModelSpec(const ModelConfig&)> describe;
};

void register_architecture(Architecture arch);
const Architecture& get_architecture(const std::string& name);     // unknown -> ConfigError listing the known ones
std::vector<std::string> architectures();

Json read_config_json(const std::string& model_dir);
std::string architecture_name(const Json& raw);                    // architectures[0]
std::unique_ptr<ModelConfig> parse_config(const Json& raw);         // chosen by the registry, validated
std::unique_ptr<ModelConfig> load_config(const std::string& model_dir);
std::string save_config(const ModelConfig& cfg, const std::string& model_dir);
ModelSpec describe(const ModelConfig& cfg);

ModelSpec describe_gpt2(const GPT2Config& cfg);

}  // namespace sandy
