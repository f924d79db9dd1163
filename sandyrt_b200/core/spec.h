// ModelSpec: an architecture described as data.
//
// An architecture's `describe(config)` returns one ModelSpec.  It lists, for every layer, which
// mixer, feed-forward and norms the layer is made of (a part kind plus its sizes and constants,
// chosen layer by layer), how the block arranges them, the names of the tensors in the weight
// file, and the order in which layers run.  The engine builds the model from this description
// alone; no part is told which model it is in.  A description can be written as JSON and read
// back, which is how architectures defined outside this library (the Python binding) hand
// theirs over.
//
// The reference writes the same information as a program in its own language
// (src/models/gpt2_small.sandy.go:1-59: functions for attention, MLP and block, a loop over
// `range(12)`, weight names through nested `weight_scope`s).
#pragma once

#include <map>
#include <optional>
#include <string>
#include <vector>

#include "json.h"

namespace sandy {

// One part: its registered kind, its sizes and constants, and where its tensors live.
// `tensors` maps the part's own tensor names ("qkv.weight") to names in the weight file
// ("h.3.attn.c_attn.weight").
struct PartSpec {
    std::string kind;
    Json params = Json::object();
    std::map<std::string, std::string> tensors;

    // typed access to params, with errors that name the part kind and the key
    int64_t get_int(const std::string& key) const;
    int64_t get_int(const std::string& key, int64_t fallback) const;
    double get_double(const std::string& key) const;
    double get_double(const std::string& key, double fallback) const;
    bool get_bool(const std::string& key, bool fallback) const;
    std::string get_string(const std::string& key) const;
    std::string get_string(const std::string& key, const std::string& fallback) const;
    std::optional<int64_t> get_optional_int(const std::string& key) const;   // absent, null or 0 -> nullopt
};

// One layer: a block arrangement over a mixer, a feed-forward and their norms.
struct LayerSpec {
    std::string block;                       // registered block kind, e.g. "pre_norm"
    PartSpec mixer;
    PartSpec feed_forward;
    std::map<std::string, PartSpec> norms;   // the block kind names the norms it wants
};

// One entry of the run order.  `layer` indexes ModelSpec::layers (a layer may be named by several
// calls: shared weights).  `cache` names the cache entry the mixer works on.  With `write_cache`
// false the call appends nothing and only reads what an earlier call of this step wrote there (a
// layer that reads another layer's keys and values).
struct LayerCall {
    int layer = 0;
    int cache = 0;
    bool write_cache = true;
};

struct ModelSpec {
    std::string architecture;
    int64_t width = 0;
    int64_t vocab_size = 0;
    std::optional<int64_t> max_positions;    // nullopt when the position encoding sets no limit
    PartSpec embedding;
    PartSpec position;
    std::vector<LayerSpec> layers;
    std::vector<LayerCall> schedule;
    PartSpec final_norm;
    PartSpec head;
    // All names in `tensors` are written without these prefixes; a file may carry one of them on
    // every name (HF stores GPT-2 both as "transformer.h.0..." and "h.0...").
    std::vector<std::string> name_prefixes{""};
    // Regular expressions for tensors that a file may hold and the model does not read.
    std::vector<std::string> ignored_tensors;
    std::optional<int64_t> eos_token_id;

    int n_caches() const;
};

Json to_json(const PartSpec& p);
Json to_json(const ModelSpec& s);
PartSpec part_spec_from_json(const Json& j);
ModelSpec model_spec_from_json(const Json& j);

}  // namespace sandy
