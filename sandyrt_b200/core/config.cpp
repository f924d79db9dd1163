#include "config.h"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "errors.h"

namespace sandy {

// ---- reading typed keys ---------------------------------------------------------------------
namespace {

const Json* present(const Json& raw, const std::string& key) {
    const Json* v = raw.find(key);
    return (v && !v->is_null()) ? v : nullptr;
}

[[noreturn]] void wrong_type(const std::string& key, const char* want, const Json& v) {
    throw ConfigError("config.json: key '" + key + "' must be " + want + ", got " + v.type_name() + " " + v.dump());
}

int64_t req_int(const Json& raw, const std::string& key) {
    const Json* v = present(raw, key);
    if (!v) throw ConfigError("config.json: required key '" + key + "' is missing");
    if (!v->is_int()) wrong_type(key, "int", *v);
    return v->as_int();
}
std::optional<int64_t> opt_int(const Json& raw, const std::string& key) {
    const Json* v = present(raw, key);
    if (!v) return std::nullopt;
    if (!v->is_int()) wrong_type(key, "int", *v);
    return v->as_int();
}
double opt_float(const Json& raw, const std::string& key, double fallback) {
    const Json* v = present(raw, key);
    if (!v) return fallback;
    if (!v->is_number()) wrong_type(key, "float", *v);
    return v->as_double();
}
std::string opt_str(const Json& raw, const std::string& key, const std::string& fallback) {
    const Json* v = present(raw, key);
    if (!v) return fallback;
    if (!v->is_string()) wrong_type(key, "str", *v);
    return v->as_string();
}
bool opt_bool(const Json& raw, const std::string& key, bool fallback) {
    const Json* v = present(raw, key);
    if (!v) return fallback;
    if (!v->is_bool()) wrong_type(key, "bool", *v);
    return v->as_bool();
}

}  // namespace

GPT2Config GPT2Config::from_json(const Json& raw) {
    if (!raw.is_object()) throw ConfigError("config.json: top level must be a JSON object");
    GPT2Config c;
    std::optional<int64_t> n_pos = opt_int(raw, "n_positions");
    if (!n_pos) n_pos = req_int(raw, "n_ctx");          // `n_ctx` is the legacy duplicate of n_positions (config.json:13)
    c.n_layer = req_int(raw, "n_layer");
    c.n_embd = req_int(raw, "n_embd");
    c.n_head = req_int(raw, "n_head");
    c.n_positions = *n_pos;
    c.vocab_size = req_int(raw, "vocab_size");
    c.n_inner = opt_int(raw, "n_inner");
    c.layer_norm_epsilon = opt_float(raw, "layer_norm_epsilon", 1e-5);
    c.activation_function = opt_str(raw, "activation_function", "gelu_new");
    c.scale_attn_weights = opt_bool(raw, "scale_attn_weights", true);
    c.scale_attn_by_inverse_layer_idx = opt_bool(raw, "scale_attn_by_inverse_layer_idx", false);
    c.tie_word_embeddings = opt_bool(raw, "tie_word_embeddings", true);
    c.bos_token_id = opt_int(raw, "bos_token_id");
    c.eos_token_id = opt_int(raw, "eos_token_id");
    return c;
}

Json GPT2Config::to_json() const {
    Json j = Json::object();
    j["activation_function"] = activation_function;
    Json archs = Json::array();
    archs.push(kArchitecture);
    j["architectures"] = archs;
    j["bos_token_id"] = bos_token_id ? Json((long long)*bos_token_id) : Json();
    j["eos_token_id"] = eos_token_id ? Json((long long)*eos_token_id) : Json();
    j["layer_norm_epsilon"] = layer_norm_epsilon;
    j["model_type"] = "gpt2";
    j["n_embd"] = (long long)n_embd;
    j["n_head"] = (long long)n_head;
    j["n_inner"] = n_inner ? Json((long long)*n_inner) : Json();
    j["n_layer"] = (long long)n_layer;
    j["n_positions"] = (long long)n_positions;
    j["scale_attn_by_inverse_layer_idx"] = scale_attn_by_inverse_layer_idx;
    j["scale_attn_weights"] = scale_attn_weights;
    j["tie_word_embeddings"] = tie_word_embeddings;
    j["vocab_size"] = (long long)vocab_size;
    return j;
}

void GPT2Config::validate() const {
    const std::pair<const char*, int64_t> sizes[] = {{"n_layer", n_layer}, {"n_embd", n_embd}, {"n_head", n_head},
                                                    {"n_positions", n_positions}, {"vocab_size", vocab_size}};
    for (const auto& s : sizes)
        if (s.second <= 0)
            throw ConfigError(std::string("config.json: '") + s.first + "' must be > 0, got " + std::to_string(s.second));
    if (n_inner && *n_inner <= 0) throw ConfigError("config.json: 'n_inner' must be > 0, got " + std::to_string(*n_inner));
    if (n_embd % n_head != 0)
        throw ConfigError("config.json: n_embd (" + std::to_string(n_embd) + ") is not divisible by n_head (" +
                          std::to_string(n_head) + ")");
    if (activation_function != "gelu_new" && activation_function != "gelu")
        throw ConfigError("config.json: activation_function '" + activation_function +
                          "' is not one of ['gelu_new', 'gelu']");
    if (!(layer_norm_epsilon > 0.0)) throw ConfigError("config.json: layer_norm_epsilon must be > 0");
    const std::pair<const char*, std::optional<int64_t>> ids[] = {{"bos_token_id", bos_token_id},
                                                                   {"eos_token_id", eos_token_id}};
    for (const auto& t : ids)
        if (t.second && !(*t.second >= 0 && *t.second < vocab_size))
            throw ConfigError(std::string("config.json: ") + t.first + "=" + std::to_string(*t.second) +
                              " is outside the vocabulary");
}

// ---- GPT-2 as a ModelSpec -----------------------------------------------------------------------
// Structure: src/models/gpt2_small.sandy.go:1-59 of the reference (token + position embedding,
// pre-LayerNorm blocks of fused-QKV causal attention and a gelu MLP, final LayerNorm, output head
// tied to the token table).  Tensor names are those of the HF checkpoint the reference converts
// from (scripts/run_gpt2.py:160-189): `wte.weight`, `wpe.weight`, `h.N.ln_1.*`,
// `h.N.attn.c_attn.*`, `h.N.attn.c_proj.*`, `h.N.ln_2.*`, `h.N.mlp.c_fc.*`, `h.N.mlp.c_proj.*`,
// `ln_f.*`, with or without a `transformer.` prefix.  Linear weights are in Conv1D layout
// [in, out] and are used as stored.  Every number below comes from the GPT2Config.
ModelSpec describe_gpt2(const GPT2Config& cfg) {
    const int64_t E = cfg.n_embd, H = cfg.n_head, D = cfg.head_dim();
    ModelSpec s;
    s.architecture = cfg.architecture();
    s.width = E;
    s.vocab_size = cfg.vocab_size;
    s.max_positions = cfg.n_positions;
    auto norm = [&](const std::string& base) {
        PartSpec p;
        p.kind = "layernorm";
        p.params["width"] = (long long)E;
        p.params["eps"] = cfg.layer_norm_epsilon;
        p.params["bias"] = true;
        p.tensors = {{"weight", base + ".weight"}, {"bias", base + ".bias"}};
        return p;
    };
    for (int64_t i = 0; i < cfg.n_layer; i++) {
        const std::string p = "h." + std::to_string(i) + ".";
        // scale_attn_weights: scores * 1/sqrt(D); scale_attn_by_inverse_layer_idx: also / (i+1).
        // The reference's attention takes this as its `scale` attribute
        // (src/core/TensorCalc.cpp:1236-1237: default 1/sqrt(D) when none is given).
        double scale = 1.0;
        if (cfg.scale_attn_weights) scale /= std::sqrt((double)D);
        if (cfg.scale_attn_by_inverse_layer_idx) scale /= (double)(i + 1);
        LayerSpec l;
        l.block = "pre_norm";
        l.mixer.kind = "causal_attention";
        l.mixer.params["width"] = (long long)E;
        l.mixer.params["n_heads"] = (long long)H;
        l.mixer.params["n_kv_heads"] = (long long)H;
        l.mixer.params["head_dim"] = (long long)D;
        l.mixer.params["scale"] = scale;
        l.mixer.params["window"] = Json();
        l.mixer.params["bias"] = true;
        l.mixer.params["weight_layout"] = "in_out";
        l.mixer.tensors = {{"qkv.weight", p + "attn.c_attn.weight"}, {"qkv.bias", p + "attn.c_attn.bias"},
                           {"out.weight", p + "attn.c_proj.weight"}, {"out.bias", p + "attn.c_proj.bias"}};
        l.feed_forward.kind = "dense_mlp";
        l.feed_forward.params["width"] = (long long)E;
        l.feed_forward.params["inner"] = (long long)cfg.inner_dim();
        l.feed_forward.params["activation"] = cfg.activation_function;
        l.feed_forward.params["bias"] = true;
        l.feed_forward.params["weight_layout"] = "in_out";
        l.feed_forward.tensors = {{"up.weight", p + "mlp.c_fc.weight"}, {"up.bias", p + "mlp.c_fc.bias"},
                                  {"down.weight", p + "mlp.c_proj.weight"}, {"down.bias", p + "mlp.c_proj.bias"}};
        l.norms["mixer"] = norm(p + "ln_1");
        l.norms["feed_forward"] = norm(p + "ln_2");
        s.layers.push_back(std::move(l));
        s.schedule.push_back(LayerCall{(int)i, (int)i, true});
    }
    s.embedding.kind = "token_embedding";
    s.embedding.params["vocab_size"] = (long long)cfg.vocab_size;
    s.embedding.params["width"] = (long long)E;
    s.embedding.tensors = {{"weight", "wte.weight"}};
    s.position.kind = "learned_absolute";
    s.position.params["width"] = (long long)E;
    s.position.params["max_positions"] = (long long)cfg.n_positions;
    s.position.tensors = {{"weight", "wpe.weight"}};
    s.final_norm = norm("ln_f");
    s.head.kind = "output_head";
    s.head.params["vocab_size"] = (long long)cfg.vocab_size;
    s.head.params["width"] = (long long)E;
    s.head.params["tied"] = cfg.tie_word_embeddings;
    if (!cfg.tie_word_embeddings) s.head.tensors = {{"weight", "lm_head.weight"}};
    s.name_prefixes = {"", "transformer."};
    s.ignored_tensors = {R"(^h\.\d+\.attn\.(bias|masked_bias)$)"};       // stored causal-mask buffers of old checkpoints
    if (cfg.tie_word_embeddings) s.ignored_tensors.push_back(R"(^lm_head\.weight$)");   // a stored copy of the tied table
    s.eos_token_id = cfg.eos_token_id;
    return s;
}

// ---- registry -------------------------------------------------------------------------------------
namespace {

std::map<std::string, Architecture>& table() {
    static std::map<std::string, Architecture> t;
    static std::once_flag once;
    std::call_once(once, [] {
        Architecture gpt2;
        gpt2.name = GPT2Config::kArchitecture;
        gpt2.parse = [](const Json& raw) { return std::unique_ptr<ModelConfig>(new GPT2Config(GPT2Config::from_json(raw))); };
        gpt2.describe = [](const ModelConfig& c) {
            const auto* g = dynamic_cast<const GPT2Config*>(&c);
            if (!g) throw ConfigError("GPT2LMHeadModel was given another architecture's configuration");
            return describe_gpt2(*g);
        };
        t[gpt2.name] = std::move(gpt2);
    });
    return t;
}
std::mutex& table_lock() { static std::mutex m; return m; }

}  // namespace

void register_architecture(Architecture arch) {
    auto& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    t[arch.name] = std::move(arch);
}

const Architecture& get_architecture(const std::string& name) {
    auto& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    auto it = t.find(name);
    if (it == t.end()) {
        std::string known;
        for (const auto& kv : t) known += (known.empty() ? "'" : ", '") + kv.first + "'";
        throw ConfigError("unknown model architecture: '" + name + "'; registered: [" + known + "]");
    }
    return it->second;
}

std::vector<std::string> architectures() {
    auto& t = table();
    std::lock_guard<std::mutex> g(table_lock());
    std::vector<std::string> out;
    for (const auto& kv : t) out.push_back(kv.first);
    return out;
}

Json read_config_json(const std::string& model_dir) {
    const std::string path = model_dir + "/config.json";
    std::ifstream f(path, std::ios::binary);
    if (!f) throw ConfigError("no config.json in model folder '" + model_dir + "'");
    std::stringstream ss;
    ss << f.rdbuf();
    Json raw;
    try {
        raw = Json::parse(ss.str());
    } catch (const ValueError& e) {
        throw ConfigError(path + ": not valid JSON (" + e.what() + ")");
    }
    if (!raw.is_object()) throw ConfigError(path + ": top level must be a JSON object");
    return raw;
}

std::string architecture_name(const Json& raw) {
    const Json* a = raw.find("architectures");
    if (!a || !a->is_array() || a->size() == 0 || !a->items()[0].is_string())
        throw ConfigError("config.json: 'architectures' must be a non-empty list of names");
    return a->items()[0].as_string();
}

std::unique_ptr<ModelConfig> parse_config(const Json& raw) {
    const Architecture& arch = get_architecture(architecture_name(raw));
    std::unique_ptr<ModelConfig> cfg = arch.parse(raw);
    cfg->validate();
    return cfg;
}

std::unique_ptr<ModelConfig> load_config(const std::string& model_dir) { return parse_config(read_config_json(model_dir)); }

static void make_dirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); i++) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty()) ::mkdir(cur.c_str(), 0777);
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
}

std::string save_config(const ModelConfig& cfg, const std::string& model_dir) {
    make_dirs(model_dir);
    const std::string path = model_dir + "/config.json";
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) throw ConfigError("cannot write " + path);
    f << cfg.to_json().dump(2) << "\n";
    return path;
}

ModelSpec describe(const ModelConfig& cfg) { return get_architecture(cfg.architecture()).describe(cfg); }

}  // namespace sandy
