#include "spec.h"

#include <algorithm>

#include "errors.h"

namespace sandy {

static const Json& need(const PartSpec& p, const std::string& key) {
    const Json* v = p.params.find(key);
    if (!v || v->is_null()) throw ConfigError(p.kind + ": parameter '" + key + "' is required");
    return *v;
}

int64_t PartSpec::get_int(const std::string& key) const {
    try { return need(*this, key).as_int(); }
    catch (const ValueError& e) { throw ConfigError(kind + ": parameter '" + key + "': " + e.what()); }
}
int64_t PartSpec::get_int(const std::string& key, int64_t fallback) const {
    const Json* v = params.find(key);
    return (!v || v->is_null()) ? fallback : get_int(key);
}
double PartSpec::get_double(const std::string& key) const {
    try { return need(*this, key).as_double(); }
    catch (const ValueError& e) { throw ConfigError(kind + ": parameter '" + key + "': " + e.what()); }
}
double PartSpec::get_double(const std::string& key, double fallback) const {
    const Json* v = params.find(key);
    return (!v || v->is_null()) ? fallback : get_double(key);
}
bool PartSpec::get_bool(const std::string& key, bool fallback) const {
    const Json* v = params.find(key);
    if (!v || v->is_null()) return fallback;
    if (v->is_bool()) return v->as_bool();
    if (v->is_int()) return v->as_int() != 0;
    throw ConfigError(kind + ": parameter '" + key + "' must be a bool");
}
std::string PartSpec::get_string(const std::string& key) const {
    try { return need(*this, key).as_string(); }
    catch (const ValueError& e) { throw ConfigError(kind + ": parameter '" + key + "': " + e.what()); }
}
std::string PartSpec::get_string(const std::string& key, const std::string& fallback) const {
    const Json* v = params.find(key);
    return (!v || v->is_null()) ? fallback : get_string(key);
}
std::optional<int64_t> PartSpec::get_optional_int(const std::string& key) const {
    const Json* v = params.find(key);
    if (!v || v->is_null()) return std::nullopt;
    const int64_t n = get_int(key);
    if (n == 0) return std::nullopt;
    return n;
}

int ModelSpec::n_caches() const {
    int n = 0;
    for (const auto& c : schedule) n = std::max(n, c.cache + 1);
    return n;
}

Json to_json(const PartSpec& p) {
    Json j = Json::object();
    j["kind"] = p.kind;
    j["params"] = p.params.is_object() ? p.params : Json::object();
    Json t = Json::object();
    for (const auto& kv : p.tensors) t[kv.first] = kv.second;
    j["tensors"] = t;
    return j;
}

Json to_json(const ModelSpec& s) {
    Json j = Json::object();
    j["architecture"] = s.architecture;
    j["width"] = (long long)s.width;
    j["vocab_size"] = (long long)s.vocab_size;
    j["max_positions"] = s.max_positions ? Json((long long)*s.max_positions) : Json();
    j["embedding"] = to_json(s.embedding);
    j["position"] = to_json(s.position);
    Json layers = Json::array();
    for (const auto& l : s.layers) {
        Json lj = Json::object();
        lj["block"] = l.block;
        lj["mixer"] = to_json(l.mixer);
        lj["feed_forward"] = to_json(l.feed_forward);
        Json norms = Json::object();
        for (const auto& kv : l.norms) norms[kv.first] = to_json(kv.second);
        lj["norms"] = norms;
        layers.push(lj);
    }
    j["layers"] = layers;
    Json sched = Json::array();
    for (const auto& c : s.schedule) {
        Json cj = Json::object();
        cj["layer"] = c.layer;
        cj["cache"] = c.cache;
        cj["write_cache"] = c.write_cache;
        sched.push(cj);
    }
    j["schedule"] = sched;
    j["final_norm"] = to_json(s.final_norm);
    j["head"] = to_json(s.head);
    Json prefixes = Json::array();
    for (const auto& p : s.name_prefixes) prefixes.push(p);
    j["name_prefixes"] = prefixes;
    Json ignored = Json::array();
    for (const auto& p : s.ignored_tensors) ignored.push(p);
    j["ignored_tensors"] = ignored;
    j["eos_token_id"] = s.eos_token_id ? Json((long long)*s.eos_token_id) : Json();
    return j;
}

PartSpec part_spec_from_json(const Json& j) {
    PartSpec p;
    try {
        p.kind = j.at("kind").as_string();
        if (const Json* params = j.find("params"))
            if (params->is_object()) p.params = *params;
        if (const Json* t = j.find("tensors"))
            if (t->is_object())
                for (const auto& m : t->members()) p.tensors[m.first] = m.second.as_string();
    } catch (const ValueError& e) {
        throw ConfigError(std::string("model description: a part is malformed: ") + e.what());
    }
    return p;
}

ModelSpec model_spec_from_json(const Json& j) {
    ModelSpec s;
    try {
        s.architecture = j.at("architecture").as_string();
        s.width = j.at("width").as_int();
        s.vocab_size = j.at("vocab_size").as_int();
        if (const Json* m = j.find("max_positions"))
            if (!m->is_null()) s.max_positions = m->as_int();
        s.embedding = part_spec_from_json(j.at("embedding"));
        s.position = part_spec_from_json(j.at("position"));
        for (const Json& lj : j.at("layers").items()) {
            LayerSpec l;
            l.block = lj.at("block").as_string();
            l.mixer = part_spec_from_json(lj.at("mixer"));
            l.feed_forward = part_spec_from_json(lj.at("feed_forward"));
            for (const auto& m : lj.at("norms").members()) l.norms[m.first] = part_spec_from_json(m.second);
            s.layers.push_back(std::move(l));
        }
        for (const Json& cj : j.at("schedule").items()) {
            LayerCall c;
            c.layer = (int)cj.at("layer").as_int();
            c.cache = (int)cj.at("cache").as_int();
            if (const Json* w = cj.find("write_cache")) c.write_cache = w->as_bool();
            s.schedule.push_back(c);
        }
        s.final_norm = part_spec_from_json(j.at("final_norm"));
        s.head = part_spec_from_json(j.at("head"));
        if (const Json* p = j.find("name_prefixes")) {
            s.name_prefixes.clear();
            for (const Json& v : p->items()) s.name_prefixes.push_back(v.as_string());
            if (s.name_prefixes.empty()) s.name_prefixes.push_back("");
        }
        if (const Json* p = j.find("ignored_tensors"))
            for (const Json& v : p->items()) s.ignored_tensors.push_back(v.as_string());
        if (const Json* e = j.find("eos_token_id"))
            if (!e->is_null()) s.eos_token_id = e->as_int();
    } catch (const ValueError& e) {
        throw ConfigError(std::string("model description is malformed: ") + e.what());
    }
    return s;
}

}  // namespace sandy
