#include "weights.h"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <set>

#include "errors.h"
#include "json.h"
#include "pattern.h"

namespace sandy {

namespace {

std::string shape_text(const std::vector<int64_t>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); i++) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}
Json shape_json(const std::vector<int64_t>& s) {
    Json a = Json::array();
    for (int64_t d : s) a.push((long long)d);
    return a;
}

// The prefix under which the file stores the model's tensors: the candidate that makes the most
// wanted names resolve.
std::string detect_prefix(const SafetensorsFile& f, const TensorRequests& wanted, const std::vector<std::string>& prefixes) {
    std::string best = prefixes.empty() ? std::string() : prefixes[0];
    long best_hits = -1;
    for (const auto& p : prefixes) {
        long hits = 0;
        for (const auto& kv : wanted)
            if (f.contains(p + kv.first)) hits++;
        if (hits > best_hits) { best = p; best_hits = hits; }
    }
    return best;
}

bool file_exists(const std::string& path) {
    struct stat st;
    return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

}  // namespace

TensorMap load_weights(const std::string& model_dir, const TensorRequests& requests,
                       const std::vector<std::string>& prefixes, const std::vector<std::string>& ignored) {
    const std::string path = model_dir + "/" + kWeightFile;
    if (!file_exists(path) && file_exists(path + ".index.json"))
        throw WeightFileError(model_dir + ": sharded weight files (model.safetensors.index.json) are not supported");
    SafetensorsFile f(path);
    const std::string prefix = detect_prefix(f, requests, prefixes.empty() ? std::vector<std::string>{""} : prefixes);
    std::vector<Pattern> ignore_res;
    for (const auto& p : ignored) ignore_res.emplace_back(p);

    std::vector<std::string> missing, unexpected;
    struct WrongShape { std::string name; std::vector<int64_t> got, want; };
    std::vector<WrongShape> wrong_shape;
    std::vector<std::pair<std::string, std::string>> wrong_kind;
    for (const auto& kv : requests) {
        const std::string full = prefix + kv.first;
        if (!f.contains(full)) { missing.push_back(full); continue; }
        if (f.shape(full) != kv.second.shape) wrong_shape.push_back({full, f.shape(full), kv.second.shape});
        if (store_dtype_is_float(f.dtype(full)) == kv.second.integer)
            wrong_kind.emplace_back(full, store_dtype_word(f.dtype(full)));
    }
    for (const auto& full : f.names()) {
        const std::string bare = (!prefix.empty() && full.compare(0, prefix.size(), prefix) == 0) ? full.substr(prefix.size()) : full;
        if (requests.count(bare) && full == prefix + bare) continue;
        bool skip = false;
        for (const auto& r : ignore_res)
            if (r.search(bare) || r.search(full)) skip = true;
        if (!skip) unexpected.push_back(full);
    }
    if (!missing.empty() || !unexpected.empty() || !wrong_shape.empty() || !wrong_kind.empty()) {
        std::sort(missing.begin(), missing.end());
        std::sort(unexpected.begin(), unexpected.end());
        std::sort(wrong_shape.begin(), wrong_shape.end(), [](const WrongShape& a, const WrongShape& b) { return a.name < b.name; });
        std::sort(wrong_kind.begin(), wrong_kind.end());
        std::string msg = path + ": weight file does not match the model";
        auto join = [](const std::vector<std::string>& v) {
            std::string out;
            for (size_t i = 0; i < v.size(); i++) out += (i ? ", " : "") + v[i];
            return out;
        };
        Json d = Json::object();
        d["path"] = path;
        Json jm = Json::array(), ju = Json::array(), js = Json::array(), jk = Json::array();
        if (!missing.empty()) msg += "\n  missing tensors (" + std::to_string(missing.size()) + "): " + join(missing);
        if (!unexpected.empty()) msg += "\n  unexpected tensors (" + std::to_string(unexpected.size()) + "): " + join(unexpected);
        if (!wrong_shape.empty()) {
            msg += "\n  wrong shapes (" + std::to_string(wrong_shape.size()) + "): ";
            for (size_t i = 0; i < wrong_shape.size(); i++)
                msg += (i ? ", " : "") + wrong_shape[i].name + " is " + shape_text(wrong_shape[i].got) + ", expected " +
                       shape_text(wrong_shape[i].want);
        }
        if (!wrong_kind.empty()) {
            msg += "\n  wrong dtypes (" + std::to_string(wrong_kind.size()) + "): ";
            for (size_t i = 0; i < wrong_kind.size(); i++) msg += (i ? ", " : "") + wrong_kind[i].first + " is " + wrong_kind[i].second;
        }
        for (const auto& n : missing) jm.push(n);
        for (const auto& n : unexpected) ju.push(n);
        for (const auto& w : wrong_shape) {
            Json row = Json::array();
            row.push(w.name); row.push(shape_json(w.got)); row.push(shape_json(w.want));
            js.push(row);
        }
        for (const auto& w : wrong_kind) {
            Json row = Json::array();
            row.push(w.first); row.push(w.second);
            jk.push(row);
        }
        d["missing"] = jm; d["unexpected"] = ju; d["wrong_shape"] = js; d["wrong_kind"] = jk;
        throw WeightBindingError(msg, d.dump());
    }
    TensorMap out;
    for (const auto& kv : requests) out[kv.first] = f.tensor(prefix + kv.first);
    return out;
}

// ---- random weights -------------------------------------------------------------------------------
namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint64_t tensor_key(uint64_t seed, const std::string& name) {
    uint64_t h = splitmix64(seed ^ 0x53616e6479525421ull);
    for (unsigned char c : name) h = splitmix64(h ^ c);
    return h;
}

// Standard normal number `index` of the stream `key` (Box-Muller over two counter-based uniforms).
inline double normal_at(uint64_t key, uint64_t index) {
    const uint64_t a = splitmix64(key + 2 * index), b = splitmix64(key + 2 * index + 1);
    const double u1 = ((double)(a >> 11) + 1.0) / 9007199254740993.0;     // (0, 1)
    const double u2 = (double)(b >> 11) / 9007199254740992.0;             // [0, 1)
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
}

}  // namespace

TensorMap random_tensors(const TensorRequests& requests, uint64_t seed, StoreDType dtype) {
    if (dtype != StoreDType::F32 && dtype != StoreDType::BF16 && dtype != StoreDType::F16)
        throw ValueError("random weights are stored as float32, bfloat16 or float16");
    TensorMap out;
    for (const auto& kv : requests) {
        const TensorRequest& req = kv.second;
        HostTensor t;
        t.shape = req.shape;
        const int64_t n = t.numel();
        if (req.integer) {
            t.dtype = StoreDType::I32;
            auto buf = std::shared_ptr<int32_t>(new int32_t[(size_t)std::max<int64_t>(n, 1)](), std::default_delete<int32_t[]>());
            t.data = buf.get();
            t.owner = buf;
            out[kv.first] = t;
            continue;
        }
        double mean = 0.0, std = 0.0;
        if (req.init == "weight") std = 0.02;
        else if (req.init == "bias") std = 0.01;
        else if (req.init == "gamma") { mean = 1.0; std = 0.02; }
        else if (req.init == "beta") std = 0.02;
        else if (req.init != "zeros") throw ValueError("tensor '" + kv.first + "': unknown init '" + req.init + "'");
        const uint64_t key = tensor_key(seed, kv.first);
        t.dtype = req.keep_32bit ? StoreDType::F32 : dtype;
        if (t.dtype == StoreDType::F32) {
            auto buf = std::shared_ptr<float>(new float[(size_t)std::max<int64_t>(n, 1)], std::default_delete<float[]>());
            for (int64_t i = 0; i < n; i++) buf.get()[i] = std == 0.0 ? (float)mean : (float)(mean + std * normal_at(key, (uint64_t)i));
            t.data = buf.get();
            t.owner = buf;
        } else {
            auto buf = std::shared_ptr<uint16_t>(new uint16_t[(size_t)std::max<int64_t>(n, 1)], std::default_delete<uint16_t[]>());
            for (int64_t i = 0; i < n; i++) {
                const float v = std == 0.0 ? (float)mean : (float)(mean + std * normal_at(key, (uint64_t)i));
                buf.get()[i] = t.dtype == StoreDType::BF16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
            }
            t.data = buf.get();
            t.owner = buf;
        }
        out[kv.first] = t;
    }
    return out;
}

// ---- conversions -----------------------------------------------------------------------------------
std::vector<float> to_f32(const HostTensor& t) {
    const int64_t n = t.numel();
    std::vector<float> out((size_t)n);
    switch (t.dtype) {
        case StoreDType::F32: std::memcpy(out.data(), t.data, (size_t)n * 4); break;
        case StoreDType::BF16: { const uint16_t* p = (const uint16_t*)t.data; for (int64_t i = 0; i < n; i++) out[i] = bf16_bits_to_f32(p[i]); break; }
        case StoreDType::F16: { const uint16_t* p = (const uint16_t*)t.data; for (int64_t i = 0; i < n; i++) out[i] = f16_bits_to_f32(p[i]); break; }
        default: throw WeightFileError("an integer tensor was asked for as floats");
    }
    return out;
}

std::vector<uint16_t> to_bf16_bits(const HostTensor& t) {
    const int64_t n = t.numel();
    std::vector<uint16_t> out((size_t)n);
    switch (t.dtype) {
        case StoreDType::BF16: std::memcpy(out.data(), t.data, (size_t)n * 2); break;
        case StoreDType::F32: { const float* p = (const float*)t.data; for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16_bits(p[i]); break; }
        case StoreDType::F16: { const uint16_t* p = (const uint16_t*)t.data; for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16_bits(f16_bits_to_f32(p[i])); break; }
        default: throw WeightFileError("an integer tensor was asked for as floats");
    }
    return out;
}

std::vector<int32_t> to_i32(const HostTensor& t) {
    const int64_t n = t.numel();
    std::vector<int32_t> out((size_t)n);
    switch (t.dtype) {
        case StoreDType::I32: std::memcpy(out.data(), t.data, (size_t)n * 4); break;
        case StoreDType::I64: { const int64_t* p = (const int64_t*)t.data; for (int64_t i = 0; i < n; i++) out[i] = (int32_t)p[i]; break; }
        case StoreDType::U8: case StoreDType::BOOL: { const uint8_t* p = (const uint8_t*)t.data; for (int64_t i = 0; i < n; i++) out[i] = p[i]; break; }
        default: throw WeightFileError("a floating-point tensor was asked for as integers");
    }
    return out;
}

}  // namespace sandy
