#include "safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "errors.h"
#include "json.h"

namespace sandy {

namespace {
struct DTypeRow { StoreDType d; const char* name; const char* word; size_t size; bool is_float; };
const DTypeRow kRows[] = {
    {StoreDType::F32, "F32", "float32", 4, true},   {StoreDType::F16, "F16", "float16", 2, true},
    {StoreDType::BF16, "BF16", "bfloat16", 2, true}, {StoreDType::I32, "I32", "int32", 4, false},
    {StoreDType::I64, "I64", "int64", 8, false},    {StoreDType::U8, "U8", "uint8", 1, false},
    {StoreDType::BOOL, "BOOL", "bool", 1, false},
};
const DTypeRow& row(StoreDType d) {
    for (const auto& r : kRows)
        if (r.d == d) return r;
    return kRows[0];
}
// A header larger than this is taken for a corrupt length field.
constexpr uint64_t kMaxHeaderBytes = 100ull * 1024 * 1024;
}  // namespace

const char* store_dtype_name(StoreDType d) { return row(d).name; }
const char* store_dtype_word(StoreDType d) { return row(d).word; }
size_t store_dtype_size(StoreDType d) { return row(d).size; }
bool store_dtype_is_float(StoreDType d) { return row(d).is_float; }
StoreDType store_dtype_from_name(const std::string& name) {
    for (const auto& r : kRows)
        if (name == r.name || name == r.word) return r.d;
    throw ValueError("unknown dtype " + name);
}

uint16_t f32_to_bf16_bits(float v) {
    uint32_t b;
    std::memcpy(&b, &v, 4);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);     // NaN stays NaN
    const uint32_t lsb = (b >> 16) & 1u;
    return (uint16_t)((b + 0x7fffu + lsb) >> 16);
}
float bf16_bits_to_f32(uint16_t h) {
    const uint32_t b = (uint32_t)h << 16;
    float v;
    std::memcpy(&v, &b, 4);
    return v;
}
float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, b;
    if (exp == 0) {
        if (man == 0) b = sign;
        else {                                   // subnormal: renormalise
            int e = -1;
            do { e++; man <<= 1; } while (!(man & 0x400u));
            b = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        b = sign | 0x7f800000u | (man << 13);
    } else {
        b = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float v;
    std::memcpy(&v, &b, 4);
    return v;
}
uint16_t f32_to_f16_bits(float v) {
    uint32_t b;
    std::memcpy(&b, &v, 4);
    const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    const uint32_t a = b & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);          // overflow (and infinity) -> infinity
    if (a < 0x33000001u) return sign;                                  // rounds to zero
    int exp = (int)(a >> 23) - 127;
    uint32_t man = (a & 0x7fffffu) | 0x800000u;
    int shift = exp < -14 ? 13 + (-14 - exp) : 13;
    uint32_t half_man = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
    uint32_t out;
    if (exp < -14) out = half_man;                                     // subnormal (a carry lands in the exponent, as it should)
    else out = ((uint32_t)(exp + 15) << 10) + (half_man - 0x400u);
    return (uint16_t)(sign | out);
}

struct SafetensorsFile::Mapping {
    void* base = nullptr;
    size_t size = 0;
    ~Mapping() {
        if (base && base != MAP_FAILED) ::munmap(base, size);
    }
};

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    struct stat st;
    if (::stat(path.c_str(), &st) != 0 || !S_ISREG(st.st_mode)) throw WeightFileError("weight file not found: " + path);
    const uint64_t size = (uint64_t)st.st_size;
    if (size < 8) throw WeightFileError(path + ": " + std::to_string(size) + " bytes is too short for a safetensors file");
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw WeightFileError(path + ": cannot open file (" + std::strerror(errno) + ")");
    map_ = std::make_shared<Mapping>();
    map_->size = (size_t)size;
    map_->base = ::mmap(nullptr, (size_t)size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map_->base == MAP_FAILED) {
        map_->base = nullptr;
        throw WeightFileError(path + ": cannot map file (" + std::strerror(errno) + ")");
    }
    const unsigned char* bytes = (const unsigned char*)map_->base;
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; i--) header_len = (header_len << 8) | bytes[i];
    if (header_len > kMaxHeaderBytes || 8 + header_len > size)
        throw WeightFileError(path + ": header length " + std::to_string(header_len) + " exceeds the file size " +
                              std::to_string(size) + " (truncated or corrupt)");
    Json header;
    try {
        header = Json::parse(std::string((const char*)bytes + 8, (size_t)header_len));
    } catch (const ValueError& e) {
        throw WeightFileError(path + ": header is not valid JSON (" + e.what() + ")");
    }
    if (!header.is_object()) throw WeightFileError(path + ": header must be a JSON object");
    data_start_ = 8 + header_len;
    const uint64_t payload = size - data_start_;
    struct Span { uint64_t b, e; std::string name; };
    std::vector<Span> spans;
    for (const auto& m : header.members()) {
        const std::string& name = m.first;
        if (name == "__metadata__") continue;
        const Json& meta = m.second;
        Entry en;
        std::string dtype_name;
        int64_t begin = 0, end = 0;
        try {
            dtype_name = meta.at("dtype").as_string();
            for (const Json& d : meta.at("shape").items()) en.shape.push_back(d.is_int() ? d.as_int() : -1);
            const auto& offs = meta.at("data_offsets").items();
            if (offs.size() != 2) throw ValueError("data_offsets must hold two numbers");
            begin = offs[0].as_int();
            end = offs[1].as_int();
        } catch (const ValueError& e) {
            throw WeightFileError(path + ": malformed header entry for '" + name + "' (" + e.what() + ")");
        }
        bool known = false;
        for (const auto& r : kRows)
            if (dtype_name == r.name) { en.dtype = r.d; known = true; }
        if (!known) throw WeightFileError(path + ": tensor '" + name + "' has unsupported dtype " + dtype_name);
        uint64_t numel = 1;
        for (int64_t d : en.shape) {
            if (d < 0) throw WeightFileError(path + ": tensor '" + name + "' has a bad shape " + meta.at("shape").dump());
            numel *= (uint64_t)d;
        }
        if (!(0 <= begin && begin <= end && (uint64_t)end <= payload))
            throw WeightFileError(path + ": tensor '" + name + "' spans bytes [" + std::to_string(begin) + "," +
                                  std::to_string(end) + ") outside the payload of " + std::to_string(payload) + " bytes");
        if ((uint64_t)(end - begin) != numel * store_dtype_size(en.dtype))
            throw WeightFileError(path + ": tensor '" + name + "' has " + std::to_string(end - begin) + " bytes, shape " +
                                  meta.at("shape").dump() + " of " + dtype_name + " needs " +
                                  std::to_string(numel * store_dtype_size(en.dtype)));
        en.begin = (uint64_t)begin;
        en.end = (uint64_t)end;
        if (end > begin) spans.push_back({en.begin, en.end, name});
        entries_[name] = std::move(en);
    }
    std::sort(spans.begin(), spans.end(), [](const Span& a, const Span& b) { return a.b < b.b || (a.b == b.b && a.e < b.e); });
    for (size_t i = 1; i < spans.size(); i++)
        if (spans[i].b < spans[i - 1].e)
            throw WeightFileError(path + ": tensors '" + spans[i - 1].name + "' and '" + spans[i].name +
                                  "' overlap in the payload");
}

std::vector<std::string> SafetensorsFile::names() const {
    std::vector<std::string> out;
    for (const auto& kv : entries_) out.push_back(kv.first);
    return out;
}
const SafetensorsFile::Entry& SafetensorsFile::entry(const std::string& name) const {
    auto it = entries_.find(name);
    if (it == entries_.end()) throw WeightFileError(path_ + ": no tensor '" + name + "'");
    return it->second;
}
const std::vector<int64_t>& SafetensorsFile::shape(const std::string& name) const { return entry(name).shape; }
StoreDType SafetensorsFile::dtype(const std::string& name) const { return entry(name).dtype; }
HostTensor SafetensorsFile::tensor(const std::string& name) const {
    const Entry& e = entry(name);
    HostTensor t;
    t.dtype = e.dtype;
    t.shape = e.shape;
    t.data = (const char*)map_->base + data_start_ + e.begin;
    t.owner = map_;
    return t;
}

void write_safetensors(const std::string& path, const std::map<std::string, HostTensor>& tensors) {
    Json header = Json::object();
    uint64_t offset = 0;
    for (const auto& kv : tensors) {            // std::map: names sorted
        const HostTensor& t = kv.second;
        Json meta = Json::object();
        meta["dtype"] = store_dtype_name(t.dtype);
        Json shape = Json::array();
        for (int64_t d : t.shape) shape.push((long long)d);
        meta["shape"] = shape;
        Json offs = Json::array();
        offs.push((long long)offset);
        offs.push((long long)(offset + t.bytes()));
        meta["data_offsets"] = offs;
        header[kv.first] = meta;
        offset += t.bytes();
    }
    std::string head = header.dump();
    head.append((8 - head.size() % 8) % 8, ' ');          // keep the payload 8-byte aligned
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) throw WeightFileError("cannot write " + tmp + " (" + std::strerror(errno) + ")");
    unsigned char len[8];
    uint64_t n = head.size();
    for (int i = 0; i < 8; i++) { len[i] = (unsigned char)(n & 0xff); n >>= 8; }
    bool ok = std::fwrite(len, 1, 8, f) == 8 && std::fwrite(head.data(), 1, head.size(), f) == head.size();
    for (const auto& kv : tensors) {
        const size_t b = kv.second.bytes();
        if (ok && b) ok = std::fwrite(kv.second.data, 1, b, f) == b;
    }
    ok = (std::fclose(f) == 0) && ok;
    if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) {
        std::remove(tmp.c_str());
        throw WeightFileError("cannot write " + path + " (" + std::strerror(errno) + ")");
    }
}

}  // namespace sandy
