// Reader and writer for the safetensors container.
//
// Format, as the reference reads it (src/weight/SafeTensorWeights.cpp:44-95 and its Python twin
// scripts/run_gpt2.py:39-83): an unsigned 64-bit little-endian header length, a JSON header
// `{name: {dtype, shape, data_offsets:[begin,end]}}` (the `__metadata__` entry is skipped), then
// the payload; offsets are relative to the end of the header.  Dtypes accepted are those of the
// reference's parse_dtype (:14-23): F32, F16, BF16, I32, I64, U8, BOOL.  Where the reference
// aborts on a bad file, every fault here is a WeightFileError that says what is wrong with which
// file.  The file is memory-mapped; a tensor is a view of the mapping until it is converted.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace sandy {

enum class StoreDType { F32, F16, BF16, I32, I64, U8, BOOL };
const char* store_dtype_name(StoreDType d);          // "F32", ...
const char* store_dtype_word(StoreDType d);          // "float32", "int64", ...
size_t store_dtype_size(StoreDType d);
bool store_dtype_is_float(StoreDType d);
StoreDType store_dtype_from_name(const std::string& name);     // throws ValueError

// A tensor on the host: a view of a mapped file or of memory its `owner` keeps alive.
struct HostTensor {
    StoreDType dtype = StoreDType::F32;
    std::vector<int64_t> shape;
    const void* data = nullptr;
    std::shared_ptr<void> owner;
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
    size_t bytes() const { return (size_t)numel() * store_dtype_size(dtype); }
};

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    const std::string& path() const { return path_; }
    std::vector<std::string> names() const;
    bool contains(const std::string& name) const { return entries_.count(name) != 0; }
    const std::vector<int64_t>& shape(const std::string& name) const;
    StoreDType dtype(const std::string& name) const;
    HostTensor tensor(const std::string& name) const;      // a view; the mapping lives as long as any view

private:
    struct Entry { StoreDType dtype; std::vector<int64_t> shape; uint64_t begin, end; };
    struct Mapping;
    const Entry& entry(const std::string& name) const;
    std::string path_;
    std::shared_ptr<Mapping> map_;
    uint64_t data_start_ = 0;
    std::map<std::string, Entry> entries_;
};

// Write `tensors` as one safetensors file, names sorted, atomically (a temporary file, then a rename).
void write_safetensors(const std::string& path, const std::map<std::string, HostTensor>& tensors);

// bfloat16 / float16 conversions used wherever a tensor changes its storage type on the host
uint16_t f32_to_bf16_bits(float v);          // round to nearest even (src/core/Tensor.h:43-49)
float bf16_bits_to_f32(uint16_t b);
uint16_t f32_to_f16_bits(float v);
float f16_bits_to_f32(uint16_t h);

}  // namespace sandy
