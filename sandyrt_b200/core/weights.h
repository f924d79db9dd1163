// Binding of weight-file tensors to a model's parts, by name, and the random-weights mode.
//
// The reference resolves `weight("h.3.attn.c_proj.weight")` against the file's descriptors and
// fails on the first name it cannot find ("weight not found: <name>",
// src/ir/MidIRMaterializer.cpp:186-194; "missing weight buffer", src/engine/Engine.cpp:1143-1147).
// Here the model states every tensor it wants with its shape up front, the file is checked
// against that list in one pass, and ONE WeightBindingError lists everything that is wrong:
// missing tensors, unexpected tensors, tensors of the wrong shape and of the wrong kind.
//
// Storage dtypes on the host after loading: floating-point tensors stay as the file stores them
// (BF16, F16 or F32: views of the mapping, nothing is rounded here); integer tables are read as
// they are and become int32 on the device.  The parts convert what feeds their matrix products to
// the engine's compute dtype when they bind, so each value is rounded at most once: an F16 file
// is widened exactly for the float32 path and rounded to bfloat16 for the bfloat16 path.  A part
// may ask that a tensor stored in 32-bit stays so (`keep_32bit`).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "safetensors.h"

namespace sandy {

// What a part expects of one tensor of the weight file.
struct TensorRequest {
    std::vector<int64_t> shape;
    bool integer = false;        // an integer table (kept as int32) rather than floats
    bool keep_32bit = false;     // if stored as F32, stay F32 whatever the compute dtype
    // How the random-weights mode fills it: "weight" N(0, 0.02), "bias" N(0, 0.01),
    // "gamma" 1 + N(0, 0.02), "beta" N(0, 0.02), "zeros".
    std::string init = "weight";
};

using TensorRequests = std::map<std::string, TensorRequest>;
using TensorMap = std::map<std::string, HostTensor>;

constexpr const char* kWeightFile = "model.safetensors";

// Open `model_dir/model.safetensors`, check it against `requests` and return the requested
// tensors by their un-prefixed names (views of the mapping).
TensorMap load_weights(const std::string& model_dir, const TensorRequests& requests,
                       const std::vector<std::string>& prefixes, const std::vector<std::string>& ignored);

// Seeded random tensors for `requests`, stored as `dtype` (F32, BF16 or F16; `keep_32bit`
// tensors stay F32).  Each tensor has its own generator keyed by (seed, tensor name), and each
// element its own counter, so a tensor's values do not depend on which other tensors the model
// has.  The distributions: matrix and table weights N(0, 0.02); biases N(0, 0.01); norm gains
// 1 + N(0, 0.02); norm offsets N(0, 0.02).  (The reference has no such mode; its tests fill
// tensors by hand, test/engine/CudaDeviceTest.cpp:302-312.)
TensorMap random_tensors(const TensorRequests& requests, uint64_t seed, StoreDType dtype);

// Convert a host tensor's floats to float32 / bfloat16 bits (any float storage type in).
std::vector<float> to_f32(const HostTensor& t);
std::vector<uint16_t> to_bf16_bits(const HostTensor& t);
std::vector<int32_t> to_i32(const HostTensor& t);

}  // namespace sandy
