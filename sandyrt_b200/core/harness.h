// A test bench for one part outside a model: builds the part from its description, binds seeded
// random tensors, keeps a small cache of its own and runs the part over hand-made steps.  Tests use
// it to compare each part alone with the plain implementation's function for it.
#pragma once

#include <memory>
#include <utility>
#include <vector>

#include "cache.h"
#include "json.h"
#include "parts.h"

namespace sandy {

class PartHarness {
public:
    // args: {"family", "part": <part description>, "position": <part description, optional>, "dtype": "float32"|"bfloat16",
    //        "page_size": 8, "max_tokens": 512, "max_requests": 8, "seed": 0}
    explicit PartHarness(const Json& args);
    ~PartHarness();
    Json tensors() const;          // {"part": {name: {"shape": [...], "address": host address of float32 values}}, "position": {...}}
    Json info() const;             // cache spec, max_positions of the position part
    // The next step: for each request its (tokens before, new tokens).  A request seen before moves on
    // (its earlier tokens are committed); ids may be null (zeros).
    void set_step(const std::vector<std::pair<int, int>>& seqs, const int* ids);
    void run_norm(const void* x, int x_rows, void* out, int n_rows, const int* rows_host);
    void run_feed_forward(const void* h, void* x);
    void run_mixer(const void* h, void* x, bool write_cache);
    void run_embedding(void* x);
private:
    Tensor view(const void* p, int64_t rows, int64_t cols, DType dt) const;
    std::string family_;
    DType dtype_ = DType::F32;
    int64_t width_ = 0;
    std::unique_ptr<Part> part_;
    std::unique_ptr<PositionEncoding> position_;
    TensorMap part_tensors_, position_tensors_;
    std::unique_ptr<CacheManager> cache_;
    Workspace workspace_;
    cudaStream_t stream_ = nullptr;
    DeviceBuffer arrays_, status_;
    StepContext ctx_;
    bool have_step_ = false;
};

}  // namespace sandy
