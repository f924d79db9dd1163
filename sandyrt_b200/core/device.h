// Device memory as the host side sees it: 2-D tensor views, owned buffers, the workspace of
// named scratch tensors, pinned host memory.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "cache.h"
#include "errors.h"
#include "safetensors.h"

namespace sandy {

void cuda_check(cudaError_t e, const char* what);        // throws KernelError

// A [rows, cols] view of device memory with a row pitch in elements.
struct Tensor {
    void* data = nullptr;
    DType dtype = DType::F32;
    int64_t rows = 0, cols = 0, ld = 0;
    bool defined() const { return data != nullptr; }
    size_t elem_size() const { return dtype_size(dtype); }
    int64_t numel() const { return rows * cols; }
    bool contiguous() const { return ld == cols; }
    Tensor col_range(int64_t c0, int64_t c1) const {
        Tensor t = *this;
        t.data = (char*)data + (size_t)c0 * elem_size();
        t.cols = c1 - c0;
        return t;
    }
    Tensor row_range(int64_t r0, int64_t r1) const {
        Tensor t = *this;
        t.data = (char*)data + (size_t)r0 * (size_t)ld * elem_size();
        t.rows = r1 - r0;
        return t;
    }
};

// Device memory that is freed with its owner.
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes);
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }
private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

// Pinned host memory.
class PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(size_t bytes);
    ~PinnedBuffer();
    PinnedBuffer(PinnedBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
    PinnedBuffer& operator=(PinnedBuffer&& o) noexcept;
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }
private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

// A weight on the device: the buffer and a 2-D view of it (a vector is [1, n]).
struct DeviceWeight {
    std::shared_ptr<DeviceBuffer> buffer;
    Tensor view;
    size_t bytes() const { return (size_t)view.numel() * view.elem_size(); }
};

// Move a loaded tensor to the device in the dtype the engine computes in (floats: float32 or
// bfloat16, one rounding at most; integers: int32; `keep_32bit` keeps a tensor stored as F32 so).
// `transpose` stores a 2-D tensor as its transpose.  Tensors of other ranks become [1, n], or
// [shape[0], rest] with `as_rows`.
DeviceWeight to_device(const HostTensor& t, DType compute, bool keep_32bit = false, bool transpose = false,
                       bool as_rows = true);

// Named scratch tensors that keep their address from step to step (so that a captured CUDA graph
// stays valid) and only ever grow.
class Workspace {
public:
    Tensor get(const std::string& name, int64_t rows, int64_t cols, DType dtype);
    void* raw(const std::string& name, size_t bytes);
    uint64_t version() const { return version_; }      // bumped whenever a buffer moves; recorded graphs check it
private:
    std::map<std::pair<std::string, int>, DeviceBuffer> bufs_;
    uint64_t version_ = 0;
};

}  // namespace sandy
