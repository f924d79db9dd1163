#include "device.h"

#include <algorithm>
#include <cstring>

#include "weights.h"

namespace sandy {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw KernelError(std::string(what) + ": " + cudaGetErrorString(e));
}

DeviceBuffer::DeviceBuffer(size_t bytes) : bytes_(bytes) {
    cuda_check(cudaMalloc(&ptr_, std::max<size_t>(bytes, 16)), "allocating device memory");
}
DeviceBuffer::~DeviceBuffer() {
    if (ptr_) cudaFree(ptr_);
}
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        if (ptr_) cudaFree(ptr_);
        ptr_ = o.ptr_;
        bytes_ = o.bytes_;
        o.ptr_ = nullptr;
        o.bytes_ = 0;
    }
    return *this;
}

PinnedBuffer::PinnedBuffer(size_t bytes) : bytes_(bytes) {
    cuda_check(cudaMallocHost(&ptr_, std::max<size_t>(bytes, 16)), "allocating pinned host memory");
    std::memset(ptr_, 0, std::max<size_t>(bytes, 16));
}
PinnedBuffer::~PinnedBuffer() {
    if (ptr_) cudaFreeHost(ptr_);
}
PinnedBuffer& PinnedBuffer::operator=(PinnedBuffer&& o) noexcept {
    if (this != &o) {
        if (ptr_) cudaFreeHost(ptr_);
        ptr_ = o.ptr_;
        bytes_ = o.bytes_;
        o.ptr_ = nullptr;
        o.bytes_ = 0;
    }
    return *this;
}

namespace {
template <typename T>
void transpose_into(const T* src, T* dst, int64_t rows, int64_t cols) {
    constexpr int64_t B = 32;
    for (int64_t r0 = 0; r0 < rows; r0 += B)
        for (int64_t c0 = 0; c0 < cols; c0 += B)
            for (int64_t r = r0; r < std::min(rows, r0 + B); r++)
                for (int64_t c = c0; c < std::min(cols, c0 + B); c++) dst[c * rows + r] = src[r * cols + c];
}
}  // namespace

DeviceWeight to_device(const HostTensor& t, DType compute, bool keep_32bit, bool transpose, bool as_rows) {
    int64_t rows = 1, cols = t.numel();
    if (t.shape.size() >= 2 && as_rows) {
        rows = t.shape[0];
        cols = rows ? t.numel() / rows : 0;
    }
    DeviceWeight w;
    const void* src = nullptr;
    std::vector<float> f32;
    std::vector<uint16_t> b16;
    std::vector<int32_t> i32;
    std::vector<char> turned;
    DType dt;
    if (!store_dtype_is_float(t.dtype)) {
        dt = DType::I32;
        i32 = to_i32(t);
        src = i32.data();
    } else if (compute == DType::F32 || (keep_32bit && t.dtype == StoreDType::F32)) {
        dt = DType::F32;
        if (t.dtype == StoreDType::F32) src = t.data;
        else { f32 = to_f32(t); src = f32.data(); }
    } else {
        dt = DType::BF16;
        if (t.dtype == StoreDType::BF16) src = t.data;
        else { b16 = to_bf16_bits(t); src = b16.data(); }
    }
    const size_t esz = dtype_size(dt);
    if (transpose) {
        if (t.shape.size() != 2) throw ValueError("only a matrix can be transposed");
        turned.resize((size_t)t.numel() * esz);
        if (esz == 2) transpose_into((const uint16_t*)src, (uint16_t*)turned.data(), rows, cols);
        else transpose_into((const uint32_t*)src, (uint32_t*)turned.data(), rows, cols);
        src = turned.data();
        std::swap(rows, cols);
    }
    w.buffer = std::make_shared<DeviceBuffer>((size_t)t.numel() * esz);
    if (t.numel())
        cuda_check(cudaMemcpy(w.buffer->get(), src, (size_t)t.numel() * esz, cudaMemcpyHostToDevice), "copying a weight to the device");
    w.view.data = w.buffer->get();
    w.view.dtype = dt;
    w.view.rows = rows;
    w.view.cols = cols;
    w.view.ld = cols;
    return w;
}

Tensor Workspace::get(const std::string& name, int64_t rows, int64_t cols, DType dtype) {
    Tensor t;
    t.data = raw(name + ":" + dtype_name(dtype), (size_t)(rows * cols) * dtype_size(dtype));
    t.dtype = dtype;
    t.rows = rows;
    t.cols = cols;
    t.ld = cols;
    return t;
}

void* Workspace::raw(const std::string& name, size_t bytes) {
    auto key = std::make_pair(name, 0);
    auto it = bufs_.find(key);
    if (it == bufs_.end() || it->second.bytes() < bytes) {
        // grow in steps, so that a slowly growing step does not move the buffer every time
        size_t want = std::max<size_t>(bytes, 256);
        if (it != bufs_.end()) want = std::max(want, it->second.bytes() + it->second.bytes() / 2);
        bufs_[key] = DeviceBuffer(want);
        version_++;
        it = bufs_.find(key);
    }
    return it->second.get();
}

}  // namespace sandy
