// Minimal stand-in for brotensor's Tensor, sufficient for the attention path.
//
// brodiffusion's model code passes 2-D row-major tensors by reference and lets
// operators resize unallocated outputs (include/brodiffusion/detail/device.h:5-25).
// This header reproduces the members those call sites use — data, rows, cols,
// dtype, device, size(), resize(), view(), clone(), deep-copying copy
// construction (src/dit/qwenimage21_forward.cpp:303-304) — on top of the CUDA
// runtime, so that the operator shims in brotensor/ops.h can be compiled and
// tested without brotensor itself.  Device tensors only: the library behind
// the shims has no CPU path.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace brotensor {

enum class Dtype { FP32 = 0, FP16 = 1, BF16 = 2, INT8 = 3 };

inline std::size_t dtype_size(Dtype d) {
    return d == Dtype::FP32 ? 4 : (d == Dtype::INT8 ? 1 : 2);
}

struct Device {
    enum Kind { CPU = 0, CUDA = 1 } kind = CUDA;
    int index = 0;
    bool is_gpu() const { return kind == CUDA; }
    bool is_cuda() const { return kind == CUDA; }
    static Device cuda(int i = 0) { return Device{CUDA, i}; }
    static Device cpu() { return Device{CPU, 0}; }
    bool operator==(const Device& o) const { return kind == o.kind && index == o.index; }
};

inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Stream every operator enqueues on (src/fused_transformer.cu:38-54).
inline void*& cuda_current_stream_slot() {
    static thread_local void* s = nullptr;
    return s;
}
inline void* cuda_current_stream() { return cuda_current_stream_slot(); }
inline void set_cuda_current_stream(void* s) { cuda_current_stream_slot() = s; }
inline void sync_all() { cuda_check(cudaDeviceSynchronize(), "sync_all"); }

struct Tensor {
    void* data = nullptr;
    int rows = 0, cols = 0;
    Dtype dtype = Dtype::FP32;
    Device device = Device::cuda();
    bool owns = false;

    Tensor() = default;
    Tensor(const Tensor& o) { *this = o.clone(); }           // copies are deep
    Tensor& operator=(const Tensor& o) {
        if (this != &o) { Tensor t = o.clone(); *this = std::move(t); }
        return *this;
    }
    Tensor(Tensor&& o) noexcept { steal(o); }
    Tensor& operator=(Tensor&& o) noexcept {
        if (this != &o) { release(); steal(o); }
        return *this;
    }
    ~Tensor() { release(); }

    std::size_t size() const { return static_cast<std::size_t>(rows) * cols; }
    std::size_t bytes() const { return size() * dtype_size(dtype); }

    // Keeps the storage when the shape and dtype already match (pointer
    // stability for captured graphs, src/unet_blocks.cpp:244-250).
    void resize(int r, int c, Dtype d) {
        if (data != nullptr && r == rows && c == cols && d == dtype) return;
        if (data != nullptr && !owns) throw std::runtime_error("Tensor::resize: cannot resize a view to a different shape");
        release();
        rows = r; cols = c; dtype = d; owns = true;
        if (bytes() > 0) cuda_check(cudaMalloc(&data, bytes()), "Tensor::resize");
    }
    static Tensor view(Device dev, void* p, int r, int c, Dtype d) {
        Tensor t; t.data = p; t.rows = r; t.cols = c; t.dtype = d; t.device = dev; t.owns = false;
        return t;
    }
    Tensor clone() const {
        Tensor t; t.device = device;
        if (data == nullptr) { t.rows = rows; t.cols = cols; t.dtype = dtype; return t; }
        t.resize(rows, cols, dtype);
        cuda_check(cudaMemcpyAsync(t.data, data, bytes(), cudaMemcpyDeviceToDevice,
                                   static_cast<cudaStream_t>(cuda_current_stream())), "Tensor::clone");
        return t;
    }
    static Tensor from_host(const float* p, int r, int c) {
        Tensor t; t.resize(r, c, Dtype::FP32);
        cuda_check(cudaMemcpy(t.data, p, t.bytes(), cudaMemcpyHostToDevice), "Tensor::from_host");
        return t;
    }
    // 16-bit tensors from their bit patterns (FP16 or BF16).
    static Tensor from_host_bits(const std::uint16_t* p, int r, int c, Dtype d) {
        Tensor t; t.resize(r, c, d);
        cuda_check(cudaMemcpy(t.data, p, t.bytes(), cudaMemcpyHostToDevice), "Tensor::from_host_bits");
        return t;
    }
    static Tensor from_host_bf16(const std::uint16_t* p, int r, int c) { return from_host_bits(p, r, c, Dtype::BF16); }
    std::vector<std::uint8_t> to_host_bytes() const {
        std::vector<std::uint8_t> v(bytes());
        cuda_check(cudaDeviceSynchronize(), "Tensor::to_host");
        if (!v.empty()) cuda_check(cudaMemcpy(v.data(), data, v.size(), cudaMemcpyDeviceToHost), "Tensor::to_host");
        return v;
    }

   private:
    void release() {
        if (owns && data != nullptr) cudaFree(data);
        data = nullptr; owns = false;
    }
    void steal(Tensor& o) {
        data = o.data; rows = o.rows; cols = o.cols; dtype = o.dtype; device = o.device; owns = o.owns;
        o.data = nullptr; o.owns = false; o.rows = o.cols = 0;
    }
};

inline std::uint16_t fp32_to_bf16_bits(float f) {
    std::uint32_t u; std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<std::uint16_t>(u >> 16);
}
inline float bf16_bits_to_fp32(std::uint16_t b) {
    std::uint32_t u = static_cast<std::uint32_t>(b) << 16; float f; std::memcpy(&f, &u, 4); return f;
}

}  // namespace brotensor
