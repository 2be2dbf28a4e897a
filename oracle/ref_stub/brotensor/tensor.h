// Host-only stand-in for the brotensor tensor type.  TEST INFRASTRUCTURE ONLY.
//
// brodiffusion's src/dit/common.cpp is plain C++ apart from the brotensor
// plumbing it calls.  brotensor itself is an external dependency whose source
// is not part of the brodiffusion tree, so this header provides just enough
// of its surface (names and signatures as common.cpp and the brodiffusion
// headers it includes use them) for that file to compile UNMODIFIED into a
// host library that the oracle is checked against.  Nothing here is a copy of
// brotensor: tensors are std::vector storage on the host, "devices" are a tag.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace brotensor {

enum class Dtype { FP32 = 0, FP16 = 1, BF16 = 2 };

struct Device {
    int kind = 0;   // 0 = host; the stand-in has no other device
    bool is_gpu() const { return false; }
    bool operator==(const Device& o) const { return kind == o.kind; }
};

inline Device default_device() { return Device{}; }
inline Dtype compute_dtype() { return Dtype::FP32; }

// bit conversions (IEEE binary16 / bfloat16, round to nearest even)
inline float bf16_bits_to_fp32(std::uint16_t b) {
    std::uint32_t u = static_cast<std::uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline std::uint16_t fp32_to_bf16_bits(float f) {
    std::uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<std::uint16_t>((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<std::uint16_t>(u >> 16);
}
inline float fp16_bits_to_fp32(std::uint16_t h) {
    const std::uint32_t sign = static_cast<std::uint32_t>(h & 0x8000u) << 16;
    std::uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
            u = sign | static_cast<std::uint32_t>(127 - 15 - e) << 23 | (man & 0x3ffu) << 13;
        }
    } else if (exp == 31) u = sign | 0x7f800000u | man << 13;
    else u = sign | (exp + 112) << 23 | man << 13;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline std::uint16_t fp32_to_fp16_bits(float f) {
    std::uint32_t u;
    std::memcpy(&u, &f, 4);
    const std::uint32_t sign = (u >> 16) & 0x8000u;
    const std::int32_t exp = static_cast<std::int32_t>((u >> 23) & 0xffu) - 127 + 15;
    std::uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xffu) == 0xffu) return static_cast<std::uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return static_cast<std::uint16_t>(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return static_cast<std::uint16_t>(sign);
        man |= 0x800000u;
        const int shift = 14 - exp;
        std::uint32_t r = man >> shift;
        const std::uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return static_cast<std::uint16_t>(sign | r);
    }
    std::uint32_t r = static_cast<std::uint32_t>(exp) << 10 | man >> 13;
    const std::uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
    return static_cast<std::uint16_t>(sign | r);
}

struct Tensor {
    // `data` is only ever compared with nullptr by the callers.
    void* data = nullptr;
    int rows = 0, cols = 0;
    Dtype dtype = Dtype::FP32;
    Device device{};
    std::vector<float> f32;            // FP32 payload
    std::vector<std::uint16_t> b16;    // FP16 / BF16 payload

    long long size() const { return static_cast<long long>(rows) * cols; }

    void resize(int r, int c, Dtype dt) {
        rows = r; cols = c; dtype = dt;
        const std::size_t n = static_cast<std::size_t>(r) * c;
        if (dt == Dtype::FP32) { f32.assign(n, 0.0f); b16.clear(); data = f32.data(); }
        else { b16.assign(n, 0); f32.clear(); data = b16.data(); }
    }
    static Tensor from_host(const float* src, int r, int c) {
        Tensor t;
        t.resize(r, c, Dtype::FP32);
        std::memcpy(t.f32.data(), src, sizeof(float) * t.f32.size());
        return t;
    }
    static Tensor from_host_fp16(const std::uint16_t* src, int r, int c) {
        Tensor t;
        t.resize(r, c, Dtype::FP16);
        std::memcpy(t.b16.data(), src, 2 * t.b16.size());
        return t;
    }
    static Tensor from_host_bf16(const std::uint16_t* src, int r, int c) {
        Tensor t;
        t.resize(r, c, Dtype::BF16);
        std::memcpy(t.b16.data(), src, 2 * t.b16.size());
        return t;
    }
    static Tensor zeros_on(Device dev, int r, int c, Dtype dt) {
        Tensor t;
        t.device = dev;
        t.resize(r, c, dt);
        return t;
    }
    Tensor to(Device dev) const {
        Tensor t = *this;
        t.device = dev;
        t.data = t.dtype == Dtype::FP32 ? static_cast<void*>(t.f32.data()) : static_cast<void*>(t.b16.data());
        return t;
    }
    void copy_to_host_fp16(std::uint16_t* dst) const { std::memcpy(dst, b16.data(), 2 * b16.size()); }
    void copy_to_host_bf16(std::uint16_t* dst) const { std::memcpy(dst, b16.data(), 2 * b16.size()); }
    std::vector<float> to_host_vector() const {
        if (dtype != Dtype::FP32) throw std::runtime_error("stand-in tensor: to_host_vector needs FP32");
        return f32;
    }
    // element access in FP32 whatever the storage type (used by the stand-in ops)
    float at(std::size_t i) const {
        if (dtype == Dtype::FP32) return f32[i];
        return dtype == Dtype::BF16 ? bf16_bits_to_fp32(b16[i]) : fp16_bits_to_fp32(b16[i]);
    }
    void set(std::size_t i, float v) {
        if (dtype == Dtype::FP32) f32[i] = v;
        else b16[i] = dtype == Dtype::BF16 ? fp32_to_bf16_bits(v) : fp32_to_fp16_bits(v);
    }
};

}  // namespace brotensor
