// Host-only stand-in for the brotensor operators named by brodiffusion's
// src/dit/common.cpp and the headers it includes.  TEST INFRASTRUCTURE ONLY.
//
// Only rope_apply does work, because dit::joint_attention_traced calls it
// before its own host loop: it is written here from the standard definition
// (pair p of a head = elements (2p, 2p+1), rotated by the angle of table entry
// (row, p)) and is NOT brotensor's code, so it pins nothing; the pin tests
// pass identity tables or compare on tensors rotated beforehand.  Every other
// operator belongs to paths that the pin does not exercise and throws.
#pragma once

#include <stdexcept>

#include "tensor.h"

namespace brotensor {

[[noreturn]] inline void not_in_pin(const char* op) {
    throw std::runtime_error(std::string("stand-in brotensor: ") + op + " is outside the pinned path");
}

inline void rope_apply(const Tensor& x, const Tensor& cos, const Tensor& sin, int head_dim, int num_heads,
                       Tensor& out) {
    const int L = x.rows, D = x.cols, half = head_dim / 2;
    if (D != head_dim * num_heads || cos.rows != L || cos.cols != half || sin.rows != L || sin.cols != half)
        throw std::runtime_error("stand-in rope_apply: shape mismatch");
    Tensor r;
    r.device = x.device;
    r.resize(L, D, x.dtype);
    for (int i = 0; i < L; ++i)
        for (int h = 0; h < num_heads; ++h)
            for (int p = 0; p < half; ++p) {
                const std::size_t c = static_cast<std::size_t>(i) * half + p;
                const std::size_t e = static_cast<std::size_t>(i) * D + static_cast<std::size_t>(h) * head_dim + 2 * p;
                const float a = x.at(e), b = x.at(e + 1), cs = cos.at(c), sn = sin.at(c);
                r.set(e, a * cs - b * sn);
                r.set(e + 1, a * sn + b * cs);
            }
    out = r;
}

inline void flash_attention_forward(const Tensor&, const Tensor&, const Tensor&, const float*, int, bool, Tensor&) {
    not_in_pin("flash_attention_forward");
}
inline void spatial_merge_2x2_forward(const Tensor&, int, int, int, int, bool, Tensor&) { not_in_pin("spatial_merge_2x2_forward"); }
inline void nchw_to_sequence(const Tensor&, int, int, int, int, Tensor&) { not_in_pin("nchw_to_sequence"); }
inline void patch_unpack_forward(const Tensor&, int, int, int, int, int, bool, Tensor&) { not_in_pin("patch_unpack_forward"); }
inline void cast(const Tensor&, Tensor&, Dtype) { not_in_pin("cast"); }
inline void copy_d2d_strided(const Tensor&, int, int, Tensor&, int, int, int, int) { not_in_pin("copy_d2d_strided"); }
inline void copy_d2d(const Tensor&, int, Tensor&, int, int) { not_in_pin("copy_d2d"); }
inline void linear_forward_batched_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&) { not_in_pin("linear_forward_batched_fp16"); }
inline void linear_forward_batched(const Tensor&, const Tensor&, const Tensor&, Tensor&) { not_in_pin("linear_forward_batched"); }
inline void layernorm_forward_inference_batched_fp16(const Tensor&, const Tensor&, const Tensor&, Tensor&, float) { not_in_pin("layernorm_forward_inference_batched_fp16"); }
inline void layernorm_forward_inference_batched(const Tensor&, const Tensor&, const Tensor&, Tensor&, float) { not_in_pin("layernorm_forward_inference_batched"); }

}  // namespace brotensor
