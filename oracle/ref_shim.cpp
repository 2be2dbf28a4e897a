// C entry points over brodiffusion's own src/dit/common.cpp, compiled UNMODIFIED
// from the reference tree against the host-only brotensor stand-in in
// ref_stub/.  TEST INFRASTRUCTURE ONLY: the result (oracle/_ref/libref.so) is
// what the oracle restatement is pinned against; the product never loads it.
//
//   ref_build_axial_rope_tables -> dit::build_axial_rope_tables (src/dit/common.cpp:116-184)
//   ref_joint_attention_traced  -> dit::joint_attention_traced  (src/dit/common.cpp:198-329)
#include <cstring>
#include <string>
#include <vector>

#include "brodiffusion/dit/common.h"
#include "brotensor/tensor.h"

namespace bt = ::brotensor;
namespace dit = ::brodiffusion::dit;

namespace {
thread_local std::string g_err;
}

extern "C" {

const char* ref_last_error(void) { return g_err.c_str(); }

// cos_out / sin_out: (txt_len + hp*wp, head_dim/2) floats.  Returns 0, or -1
// with the reference's exception text in ref_last_error().
int ref_build_axial_rope_tables(int txt_len, int hp, int wp, int head_dim, const int* axes, int n_axes,
                                float theta, float* cos_out, float* sin_out) {
    try {
        std::vector<int> ax(axes, axes + n_axes);
        dit::RopeTables t = dit::build_axial_rope_tables(txt_len, hp, wp, head_dim, ax, theta);
        std::memcpy(cos_out, t.cos.f32.data(), sizeof(float) * t.cos.f32.size());
        std::memcpy(sin_out, t.sin.f32.data(), sizeof(float) * t.sin.f32.size());
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// q, k, v: (L, D) floats; cos, sin: (L, head_dim/2); bias: (L - txt_len, txt_len)
// or null; out: (L, D); attn_avg: (L, L).  use_bf16 != 0 rounds q/k/v to BF16
// tensors first (the reference then returns a BF16 output).
int ref_joint_attention_traced(const float* q, const float* k, const float* v, const float* cos,
                               const float* sin, int L, int D, int head_dim, int num_heads, int txt_len,
                               const float* bias, int use_bf16, float* out, float* attn_avg) {
    try {
        auto make = [&](const float* src) {
            if (!use_bf16) return bt::Tensor::from_host(src, L, D);
            std::vector<std::uint16_t> bits(static_cast<std::size_t>(L) * D);
            for (std::size_t i = 0; i < bits.size(); ++i) bits[i] = bt::fp32_to_bf16_bits(src[i]);
            return bt::Tensor::from_host_bf16(bits.data(), L, D);
        };
        const bt::Tensor Q = make(q), K = make(k), V = make(v);
        const bt::Tensor C = bt::Tensor::from_host(cos, L, head_dim / 2);
        const bt::Tensor S = bt::Tensor::from_host(sin, L, head_dim / 2);
        bt::Tensor B;
        if (bias != nullptr) B = bt::Tensor::from_host(bias, L - txt_len, txt_len);
        bt::Tensor O, A, Qr, Kr;
        dit::joint_attention_traced(Q, K, V, C, S, head_dim, num_heads, O, A, Qr, Kr, txt_len,
                                    bias != nullptr ? &B : nullptr);
        for (std::size_t i = 0; i < static_cast<std::size_t>(L) * D; ++i) out[i] = O.at(i);
        for (std::size_t i = 0; i < static_cast<std::size_t>(L) * L; ++i) attn_avg[i] = A.at(i);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

}  // extern "C"
