// brodiffusion::dit shared attention bricks over the bdattn library.
// Mirrors include/brodiffusion/dit/common.h:64-153 of the reference for the
// functions on the attention path.
#pragma once

#include <vector>

#include "brotensor/ops.h"

namespace brodiffusion::dit {

namespace bt = ::brotensor;

struct RopeTables {
    bt::Tensor cos;   // (L, head_dim/2) FP32
    bt::Tensor sin;
};

// src/dit/common.cpp:116-184.  Tables are filled on the device; no host loop,
// no upload.
inline RopeTables build_axial_rope_tables(int txt_len, int hp, int wp, int head_dim,
                                          const std::vector<int>& axes_dims_rope, float theta = 10000.f) {
    RopeTables t;
    const int L = txt_len + hp * wp;
    t.cos.resize(L > 0 ? L : 1, head_dim / 2, bt::Dtype::FP32);
    t.sin.resize(L > 0 ? L : 1, head_dim / 2, bt::Dtype::FP32);
    bt::detail::bd_check(bdattn_rope_tables_flux(txt_len, hp, wp, head_dim, axes_dims_rope.data(),
                                                 static_cast<int>(axes_dims_rope.size()), theta,
                                                 static_cast<float*>(t.cos.data), static_cast<float*>(t.sin.data),
                                                 bt::detail::bd_stream()));
    return t;
}

// src/dit/common.cpp:188-196: rope(Q), rope(K), non-causal attention.
inline void joint_attention(const bt::Tensor& Q, const bt::Tensor& K, const bt::Tensor& V, const bt::Tensor& cos,
                            const bt::Tensor& sin, int head_dim, int num_heads, bt::Tensor& out, bt::Tensor& Qr,
                            bt::Tensor& Kr) {
    if (head_dim <= 0 || num_heads <= 0 || Q.cols != head_dim * num_heads)
        throw std::runtime_error("joint_attention: D must equal head_dim * num_heads");
    Qr.resize(Q.rows, Q.cols, Q.dtype);
    Kr.resize(K.rows, K.cols, K.dtype);
    // one launch rotates both tensors
    bdattn_norm_rope_job jobs[2] = {};
    jobs[0].x = Q.data; jobs[0].out = Qr.data; jobs[0].rows = Q.rows; jobs[0].x_ld = Q.cols; jobs[0].out_ld = Qr.cols;
    jobs[1].x = K.data; jobs[1].out = Kr.data; jobs[1].rows = K.rows; jobs[1].x_ld = K.cols; jobs[1].out_ld = Kr.cols;
    for (auto& j : jobs) { j.cos = static_cast<const float*>(cos.data); j.sin = static_cast<const float*>(sin.data); }
    bt::detail::bd_check(bdattn_rmsnorm_rope(jobs, 2, bt::detail::bd_dtype(Q.dtype), num_heads, head_dim, 0.0f,
                                             BDATTN_ROPE_INTERLEAVED, bt::detail::bd_stream()));
    bt::flash_attention_forward(Qr, Kr, V, /*d_mask=*/nullptr, num_heads, /*causal=*/false, out);
}

}  // namespace brodiffusion::dit
