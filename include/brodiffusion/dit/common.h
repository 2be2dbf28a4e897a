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

// src/dit/common.cpp:198-329 (include/brodiffusion/dit/common.h:117-129 of the
// reference): joint_attention plus the head-averaged softmax map (L, L) in
// attn_avg and an optional (img_len, txt_len) FP32 bias added to the scaled scores
// of image-query rows [txt_len, L) x text-key columns [0, txt_len).  The
// reference downloads Q/K/V and loops on the host; here everything stays on the
// device.  attn_avg is FP32 (the reference stores it at the pipeline's compute
// dtype; the callers only download it, src/dit/flux.cpp:505-508).
inline void joint_attention_traced(const bt::Tensor& Q, const bt::Tensor& K, const bt::Tensor& V, const bt::Tensor& cos,
                                   const bt::Tensor& sin, int head_dim, int num_heads, bt::Tensor& out,
                                   bt::Tensor& attn_avg, bt::Tensor& Qr, bt::Tensor& Kr, int txt_len = 0,
                                   const bt::Tensor* image_text_bias = nullptr) {
    const int D = Q.cols, L = Q.rows;
    if (head_dim <= 0 || num_heads <= 0 || D != head_dim * num_heads)
        throw std::runtime_error("dit::common: joint_attention_traced: D must equal head_dim * num_heads");
    if (K.rows != L || V.rows != L || K.cols != D || V.cols != D)
        throw std::runtime_error("dit::common: joint_attention_traced: Q/K/V must share shape (L, D)");
    if (image_text_bias != nullptr) {
        if (txt_len < 0 || txt_len > L)
            throw std::runtime_error("dit::common: joint_attention_traced: txt_len out of range for bias");
        if (image_text_bias->dtype != bt::Dtype::FP32)
            throw std::runtime_error("dit::common: joint_attention_traced: image_text_bias must be FP32");
        if (image_text_bias->rows != L - txt_len || image_text_bias->cols != txt_len)
            throw std::runtime_error("dit::common: joint_attention_traced: image_text_bias must be (img_len, txt_len)");
    }
    bt::rope_apply(Q, cos, sin, head_dim, num_heads, Qr);
    bt::rope_apply(K, cos, sin, head_dim, num_heads, Kr);
    out.resize(L, D, Q.dtype);
    attn_avg.resize(L, L, bt::Dtype::FP32);
    bt::Tensor ws;
    ws.resize(1, static_cast<int>(bdattn_sdpa_traced_workspace_bytes(num_heads, L)), bt::Dtype::INT8);
    bdattn_sdpa_params p{};
    p.dtype = bt::detail::bd_dtype(Q.dtype);
    p.batch = 1; p.num_heads = num_heads; p.head_dim = head_dim;
    p.n_q_seg = 1; p.q[0] = Qr.data; p.o[0] = out.data; p.q_rows[0] = L; p.q_ld[0] = D; p.o_ld[0] = D;
    p.n_kv_seg = 1; p.k[0] = Kr.data; p.v[0] = V.data; p.kv_rows[0] = L; p.k_ld[0] = D; p.v_ld[0] = D;
    bdattn_trace_params t{};
    if (image_text_bias != nullptr && txt_len > 0 && txt_len < L) {
        t.bias = static_cast<const float*>(image_text_bias->data);
        t.bias_row0 = txt_len; t.bias_rows = L - txt_len; t.bias_cols = txt_len; t.bias_ld = txt_len;
    }
    t.attn_avg = static_cast<float*>(attn_avg.data); t.map_rows = L; t.map_cols = L; t.map_ld = L;
    t.workspace = ws.data; t.workspace_bytes = ws.bytes();
    bt::detail::bd_check(bdattn_sdpa_traced_fwd(&p, &t, bt::detail::bd_stream()));
    // the statistics scratch is freed when this returns: wait for the kernels that use it
    bt::cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(bt::cuda_current_stream())), "joint_attention_traced");
}

// src/dit/common.cpp:331-377 (Krea 2): grouped-query heads, optional RoPE,
// optional key mask.  The kernel reads K/V head h / group for query head h, so
// the widened copies the reference materialises (Krep / Vrep, common.cpp:361-375)
// are not made; the two scratch arguments are kept for source compatibility and
// left untouched.
inline void gqa_attention_masked(const bt::Tensor& Q, const bt::Tensor& K, const bt::Tensor& V,
                                 const bt::Tensor* cos, const bt::Tensor* sin, int head_dim, int num_q_heads,
                                 int num_kv_heads, const float* d_mask, bt::Tensor& out, bt::Tensor& Qr,
                                 bt::Tensor& Kr, bt::Tensor& /*Krep*/, bt::Tensor& /*Vrep*/) {
    if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0)
        throw std::runtime_error("gqa_attention_masked: num_kv_heads must divide num_q_heads");
    if (head_dim <= 0 || Q.cols != head_dim * num_q_heads || K.cols != head_dim * num_kv_heads ||
        V.cols != K.cols || K.rows != V.rows)
        throw std::runtime_error("gqa_attention_masked: Q/K/V shapes do not agree with the head counts");
    const bt::Tensor* Qp = &Q;
    const bt::Tensor* Kp = &K;
    if (cos != nullptr && sin != nullptr) {
        bt::rope_apply(Q, *cos, *sin, head_dim, num_q_heads, Qr);
        bt::rope_apply(K, *cos, *sin, head_dim, num_kv_heads, Kr);
        Qp = &Qr;
        Kp = &Kr;
    }
    out.resize(Q.rows, Q.cols, Q.dtype);
    bdattn_sdpa_params p{};
    p.dtype = bt::detail::bd_dtype(Q.dtype);
    p.batch = 1; p.num_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
    p.n_q_seg = 1; p.q[0] = Qp->data; p.o[0] = out.data; p.q_rows[0] = Q.rows; p.q_ld[0] = Q.cols; p.o_ld[0] = out.cols;
    p.n_kv_seg = 1; p.k[0] = Kp->data; p.v[0] = V.data; p.kv_rows[0] = K.rows; p.k_ld[0] = K.cols; p.v_ld[0] = V.cols;
    p.mask_mode = BDATTN_MASK_NONE;
    p.key_mask = d_mask;
    bt::detail::bd_check(bdattn_sdpa_fwd(&p, bt::detail::bd_stream()));
}

}  // namespace brodiffusion::dit
