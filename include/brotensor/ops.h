// The brotensor operators the brodiffusion attention path calls, implemented
// over the bdattn C ABI.  Names, argument order and meaning follow the call
// sites cited at each function; errors surface as std::runtime_error with the
// "<op>: message" text the library produces.
#pragma once

#include "bdattn.h"
#include "brotensor/tensor.h"

namespace brotensor {

namespace detail {
inline bdattn_stream_t bd_stream() { return reinterpret_cast<bdattn_stream_t>(cuda_current_stream()); }
inline int bd_dtype(Dtype d) {
    return d == Dtype::BF16 ? BDATTN_BF16 : (d == Dtype::FP16 ? BDATTN_F16 : BDATTN_F32);
}
inline void bd_check(int rc) { if (rc != 0) throw std::runtime_error(bdattn_last_error()); }
inline void require_gpu(const Tensor& t, const char* op) {
    if (!t.device.is_gpu()) throw std::runtime_error(std::string(op) + ": CPU tensors are not supported");
}
// Per-thread scratch for the fused QKVO operators, reused across calls
// (the reference keeps thread_local scratch in its dispatchers, src/fused.cpp:71,80).
// Deliberately never destroyed: freeing device memory from a thread-exit
// destructor can run after the CUDA runtime has shut down.
inline Tensor& qkvo_scratch() { static thread_local Tensor* t = new Tensor(); return *t; }
}  // namespace detail

// src/dit/common.cpp:194, src/dit/qwenimage21_forward.cpp:648,667,674, src/dit/sana.cpp:623
inline void flash_attention_forward(const Tensor& Q, const Tensor& K, const Tensor& V, const float* d_mask,
                                    int num_heads, bool causal, Tensor& O) {
    detail::require_gpu(Q, "flash_attention_forward");
    if (num_heads <= 0 || Q.cols % num_heads != 0 || K.cols != Q.cols || V.cols != Q.cols || K.rows != V.rows)
        throw std::runtime_error("flash_attention_forward: Q/K/V shapes do not agree with num_heads");
    O.resize(Q.rows, Q.cols, Q.dtype);
    bdattn_sdpa_params p{};
    p.dtype = detail::bd_dtype(Q.dtype);
    p.batch = 1; p.num_heads = num_heads; p.head_dim = Q.cols / num_heads;
    p.n_q_seg = 1; p.q[0] = Q.data; p.o[0] = O.data; p.q_rows[0] = Q.rows; p.q_ld[0] = Q.cols; p.o_ld[0] = O.cols;
    p.n_kv_seg = 1; p.k[0] = K.data; p.v[0] = V.data; p.kv_rows[0] = K.rows; p.k_ld[0] = K.cols; p.v_ld[0] = V.cols;
    p.mask_mode = causal ? BDATTN_MASK_CAUSAL : BDATTN_MASK_NONE;
    p.key_mask = d_mask;
    detail::bd_check(bdattn_sdpa_fwd(&p, detail::bd_stream()));
}

// src/dit/qwenimage21_forward.cpp:662 — window 0: unbounded causal with q_offset = Lk - Lq
inline void flash_attention_windowed_forward(const Tensor& Q, const Tensor& K, const Tensor& V,
                                             const float* d_mask, int num_heads, int window, Tensor& O) {
    if (window != 0) throw std::runtime_error("flash_attention_windowed_forward: only window = 0 is supported");
    flash_attention_forward(Q, K, V, d_mask, num_heads, /*causal=*/true, O);
}

// src/dit/common.cpp:192-193, src/dit/qwenimage21_forward.cpp:584-585
inline void rope_apply(const Tensor& X, const Tensor& cos, const Tensor& sin, int head_dim, int num_heads,
                       Tensor& Out) {
    detail::require_gpu(X, "rope_apply");
    if (cos.dtype != Dtype::FP32 || sin.dtype != Dtype::FP32) throw std::runtime_error("rope_apply: tables must be FP32");
    if (cos.rows < X.rows || cos.cols != head_dim / 2) throw std::runtime_error("rope_apply: table shape does not match");
    Out.resize(X.rows, X.cols, X.dtype);
    bdattn_norm_rope_job j{};
    j.x = X.data; j.out = Out.data; j.rows = X.rows; j.x_ld = X.cols; j.out_ld = Out.cols;
    j.cos = static_cast<const float*>(cos.data); j.sin = static_cast<const float*>(sin.data);
    detail::bd_check(bdattn_rmsnorm_rope(&j, 1, detail::bd_dtype(X.dtype), num_heads, head_dim, 0.0f,
                                         BDATTN_ROPE_INTERLEAVED, detail::bd_stream()));
}

// src/dit/flux.cpp:467, src/dit/qwenimage21_forward.cpp:59 — X is the (L*nh, hd) per-head view
inline void rms_norm_forward(const Tensor& X, const Tensor& gain, float eps, Tensor& Out) {
    detail::require_gpu(X, "rms_norm_forward");
    if (static_cast<int>(gain.size()) != X.cols) throw std::runtime_error("rms_norm_forward: gain length must equal the column count");
    Out.resize(X.rows, X.cols, X.dtype);
    bdattn_norm_rope_job j{};
    j.x = X.data; j.out = Out.data; j.rows = X.rows; j.x_ld = X.cols; j.out_ld = Out.cols;
    j.gain = gain.data; j.gain_dtype = detail::bd_dtype(gain.dtype);
    detail::bd_check(bdattn_rmsnorm_rope(&j, 1, detail::bd_dtype(X.dtype), /*num_heads=*/1, /*head_dim=*/X.cols, eps,
                                         BDATTN_ROPE_INTERLEAVED, detail::bd_stream()));
}

namespace detail {
inline void qkvo(const char*, const Tensor& X, const Tensor* Ctx, const Tensor* Kc, const Tensor* Vc, const Tensor& Wq,
                 const Tensor* bq, const Tensor* Wk, const Tensor* bk, const Tensor* Wv, const Tensor* bv,
                 const Tensor& Wo, const Tensor* bo, const float* d_mask, int num_heads, bool causal, Tensor& Out) {
    const int inner = Wq.rows;
    const int kv_rows = Kc ? Kc->rows : (Ctx ? Ctx->rows : X.rows);
    Out.resize(X.rows, Wo.rows, X.dtype);
    const std::size_t need = bdattn_qkvo_workspace_bytes(X.rows, kv_rows, num_heads, inner / (num_heads > 0 ? num_heads : 1));
    Tensor& ws = qkvo_scratch();
    if (ws.bytes() < need) ws.resize(1, static_cast<int>(need), Dtype::INT8);
    bdattn_qkvo_params p{};
    p.dtype = bd_dtype(X.dtype); p.num_heads = num_heads; p.inner_dim = inner; p.causal = causal ? 1 : 0;
    p.x = X.data; p.x_rows = X.rows; p.x_cols = X.cols; p.x_ld = X.cols;
    if (Ctx) { p.ctx = Ctx->data; p.ctx_rows = Ctx->rows; p.ctx_cols = Ctx->cols; p.ctx_ld = Ctx->cols; }
    p.wq = Wq.data; p.bq = bq ? bq->data : nullptr;
    p.wk = Wk ? Wk->data : nullptr; p.bk = bk ? bk->data : nullptr;
    p.wv = Wv ? Wv->data : nullptr; p.bv = bv ? bv->data : nullptr;
    p.wo = Wo.data; p.bo = bo ? bo->data : nullptr;
    if (Kc) { p.k_cached = Kc->data; p.v_cached = Vc->data; p.kv_rows = Kc->rows; p.k_ld = Kc->cols; p.v_ld = Vc->cols; }
    p.key_mask = d_mask;
    p.out = Out.data; p.out_cols = Out.cols; p.out_ld = Out.cols;
    p.workspace = ws.data; p.workspace_bytes = ws.bytes();
    bd_check(bdattn_qkvo_fwd(&p, bd_stream()));
}
}  // namespace detail

// src/unet_blocks.cpp:264-271 (self-attention, Ctx == nullptr) and 320-327 (cross-attention)
inline void flash_attention_qkvo_forward(const Tensor& X, const Tensor* Ctx, const Tensor& Wq, const Tensor* bq,
                                         const Tensor& Wk, const Tensor* bk, const Tensor& Wv, const Tensor* bv,
                                         const Tensor& Wo, const Tensor* bo, const float* d_mask, int num_heads,
                                         bool causal, Tensor& Out) {
    detail::require_gpu(X, "flash_attention_qkvo_forward");
    detail::qkvo("flash_attention_qkvo_forward", X, Ctx, nullptr, nullptr, Wq, bq, &Wk, bk, &Wv, bv, Wo, bo, d_mask,
                 num_heads, causal, Out);
}

// src/unet_blocks.cpp:302-307
inline void flash_attention_q_with_kv_cached_forward(const Tensor& X, const Tensor& K, const Tensor& V,
                                                     const Tensor& Wq, const Tensor* bq, const Tensor& Wo,
                                                     const Tensor* bo, const float* d_mask, int num_heads,
                                                     bool causal, Tensor& Out) {
    detail::require_gpu(X, "flash_attention_q_with_kv_cached_forward");
    detail::qkvo("flash_attention_q_with_kv_cached_forward", X, nullptr, &K, &V, Wq, bq, nullptr, nullptr, nullptr,
                 nullptr, Wo, bo, d_mask, num_heads, causal, Out);
}

// src/unet.cpp:476-480
inline void flash_attention_project_kv(const Tensor& ctx, const Tensor& Wk, const Tensor* bk, const Tensor& Wv,
                                       const Tensor* bv, Tensor& K, Tensor& V) {
    detail::require_gpu(ctx, "flash_attention_project_kv");
    K.resize(ctx.rows, Wk.rows, ctx.dtype);
    V.resize(ctx.rows, Wv.rows, ctx.dtype);
    detail::bd_check(bdattn_project_kv(ctx.data, ctx.rows, ctx.cols, ctx.cols, Wk.data, bk ? bk->data : nullptr, Wv.data,
                                       bv ? bv->data : nullptr, K.data, V.data, K.cols, Wk.rows,
                                       detail::bd_dtype(ctx.dtype), detail::bd_stream()));
}

// src/dit/sana.cpp:441-443: C (batch, M, N) = A (batch, M, K) . B (batch, N, K)^T, the
// "A . B^T" product Sana uses to project straight into the channel-major (D, N)
// layout (A = W (D, D), B = x_mod (N, D), C = q (D, N); batch 1, strides 0).
// strideA/B/C are the element distances between batch items.  The batched
// calls inside the Sana attention core (sana.cpp:538-568) are replaced as a
// whole by bdattn_linear_attn_relu_fwd; they still run here, one launch per
// batch item.  The call sites on this path pass no bias (nullptr, 0).
inline void matmul_abt(const Tensor& A, const Tensor& B, Tensor& C, int batch, int M, int N, int K,
                       long long strideA, long long strideB, long long strideC, const Tensor* bias,
                       int bias_mode) {
    detail::require_gpu(A, "matmul_abt");
    if (bias != nullptr || bias_mode != 0) throw std::runtime_error("matmul_abt: a bias is not supported");
    if (A.dtype != B.dtype || (A.dtype != Dtype::BF16 && A.dtype != Dtype::FP16))
        throw std::runtime_error("matmul_abt: operands must both be FP16 or both BF16");
    if (batch < 1 || static_cast<long long>(A.size()) < (batch - 1) * strideA + static_cast<long long>(M) * K ||
        static_cast<long long>(B.size()) < (batch - 1) * strideB + static_cast<long long>(N) * K)
        throw std::runtime_error("matmul_abt: operand sizes do not cover batch x (M, K) and batch x (N, K)");
    if (C.data == nullptr || static_cast<long long>(C.size()) < (batch - 1) * strideC + static_cast<long long>(M) * N ||
        C.dtype != A.dtype)
        C.resize(batch == 1 ? M : batch * M, N, A.dtype);
    const std::size_t es = dtype_size(A.dtype);
    for (int b = 0; b < batch; ++b) {
        detail::bd_check(bdattn_linear_fwd(static_cast<const char*>(A.data) + b * strideA * es,
                                           static_cast<const char*>(B.data) + b * strideB * es, nullptr,
                                           static_cast<char*>(C.data) + b * strideC * es, detail::bd_dtype(A.dtype), M, N,
                                           K, K, K, N, detail::bd_stream()));
    }
}

// src/unet_blocks.cpp:282-290 (trace mode of the SD1.5 cross-attention): bias-free
// Q/K/V projections, attention with an optional FP32 (Lq, Lk) logit bias added to
// the scaled scores, bias-free output projection, and the head-averaged softmax
// map (Lq, Lk) in AttnAvg (FP32).  The reference's operator recomputes the softmax
// to expose it; here the attention kernel writes per-row statistics and a small
// kernel evaluates the map from them (bdattn_sdpa_traced_fwd).
inline void cross_attention_forward_with_attn(const Tensor& X, const Tensor& Ctx, const Tensor& Wq, const Tensor& Wk,
                                              const Tensor& Wv, const Tensor& Wo, const float* d_mask,
                                              const Tensor* attn_logit_bias, int num_heads, Tensor& Out,
                                              Tensor& AttnAvg) {
    detail::require_gpu(X, "cross_attention_forward_with_attn");
    const int Lq = X.rows, Lk = Ctx.rows, inner = Wq.rows;
    if (num_heads <= 0 || inner % num_heads != 0 || Wk.rows != inner || Wv.rows != inner || Wo.cols != inner ||
        Wq.cols != X.cols || Wk.cols != Ctx.cols || Wv.cols != Ctx.cols)
        throw std::runtime_error("cross_attention_forward_with_attn: weight shapes do not agree");
    if (attn_logit_bias != nullptr &&
        (attn_logit_bias->dtype != Dtype::FP32 || attn_logit_bias->rows != Lq || attn_logit_bias->cols != Lk))
        throw std::runtime_error("cross_attention_forward_with_attn: attn_logit_bias must be FP32 (Lq, Lk)");
    const int dt = detail::bd_dtype(X.dtype);
    Tensor Q, K, V, O, ws;
    Q.resize(Lq, inner, X.dtype); K.resize(Lk, inner, X.dtype); V.resize(Lk, inner, X.dtype); O.resize(Lq, inner, X.dtype);
    detail::bd_check(bdattn_linear_fwd(X.data, Wq.data, nullptr, Q.data, dt, Lq, inner, X.cols, X.cols, Wq.cols, inner,
                                       detail::bd_stream()));
    detail::bd_check(bdattn_project_kv(Ctx.data, Lk, Ctx.cols, Ctx.cols, Wk.data, nullptr, Wv.data, nullptr, K.data,
                                       V.data, inner, inner, dt, detail::bd_stream()));
    AttnAvg.resize(Lq, Lk, Dtype::FP32);
    const std::size_t need = bdattn_sdpa_traced_workspace_bytes(num_heads, Lq);
    ws.resize(1, static_cast<int>(need), Dtype::INT8);
    bdattn_sdpa_params p{};
    p.dtype = dt; p.batch = 1; p.num_heads = num_heads; p.head_dim = inner / num_heads;
    p.n_q_seg = 1; p.q[0] = Q.data; p.o[0] = O.data; p.q_rows[0] = Lq; p.q_ld[0] = inner; p.o_ld[0] = inner;
    p.n_kv_seg = 1; p.k[0] = K.data; p.v[0] = V.data; p.kv_rows[0] = Lk; p.k_ld[0] = inner; p.v_ld[0] = inner;
    p.key_mask = d_mask;
    bdattn_trace_params t{};
    if (attn_logit_bias != nullptr) {
        t.bias = static_cast<const float*>(attn_logit_bias->data);
        t.bias_rows = Lq; t.bias_cols = Lk; t.bias_ld = Lk;
    }
    t.attn_avg = static_cast<float*>(AttnAvg.data); t.map_rows = Lq; t.map_cols = Lk; t.map_ld = Lk;
    t.workspace = ws.data; t.workspace_bytes = ws.bytes();
    detail::bd_check(bdattn_sdpa_traced_fwd(&p, &t, detail::bd_stream()));
    Out.resize(Lq, Wo.rows, X.dtype);
    detail::bd_check(bdattn_linear_fwd(O.data, Wo.data, nullptr, Out.data, dt, Lq, Wo.rows, inner, inner, inner, Wo.rows,
                                       detail::bd_stream()));
    // the temporaries are freed when this returns: wait for the kernels that use them
    cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_current_stream())), "cross_attention_forward_with_attn");
}

// src/dit/qwenimage21_hooks.cpp:91-96 (QwenImage21PrefixCache::scale_kv)
inline void scale_inplace(Tensor& Y, float a) {
    detail::require_gpu(Y, "scale_inplace");
    detail::bd_check(bdattn_axpby_inplace(Y.data, nullptr, static_cast<long long>(Y.size()), a, 0.0f,
                                          detail::bd_dtype(Y.dtype), detail::bd_stream()));
}
// src/dit/qwenimage21_hooks.cpp:117-122 (QwenImage21PrefixCache::blend_from): y = a*y + b*x
inline void axpby_inplace(Tensor& Y, const Tensor& X, float a, float b) {
    detail::require_gpu(Y, "axpby_inplace");
    if (Y.rows != X.rows || Y.cols != X.cols || Y.dtype != X.dtype)
        throw std::runtime_error("axpby_inplace: Y and X must have the same shape and dtype");
    detail::bd_check(bdattn_axpby_inplace(Y.data, X.data, static_cast<long long>(Y.size()), a, b,
                                          detail::bd_dtype(Y.dtype), detail::bd_stream()));
}

}  // namespace brotensor
