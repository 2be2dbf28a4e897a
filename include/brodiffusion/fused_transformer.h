// SD1.5 fused transformer ops over the bdattn library.  Same entry points,
// argument meaning and refusals as include/brodiffusion/fused_transformer.h:32-61
// of the reference (16-bit GPU tensors only; CPU tensors are refused,
// src/fused.cpp:43-46).
#pragma once

#include "brotensor/ops.h"

namespace brodiffusion {

namespace bt = ::brotensor;

// Y(B, D_out) = a * gelu_exact(g), [a | g] = X W^T + b; W (2*D_out, D_in), b (2*D_out).
inline void fused_linear_geglu(const bt::Tensor& X, const bt::Tensor& W, const bt::Tensor& b, bt::Tensor& Y) {
    if (!X.device.is_gpu()) throw std::runtime_error("fused_linear_geglu: CPU tensors are not supported");
    if (W.cols != X.cols || W.rows % 2 != 0 || static_cast<int>(b.size()) != W.rows)
        throw std::runtime_error("fused_linear_geglu: W must be (2*D_out, D_in) and b (2*D_out)");
    Y.resize(X.rows, W.rows / 2, X.dtype);
    bt::detail::bd_check(bdattn_linear_geglu_fwd(X.data, W.data, b.data, Y.data, bt::detail::bd_dtype(X.dtype), X.rows,
                                                 X.cols, W.rows / 2, bt::detail::bd_stream()));
}

// Y[i] += X[i]; same shape.
inline void add_inplace_vec(bt::Tensor& Y, const bt::Tensor& X) {
    if (Y.rows != X.rows || Y.cols != X.cols) throw std::runtime_error("add_inplace_vec: Y and X must have the same shape");
    bt::detail::bd_check(bdattn_add_inplace(Y.data, X.data, static_cast<long long>(Y.size()),
                                            bt::detail::bd_dtype(Y.dtype), bt::detail::bd_stream()));
}

// Y[i, j] += bias[j]; bias has cols values, as (cols, 1) or (1, cols).
inline void add_inplace_row_bias(bt::Tensor& Y, const bt::Tensor& bias) {
    if (static_cast<int>(bias.size()) != Y.cols) throw std::runtime_error("add_inplace_row_bias: bias length must equal Y.cols");
    bt::detail::bd_check(bdattn_add_row_bias(Y.data, bias.data, Y.rows, Y.cols, Y.cols, bt::detail::bd_dtype(Y.dtype),
                                             bt::detail::bd_stream()));
}

}  // namespace brodiffusion
