// Small bandwidth-bound helpers next to the attention operators.
//   add_inplace      Y += X            (src/fused_transformer.cu:430-451)
//   add_row_bias     Y[i, j] += b[j]   (src/fused_transformer.cu:413-428)
//   axpby_inplace    Y = a*Y + b*X     (prefix-cache scale_kv / blend_from,
//                    src/dit/qwenimage21_hooks.cpp:79-124; X null: Y = a*Y)
//   pad_heads        (rows, nh*hd) -> (rows, nh*hd_pad), zero padded, for
//                    feeding cached K/V of head_dim 40 / 80 to the tensor-core
//                    attention kernel (which takes 64 / 128).
// 16-byte vectors where alignment allows; grid sized to the SM count.
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

template <bool kBf16>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    if constexpr (kBf16) {
        const float lo = __uint_as_float(a << 16) + __uint_as_float(b << 16);
        const float hi = __uint_as_float(a & 0xffff0000u) + __uint_as_float(b & 0xffff0000u);
        return pack2<true>(lo, hi);
    } else {
        __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
}
template <bool kBf16>
__device__ __forceinline__ uint16_t add1(uint16_t a, uint16_t b) {
    if constexpr (kBf16) {
        const float r = __uint_as_float(static_cast<uint32_t>(a) << 16) + __uint_as_float(static_cast<uint32_t>(b) << 16);
        __nv_bfloat16 h = __float2bfloat16_rn(r);
        return *reinterpret_cast<uint16_t*>(&h);
    } else {
        __half r = __hadd(*reinterpret_cast<const __half*>(&a), *reinterpret_cast<const __half*>(&b));
        return *reinterpret_cast<uint16_t*>(&r);
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) add_inplace_kernel(uint16_t* y, const uint16_t* x, long long n, int vec_ok) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    long long done = 0;
    if (vec_ok) {
        const long long nv = n / 8;
        uint4* yv = reinterpret_cast<uint4*>(y);
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        for (long long i = tid; i < nv; i += nthreads) {
            uint4 a = yv[i];
            const uint4 b = xv[i];
            a.x = add2<kBf16>(a.x, b.x);
            a.y = add2<kBf16>(a.y, b.y);
            a.z = add2<kBf16>(a.z, b.z);
            a.w = add2<kBf16>(a.w, b.w);
            yv[i] = a;
        }
        done = nv * 8;
    }
    for (long long i = done + tid; i < n; i += nthreads) y[i] = add1<kBf16>(y[i], x[i]);
}

// a*y + b*x with both products and the sum rounded to FP32 separately (no
// contraction), then one rounding to the storage type.
template <bool kBf16>
__device__ __forceinline__ uint16_t axpby1(uint16_t y, uint16_t x, float a, float b) {
    float fy, fx;
    if constexpr (kBf16) {
        fy = __uint_as_float(static_cast<uint32_t>(y) << 16);
        fx = __uint_as_float(static_cast<uint32_t>(x) << 16);
    } else {
        fy = __half2float(*reinterpret_cast<const __half*>(&y));
        fx = __half2float(*reinterpret_cast<const __half*>(&x));
    }
    const float r = __fadd_rn(__fmul_rn(a, fy), __fmul_rn(b, fx));
    if constexpr (kBf16) {
        __nv_bfloat16 h = __float2bfloat16_rn(r);
        return *reinterpret_cast<uint16_t*>(&h);
    } else {
        __half h = __float2half_rn(r);
        return *reinterpret_cast<uint16_t*>(&h);
    }
}
template <bool kBf16>
__device__ __forceinline__ uint32_t axpby2(uint32_t y, uint32_t x, float a, float b) {
    return static_cast<uint32_t>(axpby1<kBf16>(static_cast<uint16_t>(y & 0xffffu), static_cast<uint16_t>(x & 0xffffu), a, b)) |
           (static_cast<uint32_t>(axpby1<kBf16>(static_cast<uint16_t>(y >> 16), static_cast<uint16_t>(x >> 16), a, b)) << 16);
}

// x may be null (pure scaling): it is then never read and b is taken as 0.
template <bool kBf16>
__global__ void __launch_bounds__(256) axpby_inplace_kernel(uint16_t* y, const uint16_t* x, long long n, float a,
                                                            float b, int vec_ok) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    long long done = 0;
    if (vec_ok) {
        const long long nv = n / 8;
        uint4* yv = reinterpret_cast<uint4*>(y);
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        for (long long i = tid; i < nv; i += nthreads) {
            uint4 v = yv[i];
            const uint4 w = x != nullptr ? xv[i] : make_uint4(0, 0, 0, 0);
            v.x = axpby2<kBf16>(v.x, w.x, a, b);
            v.y = axpby2<kBf16>(v.y, w.y, a, b);
            v.z = axpby2<kBf16>(v.z, w.z, a, b);
            v.w = axpby2<kBf16>(v.w, w.w, a, b);
            yv[i] = v;
        }
        done = nv * 8;
    }
    for (long long i = done + tid; i < n; i += nthreads)
        y[i] = axpby1<kBf16>(y[i], x != nullptr ? x[i] : static_cast<uint16_t>(0), a, b);
}

template <bool kBf16>
__global__ void __launch_bounds__(256) add_row_bias_kernel(uint16_t* y, const uint16_t* bias, long long rows,
                                                           long long cols, long long ld) {
    const long long n = rows * cols;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += nthreads) {
        const long long r = i / cols, c = i - r * cols;
        y[r * ld + c] = add1<kBf16>(y[r * ld + c], bias[c]);
    }
}

__global__ void __launch_bounds__(256) pad_heads_kernel(const uint16_t* src, uint16_t* dst, int rows, int nh,
                                                        int hd, int hd_pad, long long src_ld) {
    // one thread per 8-element (16-byte) group of the padded row
    const int groups = hd_pad / 8;
    const long long n = static_cast<long long>(rows) * nh * groups;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += nthreads) {
        const int gi = static_cast<int>(i % groups);
        const long long rh = i / groups;
        const int h = static_cast<int>(rh % nh);
        const long long r = rh / nh;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (gi * 8 < hd) v = *reinterpret_cast<const uint4*>(src + r * src_ld + h * hd + gi * 8);
        *reinterpret_cast<uint4*>(dst + (r * nh + h) * hd_pad + gi * 8) = v;
    }
}

unsigned grid_for(long long work_items) {
    long long b = (work_items + 255) / 256;
    const long long cap = 148LL * 8;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return static_cast<unsigned>(b);
}

}  // namespace

cudaError_t launch_add_inplace(void* y, const void* x, long long n, bool bf16, cudaStream_t stream) {
    const int vec_ok = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
    const unsigned g = grid_for(vec_ok ? (n + 7) / 8 : n);
    if (bf16) add_inplace_kernel<true><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(x), n, vec_ok);
    else add_inplace_kernel<false><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(x), n, vec_ok);
    return cudaGetLastError();
}

cudaError_t launch_axpby_inplace(void* y, const void* x, long long n, float a, float b, bool bf16,
                                 cudaStream_t stream) {
    const int vec_ok = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
    const unsigned g = grid_for(vec_ok ? (n + 7) / 8 : n);
    if (x == nullptr) b = 0.0f;
    if (bf16) axpby_inplace_kernel<true><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(x), n, a, b, vec_ok);
    else axpby_inplace_kernel<false><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(x), n, a, b, vec_ok);
    return cudaGetLastError();
}

cudaError_t launch_add_row_bias(void* y, const void* bias, long long rows, long long cols, long long ld,
                                bool bf16, cudaStream_t stream) {
    const unsigned g = grid_for(rows * cols);
    if (bf16) add_row_bias_kernel<true><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(bias), rows, cols, ld);
    else add_row_bias_kernel<false><<<g, 256, 0, stream>>>(static_cast<uint16_t*>(y), static_cast<const uint16_t*>(bias), rows, cols, ld);
    return cudaGetLastError();
}

cudaError_t launch_pad_heads(const void* src, void* dst, int rows, int num_heads, int hd, int hd_pad,
                             long long src_ld, cudaStream_t stream) {
    const unsigned g = grid_for(static_cast<long long>(rows) * num_heads * (hd_pad / 8));
    pad_heads_kernel<<<g, 256, 0, stream>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), rows,
                                            num_heads, hd, hd_pad, src_ld);
    return cudaGetLastError();
}

}  // namespace bdattn
