// Per-head RMSNorm followed by the rotary embedding, one pass over the tensor.
//
// One warp owns one (token, head) row of head_dim elements.  Lane l handles
// rotary pairs l, l+32, ...; with the interleaved convention a pair is one
// aligned 32-bit word, so a warp reads and writes whole 128-byte lines.
// The sum of squares is accumulated in FP32 (src/dit/qwenimage21.cpp:335-337)
// and the result is rounded to the storage type once, after the rotation.
// Up to four independent jobs (tensor, gain, table offset) share one launch:
// blockIdx.y selects the job.  HBM-bound: 2 bytes read + 2 bytes written per
// element, plus the FP32 tables (shared by all heads of a token).
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

constexpr int kNormWarps = 8;

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (kBf16) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w);
        return __half22float2(h);
    }
}
template <bool kBf16>
__device__ __forceinline__ float load1(const void* p, long long i) {
    if constexpr (kBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    else return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
template <bool kBf16>
__device__ __forceinline__ void store1(void* p, long long i, float v) {
    if constexpr (kBf16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

template <bool kBf16>
__global__ void __launch_bounds__(kNormWarps * 32) norm_rope_kernel(const NormRopeArgs a) {
    const NormRopeJobDev& job = a.job[blockIdx.y];
    const int lane = threadIdx.x & 31;
    const int hd = a.head_dim;
    const int half = hd >> 1;
    const long long n_units = static_cast<long long>(job.rows) * a.num_heads;
    const long long stride = static_cast<long long>(gridDim.x) * kNormWarps;
    for (long long u = static_cast<long long>(blockIdx.x) * kNormWarps + (threadIdx.x >> 5); u < n_units;
         u += stride) {
        const int row = static_cast<int>(u / a.num_heads);
        const int head = static_cast<int>(u - static_cast<long long>(row) * a.num_heads);
        const long long xoff = static_cast<long long>(row) * job.x_ld + static_cast<long long>(head) * hd;
        const long long ooff = static_cast<long long>(row) * job.out_ld + static_cast<long long>(head) * hd;
        // Each lane keeps up to 4 pairs (head_dim <= 256).
        float xa[4], xb[4];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = lane + 32 * i;
            xa[i] = 0.0f;
            xb[i] = 0.0f;
            if (p < half) {
                if (a.pair_mode == 0) {
                    const uint32_t w = reinterpret_cast<const uint32_t*>(
                        reinterpret_cast<const uint16_t*>(job.x) + xoff)[p];
                    const float2 f = unpack2<kBf16>(w);
                    xa[i] = f.x;
                    xb[i] = f.y;
                } else {
                    xa[i] = load1<kBf16>(job.x, xoff + p);
                    xb[i] = load1<kBf16>(job.x, xoff + p + half);
                }
                ss += xa[i] * xa[i] + xb[i] * xb[i];
            }
        }
        float inv = 1.0f;
        if (job.gain != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            inv = rsqrtf(ss / static_cast<float>(hd) + a.eps);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = lane + 32 * i;
            if (p < half) {
                const int ia = a.pair_mode == 0 ? 2 * p : p;
                const int ib = a.pair_mode == 0 ? 2 * p + 1 : p + half;
                float va = xa[i], vb = xb[i];
                if (job.gain != nullptr) {
                    float ga, gb;
                    if (job.gain_is_f32) {
                        ga = reinterpret_cast<const float*>(job.gain)[ia];
                        gb = reinterpret_cast<const float*>(job.gain)[ib];
                    } else {
                        ga = load1<kBf16>(job.gain, ia);
                        gb = load1<kBf16>(job.gain, ib);
                    }
                    va = va * inv * ga;
                    vb = vb * inv * gb;
                }
                if (job.cos != nullptr) {
                    const long long t = static_cast<long long>(job.rope_row0 + row) * half + p;
                    const float c = __ldg(job.cos + t);
                    const float s = __ldg(job.sin + t);
                    const float ra = va * c - vb * s;
                    const float rb = va * s + vb * c;
                    va = ra;
                    vb = rb;
                }
                if (a.pair_mode == 0) {
                    reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(job.out) + ooff)[p] =
                        pack2<kBf16>(va, vb);
                } else {
                    store1<kBf16>(job.out, ooff + ia, va);
                    store1<kBf16>(job.out, ooff + ib, vb);
                }
            }
        }
    }
}

}  // namespace

cudaError_t launch_norm_rope(const NormRopeArgs& a, bool bf16, cudaStream_t stream) {
    long long max_units = 0;
    for (int i = 0; i < a.n_jobs; ++i) {
        const long long u = static_cast<long long>(a.job[i].rows) * a.num_heads;
        if (u > max_units) max_units = u;
    }
    long long blocks = (max_units + kNormWarps - 1) / kNormWarps;
    const long long cap = 148LL * 16;  // 16 resident 256-thread CTAs per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.n_jobs));
    if (bf16) norm_rope_kernel<true><<<grid, kNormWarps * 32, 0, stream>>>(a);
    else norm_rope_kernel<false><<<grid, kNormWarps * 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace bdattn
