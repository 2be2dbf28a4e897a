// Per-head RMSNorm followed by the rotary embedding, one pass over the tensor.
//
// Fast path (interleaved pairs, head_dim in {8, 16, 32, 64, 128, 256}, 16-byte
// aligned rows): a warp takes one token row and walks its heads; every lane owns
// 8 consecutive elements (one 16-byte vector, four rotary pairs) of a head,
// head_dim/8 neighbouring lanes share a head and reduce its sum of squares by
// shuffles, the lane's slice of the row's cos / sin entries is loaded once and
// reused for every head, and six vectors per lane are in flight so that enough
// bytes are outstanding to fill HBM.  General path: one warp per (token, head) row, lane l handles rotary
// pairs l, l+32, ...
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

// First CTA of each job in a launch that numbers its CTAs across the jobs.
struct NormRopeGrid {
    int block_begin[5];
};

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


// ---------------------------------------------------------------- fast path
// One warp per token row, all heads of the row: the row's cos / sin slice is the
// same for every head, so a lane loads it once and keeps it in registers while
// the warp walks the heads (32 / kLpu heads at a time, kUnroll vectors per lane
// in flight).  CTAs are numbered across the jobs of the launch (block_begin),
// so a short job (the 512 text rows next to 4096 image rows) brings no idle CTAs.
template <bool kBf16, int kLpu>   // kLpu = lanes per (token, head) row = head_dim / 8
__global__ void __launch_bounds__(256, 4) norm_rope_vec_kernel(const NormRopeArgs a, const NormRopeGrid g4) {
    constexpr int kUnroll = 6;
    constexpr int kHeadsPerStep = 32 / kLpu;
    dependents_may_launch();
    wait_for_prior_grid();
    int j = 0;
#pragma unroll
    for (int i = 1; i < 4; ++i) j += (i < a.n_jobs && static_cast<int>(blockIdx.x) >= g4.block_begin[i]) ? 1 : 0;
    const NormRopeJobDev& job = a.job[j];
    const int lane = threadIdx.x & 31;
    const int l = lane % kLpu;                 // this lane's 8-element slot inside the head
    const int sub = lane / kLpu;               // which head of the step
    const int hd = kLpu * 8;
    const int half = hd / 2;
    const int nh = a.num_heads;
    const int warps = blockDim.x >> 5;
    const int row_stride = (g4.block_begin[j + 1] - g4.block_begin[j]) * warps;

    float g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = 1.0f;
    if (job.gain != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            g[i] = job.gain_is_f32 ? reinterpret_cast<const float*>(job.gain)[l * 8 + i]
                                   : load1<kBf16>(job.gain, l * 8 + i);
        }
    }
    const float inv_hd = 1.0f / static_cast<float>(hd);
    const uint16_t* xin = reinterpret_cast<const uint16_t*>(job.x);
    uint16_t* xout = reinterpret_cast<uint16_t*>(job.out);

    for (int row = (static_cast<int>(blockIdx.x) - g4.block_begin[j]) * warps + (threadIdx.x >> 5); row < job.rows;
         row += row_stride) {
        float c[4] = {1.0f, 1.0f, 1.0f, 1.0f}, sn[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (job.cos != nullptr) {
            const long long t = static_cast<long long>(job.rope_row0 + row) * half + l * 4;
            const float4 cv = __ldg(reinterpret_cast<const float4*>(job.cos + t));
            const float4 sv = __ldg(reinterpret_cast<const float4*>(job.sin + t));
            c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
            sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
        }
        const uint16_t* xrow = xin + static_cast<long long>(row) * job.x_ld + l * 8;
        uint16_t* orow = xout + static_cast<long long>(row) * job.out_ld + l * 8;
        for (int h0 = 0; h0 < nh; h0 += kHeadsPerStep * kUnroll) {
            uint4 v[kUnroll];
#pragma unroll
            for (int it = 0; it < kUnroll; ++it) {
                const int head = h0 + it * kHeadsPerStep + sub;
                v[it] = head < nh ? *reinterpret_cast<const uint4*>(xrow + head * hd) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int it = 0; it < kUnroll; ++it) {
                const int head = h0 + it * kHeadsPerStep + sub;
                float2 p[4];
                p[0] = unpack2<kBf16>(v[it].x);
                p[1] = unpack2<kBf16>(v[it].y);
                p[2] = unpack2<kBf16>(v[it].z);
                p[3] = unpack2<kBf16>(v[it].w);
                if (job.gain != nullptr) {
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) ss += p[i].x * p[i].x + p[i].y * p[i].y;
#pragma unroll
                    for (int o = kLpu / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    const float inv = rsqrtf(ss * inv_hd + a.eps);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        p[i].x = p[i].x * inv * g[2 * i];
                        p[i].y = p[i].y * inv * g[2 * i + 1];
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float ra = p[i].x * c[i] - p[i].y * sn[i];
                    const float rb = p[i].x * sn[i] + p[i].y * c[i];
                    p[i].x = ra;
                    p[i].y = rb;
                }
                if (head < nh) {
                    uint4 w;
                    w.x = pack2<kBf16>(p[0].x, p[0].y);
                    w.y = pack2<kBf16>(p[1].x, p[1].y);
                    w.z = pack2<kBf16>(p[2].x, p[2].y);
                    w.w = pack2<kBf16>(p[3].x, p[3].y);
                    *reinterpret_cast<uint4*>(orow + head * hd) = w;
                }
            }
        }
    }
}

template <bool kBf16>
cudaError_t launch_vec(const NormRopeArgs& a, const NormRopeGrid& g4, int lpu, dim3 grid, cudaStream_t stream) {
    switch (lpu) {
        case 1: return launch_dependent(norm_rope_vec_kernel<kBf16, 1>, grid, dim3(256), 0, stream, a, g4);
        case 2: return launch_dependent(norm_rope_vec_kernel<kBf16, 2>, grid, dim3(256), 0, stream, a, g4);
        case 4: return launch_dependent(norm_rope_vec_kernel<kBf16, 4>, grid, dim3(256), 0, stream, a, g4);
        case 8: return launch_dependent(norm_rope_vec_kernel<kBf16, 8>, grid, dim3(256), 0, stream, a, g4);
        case 16: return launch_dependent(norm_rope_vec_kernel<kBf16, 16>, grid, dim3(256), 0, stream, a, g4);
        default: return launch_dependent(norm_rope_vec_kernel<kBf16, 32>, grid, dim3(256), 0, stream, a, g4);
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_norm_rope(const NormRopeArgs& a, bool bf16, cudaStream_t stream) {
    long long max_units = 0;
    for (int i = 0; i < a.n_jobs; ++i) {
        const long long u = static_cast<long long>(a.job[i].rows) * a.num_heads;
        if (u > max_units) max_units = u;
    }
    // Vector path when every job is 16-byte aligned and the head is a
    // power-of-two number of 8-element slots.
    const int hd = a.head_dim;
    bool vec = a.pair_mode == 0 && hd % 8 == 0 && ((hd / 8) & (hd / 8 - 1)) == 0 && hd <= 256 &&
               max_units < (1LL << 31);
    for (int i = 0; i < a.n_jobs && vec; ++i) {
        const NormRopeJobDev& j = a.job[i];
        if ((reinterpret_cast<uintptr_t>(j.x) & 15u) || (reinterpret_cast<uintptr_t>(j.out) & 15u) ||
            (j.x_ld & 7) || (j.out_ld & 7))
            vec = false;
        if (j.cos != nullptr && ((reinterpret_cast<uintptr_t>(j.cos) & 15u) ||
                                 (reinterpret_cast<uintptr_t>(j.sin) & 15u) || ((hd / 2) & 3)))
            vec = false;
    }
    if (vec) {
        const int lpu = hd / 8;
        // one warp per row; a long job is capped and its warps stride over the rows
        long long total_rows = 0;
        for (int i = 0; i < a.n_jobs; ++i) total_rows += a.job[i].rows;
        const long long cap = static_cast<long long>(sm_count()) * 64;      // CTAs of the whole launch
        NormRopeGrid g4 = {};
        int begin = 0;
        for (int i = 0; i < 4; ++i) {
            g4.block_begin[i] = begin;
            if (i < a.n_jobs) {
                long long blocks = (a.job[i].rows + 7) / 8;
                const long long share = (cap * a.job[i].rows + total_rows - 1) / total_rows;
                if (blocks > share) blocks = share;
                if (blocks < 1) blocks = 1;
                begin += static_cast<int>(blocks);
            }
        }
        g4.block_begin[4] = begin;
        for (int i = a.n_jobs; i < 4; ++i) g4.block_begin[i + 1] = begin;
        dim3 grid(static_cast<unsigned>(begin));
        return bf16 ? launch_vec<true>(a, g4, lpu, grid, stream) : launch_vec<false>(a, g4, lpu, grid, stream);
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
