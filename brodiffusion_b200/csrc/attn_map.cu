// Head-averaged softmax map for traced attention.
//
// The reference's trace mode recomputes attention on the host to expose the
// softmax (dit::joint_attention_traced, src/dit/common.cpp:198-329, keeps the
// image-query x text-key block, src/dit/flux.cpp:505-508; the U-Net uses
// brotensor::cross_attention_forward_with_attn, src/unet_blocks.cpp:282-290).
// Here the attention kernel writes each row's softmax statistics (reference
// maximum and row sum) and this kernel evaluates only the requested block of
// the map from them:  avg_h exp2((q.k * scale + bias) * log2e - m) / l.
// One CTA = 32 query rows x 32 keys, looping over the heads; CUDA-core FMA
// (the block is a small fraction of the score matrix).
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

template <bool kBf16>
__device__ __forceinline__ float map_ld16(const void* p, long long i) {
    if constexpr (kBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    else return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

template <bool kBf16>
__global__ void __launch_bounds__(128) attn_map_kernel(const AttnMapArgs a) {
    extern __shared__ float msm[];
    const int hd = a.head_dim, hdp = hd + 1;
    float* Qs = msm;               // [32][hdp]
    float* Ks = msm + 32 * hdp;    // [32][hdp]
    const int tid = threadIdx.x, r = tid >> 2, c4 = tid & 3;
    const int key0 = blockIdx.x * 32;
    const int row0 = a.map_row0 + blockIdx.y * 32;     // global query index of the tile's first row
    const int qi = row0 + r;
    const bool row_ok = qi < a.map_row0 + a.map_rows;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    const float log2e = 1.4426950408889634f;
    for (int h = 0; h < a.num_heads; ++h) {
        __syncthreads();
        for (int i = tid; i < 32 * hd; i += 128) {
            const int rr = i / hd, d = i - rr * hd;
            const int qg = row0 + rr;
            float qv = 0.0f, kv = 0.0f;
            if (qg < a.map_row0 + a.map_rows) {
                const int seg = qg >= a.q_rows[0] ? 1 : 0;
                const int lr = seg ? qg - a.q_rows[0] : qg;
                qv = map_ld16<kBf16>(seg ? a.q[1] : a.q[0], static_cast<long long>(lr) * (seg ? a.q_ld[1] : a.q_ld[0]) + h * hd + d);
            }
            const int kg = key0 + rr;
            if (kg < a.map_cols) {
                const int seg = kg >= a.kv_rows[0] ? 1 : 0;
                const int lr = seg ? kg - a.kv_rows[0] : kg;
                kv = map_ld16<kBf16>(seg ? a.k[1] : a.k[0], static_cast<long long>(lr) * (seg ? a.k_ld[1] : a.k_ld[0]) + h * hd + d);
            }
            Qs[rr * hdp + d] = qv;
            Ks[rr * hdp + d] = kv;
        }
        __syncthreads();
        float m2 = 0.0f, inv_l = 0.0f;
        if (row_ok) {
            const float* st = a.lse + (static_cast<long long>(h) * a.lq_total + qi) * 2;
            m2 = st[0];
            inv_l = st[1] > 0.0f ? 1.0f / st[1] : 0.0f;
        }
        const int br = qi - a.bias_row0;
        const bool biased = a.bias != nullptr && br >= 0 && br < a.bias_rows;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int kk = c4 * 8 + i;
            const int kg = key0 + kk;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(Qs[r * hdp + d], Ks[kk * hdp + d], dot);
            float x = dot * a.scale_log2;
            bool visible = kg < a.map_cols;
            if (visible && a.key_scale != nullptr) x *= __ldg(a.key_scale + kg);
            if (biased && kg < a.bias_cols) x += __ldg(a.bias + static_cast<long long>(br) * a.bias_ld + kg) * log2e;
            // the same visibility rules as the attention kernel: a masked key has weight 0
            if (a.mask_mode == 1 && kg > qi + a.q_offset) visible = false;
            if (visible && a.key_mask != nullptr && __ldg(a.key_mask + kg) == 0.0f) visible = false;
            // a row whose reference maximum is -inf saw no key: its map row is zero
            const float p = (!visible || m2 == -INFINITY) ? 0.0f : exp2f(x - m2) * inv_l;
            acc[i] += p;
        }
    }
    if (row_ok) {
        const float inv_h = 1.0f / static_cast<float>(a.num_heads);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int kg = key0 + c4 * 8 + i;
            if (kg < a.map_cols) a.map[static_cast<long long>(qi - a.map_row0) * a.map_ld + kg] = acc[i] * inv_h;
        }
    }
}

}  // namespace

cudaError_t launch_attn_map(const AttnMapArgs& a, bool bf16, cudaStream_t stream) {
    const size_t smem = sizeof(float) * 2 * 32 * (a.head_dim + 1);
    dim3 grid(static_cast<unsigned>((a.map_cols + 31) / 32), static_cast<unsigned>((a.map_rows + 31) / 32));
    // 2 x 32 x 257 floats at head_dim 256 is the most this kernel asks for; the
    // limit is raised to that once per device and kernel, not on every launch.
    constexpr int kMaxSmem = static_cast<int>(sizeof(float) * 2 * 32 * (256 + 1));
    if (static_cast<int>(smem) > kMaxSmem) return cudaErrorInvalidValue;
    cudaError_t e;
    if (bf16) {
        e = set_max_smem_once(attn_map_kernel<true>, kMaxSmem);
        if (e != cudaSuccess) return e;
        attn_map_kernel<true><<<grid, 128, smem, stream>>>(a);
    } else {
        e = set_max_smem_once(attn_map_kernel<false>, kMaxSmem);
        if (e != cudaSuccess) return e;
        attn_map_kernel<false><<<grid, 128, smem, stream>>>(a);
    }
    return cudaGetLastError();
}

}  // namespace bdattn
