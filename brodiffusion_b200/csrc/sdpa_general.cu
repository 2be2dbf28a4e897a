// Softmax attention forward for head dims the tensor-core kernel does not
// take (any multiple of 8 up to 256): a plain tiled online-softmax kernel on
// the CUDA cores with FP32 arithmetic.  One CTA = 32 query rows of one
// (batch, head); key/value tiles of 32 rows are staged in shared memory as
// FP32.  Thread (r, c) = (tid / 4, tid % 4) owns query row r: it computes 8 of
// the 32 scores of a tile and accumulates output columns c, c+4, c+8, ...
// Same arithmetic as src/dit/common.cpp:246-305 with FP32 scores.
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

constexpr int kGRows = 32;
constexpr int kGKeys = 32;

template <bool kBf16>
__device__ __forceinline__ float ld16(const void* p, long long i) {
    if constexpr (kBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    else return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

template <bool kBf16>
__global__ void __launch_bounds__(128) sdpa_general_kernel(const SdpaGeneralArgs a, int q_ctas0) {
    extern __shared__ float sm[];
    const int hd = a.head_dim;
    const int hdp = hd + 1;
    float* Qs = sm;                      // [32][hdp]
    float* Ks = Qs + kGRows * hdp;       // [32][hdp]
    float* Vs = Ks + kGKeys * hdp;       // [32][hd]
    float* Ps = Vs + kGKeys * hd;        // [32][33]

    const int tid = threadIdx.x;
    const int r = tid >> 2;
    const int c = tid & 3;
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int qseg = static_cast<int>(blockIdx.x) >= q_ctas0 ? 1 : 0;
    const int qrow0 = (qseg ? static_cast<int>(blockIdx.x) - q_ctas0 : static_cast<int>(blockIdx.x)) * kGRows;
    const int seg_rows = qseg ? a.q_rows[1] : a.q_rows[0];
    const int q_glob0 = (qseg ? a.q_rows[0] : 0) + qrow0;
    const void* qp = qseg ? a.q[1] : a.q[0];
    const long long q_ld = qseg ? a.q_ld[1] : a.q_ld[0];
    const long long q_bs = qseg ? a.q_bs[1] : a.q_bs[0];

    for (int i = tid; i < kGRows * hd; i += 128) {
        const int rr = i / hd, d = i - rr * hd;
        float v = 0.0f;
        if (qrow0 + rr < seg_rows)
            v = ld16<kBf16>(qp, batch * q_bs + static_cast<long long>(qrow0 + rr) * q_ld + head * hd + d);
        Qs[rr * hdp + d] = v * a.scale;
    }

    const int Lk = a.kv_rows[0] + a.kv_rows[1];
    int k_end = Lk;
    if (a.mask_mode == 1) {
        const int last = q_glob0 + min(kGRows, seg_rows - qrow0) - 1;
        k_end = max(0, min(Lk, last + a.q_offset + 1));
    }
    const int q_glob = q_glob0 + r;
    float m_run = -INFINITY, l_run = 0.0f;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.0f;

    for (int k0 = 0; k0 < k_end; k0 += kGKeys) {
        __syncthreads();
        for (int i = tid; i < kGKeys * hd; i += 128) {
            const int kk = i / hd, d = i - kk * hd;
            const int kg = k0 + kk;
            float kvv = 0.0f, vvv = 0.0f;
            if (kg < Lk) {
                const int seg = kg >= a.kv_rows[0] ? 1 : 0;
                const int rr = seg ? kg - a.kv_rows[0] : kg;
                const void* kp = seg ? a.k[1] : a.k[0];
                const void* vp = seg ? a.v[1] : a.v[0];
                const long long kld = seg ? a.k_ld[1] : a.k_ld[0];
                const long long vld = seg ? a.v_ld[1] : a.v_ld[0];
                const long long kbs = seg ? a.k_bs[1] : a.k_bs[0];
                const long long vbs = seg ? a.v_bs[1] : a.v_bs[0];
                kvv = ld16<kBf16>(kp, batch * kbs + static_cast<long long>(rr) * kld + (head / a.kv_group) * hd + d);
                vvv = ld16<kBf16>(vp, batch * vbs + static_cast<long long>(rr) * vld + (head / a.kv_group) * hd + d);
                if (a.key_scale != nullptr) kvv *= __ldg(a.key_scale + kg);
                if (a.val_scale != nullptr) vvv *= __ldg(a.val_scale + kg);
            }
            Ks[kk * hdp + d] = kvv;
            Vs[kk * hd + d] = vvv;
        }
        __syncthreads();

        float s[8];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int kk = c * 8 + i;
            const int kg = k0 + kk;
            float acc = 0.0f;
            for (int d = 0; d < hd; ++d) acc = fmaf(Qs[r * hdp + d], Ks[kk * hdp + d], acc);
            bool vis = kg < Lk;
            if (a.mask_mode == 1) vis = vis && (kg <= q_glob + a.q_offset);
            if (vis && a.key_mask != nullptr) vis = __ldg(a.key_mask + kg) != 0.0f;
            s[i] = vis ? acc : -INFINITY;
            mx = fmaxf(mx, s[i]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
        const float alpha = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_use);
        float rs = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p = __expf(s[i] - m_use);
            rs += p;
            Ps[r * 33 + c * 8 + i] = p;
        }
        rs += __shfl_xor_sync(0xffffffffu, rs, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        l_run = l_run * alpha + rs;
        m_run = m_new;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            const int d = c + 4 * i;
            if (d < hd) {
                float acc = o[i] * alpha;
                for (int kk = 0; kk < kGKeys; ++kk) acc = fmaf(Ps[r * 33 + kk], Vs[kk * hd + d], acc);
                o[i] = acc;
            }
        }
        __syncwarp();
    }

    if (qrow0 + r < seg_rows) {
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        void* op = qseg ? a.o[1] : a.o[0];
        const long long o_ld = qseg ? a.o_ld[1] : a.o_ld[0];
        const long long o_bs = qseg ? a.o_bs[1] : a.o_bs[0];
        const long long base = batch * o_bs + static_cast<long long>(qrow0 + r) * o_ld + head * hd;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            const int d = c + 4 * i;
            if (d < hd) {
                if constexpr (kBf16) reinterpret_cast<__nv_bfloat16*>(op)[base + d] = __float2bfloat16_rn(o[i] * inv);
                else reinterpret_cast<__half*>(op)[base + d] = __float2half_rn(o[i] * inv);
            }
        }
    }
}

}  // namespace

cudaError_t launch_sdpa_general(const SdpaGeneralArgs& a, int num_heads, int batch, bool bf16,
                                cudaStream_t stream) {
    const int hd = a.head_dim;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kGRows) * (hd + 1) + kGKeys * (hd + 1) +
                                         kGKeys * hd + kGRows * 33);
    const int q_ctas0 = (a.q_rows[0] + kGRows - 1) / kGRows;
    const int q_ctas1 = (a.q_rows[1] + kGRows - 1) / kGRows;
    dim3 grid(static_cast<unsigned>(q_ctas0 + q_ctas1), static_cast<unsigned>(num_heads),
              static_cast<unsigned>(batch));
    cudaError_t e;
    if (bf16) {
        e = set_max_smem_once(sdpa_general_kernel<true>, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        sdpa_general_kernel<true><<<grid, 128, smem, stream>>>(a, q_ctas0);
    } else {
        e = set_max_smem_once(sdpa_general_kernel<false>, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        sdpa_general_kernel<false><<<grid, 128, smem, stream>>>(a, q_ctas0);
    }
    return cudaGetLastError();
}

}  // namespace bdattn
