// Softmax attention forward for head_dim 64 / 128 on the sm_100a tensor cores.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the key
// tiles (128 keys each).  Roles (10 warps):
//   warps 0-3 : softmax of query tile 0   (one thread per query row)
//   warps 4-7 : softmax of query tile 1
//   warp  8   : issues every tcgen05.mma (one lane), owns the TMEM allocation
//   warp  9   : TMA producer for Q, K and V tiles (one lane)
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+HD)
// O1 [256+HD,256+2HD).  P (the exponentiated scores, 16-bit, two per column)
// is written back over the first 64 columns of its S tile and consumed from
// tensor memory as the A operand of the P.V MMA.
//
// Per key tile j and query tile t the tensor pipe runs, in this issue order,
//   PV(t, j) then QK(t, j+1)
// so the softmax of one query tile overlaps the MMAs of the other.  The
// running maximum is only raised when it grew by more than 2^8 (the factor
// is carried by P and cancels in O / l), which makes the O rescale rare; the
// rescale is done in tensor memory by the softmax warps themselves.
//
// Arithmetic follows the attention core of dit::joint_attention_traced
// (src/dit/common.cpp:246-305): scale 1/sqrt(hd), stable softmax,
// inv = denom > 0 ? 1/denom : 0, with FP32 scores and accumulation.
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {

namespace {

constexpr int kBM = 128;           // query rows per tile
constexpr int kBN = 128;           // keys per tile
constexpr int kThreads = 320;
constexpr int kChunkBytes = 128 * 128;  // one 64-column (128 B) x 128-row TMA box

template <int HD>
struct Cfg {
    static constexpr int kChunks = HD / 64;
    static constexpr int kTileBytes = kBN * HD * 2;
    static constexpr int kQBytes = kBM * HD * 2;
    static constexpr int kStages = HD == 128 ? 5 : 6;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = 2 * kQBytes + kStages * kTileBytes + kBarBytes + 1024;
};

struct TileInfo {
    int seg;
    int row0;
    int valid;
    int kbase;
};

__device__ __forceinline__ TileInfo kv_tile(const SdpaDevArgs& a, int t) {
    TileInfo ti;
    if (t < a.kv_tiles0) {
        ti.seg = 0;
        ti.row0 = t * kBN;
        ti.valid = min(kBN, a.kv_rows[0] - ti.row0);
        ti.kbase = ti.row0;
    } else {
        ti.seg = 1;
        ti.row0 = (t - a.kv_tiles0) * kBN;
        ti.valid = min(kBN, a.kv_rows[1] - ti.row0);
        ti.kbase = a.kv_rows[0] + ti.row0;
    }
    return ti;
}

template <int HD, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_tc05_kernel(const __grid_constant__ CUtensorMap tmQ0, const __grid_constant__ CUtensorMap tmQ1,
                 const __grid_constant__ CUtensorMap tmK0, const __grid_constant__ CUtensorMap tmK1,
                 const __grid_constant__ CUtensorMap tmV0, const __grid_constant__ CUtensorMap tmV1,
                 const SdpaDevArgs a) {
    using C = Cfg<HD>;
    constexpr int ST = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint8_t* smem_q = smem;
    uint8_t* smem_kv = smem + 2 * C::kQBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_kv + ST * C::kTileBytes);
    uint64_t* q_full = bars;             // [2]
    uint64_t* kv_full = bars + 2;        // [ST]
    uint64_t* kv_empty = kv_full + ST;   // [ST]
    uint64_t* s_full = kv_empty + ST;    // [2]
    uint64_t* p_full = s_full + 2;       // [2]
    uint64_t* pv_done = p_full + 2;      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int qseg = (static_cast<int>(blockIdx.x) >= a.q_ctas0) ? 1 : 0;
    const int qrow0 = (qseg ? static_cast<int>(blockIdx.x) - a.q_ctas0 : static_cast<int>(blockIdx.x)) * 2 * kBM;
    const int seg_rows = qseg ? a.q_rows[1] : a.q_rows[0];
    const int q_global0 = (qseg ? a.q_rows[0] : 0) + qrow0;

    // Key tiles this CTA has to visit.
    int n_kv = a.kv_tiles;
    if (a.mask_mode == 1) {
        const int last = q_global0 + min(2 * kBM, seg_rows - qrow0) - 1;
        const int max_key = last + a.q_offset;
        int n = 0;
        for (int t = 0; t < a.kv_tiles; ++t) {
            if (kv_tile(a, t).kbase <= max_key) n = t + 1;
        }
        n_kv = n;
    }

    if (threadIdx.x == 0) {
        mbar_init(&q_full[0], 1);
        mbar_init(&q_full[1], 1);
        for (int s = 0; s < ST; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], kBM);
            mbar_init(&pv_done[t], 1);
        }
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(qseg ? &tmQ1 : &tmQ0);
        tma_prefetch_desc(&tmK0);
        tma_prefetch_desc(&tmV0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ------------------------------------------------ softmax + epilogue
        const int t = warp >> 2;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + static_cast<uint32_t>(t * kBN);
        const uint32_t tO = tmem_base + lane_base + static_cast<uint32_t>(256 + t * HD);
        const int row_in_tile = (warp & 3) * 32 + lane;
        const int row_in_seg = qrow0 + t * kBM + row_in_tile;
        const int q_glob = q_global0 + t * kBM + row_in_tile;
        const float sl2 = a.scale_log2;
        float m_ref = -INFINITY;
        float l_sum = 0.0f;
        bool ok = true;

        for (int j = 0; j < n_kv; ++j) {
            ok = mbar_wait(&s_full[t], static_cast<uint32_t>(j & 1));
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            tc_fence_after();
            float s[kBN];
#pragma unroll
            for (int c = 0; c < kBN / 32; ++c) {
                tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            }
            tmem_wait_ld();

            const TileInfo ti = kv_tile(a, j);
            if (a.key_scale != nullptr) {
#pragma unroll
                for (int c = 0; c < kBN; ++c) {
                    if (c < ti.valid) s[c] *= __ldg(a.key_scale + ti.kbase + c);
                }
            }
            int lim = ti.valid - 1;
            if (a.mask_mode == 1) lim = min(lim, q_glob + a.q_offset - ti.kbase);
            if (__any_sync(0xffffffffu, lim < kBN - 1)) {
#pragma unroll
                for (int c = 0; c < kBN; ++c) s[c] = (c <= lim) ? s[c] : -INFINITY;
            }
            if (a.key_mask != nullptr) {
#pragma unroll
                for (int c = 0; c < kBN; ++c) {
                    if (c < ti.valid && __ldg(a.key_mask + ti.kbase + c) == 0.0f) s[c] = -INFINITY;
                }
            }

            float mx = s[0];
#pragma unroll
            for (int c = 1; c < kBN; ++c) mx = fmaxf(mx, s[c]);
            const float m_new = fmaxf(m_ref, mx);
            const bool grow = (m_new - m_ref) * sl2 > 8.0f;
            if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2((m_ref - m_new) * sl2);
                    m_ref = m_new;
                }
                l_sum *= alpha;
                if (j > 0) {
                    ok = mbar_wait(&pv_done[t], static_cast<uint32_t>((j - 1) & 1));
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(tO + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tO + c * 32, o);
                    }
                }
            }
            const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
            const float neg_ms = -m_use * sl2;
            float rs = 0.0f;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int c0 = ch * 64 + 2 * i;
                    float p0 = fast_exp2(fmaf(s[c0], sl2, neg_ms));
                    float p1 = fast_exp2(fmaf(s[c0 + 1], sl2, neg_ms));
                    rs += p0 + p1;
                    if (a.val_scale != nullptr) {
                        if (c0 < ti.valid) p0 *= __ldg(a.val_scale + ti.kbase + c0);
                        if (c0 + 1 < ti.valid) p1 *= __ldg(a.val_scale + ti.kbase + c0 + 1);
                    }
                    pk[i] = pack2<kBf16>(p0, p1);
                }
                tmem_st32(tS + ch * 32, pk);
            }
            l_sum += rs;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[t]);
        }

        if (ok && n_kv > 0) {
            ok = mbar_wait(&pv_done[t], static_cast<uint32_t>((n_kv - 1) & 1));
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
        }
        const float inv = (l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
        const bool row_ok = ok && row_in_seg < seg_rows;
        uint8_t* orow = nullptr;
        if (row_ok) {
            orow = reinterpret_cast<uint8_t*>(qseg ? a.o[1] : a.o[0]) +
                   2 * (static_cast<long long>(batch) * (qseg ? a.o_bs[1] : a.o_bs[0]) +
                        static_cast<long long>(row_in_seg) * (qseg ? a.o_ld[1] : a.o_ld[0]) +
                        static_cast<long long>(head) * a.hd_out);
        }
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            if (ok && n_kv > 0) {
                tmem_ld32(tO + c * 32, o);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
            if (row_ok) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (c * 32 + g * 8 < a.hd_out) {
                        uint4 w;
                        w.x = pack2<kBf16>(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
                        w.y = pack2<kBf16>(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
                        w.z = pack2<kBf16>(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
                        w.w = pack2<kBf16>(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + (c * 32 + g * 8) * 2) = w;
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------ MMA issuer
        constexpr int kFmt = kBf16 ? 1 : 0;
        constexpr uint32_t idesc_qk = make_idesc_f16(kFmt, kBM, kBN, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_f16(kFmt, kBM, HD, 0, 1);
        const uint32_t q_base = smem_u32(smem_q);
        const uint32_t kv_base = smem_u32(smem_kv);

        auto issue_qk = [&](int t, int slot) {
            const uint32_t qa = q_base + t * C::kQBytes;
            const uint32_t kb = kv_base + slot * C::kTileBytes;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
                umma_ss(tmem_base + t * kBN, make_smem_desc_sw128(qa + off, 16, 1024),
                        make_smem_desc_sw128(kb + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
            }
        };
        auto issue_pv = [&](int t, int slot, bool acc) {
            const uint32_t vb = kv_base + slot * C::kTileBytes;
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
                umma_ts(tmem_base + 256 + t * HD, tmem_base + t * kBN + kk * 8,
                        make_smem_desc_sw128(vb + kk * 2048, kChunkBytes, 1024), idesc_pv,
                        (acc || kk > 0) ? 1u : 0u);
            }
        };

        bool ok = n_kv > 0;
        if (ok) ok = mbar_wait(&q_full[0], 0) && mbar_wait(&q_full[1], 0);
        if (ok) ok = mbar_wait(&kv_full[0], 0);
        if (ok) {
            tc_fence_after();
            if (lane == 0) {
                issue_qk(0, 0);
                umma_commit(&s_full[0]);
                issue_qk(1, 0);
                umma_commit(&s_full[1]);
                umma_commit(&kv_empty[0]);
            }
            __syncwarp();
        }
        for (int j = 0; ok && j < n_kv; ++j) {
            const int iv = 2 * j + 1;
            const int vslot = iv % ST;
            ok = mbar_wait(&kv_full[vslot], static_cast<uint32_t>((iv / ST) & 1));
            if (!ok) break;
            const int ik = 2 * j + 2;
            const int kslot = ik % ST;
            for (int t = 0; t < 2 && ok; ++t) {
                ok = mbar_wait(&p_full[t], static_cast<uint32_t>(j & 1));
                if (!ok) break;
                if (t == 0 && j + 1 < n_kv) {
                    ok = mbar_wait(&kv_full[kslot], static_cast<uint32_t>((ik / ST) & 1));
                    if (!ok) break;
                }
                tc_fence_after();
                if (lane == 0) {
                    issue_pv(t, vslot, j > 0);
                    umma_commit(&pv_done[t]);
                    if (j + 1 < n_kv) {
                        issue_qk(t, kslot);
                        umma_commit(&s_full[t]);
                        if (t == 1) umma_commit(&kv_empty[kslot]);
                    }
                }
                __syncwarp();
            }
            if (ok && lane == 0) umma_commit(&kv_empty[vslot]);
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------- TMA producer
        if (lane == 0 && n_kv > 0) {
            const CUtensorMap* mq = qseg ? &tmQ1 : &tmQ0;
            for (int t = 0; t < 2; ++t) {
                mbar_arrive_expect_tx(&q_full[t], C::kQBytes);
                for (int c = 0; c < C::kChunks; ++c) {
                    tma_load_3d(smem_q + t * C::kQBytes + c * kChunkBytes, mq, &q_full[t],
                                head * HD + c * 64, qrow0 + t * kBM, batch);
                }
            }
            int issued = 0;
            bool ok = true;
            for (int i = 0; i < 2 * n_kv; ++i) {
                const int slot = i % ST;
                if (i >= ST) {
                    ok = mbar_wait(&kv_empty[slot], static_cast<uint32_t>(((i / ST) - 1) & 1));
                    if (!ok) break;
                }
                const TileInfo ti = kv_tile(a, i >> 1);
                const CUtensorMap* m = (i & 1) ? (ti.seg ? &tmV1 : &tmV0) : (ti.seg ? &tmK1 : &tmK0);
                mbar_arrive_expect_tx(&kv_full[slot], C::kTileBytes);
                for (int c = 0; c < C::kChunks; ++c) {
                    tma_load_3d(smem_kv + slot * C::kTileBytes + c * kChunkBytes, m, &kv_full[slot],
                                head * HD + c * 64, ti.row0, batch);
                }
                issued = i + 1;
            }
            if (!ok) {
                // Unwinding after a wait ran out: let the copies already in
                // flight land before the CTA gives its shared memory back.
                mbar_wait(&q_full[0], 0);
                mbar_wait(&q_full[1], 0);
                for (int i = max(0, issued - ST); i < issued; ++i) {
                    mbar_wait(&kv_full[i % ST], static_cast<uint32_t>((i / ST) & 1));
                }
            }
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int HD, bool kBf16>
cudaError_t launch_t(const SdpaLaunch& L, cudaStream_t stream) {
    using C = Cfg<HD>;
    auto kern = sdpa_tc05_kernel<HD, kBf16>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured_dev = dev;
    }
    dim3 grid(static_cast<unsigned>(L.q_ctas), static_cast<unsigned>(L.num_heads),
              static_cast<unsigned>(L.batch));
    kern<<<grid, kThreads, C::kSmemBytes, stream>>>(L.tmQ[0], L.tmQ[1], L.tmK[0], L.tmK[1], L.tmV[0],
                                                   L.tmV[1], L.args);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_sdpa_tc05(const SdpaLaunch& L, cudaStream_t stream) {
    if (L.head_dim == 128) return L.bf16 ? launch_t<128, true>(L, stream) : launch_t<128, false>(L, stream);
    if (L.head_dim == 64) return L.bf16 ? launch_t<64, true>(L, stream) : launch_t<64, false>(L, stream);
    return cudaErrorInvalidValue;
}

}  // namespace bdattn
