// Softmax attention forward for head_dim 64 / 128 on the sm_100a tensor cores.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the key
// tiles (128 keys each).  Roles (12 warps, three warpgroups):
//   warps 0-3  : softmax of query tile 0   (one thread per query row)
//   warps 4-7  : softmax of query tile 1
//   warp  8    : issues every tcgen05.mma (one lane), owns the TMEM allocation
//   warp  9    : TMA producer for Q, K and V tiles (one lane)
//   warps 10-11: with per-key scale vectors (kScale): multiply the rows of a K or
//                V tile in shared memory by their factors before the MMAs read it;
//                otherwise idle (they complete the third warpgroup so that
//                registers can be moved to the softmax warpgroups with setmaxnreg)
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
// What paces the kernel is the dependency chain of one query tile (scores ready
// -> softmax -> P ready -> P.V and the next Q.K^T -> scores ready), of which the
// softmax is the longest link, and the single MMA-issuing thread: tcgen05.mma
// holds its issuing thread for as long as the MMA executes (64 cycles for
// 128x128x16), so every wait, fence and commit of that thread is time the tensor
// pipe idles.  The softmax arithmetic is therefore packed two floats per
// instruction (fma/add .f32x2) and the row maximum uses the three-input max.
//
// Q, K and V are addressed through 4-D tensor maps (head element, head, row,
// batch): a head narrower than the 64 / 128 columns the kernel computes with
// (40, 72, 80, 112, ...) is zero-padded by the TMA unit itself, so such head
// dims run here without a padding pass; only the real columns are stored.
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
constexpr int kThreads = 384;
constexpr int kChunkBytes = 128 * 128;  // one 64-column (128 B) x 128-row TMA box
constexpr int kRegsSoftmax = 216;
constexpr int kRegsOther = 64;

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

// ------------------------------------------------------- packed FP32 math
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1)
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1,
                                      float c0, float c1) {
    asm("{\n"
        ".reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rb, {%4, %5};\n"
        "mov.b64 rc, {%6, %7};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\n"
        "mov.b64 {%0, %1}, rd;\n"
        "}\n"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n"
        ".reg .b64 ra, rb, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rb, {%4, %5};\n"
        "add.rn.f32x2 rd, ra, rb;\n"
        "mov.b64 {%0, %1}, rd;\n"
        "}\n"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// HOOKS: 0 = none; 1 = key_mask only; 2 = key_mask, bias and the per-row softmax
// statistics (slower softmax path).
// SCALE: key_scale / val_scale are applied to the K / V tiles in shared memory by
// warp 10 (rounded to the storage type, as the reference's scale_inplace on its
// k_full_ / v_full_ copies does, src/dit/qwenimage21_forward.cpp:606-645); the
// softmax code does not change.
template <int HD, bool kBf16, int kHooks, bool kScale>
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
    uint64_t* q_ready = pv_done + 2;     // [2]  Q tile normalised + rotated in place (fused Q path)
    uint64_t* kv_ready = q_ready + 2;    // [ST] tile landed and, where needed, scaled (kScale)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_ready + ST);

    dependents_may_launch();
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
            mbar_init(&kv_ready[s], 2);           // warps 10 and 11
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4);          // one arrival per softmax warp of the tile
            mbar_init(&pv_done[t], 1);
            mbar_init(&q_ready[t], 4);
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
    // barriers, tensor memory and descriptors are set up; from here on global memory is touched
    wait_for_prior_grid();

    if (warp < 8) {
        // ------------------------------------------------ softmax + epilogue
        setmaxnreg_inc<kRegsSoftmax>();
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

        if (a.q_fused && n_kv > 0) {
            // Per-head RMSNorm + RoPE of the query tile, in place in the (128-byte
            // swizzled) Q tile, before the first Q.K^T MMA (src/dit/flux.cpp:462-469 +
            // src/dit/common.cpp:192 applied to Q).  A warp takes its 32 rows one at a
            // time with the head's columns spread over the lanes, so that the cos / sin
            // rows are read coalesced (one row per load; a thread-per-row version
            // touched 32 cache lines per load and cost ten times as much).  Rows past
            // the segment are zero and stay zero.
            ok = __all_sync(0xffffffffu, mbar_wait(&q_full[t], 0));
            if (ok) {
                constexpr int kEpl = HD / 32;                 // elements per lane: 4 or 2
                const int hd = a.hd_out;
                const int c0 = lane * kEpl;                   // first column of this lane
                const bool live = c0 < hd;                    // hd is a multiple of 8
                const void* gain = qseg ? a.q_gain[1] : a.q_gain[0];
                float gv[kEpl];
#pragma unroll
                for (int i = 0; i < kEpl; ++i) gv[i] = 1.0f;
                if (gain != nullptr && live) {
#pragma unroll
                    for (int i = 0; i < kEpl; ++i) {
                        if (a.q_gain_is_f32) gv[i] = __ldg(reinterpret_cast<const float*>(gain) + c0 + i);
                        else {
                            const uint16_t b = __ldg(reinterpret_cast<const uint16_t*>(gain) + c0 + i);
                            gv[i] = kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                                          : __half2float(*reinterpret_cast<const __half*>(&b));
                        }
                    }
                }
                const int bofs = (c0 & 63) * 2;               // byte offset inside the 128-byte row piece
                uint8_t* qbase = smem_q + t * C::kQBytes + (c0 >> 6) * kChunkBytes + (bofs & 15);
                const int cidx = bofs >> 4;
                const float inv_hd = 1.0f / static_cast<float>(hd);
                // 16 rows at a time, every load of a batch issued before the first use:
                // a row-by-row loop is a chain of load and shuffle latencies
                constexpr int kRb = 16;
                const bool rope = a.q_cos != nullptr && live;
#pragma unroll 1
                for (int r0 = 0; r0 < 32; r0 += kRb) {
                    uint32_t w[kRb][kEpl / 2];
                    float cs[kRb][kEpl / 2], sn[kRb][kEpl / 2];
#pragma unroll
                    for (int k = 0; k < kRb; ++k) {
                        const int r = (warp & 3) * 32 + r0 + k;
                        const uint8_t* ptr = qbase + r * 128 + ((cidx ^ (r & 7)) << 4);
                        if constexpr (kEpl == 4) {
                            const uint2 u = *reinterpret_cast<const uint2*>(ptr);
                            w[k][0] = u.x; w[k][1] = u.y;
                        } else {
                            w[k][0] = *reinterpret_cast<const uint32_t*>(ptr);
                        }
#pragma unroll
                        for (int i = 0; i < kEpl / 2; ++i) { cs[k][i] = 1.0f; sn[k][i] = 0.0f; }
                        if (rope && qrow0 + t * kBM + r < seg_rows) {
                            const long long tb = static_cast<long long>(a.q_rope_row0 + q_global0 + t * kBM + r) * (hd >> 1) + (c0 >> 1);
                            if constexpr (kEpl == 4) {
                                const float2 cv = __ldg(reinterpret_cast<const float2*>(a.q_cos + tb));
                                const float2 sv = __ldg(reinterpret_cast<const float2*>(a.q_sin + tb));
                                cs[k][0] = cv.x; cs[k][1] = cv.y; sn[k][0] = sv.x; sn[k][1] = sv.y;
                            } else {
                                cs[k][0] = __ldg(a.q_cos + tb); sn[k][0] = __ldg(a.q_sin + tb);
                            }
                        }
                    }
                    float x[kRb][kEpl], ss[kRb];
#pragma unroll
                    for (int k = 0; k < kRb; ++k) {
#pragma unroll
                        for (int i = 0; i < kEpl / 2; ++i) {
                            if constexpr (kBf16) {
                                x[k][2 * i] = __uint_as_float(w[k][i] << 16);
                                x[k][2 * i + 1] = __uint_as_float(w[k][i] & 0xffff0000u);
                            } else {
                                const __half2 h = *reinterpret_cast<const __half2*>(&w[k][i]);
                                x[k][2 * i] = __low2float(h);
                                x[k][2 * i + 1] = __high2float(h);
                            }
                        }
                        ss[k] = 0.0f;
#pragma unroll
                        for (int i = 0; i < kEpl; ++i) ss[k] = fmaf(x[k][i], x[k][i], ss[k]);
                    }
                    if (gain != nullptr) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                            for (int k = 0; k < kRb; ++k) ss[k] += __shfl_xor_sync(0xffffffffu, ss[k], o);
                        }
#pragma unroll
                        for (int k = 0; k < kRb; ++k) {
                            const float inv = rsqrtf(ss[k] * inv_hd + a.q_eps);
#pragma unroll
                            for (int i = 0; i < kEpl; ++i) x[k][i] *= inv * gv[i];
                        }
                    }
#pragma unroll
                    for (int k = 0; k < kRb; ++k) {
                        const int r = (warp & 3) * 32 + r0 + k;
                        uint8_t* ptr = qbase + r * 128 + ((cidx ^ (r & 7)) << 4);
#pragma unroll
                        for (int i = 0; i < kEpl / 2; ++i) {
                            const float a0 = x[k][2 * i], b0 = x[k][2 * i + 1];
                            x[k][2 * i] = a0 * cs[k][i] - b0 * sn[k][i];
                            x[k][2 * i + 1] = a0 * sn[k][i] + b0 * cs[k][i];
                        }
                        if constexpr (kEpl == 4) {
                            uint2 u;
                            u.x = pack2<kBf16>(x[k][0], x[k][1]);
                            u.y = pack2<kBf16>(x[k][2], x[k][3]);
                            *reinterpret_cast<uint2*>(ptr) = u;
                        } else {
                            *reinterpret_cast<uint32_t*>(ptr) = pack2<kBf16>(x[k][0], x[k][1]);
                        }
                    }
                }
                fence_proxy_async_smem();      // the MMA reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&q_ready[t]);
            }
        }

        for (int j = 0; j < n_kv; ++j) {
            // Key mask of this tile as 128 bits (four ballots over one coalesced load
            // per lane), fetched before the wait for S so that its latency is hidden.
            uint32_t mbits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
            if constexpr (kHooks >= 1) {
                if (a.key_mask != nullptr) {
                    const TileInfo tm = kv_tile(a, j);
                    float mv[4];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const int c = 4 * lane + w;
                        mv[w] = c < tm.valid ? __ldg(a.key_mask + tm.kbase + c) : 1.0f;
                    }
#pragma unroll
                    for (int w = 0; w < 4; ++w) mbits[w] = __ballot_sync(0xffffffffu, mv[w] != 0.0f);
                }
            }
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
            if constexpr (kHooks == 2) {
                if (a.bias != nullptr) {
                    const int br = q_glob - a.bias_row0;
                    if (br >= 0 && br < a.bias_rows && ti.kbase < a.bias_cols) {
                        const float* brow = a.bias + static_cast<long long>(br) * a.bias_ld + ti.kbase;
#pragma unroll
                        for (int c = 0; c < kBN; ++c) {
                            if (c < ti.valid && ti.kbase + c < a.bias_cols) s[c] += __ldg(brow + c) * a.bias_mul;
                        }
                    }
                }
            }
            int lim = ti.valid - 1;
            if (a.mask_mode == 1) lim = min(lim, q_glob + a.q_offset - ti.kbase);
            if (__any_sync(0xffffffffu, lim < kBN - 1)) {
#pragma unroll
                for (int c = 0; c < kBN; ++c) s[c] = (c <= lim) ? s[c] : -INFINITY;
            }
            if constexpr (kHooks >= 1) {
                // (tiles without a masked key, the usual case away from the padded tail, skip this)
                if (a.key_mask != nullptr && (mbits[0] & mbits[1] & mbits[2] & mbits[3]) != 0xffffffffu) {
#pragma unroll
                    for (int c = 0; c < kBN; ++c) {
                        if (((mbits[c & 3] >> (c >> 2)) & 1u) == 0u) s[c] = -INFINITY;
                    }
                }
            }

            // row maximum: four independent chains of three-input max
            float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
            float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
            for (int c = 12; c + 7 < kBN; c += 8) {
                mx0 = max3(mx0, s[c], s[c + 1]);
                mx1 = max3(mx1, s[c + 2], s[c + 3]);
                mx2 = max3(mx2, s[c + 4], s[c + 5]);
                mx3 = max3(mx3, s[c + 6], s[c + 7]);
            }
            // 12 + 8*14 = 124: four scores left
            mx0 = max3(mx0, s[124], s[125]);
            mx1 = max3(mx1, s[126], s[127]);
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
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
                    // P.V of step j-1 has completed: the commit that made S of this step
                    // visible was issued after it and covers every earlier MMA of the
                    // issuing thread
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
            // p = 2^(s * scale_log2 - m * scale_log2); row sum in four packed chains
            float rs[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) rs[i] = 0.0f;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int c0 = ch * 32 + 2 * i;
                    float x0, x1, p0, p1;
                    ffma2(x0, x1, s[c0], s[c0 + 1], sl2, sl2, neg_ms, neg_ms);
                    p0 = fast_exp2(x0);
                    p1 = fast_exp2(x1);
                    fadd2(rs[2 * (i & 3)], rs[2 * (i & 3) + 1], rs[2 * (i & 3)], rs[2 * (i & 3) + 1], p0, p1);
                    pk[i] = pack2<kBf16>(p0, p1);
                }
                tmem_st16(tS + ch * 16, pk);
            }
            l_sum += ((rs[0] + rs[1]) + (rs[2] + rs[3])) + ((rs[4] + rs[5]) + (rs[6] + rs[7]));
            tmem_wait_st();
            tc_fence_before();
            // one elected arrival per warp: 32 lanes arriving on the same barrier
            // word serialise and delay the hand-over to the MMA warp
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
        }

        if (ok && n_kv > 0) {
            ok = mbar_wait(&pv_done[t], 0u);       // committed once, after the last P.V
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
        }
        const float inv = (l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
        if constexpr (kHooks == 2) {
            if (a.lse != nullptr && ok && row_in_seg < seg_rows) {
                float* st = a.lse + ((static_cast<long long>(batch) * gridDim.y + head) * a.lq_total + q_glob) * 2;
                st[0] = m_ref * sl2;
                st[1] = l_sum;
            }
        }
        // Epilogue: O / l goes through shared memory (this tile's Q buffer, no longer
        // read: all Q.K^T MMAs have completed) so that global stores are whole
        // rows: 16-byte chunk c of row r sits at chunk c ^ (r mod chunks) to keep
        // the row-per-thread writes and the row-major reads free of bank conflicts.
        constexpr int kRowChunks = HD / 8;
        uint8_t* stg = smem_q + t * C::kQBytes;
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
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint4 w;
                w.x = pack2<kBf16>(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
                w.y = pack2<kBf16>(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
                w.z = pack2<kBf16>(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
                w.w = pack2<kBf16>(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
                const int cg = c * 4 + g;
                *reinterpret_cast<uint4*>(stg + row_in_tile * (HD * 2) + ((cg ^ (row_in_tile & (kRowChunks - 1))) << 4)) = w;
            }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");   // the 128 threads of this query tile
        if (ok) {
            uint8_t* obase = reinterpret_cast<uint8_t*>(qseg ? a.o[1] : a.o[0]);
            const long long o_ld = qseg ? a.o_ld[1] : a.o_ld[0];
            const long long o_bs = qseg ? a.o_bs[1] : a.o_bs[0];
            const int out_chunks = a.hd_out >> 3;
            for (int idx = row_in_tile; idx < kBM * kRowChunks; idx += kBM) {
                const int r = idx / kRowChunks;
                const int cg = idx - r * kRowChunks;
                const int rs = qrow0 + t * kBM + r;
                if (rs < seg_rows && cg < out_chunks) {
                    const uint4 w = *reinterpret_cast<const uint4*>(stg + r * (HD * 2) + ((cg ^ (r & (kRowChunks - 1))) << 4));
                    const long long off = 2 * (static_cast<long long>(batch) * o_bs + static_cast<long long>(rs) * o_ld +
                                               static_cast<long long>(head) * a.hd_out + cg * 8);
                    uint8_t* const mc = reinterpret_cast<uint8_t*>(qseg ? a.o_mc[1] : a.o_mc[0]);
                    if (mc != nullptr) {
                        // fused all-gather through the switch: one store to the multicast
                        // address lands in every GPU's copy of the output, this one's included
                        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                                     ::"l"(mc + off), "f"(__uint_as_float(w.x)), "f"(__uint_as_float(w.y)),
                                       "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
                                     : "memory");
                    } else {
                        *reinterpret_cast<uint4*>(obase + off) = w;
                        // fused all-gather: the same vector goes to every peer's copy of the
                        // output (plain stores over NVLink; no TMA, no peer reads)
                        for (int pi = 0; pi < a.n_peers; ++pi) {
                            uint8_t* pb = reinterpret_cast<uint8_t*>(qseg ? a.o_peer[1][pi] : a.o_peer[0][pi]);
                            *reinterpret_cast<uint4*>(pb + off) = w;
                        }
                    }
                }
            }
        }
    } else {
        setmaxnreg_dec<kRegsOther>();
        if (warp == 8) {
            // -------------------------------------------------- MMA issuer
            // tcgen05.mma issue blocks while the pipe is busy, and everything this
            // warp does between two batches of MMAs (barrier waits, commits, index
            // arithmetic) is time the tensor pipe idles, so the loop is kept short:
            // ring slots and phases are walked without divisions, the K/V waits sit
            // before the wait for P, and descriptors are formed from per-tile bases.
            // (Two issuing warps, one per query tile, were slower: MMAs of the two
            // tiles then interleave in the pipe and lose their back-to-back runs on
            // one accumulator.)
            constexpr int kFmt = kBf16 ? 1 : 0;
            constexpr uint32_t idesc_qk = make_idesc_f16(kFmt, kBM, kBN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(kFmt, kBM, HD, 0, 1);
            const uint32_t q_base = smem_u32(smem_q);
            const uint32_t kv_base = smem_u32(smem_kv);
            uint64_t* const kv_rdy = kScale ? kv_ready : kv_full;

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
            if (ok && a.q_fused) ok = mbar_wait(&q_ready[0], 0) && mbar_wait(&q_ready[1], 0);
            if (ok) ok = mbar_wait(&kv_rdy[0], 0);
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
            // slot and phase of the V tile of step j (ring item 2j+1) and of the K tile
            // of step j+1 (item 2j+2)
            int vslot = 1 % ST, vphase = 0;
            for (int j = 0; ok && j < n_kv; ++j) {
                int kslot = vslot + 1, kphase = vphase;
                if (kslot == ST) { kslot = 0; kphase ^= 1; }
                const bool more = j + 1 < n_kv;
                ok = mbar_wait(&kv_rdy[vslot], static_cast<uint32_t>(vphase));
                if (ok && more) ok = mbar_wait(&kv_rdy[kslot], static_cast<uint32_t>(kphase));
                if (ok) ok = mbar_wait(&p_full[0], static_cast<uint32_t>(j & 1));
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    issue_pv(0, vslot, j > 0);
                    if (more) {
                        issue_qk(0, kslot);
                        umma_commit(&s_full[0]);
                    } else {
                        umma_commit(&pv_done[0]);    // only the last step needs its own signal
                    }
                }
                __syncwarp();
                ok = mbar_wait(&p_full[1], static_cast<uint32_t>(j & 1));
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    issue_pv(1, vslot, j > 0);
                    if (!more) umma_commit(&pv_done[1]);
                    umma_commit(&kv_empty[vslot]);
                    if (more) {
                        issue_qk(1, kslot);
                        umma_commit(&s_full[1]);
                        umma_commit(&kv_empty[kslot]);
                    }
                }
                __syncwarp();
                vslot = kslot + 1; vphase = kphase;
                if (vslot == ST) { vslot = 0; vphase ^= 1; }
            }
        } else if (warp == 9) {
            // ------------------------------------------------ TMA producer
            if (lane == 0 && n_kv > 0) {
                const CUtensorMap* mq = qseg ? &tmQ1 : &tmQ0;
                for (int t = 0; t < 2; ++t) {
                    mbar_arrive_expect_tx(&q_full[t], C::kQBytes);
                    for (int c = 0; c < C::kChunks; ++c) {
                        tma_load_4d(smem_q + t * C::kQBytes + c * kChunkBytes, mq, &q_full[t],
                                    c * 64, head, qrow0 + t * kBM, batch);
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
                    const int kv_head = head / a.kv_group;
                    const CUtensorMap* m = (i & 1) ? (ti.seg ? &tmV1 : &tmV0) : (ti.seg ? &tmK1 : &tmK0);
                    mbar_arrive_expect_tx(&kv_full[slot], C::kTileBytes);
                    for (int c = 0; c < C::kChunks; ++c) {
                        tma_load_4d(smem_kv + slot * C::kTileBytes + c * kChunkBytes, m, &kv_full[slot],
                                    c * 64, kv_head, ti.row0, batch);
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
        } else if (warp >= 10) {
            // ------------------------------------------- K / V row scaling
            // Warps 10 and 11 both walk the ring items in order (each sees every phase
            // of the barriers it waits on) and take half of a tile each.  The row
            // factors of an item are fetched before the wait for its tile.  A tile
            // none of whose factors differs from one is passed on as it is; otherwise
            // every row is multiplied by its factor (FP32 product rounded to the
            // storage type).
            if constexpr (kScale) {
                const int half_id = warp - 10;
                bool ok = true;
                // row factors of item i (rows lane, lane + 32, ...), fetched one item ahead
                auto fetch = [&](int i, float (&f)[4]) {
#pragma unroll
                    for (int w = 0; w < 4; ++w) f[w] = 1.0f;
                    const float* sc = (i & 1) ? a.val_scale : a.key_scale;
                    if (sc != nullptr && i < 2 * n_kv) {
                        const TileInfo ti = kv_tile(a, i >> 1);
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            const int r = lane + 32 * w;
                            if (r < ti.valid) f[w] = __ldg(sc + ti.kbase + r);
                        }
                    }
                };
                float f[4], fn[4];
                fetch(0, fn);
                for (int i = 0; ok && i < 2 * n_kv; ++i) {
                    const int slot = i % ST;
#pragma unroll
                    for (int w = 0; w < 4; ++w) f[w] = fn[w];
                    fetch(i + 1, fn);
                    const bool ne = f[0] != 1.0f || f[1] != 1.0f || f[2] != 1.0f || f[3] != 1.0f;
                    const bool scale_tile = __any_sync(0xffffffffu, ne);
                    ok = mbar_wait(&kv_full[slot], static_cast<uint32_t>((i / ST) & 1));
                    if (!ok) break;
                    if (scale_tile) {
                        uint8_t* tile = smem_kv + slot * C::kTileBytes;
                        // A lane owns whole rows (lane, lane + 32, ...: the rows whose factors it
                        // holds).  Within a 64-column chunk a row is one 128-byte line whose 16-byte
                        // pieces the swizzle permutes; the factor is the same for all of them, so
                        // the pieces are walked in physical order, rotated by the lane's row so that
                        // the 32 rows of one access fall into different banks.  The (row group,
                        // chunk) pairs alternate between the two warps.
#pragma unroll
                        for (int pi = 0; pi < 4 * C::kChunks; ++pi) {
                            const int w = pi / C::kChunks, ch = pi % C::kChunks;
                            if ((pi & 1) != half_id) continue;
                            if (!__any_sync(0xffffffffu, f[w] != 1.0f)) continue;
                            uint8_t* line = tile + ch * kChunkBytes + (lane + 32 * w) * 128;
                            const float fw = f[w];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint4 v[4];
#pragma unroll
                                for (int b = 0; b < 4; ++b)
                                    v[b] = *reinterpret_cast<const uint4*>(line + (((h * 4 + b) ^ (lane & 7)) << 4));
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    uint32_t* w32 = reinterpret_cast<uint32_t*>(&v[b]);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        float lo, hi;
                                        if constexpr (kBf16) {
                                            lo = __uint_as_float(w32[e] << 16);
                                            hi = __uint_as_float(w32[e] & 0xffff0000u);
                                        } else {
                                            const __half2 hh = *reinterpret_cast<const __half2*>(&w32[e]);
                                            lo = __low2float(hh);
                                            hi = __high2float(hh);
                                        }
                                        // x * f + (-0) = x * f with the sign of a zero product kept
                                        ffma2(lo, hi, lo, hi, fw, fw, -0.0f, -0.0f);
                                        w32[e] = pack2<kBf16>(lo, hi);
                                    }
                                }
#pragma unroll
                                for (int b = 0; b < 4; ++b)
                                    *reinterpret_cast<uint4*>(line + (((h * 4 + b) ^ (lane & 7)) << 4)) = v[b];
                            }
                        }
                        fence_proxy_async_smem();      // the MMA reads the tile through the async proxy
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&kv_ready[slot]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int HD, bool kBf16, int kHooks, bool kScale>
cudaError_t launch_t(const SdpaLaunch& L, cudaStream_t stream) {
    using C = Cfg<HD>;
    auto kern = sdpa_tc05_kernel<HD, kBf16, kHooks, kScale>;
    cudaError_t e = set_max_smem_once(kern, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    dim3 grid(static_cast<unsigned>(L.q_ctas), static_cast<unsigned>(L.num_heads),
              static_cast<unsigned>(L.batch));
    return launch_dependent(kern, grid, dim3(kThreads), C::kSmemBytes, stream, L.tmQ[0], L.tmQ[1], L.tmK[0],
                            L.tmK[1], L.tmV[0], L.tmV[1], L.args);
}

template <int HD, bool kBf16>
cudaError_t launch_hd(const SdpaLaunch& L, cudaStream_t stream) {
    // 2: every softmax hook; 1: key mask only (the common case: padded captions), kept
    // free of the other hooks' code; 0: none.  The per-key scale vectors are handled
    // outside the softmax (kScale) and combine with 0 or 2.
    const bool all_hooks = L.args.bias != nullptr || L.args.lse != nullptr;
    const bool scale = L.args.key_scale != nullptr || L.args.val_scale != nullptr;
    if (scale) {
        if (all_hooks || L.args.key_mask != nullptr) return launch_t<HD, kBf16, 2, true>(L, stream);
        return launch_t<HD, kBf16, 0, true>(L, stream);
    }
    if (all_hooks) return launch_t<HD, kBf16, 2, false>(L, stream);
    if (L.args.key_mask != nullptr) return launch_t<HD, kBf16, 1, false>(L, stream);
    return launch_t<HD, kBf16, 0, false>(L, stream);
}

}  // namespace

cudaError_t launch_sdpa_tc05(const SdpaLaunch& L, cudaStream_t stream) {
    if (L.head_dim == 128) return L.bf16 ? launch_hd<128, true>(L, stream) : launch_hd<128, false>(L, stream);
    if (L.head_dim == 64) return L.bf16 ? launch_hd<64, true>(L, stream) : launch_hd<64, false>(L, stream);
    return cudaErrorInvalidValue;
}

}  // namespace bdattn
