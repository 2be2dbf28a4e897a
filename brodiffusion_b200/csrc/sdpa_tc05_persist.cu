// Softmax attention forward for head_dim 64 / 128 on the sm_100a tensor cores:
// the persistent variant, used for the head-sharded call whose output also goes
// to the other GPUs (fused all-gather).  Arithmetic, tiles, tensor-memory layout
// and warp roles are those of sdpa_tc05.cu; what differs:
//
//   * The grid is persistent: one CTA per SM takes the work items (two 128-row
//     query tiles of one (batch, head)) blockIdx.x, blockIdx.x + gridDim.x, ...;
//     tensor memory, the barriers (running phases) and the K/V ring carry on from
//     item to item.  The queries and first K/V tiles of the next item load while
//     the current one finishes (q_empty tells the producer that the last Q.K^T of
//     an item has completed), and its first Q.K^T runs under the epilogue.
//   * The epilogue stages O / l in a tile of its own (32 KB, shared by the two
//     query tiles of the CTA through named barriers 3 and 4) instead of the Q
//     buffers, which are being refilled by then; the K/V ring has four tiles.
//   * Warps 10-11, idle in the other kernel, forward finished tiles to the peers:
//     once the softmax warps have stored a tile's rows to this GPU's copy of the
//     output they signal out_done; warps 10-11 read the rows back (L2) and store
//     them to the same place in every peer's copy, plain 16-byte stores over
//     NVLink, while the attention of the next items runs.  In the one-item-per-CTA
//     kernel those stores are issued by the softmax warps at the end of each CTA
//     and leave in a burst at the end of each wave (0.21 of 0.97 ms per call on
//     8 GPUs at 3 heads per GPU); here they run behind the computation.  (With
//     per-key scale vectors warps 10-11 scale K / V tiles instead and the softmax
//     warps keep the peer stores.)
//   * The MMA-issuing role is a function of its own, not inlined: that warp has no
//     latency hiding, and inside the item loop of the kernel body its batches ran
//     up to 80 % longer than as a separate function.
//
// On one GPU this variant is about 3 % slower per call than sdpa_tc05.cu (its
// steady state is slower than what hiding prologue and epilogue wins back), which
// is why it is used for the fused all-gather only.
#include "sdpa_tc05_common.cuh"

namespace bdattn {
namespace persist {
namespace {

using namespace sdpa_tc;

template <int HD>
struct Cfg {
    static constexpr int kChunks = HD / 64;
    static constexpr int kTileBytes = kBN * HD * 2;
    static constexpr int kQBytes = kBM * HD * 2;
    static constexpr int kStages = HD == 128 ? 4 : 6;   // four 32 KB tiles lose nothing against five
    static constexpr int kStageBytes = kBM * HD * 2;    // output staging tile, shared by the two query tiles
    static constexpr int kBarBytes = 512;
    static constexpr int kSmemBytes = 2 * kQBytes + kStages * kTileBytes + kStageBytes + kBarBytes + 1024;
};

// One work item = two 128-row query tiles of one (batch, head).  A CTA walks the
// items blockIdx.x, blockIdx.x + gridDim.x, ...; query tiles are the fastest index,
// so the CTAs that run side by side share the K/V of a head in L2.
struct Item {
    int head, batch, qseg, qrow0, seg_rows, q_global0, n_kv;
};
__device__ __forceinline__ Item decode_item(const SdpaDevArgs& a, int w) {
    Item it;
    const int qc = w % a.item_q_ctas;
    const int hb = w / a.item_q_ctas;
    it.head = hb % a.item_heads;
    it.batch = hb / a.item_heads;
    it.qseg = qc >= a.q_ctas0 ? 1 : 0;
    it.qrow0 = (it.qseg ? qc - a.q_ctas0 : qc) * 2 * kBM;
    it.seg_rows = it.qseg ? a.q_rows[1] : a.q_rows[0];
    it.q_global0 = (it.qseg ? a.q_rows[0] : 0) + it.qrow0;
    // key tiles the item has to visit
    it.n_kv = a.kv_tiles;
    if (a.mask_mode == 1) {
        const int last = it.q_global0 + min(2 * kBM, it.seg_rows - it.qrow0) - 1;
        const int max_key = last + a.q_offset;
        int n = 0;
        for (int t = 0; t < a.kv_tiles; ++t) {
            if (kv_tile(a, t).kbase <= max_key) n = t + 1;
        }
        it.n_kv = n;
    }
    return it;
}
__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct MmaCtx {
    uint64_t *q_full, *q_ready, *kv_rdy, *kv_empty, *s_full, *p_full, *pv_done, *q_empty;
    uint32_t tmem_base, q_base_addr, kv_base_addr;
    int n_items, w0, wstep, lane;
};

// The MMA-issuing role as a function of its own (not inlined): its instructions
// stay together whatever the rest of the kernel looks like.
template <int HD, bool kBf16, int ST>
__device__ __noinline__ void mma_role(const SdpaDevArgs& a, const MmaCtx& cx) {
    using C = Cfg<HD>;
    uint64_t* const q_full = cx.q_full; uint64_t* const q_ready = cx.q_ready; uint64_t* const kv_rdy = cx.kv_rdy;
    uint64_t* const kv_empty = cx.kv_empty; uint64_t* const s_full = cx.s_full; uint64_t* const p_full = cx.p_full;
    uint64_t* const pv_done = cx.pv_done; uint64_t* const q_empty = cx.q_empty;
    const uint32_t tmem_base = cx.tmem_base;
    const int n_items = cx.n_items, w0 = cx.w0, wstep = cx.wstep, lane = cx.lane;
            constexpr int kFmt = kBf16 ? 1 : 0;
            constexpr uint32_t idesc_qk = make_idesc_f16(kFmt, kBM, kBN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(kFmt, kBM, HD, 0, 1);
            const uint32_t q_base = cx.q_base_addr;
            const uint32_t kv_base = cx.kv_base_addr;

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

            bool ok = true;
            int jb = 0, qn = 0;      // as in the softmax warps
            // slot and phase of the next K/V ring item to consume: K_0 of the first item
            int vslot = 0, vphase = 0;
#pragma unroll 1
            for (int w = w0; ok && w < n_items; w += wstep) {
                const int n_kv = decode_item(a, w).n_kv;
                if (n_kv == 0) continue;
                const uint32_t qph = static_cast<uint32_t>(qn & 1);
                ok = mbar_wait(&q_full[0], qph) && mbar_wait(&q_full[1], qph);
                if (ok && a.q_fused) ok = mbar_wait(&q_ready[0], qph) && mbar_wait(&q_ready[1], qph);
                if (ok) ok = mbar_wait(&kv_rdy[vslot], static_cast<uint32_t>(vphase));
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    issue_qk(0, vslot);
                    umma_commit(&s_full[0]);
                    issue_qk(1, vslot);
                    umma_commit(&s_full[1]);
                    umma_commit(&kv_empty[vslot]);
                    if (n_kv == 1) umma_commit(q_empty);
                }
                __syncwarp();
                // slot and phase of the V tile of step j and of the K tile of step j+1
                ++vslot;
                if (vslot == ST) { vslot = 0; vphase ^= 1; }
#pragma unroll 1
                for (int j = 0; ok && j < n_kv; ++j) {
                    int kslot = vslot + 1, kphase = vphase;
                    if (kslot == ST) { kslot = 0; kphase ^= 1; }
                    const bool more = j + 1 < n_kv;
                    ok = mbar_wait(&kv_rdy[vslot], static_cast<uint32_t>(vphase));
                    if (ok && more) ok = mbar_wait(&kv_rdy[kslot], static_cast<uint32_t>(kphase));
                    if (ok) ok = mbar_wait(&p_full[0], static_cast<uint32_t>((jb + j) & 1));
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
                    ok = mbar_wait(&p_full[1], static_cast<uint32_t>((jb + j) & 1));
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
                    if (more) {
                        vslot = kslot + 1; vphase = kphase;
                        if (vslot == ST) { vslot = 0; vphase ^= 1; }
                        // the last Q.K^T of the item has been issued: the Q tiles can be refilled
                        if (j + 2 == n_kv && lane == 0) umma_commit(q_empty);
                    } else {
                        vslot = kslot; vphase = kphase;      // the next ring item is K_0 of the next work item
                    }
                }
                jb += n_kv;
                ++qn;
            }
}
// HOOKS: 0 = none; 1 = key_mask only; 2 = key_mask, bias and the per-row softmax
// statistics (slower softmax path).
// SCALE: key_scale / val_scale are applied to the K / V tiles in shared memory by
// warp 10 (rounded to the storage type, as the reference's scale_inplace on its
// k_full_ / v_full_ copies does, src/dit/qwenimage21_forward.cpp:606-645); the
// softmax code does not change.
template <int HD, bool kBf16, int kHooks, bool kScale>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_tc05_persistent_kernel(const __grid_constant__ CUtensorMap tmQ0, const __grid_constant__ CUtensorMap tmQ1,
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
    uint8_t* smem_stage = smem_kv + ST * C::kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_stage + C::kStageBytes);
    uint64_t* q_full = bars;             // [2]
    uint64_t* kv_full = bars + 2;        // [ST]
    uint64_t* kv_empty = kv_full + ST;   // [ST]
    uint64_t* s_full = kv_empty + ST;    // [2]
    uint64_t* p_full = s_full + 2;       // [2]
    uint64_t* pv_done = p_full + 2;      // [2]
    uint64_t* q_ready = pv_done + 2;     // [2]  Q tile normalised + rotated in place (fused Q path)
    uint64_t* kv_ready = q_ready + 2;    // [ST] tile landed and, where needed, scaled (kScale)
    uint64_t* q_empty = kv_ready + ST;   // [1]  every Q.K^T MMA of the item has been issued and completed
    uint64_t* out_done = q_empty + 1;    // [2]  a tile's rows are in the local output (peer push)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(out_done + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_items = a.n_items;
    const int w0 = static_cast<int>(blockIdx.x), wstep = static_cast<int>(gridDim.x);
    // warps 10-11 copy finished tiles to the peers' replicas (fused all-gather) unless they
    // are busy scaling K / V tiles
    const bool push_peers = !kScale && a.n_peers > 0;

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
            mbar_init(&out_done[t], 4);
        }
        mbar_init(q_empty, 1);
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tmQ0);
        tma_prefetch_desc(&tmQ1);
        tma_prefetch_desc(&tmK0);
        tma_prefetch_desc(&tmV0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ------------------------------------------------ softmax + epilogue
        setmaxnreg_inc<kRegsSoftmax>();
        const int t = warp >> 2;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + static_cast<uint32_t>(t * kBN);
        const uint32_t tO = tmem_base + lane_base + static_cast<uint32_t>(256 + t * HD);
        const int row_in_tile = (warp & 3) * 32 + lane;
        const float sl2 = a.scale_log2;
        bool ok = true;
        int jb = 0;     // key steps of the earlier items: the phase of s_full / p_full carries on
        int qn = 0;     // earlier items that had key tiles: phase of q_full, q_ready, pv_done
        for (int w = w0, item_no = 0; w < n_items; w += wstep, ++item_no) {
        const Item im = decode_item(a, w);
        const int head = im.head, batch = im.batch, qseg = im.qseg, qrow0 = im.qrow0, seg_rows = im.seg_rows;
        const int q_global0 = im.q_global0, n_kv = im.n_kv;
        const int row_in_seg = qrow0 + t * kBM + row_in_tile;
        const int q_glob = q_global0 + t * kBM + row_in_tile;
        float m_ref = -INFINITY;
        float l_sum = 0.0f;

        if (ok && a.q_fused && n_kv > 0) {
            // Per-head RMSNorm + RoPE of the query tile, in place in the (128-byte
            // swizzled) Q tile, before the first Q.K^T MMA (src/dit/flux.cpp:462-469 +
            // src/dit/common.cpp:192 applied to Q).  A warp takes its 32 rows one at a
            // time with the head's columns spread over the lanes, so that the cos / sin
            // rows are read coalesced (one row per load; a thread-per-row version
            // touched 32 cache lines per load and cost ten times as much).  Rows past
            // the segment are zero and stay zero.
            ok = __all_sync(0xffffffffu, mbar_wait(&q_full[t], static_cast<uint32_t>(qn & 1)));
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

        for (int j = 0; ok && j < n_kv; ++j) {
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
            ok = mbar_wait(&s_full[t], static_cast<uint32_t>((jb + j) & 1));
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
            ok = mbar_wait(&pv_done[t], static_cast<uint32_t>(qn & 1));   // committed once per item, after the last P.V
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
        }
        const float inv = (l_sum > 0.0f) ? 1.0f / l_sum : 0.0f;
        if constexpr (kHooks == 2) {
            if (a.lse != nullptr && ok && row_in_seg < seg_rows) {
                float* st = a.lse + ((static_cast<long long>(batch) * a.item_heads + head) * a.lq_total + q_glob) * 2;
                st[0] = m_ref * sl2;
                st[1] = l_sum;
            }
        }
        // Epilogue: O / l goes through a staging tile in shared memory so that global
        // stores are whole rows: 16-byte chunk c of row r sits at chunk c ^ (r mod chunks)
        // to keep the row-per-thread writes and the row-major reads free of bank
        // conflicts.  The two query tiles of a CTA share the one staging tile: tile 0
        // finishes half a key step ahead, hands it to tile 1 (named barrier 3), and gets
        // it back for the next item (named barrier 4).  The Q buffers are not touched,
        // so the next item's queries load while this one drains.
        constexpr int kRowChunks = HD / 8;
        uint8_t* stg = smem_stage;
        const bool has_next = w + wstep < n_items;
        if (t == 0) { if (item_no > 0) named_sync(4, 256); }
        else named_sync(3, 256);
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
                uint4 w4;
                w4.x = pack2<kBf16>(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
                w4.y = pack2<kBf16>(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
                w4.z = pack2<kBf16>(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
                w4.w = pack2<kBf16>(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
                const int cg = c * 4 + g;
                *reinterpret_cast<uint4*>(stg + row_in_tile * (HD * 2) + ((cg ^ (row_in_tile & (kRowChunks - 1))) << 4)) = w4;
            }
        }
        // the accumulator has been read: P.V of the next item may overwrite it (it is
        // issued only after this thread's next arrival on p_full, which comes later)
        tc_fence_before();
        named_sync(1 + t, 128);                     // the 128 threads of this query tile
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
                    const uint4 w4 = *reinterpret_cast<const uint4*>(stg + r * (HD * 2) + ((cg ^ (r & (kRowChunks - 1))) << 4));
                    const long long off = 2 * (static_cast<long long>(batch) * o_bs + static_cast<long long>(rs) * o_ld +
                                               static_cast<long long>(head) * a.hd_out + cg * 8);
                    *reinterpret_cast<uint4*>(obase + off) = w4;
                    if (!push_peers) {
                        // fused all-gather by the softmax warps themselves (only when warps
                        // 10-11 are taken by the K / V scaling): plain stores over NVLink
                        for (int pi = 0; pi < a.n_peers; ++pi) {
                            uint8_t* pb = reinterpret_cast<uint8_t*>(qseg ? a.o_peer[1][pi] : a.o_peer[0][pi]);
                            *reinterpret_cast<uint4*>(pb + off) = w4;
                        }
                    }
                }
            }
        }
        if (push_peers) {
            // the tile's rows are in the local copy: warps 10-11 forward them to the peers
            __threadfence();
            __syncwarp();
            if (lane == 0) mbar_arrive(&out_done[t]);
        }
        if (t == 0) named_arrive(3, 256);
        else if (has_next) named_arrive(4, 256);
        if (n_kv > 0) { jb += n_kv; ++qn; }
        }   // items
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
            MmaCtx cx;
            cx.q_full = q_full; cx.q_ready = q_ready; cx.kv_rdy = kScale ? kv_ready : kv_full; cx.kv_empty = kv_empty;
            cx.s_full = s_full; cx.p_full = p_full; cx.pv_done = pv_done; cx.q_empty = q_empty;
            cx.tmem_base = tmem_base; cx.q_base_addr = smem_u32(smem_q); cx.kv_base_addr = smem_u32(smem_kv);
            cx.n_items = n_items; cx.w0 = w0; cx.wstep = wstep; cx.lane = lane;
            mma_role<HD, kBf16, ST>(a, cx);
        } else if (warp == 9) {
            // ------------------------------------------------ TMA producer
            if (lane == 0) {
                bool ok = true;
                int qn = 0;          // earlier items with key tiles (phase of q_full / q_empty)
                int gi = 0;          // ring items issued so far, over all items
                int q_issued = 0;    // Q loads issued so far
                for (int w = w0; ok && w < n_items; w += wstep) {
                    const Item im = decode_item(a, w);
                    const int n_kv = im.n_kv;
                    if (n_kv == 0) continue;
                    // the Q tiles are free once every Q.K^T MMA of the previous item has completed
                    if (qn > 0) {
                        ok = mbar_wait(q_empty, static_cast<uint32_t>((qn - 1) & 1));
                        if (!ok) break;
                    }
                    const CUtensorMap* mq = im.qseg ? &tmQ1 : &tmQ0;
                    for (int t = 0; t < 2; ++t) {
                        mbar_arrive_expect_tx(&q_full[t], C::kQBytes);
                        for (int c = 0; c < C::kChunks; ++c) {
                            tma_load_4d(smem_q + t * C::kQBytes + c * kChunkBytes, mq, &q_full[t],
                                        c * 64, im.head, im.qrow0 + t * kBM, im.batch);
                        }
                    }
                    ++q_issued;
                    const int kv_head = im.head / a.kv_group;
                    for (int i = 0; i < 2 * n_kv; ++i, ++gi) {
                        const int slot = gi % ST;
                        if (gi >= ST) {
                            ok = mbar_wait(&kv_empty[slot], static_cast<uint32_t>(((gi / ST) - 1) & 1));
                            if (!ok) break;
                        }
                        const TileInfo ti = kv_tile(a, i >> 1);
                        const CUtensorMap* m = (i & 1) ? (ti.seg ? &tmV1 : &tmV0) : (ti.seg ? &tmK1 : &tmK0);
                        mbar_arrive_expect_tx(&kv_full[slot], C::kTileBytes);
                        for (int c = 0; c < C::kChunks; ++c) {
                            tma_load_4d(smem_kv + slot * C::kTileBytes + c * kChunkBytes, m, &kv_full[slot],
                                        c * 64, kv_head, ti.row0, im.batch);
                        }
                    }
                    if (!ok) break;
                    ++qn;
                }
                if (!ok) {
                    // Unwinding after a wait ran out: let the copies already in
                    // flight land before the CTA gives its shared memory back.
                    if (q_issued > 0) {
                        mbar_wait(&q_full[0], static_cast<uint32_t>((q_issued - 1) & 1));
                        mbar_wait(&q_full[1], static_cast<uint32_t>((q_issued - 1) & 1));
                    }
                    for (int i = max(0, gi - ST); i < gi; ++i) {
                        mbar_wait(&kv_full[i % ST], static_cast<uint32_t>((i / ST) & 1));
                    }
                }
            }
            __syncwarp();
        } else if (warp >= 10) {
            // ------------------------------------------- K / V row scaling
            // Warps 10 and 11 both walk the ring items in order (each sees every phase
            // of the barriers it waits on) and take half of a tile's lines each.  The
            // row factors of an item are fetched before the wait for its tile.  A tile
            // none of whose factors differs from one is passed on as it is; otherwise
            // every 128-byte line (one row of a 64-column chunk; the swizzle permutes
            // inside the line only) is multiplied by its row's factor.
            if constexpr (kScale) {
                const int half_id = warp - 10;
                bool ok = true;
                int gi = 0;      // ring items seen so far, over all work items
                for (int w = w0; ok && w < n_items; w += wstep) {
                const int n_kv = decode_item(a, w).n_kv;
                // row factors of ring item i (rows lane, lane + 32, ...), fetched one item ahead
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
                for (int i = 0; ok && i < 2 * n_kv; ++i, ++gi) {
                    const int slot = gi % ST;
#pragma unroll
                    for (int w = 0; w < 4; ++w) f[w] = fn[w];
                    fetch(i + 1, fn);
                    const bool ne = f[0] != 1.0f || f[1] != 1.0f || f[2] != 1.0f || f[3] != 1.0f;
                    const bool scale_tile = __any_sync(0xffffffffu, ne);
                    ok = mbar_wait(&kv_full[slot], static_cast<uint32_t>((gi / ST) & 1));
                    if (!ok) break;
                    if (scale_tile) {
                        uint8_t* tile = smem_kv + slot * C::kTileBytes;
                        // lane -> 16-byte piece (lane & 7) of row 4 * g + (lane >> 3) of a chunk;
                        // this warp takes the row groups g of its parity
                        constexpr int kIters = 16 * C::kChunks;
                        constexpr int kBatch = 4;       // loads of a batch are issued before its stores
#pragma unroll 1
                        for (int it0 = 0; it0 < kIters; it0 += kBatch) {
                            uint4 v[kBatch];
                            float fr[kBatch];
#pragma unroll
                            for (int b = 0; b < kBatch; ++b) {
                                const int it = it0 + b;
                                const int g = ((it & 15) << 1) + half_id;      // row group 0..31
                                const int r = (g << 2) + (lane >> 3);
                                const int fw = g >> 3;                          // = r >> 5, the same for the whole warp
                                const float fsel = fw == 0 ? f[0] : (fw == 1 ? f[1] : (fw == 2 ? f[2] : f[3]));
                                fr[b] = __shfl_sync(0xffffffffu, fsel, r & 31);
                                v[b] = *reinterpret_cast<const uint4*>(tile + (it >> 4) * kChunkBytes + r * 128 + ((lane & 7) << 4));
                            }
#pragma unroll
                            for (int b = 0; b < kBatch; ++b) {
                                uint32_t* w32 = reinterpret_cast<uint32_t*>(&v[b]);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float lo, hi;
                                    if constexpr (kBf16) {
                                        lo = __uint_as_float(w32[e] << 16);
                                        hi = __uint_as_float(w32[e] & 0xffff0000u);
                                    } else {
                                        const __half2 h = *reinterpret_cast<const __half2*>(&w32[e]);
                                        lo = __low2float(h);
                                        hi = __high2float(h);
                                    }
                                    w32[e] = pack2<kBf16>(lo * fr[b], hi * fr[b]);
                                }
                            }
#pragma unroll
                            for (int b = 0; b < kBatch; ++b) {
                                const int it = it0 + b;
                                const int r = ((((it & 15) << 1) + half_id) << 2) + (lane >> 3);
                                *reinterpret_cast<uint4*>(tile + (it >> 4) * kChunkBytes + r * 128 + ((lane & 7) << 4)) = v[b];
                            }
                        }
                        fence_proxy_async_smem();      // the MMA reads the tile through the async proxy
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&kv_ready[slot]);
                }
                }   // work items
            } else if (push_peers) {
                // ------------------------------------- fused all-gather: peer push
                // Once a tile's rows are in this GPU's copy of the output (signalled by
                // its softmax warps), these two warps read them back (L2) and store them
                // to the same place in every peer's copy: plain 16-byte loads of local
                // memory and stores over NVLink, running behind the attention of the
                // following items instead of holding up the softmax warps.
                const int lane64 = (warp - 10) * 32 + lane;
                bool ok = true;
                for (int w = w0, item_no = 0; ok && w < n_items; w += wstep, ++item_no) {
                    const Item im = decode_item(a, w);
                    const uint8_t* obase = reinterpret_cast<const uint8_t*>(im.qseg ? a.o[1] : a.o[0]);
                    const long long o_ld = im.qseg ? a.o_ld[1] : a.o_ld[0];
                    const long long o_bs = im.qseg ? a.o_bs[1] : a.o_bs[0];
                    const int out_chunks = a.hd_out >> 3;
                    for (int t = 0; t < 2 && ok; ++t) {
                        ok = __all_sync(0xffffffffu, mbar_wait(&out_done[t], static_cast<uint32_t>(item_no & 1)));
                        if (!ok) break;
                        const int rows = min(kBM, im.seg_rows - (im.qrow0 + t * kBM));
                        for (int idx = lane64; idx < rows * out_chunks; idx += 64) {
                            const int r = idx / out_chunks;
                            const int cg = idx - r * out_chunks;
                            const long long off = 2 * (static_cast<long long>(im.batch) * o_bs +
                                                       static_cast<long long>(im.qrow0 + t * kBM + r) * o_ld +
                                                       static_cast<long long>(im.head) * a.hd_out + cg * 8);
                            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(obase + off));
                            for (int pi = 0; pi < a.n_peers; ++pi) {
                                uint8_t* pb = reinterpret_cast<uint8_t*>(im.qseg ? a.o_peer[1][pi] : a.o_peer[0][pi]);
                                *reinterpret_cast<uint4*>(pb + off) = v;
                            }
                        }
                    }
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
    auto kern = sdpa_tc05_persistent_kernel<HD, kBf16, kHooks, kScale>;
    cudaError_t e = set_max_smem_once(kern, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    SdpaDevArgs args = L.args;
    args.item_q_ctas = L.q_ctas;
    args.item_heads = L.num_heads;
    const long long n_items = static_cast<long long>(L.q_ctas) * L.num_heads * L.batch;
    if (n_items < 1 || n_items > 0x7fffffffLL) return cudaErrorInvalidValue;
    args.n_items = static_cast<int>(n_items);
    // persistent grid: one CTA per SM (shared and tensor memory allow no more), fewer for small calls
    const int sms = sm_count();
    const unsigned grid = static_cast<unsigned>(n_items < sms ? n_items : sms);
    kern<<<grid, kThreads, C::kSmemBytes, stream>>>(L.tmQ[0], L.tmQ[1], L.tmK[0], L.tmK[1], L.tmV[0],
                                                   L.tmV[1], args);
    return cudaGetLastError();
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
}  // namespace persist

cudaError_t launch_sdpa_tc05_persistent(const SdpaLaunch& L, cudaStream_t stream) {
    if (L.head_dim == 128) return L.bf16 ? persist::launch_hd<128, true>(L, stream) : persist::launch_hd<128, false>(L, stream);
    if (L.head_dim == 64) return L.bf16 ? persist::launch_hd<64, true>(L, stream) : persist::launch_hd<64, false>(L, stream);
    return cudaErrorInvalidValue;
}

}  // namespace bdattn
