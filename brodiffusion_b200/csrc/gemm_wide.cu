// Persistent wide-tile linear layer for the large projections (Q/K/V of a
// DiT block: src/dit/flux.cpp:471-484; out-projection: src/dit/flux.cpp:519-525):
//   C[M,N] = A[M,K] . W[N,K]^T (+ bias) [-> per-head RMSNorm -> RoPE]
// Same operand layout and epilogue arithmetic as gemm_tc05_kernel; what differs
// is the schedule, chosen for problems with at least one 128 x 256 tile per SM:
//   * one CTA per SM walks a list of 128-row x 256-column tiles (up to three
//     problems in one launch, tiles of one column block adjacent so that the
//     CTAs running together share a few weight tiles in L2);
//   * an MMA of N = 256 reads 12 KB of shared memory per 128 tensor-pipe
//     cycles instead of 8 KB per 64, which keeps the operand reads and the TMA
//     fill of the next stage inside the shared-memory bandwidth;
//   * the accumulator is double-buffered in tensor memory (2 x 256 columns),
//     so the epilogue of tile i (bias, RMSNorm, RoPE, stores) runs while the
//     MMAs of tile i+1 are issued.
// GEGLU (src/fused_transformer.cu:89-92,275-282) runs here too: a tile is then
// 128 value columns + their 128 gate columns (weight rows n0.. and D_out + n0..
// loaded as the two halves of the B stage), one N = 256 MMA computes both and
// the epilogue stores value * gelu_exact(gate).
// Roles: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer and TMEM owner,
// warps 2-9 = epilogue (warp w owns TMEM lanes 32 * (w % 4)..; warps 2-5 take
// the first half of a tile's output columns, warps 6-9 the second half).
#include <cstdlib>

#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

constexpr int kWThreads = 320;
constexpr int kWStages = 4;
constexpr int kWTileN = 256;
constexpr int kWABytes = 128 * 64 * 2;        // A stage: 128 rows x 64 columns
constexpr int kWBBytes = kWTileN * 64 * 2;    // B stage: 256 weight rows x 64 columns
constexpr int kWStageBytes = kWABytes + kWBBytes;
constexpr int kWSmemBytes = kWStages * kWStageBytes + 256 + 3 * 128 * 4 + 1024;

struct WideTile {
    int z, m0, n0;
};

// Output columns of one tile: 256, or 128 for GEGLU (the other 128 accumulator
// columns hold the gate).
__host__ __device__ __forceinline__ int wide_out_cols(const GemmProblem& p) {
    return p.geglu_offset > 0 ? kWTileN / 2 : kWTileN;
}

__device__ __forceinline__ WideTile wide_tile(const GemmArgs& g, int tile) {
    int z = 0;
    int local = tile;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int cnt = g.p[i].tiles_m * (g.p[i].N / wide_out_cols(g.p[i]));
        if (z == i && local >= cnt) {
            local -= cnt;
            z = i + 1;
        }
    }
    const int tm = z == 0 ? g.p[0].tiles_m : (z == 1 ? g.p[1].tiles_m : g.p[2].tiles_m);
    const int wn = z == 0 ? wide_out_cols(g.p[0]) : (z == 1 ? wide_out_cols(g.p[1]) : wide_out_cols(g.p[2]));
    WideTile t;
    t.z = z;
    t.n0 = (local / tm) * wn;
    t.m0 = (local % tm) * 128;
    return t;
}

template <bool kBf16>
__device__ __forceinline__ float load16(const void* base, long long i) {
    const uint16_t b = reinterpret_cast<const uint16_t*>(base)[i];
    return kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                 : __half2float(*reinterpret_cast<const __half*>(&b));
}

// Epilogue of a tile that holds 256 / HD whole heads; this thread owns one
// token's row of each: RMSNorm over the head and the rotary embedding are
// thread-local (src/dit/flux.cpp:462-469, src/dit/common.cpp:192-193).  Two
// passes over the accumulator (tensor memory reads are cheap): sum of squares
// per head first, then 32 columns at a time so that one load of the token's
// cos / sin serves every head of the tile.  gain_s: the HD gains in shared
// memory as FP32, or null for no RMSNorm.
template <int HD, bool kBf16>
__device__ __forceinline__ void epilogue_heads(const GemmProblem& p, uint32_t tacc, uint16_t* crow, int row,
                                               int n0, const float* gain_s, int half) {
    // this warp group's share of the tile: half of its heads
    constexpr int kHeads = kWTileN / HD / 2;
    tacc += static_cast<uint32_t>(half * (kWTileN / 2));
    crow += half * (kWTileN / 2);
    n0 += half * (kWTileN / 2);
    float inv[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) inv[h] = 1.0f;
    if (gain_s != nullptr) {
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            float ss0 = 0.0f, ss1 = 0.0f;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tacc + h * HD + c * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
                    if (p.bias != nullptr) {
                        x0 += load16<kBf16>(p.bias, n0 + h * HD + c * 32 + i);
                        x1 += load16<kBf16>(p.bias, n0 + h * HD + c * 32 + i + 1);
                    }
                    ss0 = fmaf(x0, x0, ss0);
                    ss1 = fmaf(x1, x1, ss1);
                }
            }
            inv[h] = rsqrtf((ss0 + ss1) / static_cast<float>(HD) + p.eps);
        }
    }
    const bool rope = p.cos != nullptr;
    const long long tb = static_cast<long long>(p.rope_row0 + row) * (HD / 2);
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
        float cs[16], sn[16];
        if (rope && row < p.M) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(p.cos + tb + c * 16) + i);
                const float4 b = __ldg(reinterpret_cast<const float4*>(p.sin + tb + c * 16) + i);
                cs[4 * i] = a.x; cs[4 * i + 1] = a.y; cs[4 * i + 2] = a.z; cs[4 * i + 3] = a.w;
                sn[4 * i] = b.x; sn[4 * i + 1] = b.y; sn[4 * i + 2] = b.z; sn[4 * i + 3] = b.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) { cs[i] = 1.0f; sn[i] = 0.0f; }
        }
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            uint32_t v[32];
            tmem_ld32(tacc + h * HD + c * 32, v);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float x = __uint_as_float(v[i]);
                if (p.bias != nullptr) x += load16<kBf16>(p.bias, n0 + h * HD + c * 32 + i);
                if (gain_s != nullptr) x *= inv[h] * gain_s[c * 32 + i];
                f[i] = x;
            }
            if (rope) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a0 = f[2 * i], b0 = f[2 * i + 1];
                    f[2 * i] = a0 * cs[i] - b0 * sn[i];
                    f[2 * i + 1] = a0 * sn[i] + b0 * cs[i];
                }
            }
            if (row < p.M) {
#pragma unroll
                for (int v8 = 0; v8 < 4; ++v8) {
                    uint4 w;
                    w.x = pack2<kBf16>(f[v8 * 8 + 0], f[v8 * 8 + 1]);
                    w.y = pack2<kBf16>(f[v8 * 8 + 2], f[v8 * 8 + 3]);
                    w.z = pack2<kBf16>(f[v8 * 8 + 4], f[v8 * 8 + 5]);
                    w.w = pack2<kBf16>(f[v8 * 8 + 6], f[v8 * 8 + 7]);
                    *reinterpret_cast<uint4*>(crow + h * HD + c * 32 + v8 * 8) = w;
                }
            }
        }
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(kWThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB0,
                 const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
                 const GemmArgs g, const int total_tiles) {
    extern __shared__ uint8_t gemm_wide_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_wide_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWStages * kWStageBytes);
    uint64_t* full = bars;                   // [kWStages]
    uint64_t* empty = bars + kWStages;       // [kWStages]
    uint64_t* acc_full = empty + kWStages;   // [2]
    uint64_t* acc_empty = acc_full + 2;      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    float* gain_s = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);   // [3][128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 256);
        }
        fence_mbar_init();
    }
    // RMSNorm gains of the three problems as FP32 (read by every epilogue thread)
    for (int idx = threadIdx.x; idx < 3 * 128; idx += kWThreads) {
        const GemmProblem& gp = idx < 128 ? g.p[0] : (idx < 256 ? g.p[1] : g.p[2]);
        const int i = idx & 127;
        float gv = 1.0f;
        if (gp.norm_rope && gp.gain != nullptr && i < gp.n_tile)
            gv = gp.gain_is_f32 ? __ldg(reinterpret_cast<const float*>(gp.gain) + i) : load16<kBf16>(gp.gain, i);
        gain_s[idx] = gv;
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmA0);
        tma_prefetch_desc(&tmB0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------- TMA producer
        if (lane == 0) {
            int it = 0;          // stage uses so far, over all tiles of this CTA
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const WideTile t = wide_tile(g, tile);
                const CUtensorMap* tmA = t.z == 0 ? &tmA0 : (t.z == 1 ? &tmA1 : &tmA2);
                const CUtensorMap* tmB = t.z == 0 ? &tmB0 : (t.z == 1 ? &tmB1 : &tmB2);
                const int K = t.z == 0 ? g.p[0].K : (t.z == 1 ? g.p[1].K : g.p[2].K);
                const int geglu_off = t.z == 0 ? g.p[0].geglu_offset : (t.z == 1 ? g.p[1].geglu_offset : g.p[2].geglu_offset);
                const int k_blocks = (K + 63) / 64;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kWStages;
                    if (it >= kWStages) {
                        ok = mbar_wait(&empty[s], static_cast<uint32_t>(((it / kWStages) - 1) & 1));
                        if (!ok) break;
                    }
                    uint8_t* st = smem + s * kWStageBytes;
                    mbar_arrive_expect_tx(&full[s], kWStageBytes);
                    tma_load_2d(st, tmA, &full[s], kb * 64, t.m0);
                    if (geglu_off > 0) {
                        // value rows, then the gate rows of the same output columns (128-row boxes)
                        tma_load_2d(st + kWABytes, tmB, &full[s], kb * 64, t.n0);
                        tma_load_2d(st + kWABytes + kWBBytes / 2, tmB, &full[s], kb * 64, geglu_off + t.n0);
                    } else {
                        tma_load_2d(st + kWABytes, tmB, &full[s], kb * 64, t.n0);
                    }
                }
            }
            if (!ok) {
                // a wait ran out: let the copies in flight land before the CTA ends
                for (int i = max(0, it - kWStages); i < it; ++i)
                    mbar_wait(&full[i % kWStages], static_cast<uint32_t>((i / kWStages) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = make_idesc_f16(kBf16 ? 1 : 0, 128, kWTileN, 0, 0);
        int it = 0;
        int ti = 0;              // tiles done by this CTA
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++ti) {
            const WideTile t = wide_tile(g, tile);
            const int K = t.z == 0 ? g.p[0].K : (t.z == 1 ? g.p[1].K : g.p[2].K);
            const int k_blocks = (K + 63) / 64;
            const int as = ti & 1;
            if (ti >= 2) {       // the epilogue must have drained this accumulator (tile ti - 2)
                ok = mbar_wait(&acc_empty[as], static_cast<uint32_t>(((ti >> 1) - 1) & 1));
                if (!ok) break;
                tc_fence_after();
            }
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(as * kWTileN);
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % kWStages;
                ok = mbar_wait(&full[s], static_cast<uint32_t>((it / kWStages) & 1));
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t ab = smem_u32(smem + s * kWStageBytes);
                    const uint32_t bb = ab + kWABytes;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        umma_ss(d_tmem, make_smem_desc_sw128(ab + kk * 32, 16, 1024),
                                make_smem_desc_sw128(bb + kk * 32, 16, 1024), idesc,
                                (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                    if (kb == k_blocks - 1) umma_commit(&acc_full[as]);
                }
                __syncwarp();
            }
        }
    } else {
        // -------------------------------------------------------- epilogue
        const int q = warp & 3;             // TMEM lane quarter of this warp
        const int half = (warp - 2) >> 2;   // which half of the tile's output columns
        int ti = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
            const WideTile t = wide_tile(g, tile);
            const GemmProblem& p = t.z == 0 ? g.p[0] : (t.z == 1 ? g.p[1] : g.p[2]);
            const int as = ti & 1;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[as], static_cast<uint32_t>((ti >> 1) & 1)));
            if (!ok) break;
            tc_fence_after();
            const int row = t.m0 + q * 32 + lane;
            const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(as * kWTileN);
            uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(row) * p.ldc + t.n0;
            if (p.norm_rope) {
                const float* gs = p.gain != nullptr ? gain_s + t.z * 128 : nullptr;
                if (p.n_tile == 128) epilogue_heads<128, kBf16>(p, tacc, crow, row, t.n0, gs, half);
                else epilogue_heads<64, kBf16>(p, tacc, crow, row, t.n0, gs, half);
            } else if (p.geglu_offset > 0) {
                // value in accumulator columns [0, 128), gate in [128, 256); this group
                // stores 64 of the tile's 128 output columns
                for (int c = half * 64; c < half * 64 + 64; c += 32) {
                    uint32_t v[32], gt[32];
                    tmem_ld32(tacc + c, v);
                    tmem_ld32(tacc + 128 + c, gt);
                    tmem_wait_ld();
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float x = __uint_as_float(v[i]);
                        float gate = __uint_as_float(gt[i]);
                        if (p.bias != nullptr) {
                            x += load16<kBf16>(p.bias, t.n0 + c + i);
                            gate += load16<kBf16>(p.bias, p.geglu_offset + t.n0 + c + i);
                        }
                        f[i] = x * (0.5f * gate * (1.0f + erff(gate * 0.7071067811865475f)));
                    }
                    if (row < p.M) {
#pragma unroll
                        for (int v8 = 0; v8 < 4; ++v8) {
                            uint4 w;
                            w.x = pack2<kBf16>(f[v8 * 8 + 0], f[v8 * 8 + 1]);
                            w.y = pack2<kBf16>(f[v8 * 8 + 2], f[v8 * 8 + 3]);
                            w.z = pack2<kBf16>(f[v8 * 8 + 4], f[v8 * 8 + 5]);
                            w.w = pack2<kBf16>(f[v8 * 8 + 6], f[v8 * 8 + 7]);
                            *reinterpret_cast<uint4*>(crow + c + v8 * 8) = w;
                        }
                    }
                }
            } else {
                for (int c = half * (kWTileN / 2); c < (half + 1) * (kWTileN / 2); c += 32) {
                    uint32_t v[32];
                    tmem_ld32(tacc + c, v);
                    tmem_wait_ld();
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float x = __uint_as_float(v[i]);
                        if (p.bias != nullptr) x += load16<kBf16>(p.bias, t.n0 + c + i);
                        f[i] = x;
                    }
                    if (row < p.M) {
#pragma unroll
                        for (int v8 = 0; v8 < 4; ++v8) {
                            uint4 w;
                            w.x = pack2<kBf16>(f[v8 * 8 + 0], f[v8 * 8 + 1]);
                            w.y = pack2<kBf16>(f[v8 * 8 + 2], f[v8 * 8 + 3]);
                            w.z = pack2<kBf16>(f[v8 * 8 + 4], f[v8 * 8 + 5]);
                            w.w = pack2<kBf16>(f[v8 * 8 + 6], f[v8 * 8 + 7]);
                            *reinterpret_cast<uint4*>(crow + c + v8 * 8) = w;
                        }
                    }
                }
            }
            // this accumulator may be overwritten by the MMAs of tile ti + 2
            tc_fence_before();
            mbar_arrive(&acc_empty[as]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

int gemm_wide_tiles(const GemmLaunch& L) {
    int total = 0;
    for (int i = 0; i < L.n_problems; ++i) total += L.args.p[i].tiles_m * (L.args.p[i].N / wide_out_cols(L.args.p[i]));
    return total;
}

cudaError_t launch_gemm_wide(const GemmLaunch& L, cudaStream_t stream) {
    const int total = gemm_wide_tiles(L);
    const int sms = sm_count();
    cudaError_t e;
    const int grid = total < sms ? total : sms;
    if (L.bf16) {
        e = set_max_smem_once(gemm_wide_kernel<true>, kWSmemBytes);
        if (e != cudaSuccess) return e;
        gemm_wide_kernel<true><<<grid, kWThreads, kWSmemBytes, stream>>>(
            L.tmA[0], L.tmA[1], L.tmA[2], L.tmBw[0], L.tmBw[1], L.tmBw[2], L.args, total);
    } else {
        e = set_max_smem_once(gemm_wide_kernel<false>, kWSmemBytes);
        if (e != cudaSuccess) return e;
        gemm_wide_kernel<false><<<grid, kWThreads, kWSmemBytes, stream>>>(
            L.tmA[0], L.tmA[1], L.tmA[2], L.tmBw[0], L.tmBw[1], L.tmBw[2], L.args, total);
    }
    return cudaGetLastError();
}

// BDATTN_GEMM_WIDE=0 keeps every problem on the one-tile-per-CTA kernel (tuning runs).
cudaError_t launch_gemm(const GemmLaunch& L, cudaStream_t stream) {
    static const int mode = [] {
        const char* e = std::getenv("BDATTN_GEMM_WIDE");
        return e != nullptr ? std::atoi(e) : 1;
    }();
    bool wide = mode != 0 && L.n_problems > 0;
    for (int i = 0; i < L.n_problems; ++i) wide = wide && L.wide[i];
    if (wide) {
        if (gemm_wide_tiles(L) >= sm_count()) return launch_gemm_wide(L, stream);
    }
    return launch_gemm_tc05(L, stream);
}

}  // namespace bdattn
