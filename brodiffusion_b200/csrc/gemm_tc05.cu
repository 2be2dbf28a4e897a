// Linear layers on the sm_100a tensor cores:  C[M,N] = A[M,K] . B[N,K]^T (+ bias)
// with 16-bit operands, FP32 accumulation in tensor memory and a fused
// epilogue.  Weights are stored (out_features, in_features) as in the
// reference (src/unet_blocks.cpp:264-271), so both operands are K-major and
// are staged by TMA with the 128-byte swizzle.
//
// Up to three independent problems share one launch (blockIdx.z): the Q, K
// and V projections of one attention call.  A CTA computes one 128-row x
// n_tile-column tile:
//   warp 0     TMA producer (A tile 128 x 64, B tile n_tile x 64 per K block)
//   warp 1     tcgen05.mma issuer, owns the TMEM allocation
//   warps 2-5  epilogue: tcgen05.ld -> bias / GEGLU -> 16-byte stores
// Tiles may be head-aligned: tile t starts at weight row t * n_step and its
// n_valid columns land at output column t * c_step, zero-filled up to c_fill.
// That writes Q/K/V with every head padded to the width the attention kernel
// takes (40 -> 64, 80 -> 128) without a separate padding pass.
//
// GEGLU mode (src/fused_transformer.cu:89-92,275-282): a second B tile from
// weight row n0 + D_out feeds a second accumulator and the epilogue stores
// value * gelu_exact(gate), so the (B, 2*D_out) intermediate never exists.
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

constexpr int kGemmThreads = 192;
constexpr int kGemmMaxStages = 4;
constexpr int kGemmABytes = 128 * 64 * 2;   // A stage
// A B (or gate) tile is n_tile rows x 128 B; a stage holds A, B and, for GEGLU,
// the gate tile, rounded up to the 1024-byte swizzle period.  Sizing the stage by
// the tile shape keeps a 64-column GEMM at 96 KB so that two CTAs share an SM.
__host__ __device__ inline int gemm_b_bytes(int n_tile) { return (n_tile * 128 + 1023) / 1024 * 1024; }
__host__ __device__ inline int gemm_stage_bytes(int n_tile, bool geglu) {
    return kGemmABytes + (geglu ? 2 : 1) * gemm_b_bytes(n_tile);
}

// One instantiation per epilogue (plain, GEGLU, norm + RoPE): the GEGLU and the norm +
// RoPE code are long, and an epilogue that only branches around them spent more time
// fetching instructions than storing (5.6 us for one 128 x 128 tile against 2.3 us).
template <bool kBf16, bool kGeglu, bool kNormRope>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB0,
                 const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
                 const GemmArgs g) {
    const int z = blockIdx.z;
    const GemmProblem& p = z == 0 ? g.p[0] : (z == 1 ? g.p[1] : g.p[2]);
    const CUtensorMap* tmA = z == 0 ? &tmA0 : (z == 1 ? &tmA1 : &tmA2);
    const CUtensorMap* tmB = z == 0 ? &tmB0 : (z == 1 ? &tmB1 : &tmB2);
    const int tile_n = blockIdx.x;
    const int tile_m = blockIdx.y;
    if (tile_n >= p.tiles_n || tile_m >= p.tiles_m) return;

    extern __shared__ uint8_t gemm_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int kGemmStages = g.stages;
    const int kGemmBBytes = gemm_b_bytes(g.n_tile_max);
    const int kGemmStageBytes = gemm_stage_bytes(g.n_tile_max, g.any_geglu != 0);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kGemmStages * kGemmStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + kGemmMaxStages;
    uint64_t* acc_done = empty + kGemmMaxStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = (p.K + 63) / 64;
    const int n0 = tile_n * p.n_step;
    const int m0 = tile_m * 128;
    const bool geglu = kGeglu && p.geglu_offset > 0;
    constexpr uint32_t kTmemCols = kGeglu ? 256 : 128;     // the gate accumulator sits 128 columns up

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_done, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t bytes = kGemmABytes + (geglu ? 2u : 1u) * static_cast<uint32_t>(p.n_tile) * 128u;
            bool ok = true;
            int issued = 0;
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % kGemmStages;
                if (kb >= kGemmStages) {
                    ok = mbar_wait(&empty[s], static_cast<uint32_t>(((kb / kGemmStages) - 1) & 1));
                    if (!ok) break;
                }
                uint8_t* st = smem + s * kGemmStageBytes;
                mbar_arrive_expect_tx(&full[s], bytes);
                tma_load_2d(st, tmA, &full[s], kb * 64, m0);
                tma_load_2d(st + kGemmABytes, tmB, &full[s], kb * 64, n0);
                if (geglu) tma_load_2d(st + kGemmABytes + kGemmBBytes, tmB, &full[s], kb * 64, n0 + p.geglu_offset);
                issued = kb + 1;
            }
            if (!ok) {
                for (int kb = max(0, issued - kGemmStages); kb < issued; ++kb)
                    mbar_wait(&full[kb % kGemmStages], static_cast<uint32_t>((kb / kGemmStages) & 1));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_f16(kBf16 ? 1 : 0, 128, p.n_tile, 0, 0);
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int s = kb % kGemmStages;
            ok = mbar_wait(&full[s], static_cast<uint32_t>((kb / kGemmStages) & 1));
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t ab = smem_u32(smem + s * kGemmStageBytes);
                const uint32_t bb = ab + kGemmABytes;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t ad = make_smem_desc_sw128(ab + kk * 32, 16, 1024);
                    umma_ss(tmem_base, ad, make_smem_desc_sw128(bb + kk * 32, 16, 1024), idesc,
                            (kb > 0 || kk > 0) ? 1u : 0u);
                    if (geglu)
                        umma_ss(tmem_base + 128, ad, make_smem_desc_sw128(bb + kGemmBBytes + kk * 32, 16, 1024),
                                idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
                if (kb == k_blocks - 1) umma_commit(acc_done);
            }
            __syncwarp();
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32 * (w % 4) ..
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        bool ok = mbar_wait(acc_done, 0);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        const long long c0 = static_cast<long long>(tile_n) * p.c_step;
        uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(row) * p.ldc + c0;
        const int n_valid = min(p.n_valid, p.N - n0);
        // plain tiles stop at the matrix edge; head tiles own their padded slot
        const int c_lim = p.c_step == p.n_step ? min(p.c_fill, p.N - n0) : p.c_fill;
        if (kNormRope && ok && p.norm_rope) {
            // The tile is one head and this thread holds one token's row of it:
            // RMSNorm over the head and the rotary embedding are thread-local
            // (src/dit/flux.cpp:462-469 + src/dit/common.cpp:192-193 fused into
            // the projection, so Q and K never travel to HBM un-normalised).
            float f[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (c * 32 < p.n_tile) {
                    uint32_t v[32];
                    tmem_ld32(tacc + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float x = __uint_as_float(v[i]);
                        if (p.bias != nullptr) {
                            const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[n0 + c * 32 + i];
                            x += kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                                       : __half2float(*reinterpret_cast<const __half*>(&b));
                        }
                        f[c * 32 + i] = x;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[c * 32 + i] = 0.0f;
                }
            }
            if (p.gain != nullptr) {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 128; ++i) ss = fmaf(f[i], f[i], ss);
                const float inv = rsqrtf(ss / static_cast<float>(p.n_tile) + p.eps);
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    if (i < p.n_tile) {
                        float gv;
                        if (p.gain_is_f32) gv = __ldg(reinterpret_cast<const float*>(p.gain) + i);
                        else {
                            const uint16_t b = reinterpret_cast<const uint16_t*>(p.gain)[i];
                            gv = kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                                       : __half2float(*reinterpret_cast<const __half*>(&b));
                        }
                        f[i] *= inv * gv;
                    }
                }
            }
            if (p.cos != nullptr && row < p.M) {
                const long long t = static_cast<long long>(p.rope_row0 + row) * (p.n_tile / 2);
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    if (2 * i < p.n_tile) {
                        const float cv = __ldg(p.cos + t + i), sv = __ldg(p.sin + t + i);
                        const float a0 = f[2 * i], b0 = f[2 * i + 1];
                        f[2 * i] = a0 * cv - b0 * sv;
                        f[2 * i + 1] = a0 * sv + b0 * cv;
                    }
                }
            }
            if (row < p.M) {
#pragma unroll
                for (int v8 = 0; v8 < 16; ++v8) {
                    if (v8 * 8 < p.n_tile) {
                        uint4 w;
                        w.x = pack2<kBf16>(f[v8 * 8 + 0], f[v8 * 8 + 1]);
                        w.y = pack2<kBf16>(f[v8 * 8 + 2], f[v8 * 8 + 3]);
                        w.z = pack2<kBf16>(f[v8 * 8 + 4], f[v8 * 8 + 5]);
                        w.w = pack2<kBf16>(f[v8 * 8 + 6], f[v8 * 8 + 7]);
                        *reinterpret_cast<uint4*>(crow + v8 * 8) = w;
                    }
                }
            }
        } else if (ok) {
            for (int c = 0; c < c_lim; c += 32) {
                uint32_t v[32], gt[32];
                if (c < p.n_tile) {
                    tmem_ld32(tacc + c, v);
                    if (geglu) tmem_ld32(tacc + 128 + c, gt);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                // the 32 bias values of this piece (and of its gate), zero where there is none
                float bx[32], bg[kGeglu ? 32 : 1];
                const bool whole = c + 32 <= n_valid;
                if (p.bias != nullptr && whole) {
                    load32_as_float<kBf16>(p.bias, n0 + c, bx);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        bx[i] = 0.0f;
                        if (p.bias != nullptr && c + i < n_valid) {
                            const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[n0 + c + i];
                            bx[i] = kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                                          : __half2float(*reinterpret_cast<const __half*>(&b));
                        }
                    }
                }
                if constexpr (kGeglu) {
                    if (p.bias != nullptr && geglu && whole) {
                        load32_as_float<kBf16>(p.bias, n0 + p.geglu_offset + c, bg);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            bg[i] = 0.0f;
                            if (p.bias != nullptr && geglu && c + i < n_valid) {
                                const uint16_t b = reinterpret_cast<const uint16_t*>(p.bias)[n0 + p.geglu_offset + c + i];
                                bg[i] = kBf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16)
                                              : __half2float(*reinterpret_cast<const __half*>(&b));
                            }
                        }
                    }
                }
                float f[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float x = __uint_as_float(v[i]) + bx[i];
                    if constexpr (kGeglu) {
                        if (geglu) {
                            const float gate = __uint_as_float(gt[i]) + bg[i];
                            x *= 0.5f * gate * (1.0f + erff(gate * 0.7071067811865475f));
                        }
                    }
                    f[i] = c + i < n_valid ? x : 0.0f;
                }
                if (row < p.M) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        if (c + v8 * 8 < c_lim) {
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
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

cudaError_t launch_gemm_tc05(const GemmLaunch& L, cudaStream_t stream) {
    int tn = 0, tm = 0, nt_max = 16, any_geglu = 0, any_norm_rope = 0;
    for (int i = 0; i < L.n_problems; ++i) {
        tn = L.args.p[i].tiles_n > tn ? L.args.p[i].tiles_n : tn;
        tm = L.args.p[i].tiles_m > tm ? L.args.p[i].tiles_m : tm;
        nt_max = L.args.p[i].n_tile > nt_max ? L.args.p[i].n_tile : nt_max;
        any_geglu |= L.args.p[i].geglu_offset > 0 ? 1 : 0;
        any_norm_rope |= L.args.p[i].norm_rope ? 1 : 0;
    }
    GemmArgs args = L.args;
    args.n_tile_max = nt_max;
    args.any_geglu = any_geglu;
    // three stages with the gate tile: the stage ring stays below 114 KB and two CTAs fit per SM
    args.stages = any_geglu ? 3 : kGemmMaxStages;
    // Short K and more tiles than SMs: a ring of two (64 KB) lets up to three CTAs share an SM,
    // so that one CTA's epilogue runs under the others' loads (4096 x 320 -> 960: 18.1 -> 12.2 us).
    int k_max = 0;
    for (int i = 0; i < L.n_problems; ++i) k_max = L.args.p[i].K > k_max ? L.args.p[i].K : k_max;
    if (!any_geglu && k_max <= 512 && static_cast<long long>(tn) * tm * L.n_problems > sm_count()) args.stages = 2;
    const int kGemmSmemBytes = args.stages * gemm_stage_bytes(nt_max, any_geglu != 0) + 256 + 1024;
    dim3 grid(static_cast<unsigned>(tn), static_cast<unsigned>(tm), static_cast<unsigned>(L.n_problems));
    cudaError_t e = cudaSuccess;
    auto go = [&](auto kern) {
        e = set_max_smem_once(kern, 227 * 1024);
        if (e != cudaSuccess) return;
        kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(L.tmA[0], L.tmA[1], L.tmA[2], L.tmB[0], L.tmB[1],
                                                            L.tmB[2], args);
    };
    if (L.bf16) {
        if (any_norm_rope) go(gemm_tc05_kernel<true, false, true>);
        else if (any_geglu) go(gemm_tc05_kernel<true, true, false>);
        else go(gemm_tc05_kernel<true, false, false>);
    } else {
        if (any_norm_rope) go(gemm_tc05_kernel<false, false, true>);
        else if (any_geglu) go(gemm_tc05_kernel<false, true, false>);
        else go(gemm_tc05_kernel<false, false, false>);
    }
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace bdattn
