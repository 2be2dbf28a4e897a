// Sana ReLU linear attention (head_dim 32, BF16 storage, FP32 state).
//
// Math (src/dit/sana.cpp:470-520), per (batch, head), channel-major (32, N)
// operands Q, K, V:
//   [S; z] = [V; 1] relu(K)^T            (33 x 32, summed over the N tokens)
//   out    = (S relu(Q)) / (z relu(Q) + eps)
//
// One thread-block cluster of CS CTAs (CS in {1, 2, 4, 8}, picked so that
// batch * heads * CS fills the SMs; one CTA per SM) owns one (batch, head).
// A CTA has two groups of eight consumer warps that take the ring items in
// turn, and streams its share of the tokens twice:
//   pass A  K and V chunks (128 tokens) -> partial [S; z] on the legacy
//           tensor path (mma.sync m16n8k16, FP32 accumulate; the matrices are
//           32 x 32, far below a tcgen05 tile), ReLU applied to the B
//           fragments in registers, z summed from the same fragments;
//   reduce  warps -> CTA in shared memory, CTA -> cluster through distributed
//           shared memory (no global scratch);
//   pass B  Q chunks -> out = [S; z] relu(Q) with the state rounded to BF16
//           (FP32 accumulation), division by the z row; every warp stages its
//           own 32-row x 32-token BF16 piece of a 256-token item in shared memory
//           and sends it off with its own TMA store.
// Tiles arrive by TMA (64-token x 32-row boxes, 128-byte swizzle) into a ring
// shared by both passes and fed by a dedicated producer warp (full / empty
// mbarriers, no CTA-wide barrier in the loops), so the first Q chunks are in
// flight during the reduction.  HBM-bound: 4 * N * 32 * 2 bytes per (batch, head).
#include <cooperative_groups.h>

#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

namespace cg = cooperative_groups;

constexpr int kLaItemWarps = 8;               // consumer warps that work on one ring item
constexpr int kLaWarps = 16;                  // consumer warps: two groups of 8 take the ring items in turn, so
                                              // that twice as many independent instruction streams hide the
                                              // latencies of a chunk; one more warp feeds the ring by TMA
constexpr int kLaThreads = (kLaWarps + 1) * 32;
constexpr int kLaGroups = kLaWarps / kLaItemWarps;
constexpr int kLaChunk = 128;                 // tokens per ring item
constexpr int kLaMaxStages = 8;               // ring of 16 KB items; a multiple of the number of warp groups, so that
                                              // a group always meets the same slots and sees every phase of their
                                              // barriers (a ring of nine, where the groups alternate on every slot,
                                              // ended one run with a launch failure and is refused by the launcher)
constexpr int kLaBoxBytes = 32 * 64 * 2;      // one 64-token x 32-row box
constexpr int kLaSlotBytes = 4 * kLaBoxBytes; // K (2 boxes) + V (2 boxes)
constexpr int kLaPieceBytes = 32 * 32 * 2;    // output piece of one warp and item: 32 rows x 32 tokens (64-byte rows)
constexpr int kLaState = 33 * 32;             // [S; z] floats
constexpr int kLaStLd = 40;                   // row stride of the state tile in shared memory: the fragment
                                              // loads of the apply pass (rows over g, columns over q4) then
                                              // meet at most two to a bank instead of eight

struct LaSmem {
    union {
        float partial[kLaWarps][kLaState];                          // reduction between the passes
        alignas(1024) uint8_t out_stage[kLaWarps][2][kLaPieceBytes];  // pass B: two output pieces per warp
    };
    float local_state[kLaState];
    float state[48 * kLaStLd];   // rows 33..47 zero
    uint64_t full[kLaMaxStages];
    uint64_t empty[kLaMaxStages];
    alignas(1024) uint8_t ring[1][kLaSlotBytes];   // a.stages items follow (dynamic shared memory)
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// ReLU of two packed BF16 values: the fused multiply-add with the ReLU modifier
// (x * 1 + 0) runs on the FMA pipe; the packed maximum against zero issues at a
// quarter of that rate on this part.
__device__ __forceinline__ uint32_t relu2(uint32_t w) {
    uint32_t r;
    asm("fma.rn.relu.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0x3f803f80u), "r"(0u));
    return r;
}
__device__ __forceinline__ float sum2(uint32_t w) {
    return __uint_as_float(w << 16) + __uint_as_float(w & 0xffff0000u);
}
// Byte offset of (row, 16-byte chunk) inside a 128-byte-swizzled 32 x 64 box.
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(kLaThreads, 1)
linear_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                   const LinearAttnArgs a) {
    extern __shared__ uint8_t la_raw[];
    constexpr int kGroups = kLaGroups;      // group (item mod kGroups) takes an item
    LaSmem& sm = *reinterpret_cast<LaSmem*>((reinterpret_cast<uintptr_t>(la_raw) + 1023) &
                                            ~static_cast<uintptr_t>(1023));
    cg::cluster_group cluster = cg::this_cluster();
    const int cs = static_cast<int>(cluster.num_blocks());
    // Phase barrier of everything that shares this (batch, head): the cluster
    // barrier, or, for a cluster of one CTA, a plain block barrier (the hardware
    // cluster barrier costs microseconds even when it has a single member).
    auto phase_sync = [&]() {
        if (cs == 1) __syncthreads();
        else cluster.sync();
    };
    const int rank = static_cast<int>(cluster.block_rank());
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int q4 = lane & 3;

    const int chunks = (a.n_tokens + kLaChunk - 1) / kLaChunk;
    const int cpc = (chunks + cs - 1) / cs;
    const int c_begin = min(rank * cpc, chunks);
    const int c_end = min(c_begin + cpc, chunks);
    const int n_mine = c_end - c_begin;
    const int n_b = (n_mine + 1) / 2;  // pass B items carry two 128-token Q chunks (16 KB, like a pass A item)
    const int n_items = n_mine + n_b;  // pass A items (K + V chunks), then pass B items
    const int row0 = head * 32;
    const int kLaStages = a.stages;
    uint8_t* const ring_base = &sm.ring[0][0];     // a.stages items of kLaSlotBytes

    // Programmatic dependent launch: the next kernel of the stream (if it was
    // launched with the same attribute) may become resident as CTAs of this one
    // retire and run its own set-up; its griddepcontrol.wait holds it back until
    // this grid has completed and its writes are visible.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int s = 0; s < kLaStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kLaItemWarps);
        }
        fence_mbar_init();
    }
    for (int i = tid; i < 48 * kLaStLd; i += kLaThreads) sm.state[i] = 0.0f;
    if (tid == kLaWarps * 32) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmO);
    }
    // Everything above touched shared memory only.  No global read or write of this
    // kernel is issued before the preceding kernel of the stream has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    if (warp == kLaWarps) {
        // ------------------------------------------------------- TMA producer
        bool ok = true;
        auto issue = [&](int item) {
            const int slot = item % kLaStages;
            if (item >= kLaStages) {
                ok = mbar_wait(&sm.empty[slot], static_cast<uint32_t>(((item / kLaStages) - 1) & 1));
                if (!ok) return;
            }
            uint8_t* dst = ring_base + slot * kLaSlotBytes;
            if (item < n_mine) {
                const int tok = (c_begin + item) * kLaChunk;
                mbar_arrive_expect_tx(&sm.full[slot], 4 * kLaBoxBytes);
                tma_load_3d(dst, &tmK, &sm.full[slot], tok, row0, batch);
                tma_load_3d(dst + kLaBoxBytes, &tmK, &sm.full[slot], tok + 64, row0, batch);
                tma_load_3d(dst + 2 * kLaBoxBytes, &tmV, &sm.full[slot], tok, row0, batch);
                tma_load_3d(dst + 3 * kLaBoxBytes, &tmV, &sm.full[slot], tok + 64, row0, batch);
            } else {
                const int tok = (c_begin + 2 * (item - n_mine)) * kLaChunk;
                mbar_arrive_expect_tx(&sm.full[slot], 4 * kLaBoxBytes);
#pragma unroll
                for (int bx = 0; bx < 4; ++bx)
                    tma_load_3d(dst + bx * kLaBoxBytes, &tmQ, &sm.full[slot], tok + 64 * bx, row0, batch);
            }
        };
        // Items whose ring slot is freed during pass A can be issued before the
        // cluster-wide reduction; the rest follow it (their slots free up in pass B).
        const int first = min(n_items, n_mine + kLaStages);
        int issued = 0;
        if (lane == 0) {
            for (int it = 0; it < first && ok; ++it) { issue(it); if (ok) issued = it + 1; }
        }
        __syncwarp();
        phase_sync();
        phase_sync();
        if (lane == 0) {
            for (int it = first; it < n_items && ok; ++it) { issue(it); if (ok) issued = it + 1; }
            if (!ok) {
                // Unwinding after a wait ran out: let copies in flight land.
                for (int it = max(0, issued - kLaStages); it < issued; ++it)
                    mbar_wait(&sm.full[it % kLaStages], static_cast<uint32_t>((it / kLaStages) & 1));
            }
        }
        __syncwarp();
        phase_sync();
        return;
    }

    // ----------------------------------------------------------- consumers
    bool ok = true;
    float acc[2][4][4];
    float zacc[4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) zacc[nt] = 0.0f;

    const int group = warp / kLaItemWarps;   // which items this warp works on
    const int wg = warp % kLaItemWarps;      // its place among the eight warps of an item
    const int box = wg >> 2;             // which 64-token box of the chunk
    const int chunk0 = (wg & 3) * 2;     // first 16-byte chunk of this warp's 16 tokens
    // pass A
    for (int it = group; it < n_mine; it += kGroups) {
        const int slot = it % kLaStages;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.full[slot], static_cast<uint32_t>((it / kLaStages) & 1)));
        if (ok) {
            const uint32_t kb = smem_u32(ring_base + slot * kLaSlotBytes) + box * kLaBoxBytes;
            const uint32_t vb = kb + 2 * kLaBoxBytes;
            uint32_t af[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                const int row = mt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                ldsm_x4(vb + swz(row, chunk0 + (lane >> 4)), af[mt][0], af[mt][1], af[mt][2], af[mt][3]);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const int mi = lane >> 3;
                const int row = np * 16 + (mi >> 1) * 8 + (lane & 7);
                uint32_t b[4];
                ldsm_x4(kb + swz(row, chunk0 + (mi & 1)), b[0], b[1], b[2], b[3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) b[i] = relu2(b[i]);
                zacc[2 * np] += sum2(b[0]) + sum2(b[1]);
                zacc[2 * np + 1] += sum2(b[2]) + sum2(b[3]);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma_bf16(acc[mt][2 * np], af[mt][0], af[mt][1], af[mt][2], af[mt][3], b[0], b[1]);
                    mma_bf16(acc[mt][2 * np + 1], af[mt][0], af[mt][1], af[mt][2], af[mt][3], b[2], b[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[slot]);   // the operands are in registers
    }

    // reduce: warps -> CTA (shared memory) -> cluster (distributed shared memory)
    // accumulators are parked in fragment order (register slot x lane: every store
    // is 32 consecutive floats, no bank conflicts); the sum over the warps below
    // puts each element at its place in the matrix
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) sm.partial[warp][((mt * 4 + nt) * 4 + r) * 32 + lane] = acc[mt][nt][r];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        float z = zacc[nt];
        z += __shfl_xor_sync(0xffffffffu, z, 1);
        z += __shfl_xor_sync(0xffffffffu, z, 2);
        if (q4 == 0) sm.partial[warp][32 * 32 + nt * 8 + g] = z;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kLaWarps * 32) : "memory");
    for (int i = tid; i < kLaState; i += kLaWarps * 32) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kLaWarps; ++w) s += sm.partial[w][i];
        int at = i;                                   // the z row is stored in place
        if (i < 32 * 32) {
            const int slot = i >> 5, ln = i & 31;     // slot = (mt * 4 + nt) * 4 + r
            const int row = (slot >> 4) * 16 + (ln >> 2) + ((slot >> 1) & 1) * 8;
            const int col = ((slot >> 2) & 3) * 8 + (ln & 3) * 2 + (slot & 1);
            at = row * 32 + col;
        }
        if (cs == 1) {
            // no partner CTA: this is the final state (capture / inject seam applied here)
            const long long so = (static_cast<long long>(batch) * a.num_heads + head) * kLaState + at;
            if (a.sz_out != nullptr) a.sz_out[so] = s;
            if (a.sz_in != nullptr) s += a.w_in * a.sz_in[so];
            sm.state[(at >> 5) * kLaStLd + (at & 31)] = s;
        } else {
            sm.local_state[at] = s;
        }
    }
    phase_sync();
    if (cs > 1) {
        // every thread owns up to five state elements; all remote (distributed
        // shared memory) loads are issued before the first add so that their
        // latencies overlap
        constexpr int kPer = (kLaState + kLaWarps * 32 - 1) / (kLaWarps * 32);
        float part[kPer][8];
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const int i = tid + e * kLaWarps * 32;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                part[e][r] = 0.0f;
                if (r < cs && i < kLaState) {
                    const float* remote = cluster.map_shared_rank(sm.local_state, r);
                    part[e][r] = remote[i];
                }
            }
        }
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const int i = tid + e * kLaWarps * 32;
            if (i < kLaState) {
                float s = 0.0f;
#pragma unroll
                for (int r = 0; r < 8; ++r) s += part[e][r];      // rank order, as before
                const long long so = (static_cast<long long>(batch) * a.num_heads + head) * kLaState + i;
                if (a.sz_out != nullptr && rank == 0) a.sz_out[so] = s;
                if (a.sz_in != nullptr) s += a.w_in * a.sz_in[so];
                sm.state[(i >> 5) * kLaStLd + (i & 31)] = s;
            }
        }
    }
    phase_sync();

    // pass B: A fragments of [S; z] (48 x 32, rows 33.. zero) rounded to BF16.
    // The output is rounded to BF16 anyway (2^-9 relative per element); rounding
    // the 32 state terms of a dot product adds about 2^-9 / sqrt(32) to that, and
    // the reference's own batched path keeps S and z in BF16 (src/dit/sana.cpp:538-546).
    // A second MMA with the rounding residue doubled the work of this pass, which
    // is bound by the legacy tensor path (one m16n8k16 per 16 cycles and scheduler).
    uint32_t ah[3][2][4];
#pragma unroll
    for (int mt = 0; mt < 3; ++mt)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = mt * 16 + g + (r & 1) * 8;
                const int col = ks * 16 + q4 * 2 + (r >> 1) * 8;
                const float2 xx = *reinterpret_cast<const float2*>(&sm.state[row * kLaStLd + col]);
                const float x0 = xx.x, x1 = xx.y;
                ah[mt][ks][r] = pack2<true>(x0, x1);
            }

    // Warp w of an item's eight owns tokens [32 w, 32 w + 32) of the 256-token item (half of box w / 2)
    // and stages and stores that piece by itself (TMA store issued by its lane 0),
    // so no barrier of the CTA sits between items and the warps drift apart, which
    // hides the latency chain of a piece (tile load, MMAs, reciprocal, packing).
    // Two pieces per warp alternate: before a piece is overwritten, the store that
    // last read it has finished reading.  The pieces lie where the partial states
    // of the reduction were: every warp is past the barrier that followed it.
    // (an item belongs to group item mod kGroups in both passes: with a ring that is a
    // multiple of kGroups a group always meets the same slots and every phase of their barriers)
    int mine_b = 0;                                   // pass B items this group has taken
    for (int it = n_mine + (group + kGroups - n_mine % kGroups) % kGroups; it < n_items; it += kGroups, ++mine_b) {
        const int bi = it - n_mine;
        const int slot = it % kLaStages;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.full[slot], static_cast<uint32_t>((it / kLaStages) & 1)));
        if (2 * bi + (wg >> 2) < n_mine) {            // this warp's 128-token chunk exists
            uint8_t* stage = sm.out_stage[warp][mine_b & 1];
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            if (ok) {
                const uint32_t qb = smem_u32(ring_base + slot * kLaSlotBytes) + (wg >> 1) * kLaBoxBytes;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    uint32_t b[4];
                    ldsm_x4_trans(qb + swz(lane, (wg & 1) * 4 + nt), b[0], b[1], b[2], b[3]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) b[i] = relu2(b[i]);
                    float o[3][4];
#pragma unroll
                    for (int mt = 0; mt < 3; ++mt) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[mt][i] = 0.0f;
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {
                            mma_bf16(o[mt], ah[mt][ks][0], ah[mt][ks][1], ah[mt][ks][2], ah[mt][ks][3],
                                     b[2 * ks], b[2 * ks + 1]);
                        }
                    }
                    // Row 32 (z . relu(q)) sits in row 0 of the third tile: lanes 0..3.
                    const float den0 = __shfl_sync(0xffffffffu, o[2][0], q4);
                    const float den1 = __shfl_sync(0xffffffffu, o[2][1], q4);
                    const float r0 = 1.0f / (den0 + a.eps);
                    const float r1 = 1.0f / (den1 + a.eps);
                    // 64-byte rows under the 64-byte swizzle of the store's tensor map
                    // (16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3)): the
                    // eight rows and four words of one store fall into 32 different banks
                    uint8_t* sp = stage + q4 * 4;
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        const int i0 = mt * 16 + g;
                        *reinterpret_cast<uint32_t*>(sp + i0 * 64 + (((nt ^ (i0 >> 1)) & 3) << 4)) =
                            pack2<true>(o[mt][0] * r0, o[mt][1] * r1);
                        *reinterpret_cast<uint32_t*>(sp + (i0 + 8) * 64 + (((nt ^ ((i0 + 8) >> 1)) & 3) << 4)) =
                            pack2<true>(o[mt][2] * r0, o[mt][3] * r1);
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (ok && lane == 0) {
                const int tok = (c_begin + 2 * bi) * kLaChunk + wg * 32;
                if (tok < a.n_tokens) tma_store_3d(&tmO, stage, tok, row0, batch);
                tma_store_commit();
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[slot]);
    }
    if (lane == 0) tma_store_wait_all();    // shared memory stays valid until the last store has left
    phase_sync();
}

}  // namespace

cudaError_t launch_linear_attn(const LinearAttnArgs& a, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                               const CUtensorMap& tmV, const CUtensorMap& tmO, int cluster_size,
                               cudaStream_t stream) {
    const size_t smem = sizeof(LaSmem) + static_cast<size_t>(a.stages - 1) * kLaSlotBytes + 1024;
    // the largest ring is set once per device; every launch fits under it
    constexpr int kMaxSmem = static_cast<int>(sizeof(LaSmem) + (kLaMaxStages - 1) * kLaSlotBytes + 1024);
    static_assert(kLaMaxStages % kLaGroups == 0, "every warp group must own a fixed set of ring slots");
    if (a.stages < kLaGroups || a.stages % kLaGroups != 0 || static_cast<int>(smem) > kMaxSmem)
        return cudaErrorInvalidValue;
    cudaError_t e = set_max_smem_once(linear_attn_kernel, kMaxSmem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(cluster_size), static_cast<unsigned>(a.num_heads),
                       static_cast<unsigned>(a.batch));
    cfg.blockDim = dim3(kLaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster_size);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    // set-up of this launch may overlap the tail of the kernel before it (see the kernel's first lines)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, linear_attn_kernel, tmQ, tmK, tmV, tmO, a);
}

}  // namespace bdattn
