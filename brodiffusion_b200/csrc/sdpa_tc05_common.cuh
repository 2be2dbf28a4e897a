// Pieces shared by the two softmax-attention kernels for the sm_100a tensor cores
// (sdpa_tc05.cu: one work item per CTA; sdpa_tc05_persist.cu: persistent grid with
// the peer push of the fused all-gather): tile geometry, the walk over the one or
// two key segments, packed FP32 arithmetic, register re-allocation.
#pragma once

#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace sdpa_tc {

constexpr int kBM = 128;           // query rows per tile
constexpr int kBN = 128;           // keys per tile
constexpr int kThreads = 384;
constexpr int kChunkBytes = 128 * 128;  // one 64-column (128 B) x 128-row TMA box
constexpr int kRegsSoftmax = 216;
constexpr int kRegsOther = 64;

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

}  // namespace sdpa_tc
}  // namespace bdattn
