// Axial RoPE cos/sin tables built on the device.
//
// The reference builds these on the host every forward and uploads them
// (src/dit/flux.cpp:760 -> src/dit/common.cpp:116-184;
// src/dit/qwenimage21_forward.cpp:301-302 -> 124-200).  Here one thread
// computes one (token, pair) cell with the same double-precision formula, so
// the tables never cross PCIe.  Tables are FP32 (rows, head_dim / 2).
#include "sdpa_internal.h"
#include "tc05.cuh"

namespace bdattn {
namespace {

__global__ void rope_tables_kernel(const RopeTableArgs a) {
    const int half = a.half;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(a.rows) * half) return;
    const int row = static_cast<int>(idx / half);
    const int p = static_cast<int>(idx - static_cast<long long>(row) * half);
    // axis that owns pair p, and the pair's index inside the axis
    int axis = 0, pl = p;
    while (axis < a.n_axes - 1 && pl >= a.axes[axis] / 2) {
        pl -= a.axes[axis] / 2;
        ++axis;
    }
    // segment of the row
    int s = 0;
    while (s < a.n_seg - 1 && row >= a.seg_row0[s + 1]) ++s;
    const int t = row - a.seg_row0[s];
    int pos;
    if (a.seg_kind[s] == 0) {                 // text
        pos = a.flux ? 0 : a.seg_pos0[s] + t;
    } else {                                  // image grid
        const int w = a.seg_w[s];
        const int i = t / w, j = t - i * w;
        if (a.flux) {
            pos = axis == 0 ? 0 : (axis == 1 ? i : j);
        } else {
            const int h = a.seg_h[s];
            pos = axis == 0 ? a.seg_pos0[s] : (axis == 1 ? i - (h - h / 2) : j - (w - w / 2));
        }
    }
    double c = 1.0, sn = 0.0;
    if (a.flux) {
        if (a.seg_kind[s] != 0 && axis < 3) {
            const double omega = 1.0 / pow(static_cast<double>(a.theta),
                                           (2.0 * pl) / static_cast<double>(a.axes[axis]));
            const double ang = static_cast<double>(pos) * omega;
            c = cos(ang);
            sn = sin(ang);
        }
    } else {
        const double freq = pow(static_cast<double>(a.theta),
                                -2.0 * static_cast<double>(pl) / static_cast<double>(a.axes[axis]));
        const double ang = static_cast<double>(pos) * freq;
        c = cos(ang);
        sn = sin(ang);
    }
    a.cos_out[idx] = static_cast<float>(c);
    a.sin_out[idx] = static_cast<float>(sn);
}

}  // namespace

cudaError_t launch_rope_tables(const RopeTableArgs& a, cudaStream_t stream) {
    const long long n = static_cast<long long>(a.rows) * a.half;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    rope_tables_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace bdattn
