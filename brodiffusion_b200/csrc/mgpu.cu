// Multi-GPU set-up for a single-process caller that drives one GPU per host
// thread: peer access between the GPUs, head-sharded attention that stores into
// every GPU's copy of the output, and a cross-GPU barrier on the stream.
//
// The barrier is a one-CTA kernel per GPU.  Rank r adds nothing to shared state
// on the host: it writes its epoch number into slot [r] of every peer's arrival
// array (a plain store through the peer mapping, after a system-wide fence) and
// then polls its own array until every slot has reached the epoch.  The poll is
// bounded by wall time; when it runs out the kernel sets the wait-timeout bit of
// its GPU's status word and returns, so the context stays usable and the host
// learns of the missing rank from bdattn_device_status.  No multimem, no NVLS,
// no TMA: plain loads of local memory and plain stores to peer memory.
#include "../../include/bdattn.h"

#include <cstdio>
#include <mutex>
#include <new>

#include "sdpa_internal.h"
#include "tc05.cuh"

struct bdattn_mgpu {
    int n = 0;
    int device[BDATTN_MGPU_MAX] = {};
    unsigned long long* arrive[BDATTN_MGPU_MAX] = {};   // on device[g]: n slots, slot r written by rank r
    unsigned long long epoch[BDATTN_MGPU_MAX] = {};      // barriers enqueued so far by rank g (host side)
};

namespace bdattn {
namespace {

struct BarrierArgs {
    unsigned long long* peer_slot[BDATTN_MGPU_MAX];   // slot [rank] inside every GPU's arrival array
    const unsigned long long* mine;                   // this GPU's arrival array
    int n;
    unsigned long long epoch;
    unsigned long long timeout_ns;
};

__global__ void __launch_bounds__(32) mgpu_barrier_kernel(const BarrierArgs a) {
    const int t = threadIdx.x;
    if (t < a.n) {
        // everything this GPU wrote before the barrier (peer stores of the attention
        // epilogue included) is performed before the arrival becomes visible
        __threadfence_system();
        *reinterpret_cast<volatile unsigned long long*>(a.peer_slot[t]) = a.epoch;
        const volatile unsigned long long* slot = a.mine + t;
        const uint64_t t0 = global_timer_ns();
        bool seen = *slot >= a.epoch;
        while (!seen) {
#pragma unroll 1
            for (int i = 0; i < 64 && !seen; ++i) seen = *slot >= a.epoch;
            if (!seen && global_timer_ns() - t0 > a.timeout_ns) {
                atomicOr(&g_device_status, kStatusWaitTimeout);
                break;
            }
        }
        __threadfence_system();
    }
}

}  // namespace
}  // namespace bdattn

// This file is compiled in the same translation unit as capi.cu and after it:
// fail() (per-thread error message) and sdpa_fwd_impl() are the ones defined there.

extern "C" {

int bdattn_mgpu_init(bdattn_mgpu** out, const int* devices, int n_gpus) {
    const char* op = "bdattn_mgpu_init";
    if (out == nullptr || devices == nullptr) return fail("%s: null argument", op);
    if (n_gpus < 1 || n_gpus > BDATTN_MGPU_MAX) return fail("%s: n_gpus must be in [1, %d]", op, BDATTN_MGPU_MAX);
    int prev = 0;
    cudaGetDevice(&prev);
    bdattn_mgpu* c = new (std::nothrow) bdattn_mgpu();
    if (c == nullptr) return fail("%s: out of host memory", op);
    c->n = n_gpus;
    int rc = 0;
    for (int g = 0; g < n_gpus && rc == 0; ++g) {
        c->device[g] = devices[g];
        for (int h = 0; h < g; ++h)
            if (devices[h] == devices[g]) rc = fail("%s: device %d is listed twice", op, devices[g]);
    }
    for (int g = 0; g < n_gpus && rc == 0; ++g) {
        cudaError_t e = cudaSetDevice(devices[g]);
        if (e != cudaSuccess) { rc = fail("%s: cudaSetDevice(%d) failed", op, devices[g]); break; }
        for (int h = 0; h < n_gpus; ++h) {
            if (h == g) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, devices[g], devices[h]);
            if (!can) { rc = fail("%s: device %d cannot access device %d as a peer", op, devices[g], devices[h]); break; }
            e = cudaDeviceEnablePeerAccess(devices[h], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
            if (e != cudaSuccess) { rc = fail("%s: enabling peer access %d -> %d failed", op, devices[g], devices[h]); break; }
        }
        if (rc != 0) break;
        e = cudaMalloc(&c->arrive[g], sizeof(unsigned long long) * BDATTN_MGPU_MAX);
        if (e == cudaSuccess) e = cudaMemset(c->arrive[g], 0, sizeof(unsigned long long) * BDATTN_MGPU_MAX);
        if (e != cudaSuccess) rc = fail("%s: allocating the arrival array on device %d failed", op, devices[g]);
    }
    for (int g = 0; g < n_gpus && rc == 0; ++g) {      // the zeroed arrays are in place before anyone signals
        cudaSetDevice(devices[g]);
        if (cudaDeviceSynchronize() != cudaSuccess) rc = fail("%s: device %d failed to synchronise", op, devices[g]);
    }
    cudaSetDevice(prev);
    if (rc != 0) {
        bdattn_mgpu_destroy(c);
        return -1;
    }
    *out = c;
    return 0;
}

int bdattn_mgpu_destroy(bdattn_mgpu* c) {
    if (c == nullptr) return 0;
    int prev = 0;
    cudaGetDevice(&prev);
    for (int g = 0; g < c->n; ++g) {
        if (c->arrive[g] != nullptr) {
            cudaSetDevice(c->device[g]);
            cudaDeviceSynchronize();
            cudaFree(c->arrive[g]);
        }
    }
    cudaSetDevice(prev);
    delete c;
    return 0;
}

int bdattn_mgpu_size(const bdattn_mgpu* c) { return c != nullptr ? c->n : 0; }

int bdattn_mgpu_barrier(bdattn_mgpu* c, int rank, int timeout_ms, bdattn_stream_t stream) {
    const char* op = "bdattn_mgpu_barrier";
    if (c == nullptr) return fail("%s: context is null", op);
    if (rank < 0 || rank >= c->n) return fail("%s: rank %d is not in [0, %d)", op, rank, c->n);
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != c->device[rank]) return fail("%s: rank %d must be called with device %d current", op, rank, c->device[rank]);
    bdattn::BarrierArgs a = {};
    for (int g = 0; g < c->n; ++g) a.peer_slot[g] = c->arrive[g] + rank;
    a.mine = c->arrive[rank];
    a.n = c->n;
    a.epoch = ++c->epoch[rank];     // each rank's thread owns its own counter
    a.timeout_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
    bdattn::mgpu_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", op, cudaGetErrorString(e));
    return 0;
}

int bdattn_mgpu_sdpa_fwd_headsharded(bdattn_mgpu* c, int rank, const bdattn_sdpa_params* p, void* const* replicas,
                                     long long replica_ld, long long replica_batch_stride, int total_heads,
                                     bdattn_stream_t stream) {
    const char* op = "bdattn_mgpu_sdpa_fwd_headsharded";
    if (c == nullptr || p == nullptr || replicas == nullptr) return fail("%s: null argument", op);
    if (rank < 0 || rank >= c->n) return fail("%s: rank %d is not in [0, %d)", op, rank, c->n);
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != c->device[rank]) return fail("%s: rank %d must be called with device %d current", op, rank, c->device[rank]);
    if (total_heads < 1 || total_heads % c->n != 0 || p->num_heads != total_heads / c->n)
        return fail("%s: params must describe this rank's share of the heads (%d of %d)", op,
                    total_heads / (c->n > 0 ? c->n : 1), total_heads);
    if (replica_ld < static_cast<long long>(total_heads) * p->head_dim)
        return fail("%s: replica_ld is smaller than total_heads * head_dim", op);
    const size_t es = 2;
    const long long col0 = static_cast<long long>(rank) * p->num_heads * p->head_dim;
    bdattn_sdpa_params q = *p;
    void* peers[2][BDATTN_MGPU_MAX] = {};
    long long row0 = 0;
    for (int s = 0; s < p->n_q_seg && s < 2; ++s) {
        int np = 0;
        for (int g = 0; g < c->n; ++g) {
            if (replicas[g] == nullptr) return fail("%s: replica %d is null", op, g);
            char* base = static_cast<char*>(replicas[g]) + (row0 * replica_ld + col0) * es;
            if (g == rank) q.o[s] = base;
            else peers[s][np++] = base;
        }
        q.o_ld[s] = replica_ld;
        q.o_batch_stride[s] = replica_batch_stride;
        row0 += p->q_rows[s];
    }
    return sdpa_fwd_impl(op, &q, peers[0], peers[1], c->n - 1, nullptr, stream);
}

}  // extern "C"
