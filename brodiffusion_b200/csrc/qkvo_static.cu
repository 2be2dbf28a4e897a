// bdattn_qkvo_fwd_static: the SD1.5 attention block for callers that cannot
// give the library any scratch memory of their own.
//
// bdattn_qkvo_fwd needs device scratch for the projected Q, K, V and the
// attention output, and takes it from the caller.  Some callers have nothing
// to give: a plugin loaded into a host application that has already handed all
// device memory to its own pool and forbids cudaMalloc from plugins, or a
// latency-critical loop in which cudaMalloc/cudaFree are banned because they
// synchronise the whole device.  For them this entry point runs the same
// kernels with the scratch placed in a fixed array that is part of the
// library's device image.
//
// The array, the lookup of its device address and the entry point live in this
// one file on purpose: in host code the array's name is only a handle for the
// runtime, not a device address, so the address is asked for with
// cudaGetSymbolAddress (once per device, with that device current) and that
// pointer is what the kernels receive.
#include <mutex>

namespace {

// Scratch capacity: 16 MiB, enough for every SD1.5 attention call at 512 px
// (the largest, 4096 tokens x 8 heads of 40, needs 14.5 MiB).  Each GPU that
// loads the library keeps this much memory reserved until the process exits.
constexpr size_t kQkvoStaticBytes = static_cast<size_t>(16) << 20;

static __device__ __align__(256) unsigned char g_qkvo_static_scratch[kQkvoStaticBytes];

constexpr int kQkvoMaxDevices = 64;
void* g_qkvo_static_ptr[kQkvoMaxDevices] = {};
std::mutex g_qkvo_static_mu;

// Device address of the scratch array on the current device.  The first call
// on a device resolves it (cudaGetSymbolAddress); later calls read the cache.
int qkvo_static_scratch(const char* op, void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(op, e);
    if (dev < 0 || dev >= kQkvoMaxDevices) return fail("%s: device index %d out of range", op, dev);
    std::lock_guard<std::mutex> lock(g_qkvo_static_mu);
    if (g_qkvo_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_qkvo_static_scratch);
        if (e != cudaSuccess) return cuda_fail(op, e);
        if (p == nullptr) return fail("%s: the runtime returned a null address for the scratch array", op);
        g_qkvo_static_ptr[dev] = p;
    }
    *out = g_qkvo_static_ptr[dev];
    return 0;
}

}  // namespace

extern "C" {

size_t bdattn_qkvo_static_capacity(void) { return kQkvoStaticBytes; }

int bdattn_qkvo_fwd_static(const bdattn_qkvo_params* p, bdattn_stream_t stream) {
    const char* op = "bdattn_qkvo_fwd_static";
    if (p == nullptr) return fail("%s: params is null", op);
    if (require_sm100(op)) return -1;
    if (p->num_heads < 1 || p->inner_dim < 1 || p->inner_dim % p->num_heads != 0)
        return fail("%s: inner_dim must be a positive multiple of num_heads", op);
    const bool cached = p->k_cached != nullptr || p->v_cached != nullptr;
    const int kv_rows = cached ? p->kv_rows : (p->ctx != nullptr ? p->ctx_rows : p->x_rows);
    const size_t need = bdattn_qkvo_workspace_bytes(p->x_rows, kv_rows, p->num_heads,
                                                    p->inner_dim / p->num_heads);
    if (need > kQkvoStaticBytes)
        return fail("%s: this call needs %zu bytes of scratch but the built-in array holds %zu; use "
                    "bdattn_qkvo_fwd with caller-provided scratch for shapes this large",
                    op, need, kQkvoStaticBytes);
    void* scratch = nullptr;
    if (qkvo_static_scratch(op, &scratch)) return -1;
    bdattn_qkvo_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = kQkvoStaticBytes;
    return bdattn_qkvo_fwd(&q, stream);
}

}  // extern "C"
