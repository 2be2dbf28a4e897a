// C-ABI layer: argument validation, tensor-map construction and kernel
// dispatch.  No device memory is allocated here; every kernel runs on the
// stream the caller passes.
#include "../../include/bdattn.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "sdpa_internal.h"
#include "tc05.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return -1;
}

int cuda_fail(const char* op, cudaError_t e) {
    return fail("%s: CUDA error: %s", op, cudaGetErrorString(e));
}

// The current device must be a Blackwell data-centre part (sm_100): the
// kernels are sm_100a-only and there is no other path.
int require_sm100(const char* op) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(op, e);
    static thread_local int checked_dev = -1;
    if (checked_dev == dev) return 0;
    int major = 0, minor = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(op, e);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (major != 10) {
        return fail("%s: device %d is sm_%d%d; this library only runs on sm_100 (B200) and has no "
                    "other path", op, dev, major, minor);
    }
    checked_dev = dev;
    return 0;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// (cols, rows, batch) row-major 16-bit tensor, box = box_cols columns x box_rows rows,
// 128-byte swizzle (or 64-byte, or none when swizzle_bytes is 0), zero fill outside the tensor.
int make_map_3d(const char* op, CUtensorMap* m, const void* base, bool bf16, long long cols,
                long long rows, long long batch, long long ld, long long batch_stride,
                int box_rows, int box_cols = 64, int swizzle_bytes = 128) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail("%s: cuTensorMapEncodeTiled is not available from the driver", op);
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(batch)};
    if (batch_stride <= 0) batch_stride = rows * ld;
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                         : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail("%s: cuTensorMapEncodeTiled failed (CUresult %d) for base=%p cols=%lld rows=%lld "
                    "batch=%lld ld=%lld batch_stride=%lld", op, static_cast<int>(r), base, cols, rows,
                    batch, ld, batch_stride);
    }
    return 0;
}

// Attention operand: (head_dim, heads, rows, batch) view of a row-major
// (rows, heads * head_dim) 16-bit tensor; box = 64 head elements x 1 head x
// box_rows rows, 128-byte swizzle.  Head elements beyond head_dim read as zero.
int make_map_heads(const char* op, CUtensorMap* m, const void* base, bool bf16, int head_dim,
                   int num_heads, long long rows, long long batch, long long ld,
                   long long batch_stride, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail("%s: cuTensorMapEncodeTiled is not available from the driver", op);
    if (batch_stride <= 0) batch_stride = rows * ld;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(num_heads),
                          static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(ld) * 2,
                             static_cast<cuuint64_t>(batch_stride) * 2};
    cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail("%s: cuTensorMapEncodeTiled failed (CUresult %d) for base=%p head_dim=%d heads=%d "
                    "rows=%lld batch=%lld ld=%lld", op, static_cast<int>(r), base, head_dim, num_heads,
                    rows, batch, ld);
    return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// (cols, rows) row-major 16-bit matrix, box = 64 columns x box_rows rows,
// 128-byte swizzle, zero fill outside.
int make_map_2d(const char* op, CUtensorMap* m, const void* base, bool bf16, long long cols,
                long long rows, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail("%s: cuTensorMapEncodeTiled is not available from the driver", op);
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail("%s: cuTensorMapEncodeTiled failed (CUresult %d) for base=%p cols=%lld rows=%lld ld=%lld",
                    op, static_cast<int>(r), base, cols, rows, ld);
    return 0;
}

int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Width each head is padded to for the tensor-core attention kernel (0: the
// general kernel is used and heads stay unpadded).
int padded_head_dim(int hd) {
    if (hd % 8 != 0) return 0;
    if (hd <= 64) return 64;
    if (hd <= 128) return 128;
    return 0;
}

// One GEMM problem  C[M, N] = A[M, K] . W[N, K]^T (+ bias).  head_dim > 0 cuts
// the N dimension into per-head tiles whose results land head_pad columns
// apart (zero filled); head_dim == 0 uses plain 64-column tiles.
int add_gemm_problem(const char* op, bdattn::GemmLaunch& L, int idx, const void* A, long long lda,
                     const void* W, long long ldw, const void* bias, void* Cout, long long ldc, int M,
                     int N, int K, int head_dim, int head_pad, int geglu_offset) {
    if (A == nullptr || W == nullptr || Cout == nullptr) return fail("%s: null matrix pointer", op);
    if (M < 1 || N < 1 || K < 1) return fail("%s: empty matrix (M=%d N=%d K=%d)", op, M, N, K);
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ldc % 8 != 0 || lda < K || ldw < K)
        return fail("%s: inner size and row strides must be multiples of 8 elements (K=%d lda=%lld ldw=%lld "
                    "ldc=%lld)", op, K, lda, ldw, ldc);
    if (!aligned16(A) || !aligned16(W) || !aligned16(Cout)) return fail("%s: matrices must be 16-byte aligned", op);
    {
        // columns one output row receives: N, or head_pad per head for head tiles
        const long long written = head_dim > 0 ? static_cast<long long>(N / head_dim) * head_pad : N;
        if (ldc < written)
            return fail("%s: output row stride %lld is smaller than the %lld columns written per row", op, ldc, written);
    }
    bdattn::GemmProblem& p = L.args.p[idx];
    p.M = M; p.N = N; p.K = K; p.C = Cout; p.ldc = ldc; p.bias = bias;
    p.tiles_m = (M + 127) / 128;
    p.geglu_offset = geglu_offset;
    if (head_dim > 0) {
        if (N % head_dim != 0) return fail("%s: output width %d is not a multiple of head_dim %d", op, N, head_dim);
        p.n_tile = round_up(head_dim, 16);
        p.n_step = head_dim;
        p.n_valid = head_dim;
        p.c_step = head_pad;
        p.c_fill = head_pad;
        p.tiles_n = N / head_dim;
    } else {
        if (N % 8 != 0) return fail("%s: output width must be a multiple of 8 (got %d)", op, N);
        // 128-column tiles once the output is wide enough to fill the SMs with them
        const int tile = (geglu_offset == 0 && static_cast<long long>((M + 127) / 128) * ((N + 127) / 128) >= 148) ? 128 : 64;
        p.n_tile = tile;
        p.n_step = tile;
        p.n_valid = tile;
        p.c_step = tile;
        p.c_fill = tile;      // the epilogue stops at the matrix edge on a ragged last tile
        p.tiles_n = (N + tile - 1) / tile;
    }
    if (make_map_2d(op, &L.tmA[idx], A, L.bf16, K, M, lda, 128)) return -1;
    // the weight matrix has N (+ D_out for GEGLU) rows
    const long long w_rows = geglu_offset > 0 ? static_cast<long long>(N) + geglu_offset : N;
    if (make_map_2d(op, &L.tmB[idx], W, L.bf16, K, w_rows, ldw, p.n_tile)) return -1;
    // 128 x 256 tiles need whole tiles along N and, for head tiles, unpadded heads of 64 or 128
    // (GEGLU: a tile is 128 value columns + their 128 gate columns, two 128-row boxes)
    L.wide[idx] = geglu_offset > 0
                      ? N % 128 == 0
                      : N % 256 == 0 && (head_dim == 0 || (head_dim == head_pad && (head_dim == 64 || head_dim == 128)));
    if (L.wide[idx] && make_map_2d(op, &L.tmBw[idx], W, L.bf16, K, w_rows, ldw, geglu_offset > 0 ? 128 : 256)) return -1;
    return 0;
}

void finish_gemm_launch(bdattn::GemmLaunch& L, int n) {
    L.n_problems = n;
    for (int i = n; i < 3; ++i) {
        L.args.p[i] = L.args.p[0];
        L.args.p[i].tiles_m = 0;
        L.args.p[i].tiles_n = 0;
        L.tmA[i] = L.tmA[0];
        L.tmB[i] = L.tmB[0];
        L.tmBw[i] = L.tmBw[0];
        L.wide[i] = L.wide[0];
    }
}

}  // namespace

extern "C" {

int bdattn_version(void) { return 100; }

const char* bdattn_last_error(void) { return g_err; }

int bdattn_device_status(int* status, int clear) {
    if (status == nullptr) return fail("bdattn_device_status: status is null");
    if (require_sm100("bdattn_device_status")) return -1;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail("bdattn_device_status", e);
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, bdattn::g_device_status, sizeof(int));
    if (e != cudaSuccess) return cuda_fail("bdattn_device_status", e);
    *status = v;
    if (clear && v != 0) {
        int z = 0;
        e = cudaMemcpyToSymbol(bdattn::g_device_status, &z, sizeof(int));
        if (e != cudaSuccess) return cuda_fail("bdattn_device_status", e);
    }
    return 0;
}

static int sdpa_fwd_impl(const char* op, const bdattn_sdpa_params* p, void* const* peer_o0,
                         void* const* peer_o1, int n_peers, const bdattn_trace_params* tr,
                         bdattn_stream_t stream, void* const* mc_o = nullptr) {
    if (p == nullptr) return fail("%s: params is null", op);
    if (n_peers < 0 || n_peers > 8) return fail("%s: n_peers must be in [0, 8]", op);
    if (require_sm100(op)) return -1;
    if (p->dtype != BDATTN_BF16 && p->dtype != BDATTN_F16)
        return fail("%s: dtype must be BF16 or F16 (got %d)", op, p->dtype);
    if (p->batch < 1 || p->num_heads < 1) return fail("%s: batch and num_heads must be >= 1", op);
    const int hd = p->head_dim;
    if (hd < 8 || hd > 256 || hd % 8 != 0)
        return fail("%s: head_dim must be a multiple of 8 in [8, 256] (got %d)", op, hd);
    if (p->n_q_seg < 1 || p->n_q_seg > 2 || p->n_kv_seg < 1 || p->n_kv_seg > 2)
        return fail("%s: n_q_seg and n_kv_seg must be 1 or 2", op);
    if (p->mask_mode != BDATTN_MASK_NONE && p->mask_mode != BDATTN_MASK_CAUSAL)
        return fail("%s: unknown mask_mode %d", op, p->mask_mode);
    const long long D = static_cast<long long>(p->num_heads) * hd;
    const int nkv = p->num_kv_heads > 0 ? p->num_kv_heads : p->num_heads;
    if (p->num_kv_heads < 0 || p->num_heads % nkv != 0)
        return fail("%s: num_kv_heads must divide num_heads (got %d and %d)", op, p->num_kv_heads, p->num_heads);
    const long long Dkv = static_cast<long long>(nkv) * hd;
    long long Lq = 0, Lk = 0;
    for (int s = 0; s < p->n_q_seg; ++s) {
        if (p->q[s] == nullptr || p->o[s] == nullptr) return fail("%s: q/o segment %d is null", op, s);
        if (p->q_rows[s] < 1) return fail("%s: q_rows[%d] must be >= 1", op, s);
        if (p->q_ld[s] < D || p->o_ld[s] < D)
            return fail("%s: q_ld/o_ld of segment %d smaller than num_heads*head_dim", op, s);
        if (p->q_ld[s] % 8 || p->o_ld[s] % 8 || !aligned16(p->q[s]) || !aligned16(p->o[s]) ||
            p->q_batch_stride[s] % 8 || p->o_batch_stride[s] % 8)
            return fail("%s: q/o segment %d must be 16-byte aligned with strides that are multiples of 8 "
                        "elements", op, s);
        Lq += p->q_rows[s];
    }
    for (int s = 0; s < p->n_kv_seg; ++s) {
        if (p->k[s] == nullptr || p->v[s] == nullptr) return fail("%s: k/v segment %d is null", op, s);
        if (p->kv_rows[s] < 1) return fail("%s: kv_rows[%d] must be >= 1", op, s);
        if (p->k_ld[s] < Dkv || p->v_ld[s] < Dkv)
            return fail("%s: k_ld/v_ld of segment %d smaller than num_kv_heads*head_dim", op, s);
        if (p->k_ld[s] % 8 || p->v_ld[s] % 8 || !aligned16(p->k[s]) || !aligned16(p->v[s]) ||
            p->k_batch_stride[s] % 8 || p->v_batch_stride[s] % 8)
            return fail("%s: k/v segment %d must be 16-byte aligned with strides that are multiples of 8 "
                        "elements", op, s);
        Lk += p->kv_rows[s];
    }
    const float scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(hd));
    const bool bf16 = p->dtype == BDATTN_BF16;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool q_fused = p->q_gain[0] != nullptr || p->q_gain[1] != nullptr || p->q_cos != nullptr ||
                         p->q_sin != nullptr;
    if (q_fused) {
        if ((p->q_cos == nullptr) != (p->q_sin == nullptr)) return fail("%s: q_cos and q_sin must both be given", op);
        if (!aligned16(p->q_cos) || !aligned16(p->q_sin)) return fail("%s: q_cos and q_sin must be 16-byte aligned", op);
        if ((p->q_gain[0] != nullptr || p->q_gain[1] != nullptr) && p->q_gain_dtype != BDATTN_F32 &&
            p->q_gain_dtype != p->dtype)
            return fail("%s: q_gain_dtype must be F32 or the tensor dtype", op);
        if (!aligned16(p->q_gain[0]) || !aligned16(p->q_gain[1])) return fail("%s: q_gain must be 16-byte aligned", op);
        if (p->q_rope_row0 < 0) return fail("%s: q_rope_row0 must be >= 0", op);
        if (hd > 128) return fail("%s: the fused query RMSNorm/RoPE needs head_dim <= 128", op);
    }

    if (hd <= 128) {
        // tensor-core path: the kernel computes with 64 or 128 columns per head and
        // the TMA unit zero-pads narrower heads
        const int hd_kernel = hd <= 64 ? 64 : 128;
        bdattn::SdpaLaunch L;
        std::memset(&L, 0, sizeof(L));
        for (int s = 0; s < 2; ++s) {
            const int qs = s < p->n_q_seg ? s : 0;
            const int ks = s < p->n_kv_seg ? s : 0;
            if (make_map_heads(op, &L.tmQ[s], p->q[qs], bf16, hd, p->num_heads, p->q_rows[qs], p->batch,
                               p->q_ld[qs], p->q_batch_stride[qs], 128))
                return -1;
            if (make_map_heads(op, &L.tmK[s], p->k[ks], bf16, hd, nkv, p->kv_rows[ks], p->batch,
                               p->k_ld[ks], p->k_batch_stride[ks], 128))
                return -1;
            if (make_map_heads(op, &L.tmV[s], p->v[ks], bf16, hd, nkv, p->kv_rows[ks], p->batch,
                               p->v_ld[ks], p->v_batch_stride[ks], 128))
                return -1;
        }
        bdattn::SdpaDevArgs& a = L.args;
        for (int s = 0; s < 2; ++s) {
            const bool have_q = s < p->n_q_seg;
            const bool have_k = s < p->n_kv_seg;
            a.q_rows[s] = have_q ? p->q_rows[s] : 0;
            a.o[s] = have_q ? p->o[s] : nullptr;
            a.o_ld[s] = have_q ? p->o_ld[s] : 0;
            a.o_bs[s] = have_q ? p->o_batch_stride[s] : 0;
            a.kv_rows[s] = have_k ? p->kv_rows[s] : 0;
        }
        a.q_ctas0 = (a.q_rows[0] + 255) / 256;
        const int q_ctas1 = (a.q_rows[1] + 255) / 256;
        a.kv_tiles0 = (a.kv_rows[0] + 127) / 128;
        a.kv_tiles = a.kv_tiles0 + (a.kv_rows[1] + 127) / 128;
        a.mask_mode = p->mask_mode;
        a.q_offset = static_cast<int>(Lk - Lq);
        a.hd_out = hd;
        a.kv_group = p->num_heads / nkv;
        a.q_fused = q_fused ? 1 : 0;
        a.q_gain[0] = p->q_gain[0];
        a.q_gain[1] = p->n_q_seg > 1 ? p->q_gain[1] : p->q_gain[0];
        a.q_gain_is_f32 = p->q_gain_dtype == BDATTN_F32 ? 1 : 0;
        a.q_eps = p->q_eps;
        a.q_cos = p->q_cos; a.q_sin = p->q_sin; a.q_rope_row0 = p->q_rope_row0;
        a.key_mask = p->key_mask;
        a.key_scale = p->key_scale;
        a.val_scale = p->val_scale;
        a.scale_log2 = scale * 1.4426950408889634f;
        if (tr != nullptr) {
            a.bias = tr->bias;
            a.bias_row0 = tr->bias_row0; a.bias_rows = tr->bias_rows; a.bias_cols = tr->bias_cols;
            a.bias_ld = tr->bias_ld > 0 ? tr->bias_ld : tr->bias_cols;
            a.bias_mul = 1.0f / scale;
            a.lse = static_cast<float*>(tr->workspace);
            a.lq_total = static_cast<int>(Lq);
        }
        a.n_peers = n_peers;
        for (int i = 0; i < n_peers; ++i) {
            if (peer_o0 == nullptr || peer_o0[i] == nullptr || !aligned16(peer_o0[i]))
                return fail("%s: peer output %d of segment 0 is null or not 16-byte aligned", op, i);
            a.o_peer[0][i] = peer_o0[i];
            if (p->n_q_seg > 1) {
                if (peer_o1 == nullptr || peer_o1[i] == nullptr || !aligned16(peer_o1[i]))
                    return fail("%s: peer output %d of segment 1 is null or not 16-byte aligned", op, i);
                a.o_peer[1][i] = peer_o1[i];
            }
        }
        if (mc_o != nullptr) {
            for (int s = 0; s < p->n_q_seg; ++s) {
                if (mc_o[s] == nullptr || !aligned16(mc_o[s]))
                    return fail("%s: multicast output of segment %d is null or not 16-byte aligned", op, s);
                a.o_mc[s] = mc_o[s];
            }
        }
        L.q_ctas = a.q_ctas0 + q_ctas1;
        L.num_heads = p->num_heads;
        L.batch = p->batch;
        L.head_dim = hd_kernel;
        L.bf16 = bf16;
        if (L.num_heads > 65535 || L.batch > 65535) return fail("%s: num_heads/batch too large", op);
        cudaError_t e = bdattn::launch_sdpa_tc05(L, st);
        if (e != cudaSuccess) return cuda_fail(op, e);
        return 0;
    }

    if (n_peers > 0 || mc_o != nullptr) return fail("%s: the fused all-gather needs head_dim <= 128", op);
    if (tr != nullptr) return fail("%s: traced attention needs head_dim <= 128", op);
    bdattn::SdpaGeneralArgs g;
    std::memset(&g, 0, sizeof(g));
    for (int s = 0; s < 2; ++s) {
        if (s < p->n_q_seg) {
            g.q[s] = p->q[s]; g.o[s] = p->o[s]; g.q_rows[s] = p->q_rows[s];
            g.q_ld[s] = p->q_ld[s]; g.o_ld[s] = p->o_ld[s];
            g.q_bs[s] = p->q_batch_stride[s]; g.o_bs[s] = p->o_batch_stride[s];
        }
        if (s < p->n_kv_seg) {
            g.k[s] = p->k[s]; g.v[s] = p->v[s]; g.kv_rows[s] = p->kv_rows[s];
            g.k_ld[s] = p->k_ld[s]; g.v_ld[s] = p->v_ld[s];
            g.k_bs[s] = p->k_batch_stride[s]; g.v_bs[s] = p->v_batch_stride[s];
        }
    }
    g.mask_mode = p->mask_mode;
    g.q_offset = static_cast<int>(Lk - Lq);
    g.head_dim = hd;
    g.kv_group = p->num_heads / nkv;
    g.key_mask = p->key_mask;
    g.key_scale = p->key_scale;
    g.val_scale = p->val_scale;
    g.scale = scale;
    cudaError_t e = bdattn::launch_sdpa_general(g, p->num_heads, p->batch, bf16, st);
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_sdpa_fwd(const bdattn_sdpa_params* p, bdattn_stream_t stream) {
    return sdpa_fwd_impl("bdattn_sdpa_fwd", p, nullptr, nullptr, 0, nullptr, stream);
}

int bdattn_sdpa_fwd_allgather(const bdattn_sdpa_params* p, void* const* peer_o0, void* const* peer_o1,
                              int n_peers, bdattn_stream_t stream) {
    return sdpa_fwd_impl("bdattn_sdpa_fwd_allgather", p, peer_o0, peer_o1, n_peers, nullptr, stream);
}

int bdattn_sdpa_fwd_allgather_multicast(const bdattn_sdpa_params* p, void* mc_o0, void* mc_o1,
                                        bdattn_stream_t stream) {
    void* mc[2] = {mc_o0, mc_o1};
    return sdpa_fwd_impl("bdattn_sdpa_fwd_allgather_multicast", p, nullptr, nullptr, 0, nullptr, stream, mc);
}

size_t bdattn_sdpa_traced_workspace_bytes(int num_heads, int q_rows_total) {
    if (num_heads < 1 || q_rows_total < 1) return 0;
    return static_cast<size_t>(num_heads) * q_rows_total * 2 * sizeof(float);
}

int bdattn_sdpa_traced_fwd(const bdattn_sdpa_params* p, const bdattn_trace_params* t,
                           bdattn_stream_t stream) {
    const char* op = "joint_attention_traced";
    if (p == nullptr || t == nullptr) return fail("%s: params is null", op);
    if (p->batch != 1) return fail("%s: batch must be 1", op);
    long long Lq = 0, Lk = 0;
    for (int s = 0; s < p->n_q_seg && s < 2; ++s) Lq += p->q_rows[s];
    for (int s = 0; s < p->n_kv_seg && s < 2; ++s) Lk += p->kv_rows[s];
    if (t->bias != nullptr) {
        if (t->bias_rows < 1 || t->bias_cols < 1 || t->bias_row0 < 0 || t->bias_row0 + t->bias_rows > Lq ||
            t->bias_cols > Lk)
            return fail("%s: bias block (rows %d..%d, %d cols) does not fit the %lld x %lld score matrix", op,
                        t->bias_row0, t->bias_row0 + t->bias_rows, t->bias_cols, Lq, Lk);
    }
    if (t->attn_avg != nullptr) {
        if (t->map_rows < 1 || t->map_cols < 1 || t->map_row0 < 0 || t->map_row0 + t->map_rows > Lq ||
            t->map_cols > Lk)
            return fail("%s: map block (rows %d..%d, %d cols) does not fit the %lld x %lld score matrix", op,
                        t->map_row0, t->map_row0 + t->map_rows, t->map_cols, Lq, Lk);
    }
    if (p->num_kv_heads > 0 && p->num_kv_heads != p->num_heads)
        return fail("%s: grouped-query heads are not supported by the traced path", op);
    const size_t need = bdattn_sdpa_traced_workspace_bytes(p->num_heads, static_cast<int>(Lq));
    if (t->workspace == nullptr || t->workspace_bytes < need)
        return fail("%s: workspace of %zu bytes needed (got %zu)", op, need, t->workspace_bytes);
    if (sdpa_fwd_impl(op, p, nullptr, nullptr, 0, t, stream)) return -1;
    if (t->attn_avg == nullptr) return 0;
    const int hd = p->head_dim;
    bdattn::AttnMapArgs m;
    std::memset(&m, 0, sizeof(m));
    for (int s = 0; s < 2; ++s) {
        if (s < p->n_q_seg) { m.q[s] = p->q[s]; m.q_rows[s] = p->q_rows[s]; m.q_ld[s] = p->q_ld[s]; }
        if (s < p->n_kv_seg) { m.k[s] = p->k[s]; m.kv_rows[s] = p->kv_rows[s]; m.k_ld[s] = p->k_ld[s]; }
    }
    if (p->n_q_seg == 1) m.q_rows[0] = static_cast<int>(Lq);
    if (p->n_kv_seg == 1) m.kv_rows[0] = static_cast<int>(Lk);
    m.num_heads = p->num_heads; m.head_dim = hd;
    const float scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(hd));
    m.scale_log2 = scale * 1.4426950408889634f;
    m.lse = static_cast<const float*>(t->workspace); m.lq_total = static_cast<int>(Lq);
    m.bias = t->bias; m.bias_row0 = t->bias_row0; m.bias_rows = t->bias_rows; m.bias_cols = t->bias_cols;
    m.bias_ld = t->bias_ld > 0 ? t->bias_ld : t->bias_cols;
    m.map = t->attn_avg; m.map_row0 = t->map_row0; m.map_rows = t->map_rows; m.map_cols = t->map_cols;
    m.map_ld = t->map_ld > 0 ? t->map_ld : t->map_cols;
    m.mask_mode = p->mask_mode;
    m.q_offset = static_cast<int>(Lk - Lq);
    m.key_mask = p->key_mask;
    m.key_scale = p->key_scale;
    cudaError_t e = bdattn::launch_attn_map(m, p->dtype == BDATTN_BF16, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_rmsnorm_rope(const bdattn_norm_rope_job* jobs, int n_jobs, int dtype, int num_heads,
                        int head_dim, float eps, int pair_mode, bdattn_stream_t stream) {
    const char* op = "bdattn_rmsnorm_rope";
    if (require_sm100(op)) return -1;
    if (jobs == nullptr || n_jobs < 1 || n_jobs > BDATTN_MAX_NORM_JOBS)
        return fail("%s: n_jobs must be in [1, %d]", op, BDATTN_MAX_NORM_JOBS);
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: dtype must be BF16 or F16", op);
    if (num_heads < 1 || head_dim < 2 || head_dim > 256 || head_dim % 2 != 0)
        return fail("%s: head_dim must be even and <= 256 (got %d)", op, head_dim);
    if (pair_mode != BDATTN_ROPE_INTERLEAVED && pair_mode != BDATTN_ROPE_HALF_SPLIT)
        return fail("%s: unknown pair_mode %d", op, pair_mode);
    bdattn::NormRopeArgs a;
    std::memset(&a, 0, sizeof(a));
    const long long D = static_cast<long long>(num_heads) * head_dim;
    for (int i = 0; i < n_jobs; ++i) {
        const bdattn_norm_rope_job& j = jobs[i];
        if (j.x == nullptr || j.out == nullptr) return fail("%s: job %d: x/out is null", op, i);
        if (j.rows < 1) return fail("%s: job %d: rows must be >= 1", op, i);
        if (j.x_ld < D || j.out_ld < D) return fail("%s: job %d: ld smaller than num_heads*head_dim", op, i);
        if ((j.cos == nullptr) != (j.sin == nullptr)) return fail("%s: job %d: cos and sin must both be given", op, i);
        if (j.gain != nullptr && j.gain_dtype != BDATTN_F32 && j.gain_dtype != dtype)
            return fail("%s: job %d: gain_dtype must be F32 or the tensor dtype", op, i);
        if ((reinterpret_cast<uintptr_t>(j.x) & 3u) || (reinterpret_cast<uintptr_t>(j.out) & 3u) ||
            (j.x_ld & 1) || (j.out_ld & 1))
            return fail("%s: job %d: x/out must be 4-byte aligned with even ld", op, i);
        bdattn::NormRopeJobDev& d = a.job[i];
        d.x = j.x; d.out = j.out; d.rows = j.rows; d.x_ld = j.x_ld; d.out_ld = j.out_ld;
        d.gain = j.gain; d.gain_is_f32 = j.gain_dtype == BDATTN_F32 ? 1 : 0;
        d.cos = j.cos; d.sin = j.sin; d.rope_row0 = j.rope_row0;
    }
    a.n_jobs = n_jobs;
    a.num_heads = num_heads;
    a.head_dim = head_dim;
    a.eps = eps;
    a.pair_mode = pair_mode;
    cudaError_t e = bdattn::launch_norm_rope(a, dtype == BDATTN_BF16, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_rope_tables_flux(int txt_len, int hp, int wp, int head_dim, const int* axes_dims,
                            int n_axes, float theta, float* cos, float* sin,
                            bdattn_stream_t stream) {
    const char* op = "build_axial_rope_tables";
    if (require_sm100(op)) return -1;
    if (head_dim < 2 || head_dim % 2 != 0) return fail("%s: head_dim must be even", op);
    if (axes_dims == nullptr || n_axes < 1 || n_axes > 3) return fail("%s: n_axes must be 1..3", op);
    int sum = 0;
    for (int i = 0; i < n_axes; ++i) {
        if (axes_dims[i] < 0 || axes_dims[i] % 2 != 0) return fail("%s: axes_dims_rope entries must be even", op);
        sum += axes_dims[i];
    }
    if (sum != head_dim) return fail("%s: axes_dims_rope must sum to head_dim", op);
    if (txt_len < 0 || hp < 0 || wp < 0 || txt_len + static_cast<long long>(hp) * wp < 1)
        return fail("%s: empty sequence", op);
    if (cos == nullptr || sin == nullptr) return fail("%s: cos/sin must not be null", op);
    bdattn::RopeTableArgs a;
    std::memset(&a, 0, sizeof(a));
    a.flux = 1;
    a.rows = txt_len + hp * wp;
    a.half = head_dim / 2;
    a.n_axes = n_axes;
    for (int i = 0; i < n_axes; ++i) a.axes[i] = axes_dims[i];
    a.theta = theta;
    a.n_seg = 2;
    a.seg_kind[0] = 0; a.seg_row0[0] = 0;
    a.seg_kind[1] = 1; a.seg_row0[1] = txt_len; a.seg_h[1] = hp; a.seg_w[1] = wp > 0 ? wp : 1;
    a.cos_out = cos; a.sin_out = sin;
    cudaError_t e = bdattn::launch_rope_tables(a, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_rope_rows_qwen(const bdattn_rope_segment* prefix, int n_prefix, int hp, int wp) {
    long long rows = static_cast<long long>(hp) * wp;
    for (int i = 0; i < n_prefix; ++i)
        rows += prefix[i].kind == 0 ? prefix[i].n_tokens : static_cast<long long>(prefix[i].h) * prefix[i].w;
    return static_cast<int>(rows);
}

int bdattn_rope_tables_qwen(const bdattn_rope_segment* prefix, int n_prefix, int hp, int wp,
                            int head_dim, const int* axes_dims3, float theta, float* cos,
                            float* sin, bdattn_stream_t stream) {
    const char* op = "build_rope_tables";
    if (require_sm100(op)) return -1;
    if (n_prefix < 0 || (n_prefix > 0 && prefix == nullptr)) return fail("%s: bad prefix", op);
    if (n_prefix + 1 > bdattn::kMaxRopeSegments)
        return fail("%s: at most %d prefix segments", op, bdattn::kMaxRopeSegments - 1);
    if (head_dim < 2 || head_dim % 2 != 0 || axes_dims3 == nullptr) return fail("%s: head_dim must be even", op);
    if (axes_dims3[0] + axes_dims3[1] + axes_dims3[2] != head_dim)
        return fail("%s: axes_dims_rope must sum to head_dim", op);
    if (hp < 1 || wp < 1) return fail("%s: target grid must be at least 1x1", op);
    if (cos == nullptr || sin == nullptr) return fail("%s: cos/sin must not be null", op);
    bdattn::RopeTableArgs a;
    std::memset(&a, 0, sizeof(a));
    a.flux = 0;
    a.half = head_dim / 2;
    a.n_axes = 3;
    for (int i = 0; i < 3; ++i) a.axes[i] = axes_dims3[i];
    a.theta = theta;
    int row = 0, pos = 0;
    for (int i = 0; i <= n_prefix; ++i) {
        const bool target = i == n_prefix;
        const int kind = target ? 1 : prefix[i].kind;
        const int h = target ? hp : prefix[i].h;
        const int w = target ? wp : prefix[i].w;
        a.seg_kind[i] = kind; a.seg_row0[i] = row; a.seg_pos0[i] = pos;
        if (kind == 0) {
            if (prefix[i].n_tokens < 0) return fail("%s: negative segment length", op);
            row += prefix[i].n_tokens; pos += prefix[i].n_tokens;
        } else {
            if (h < 1 || w < 1) return fail("%s: image segment %d must be at least 1x1", op, i);
            a.seg_h[i] = h; a.seg_w[i] = w;
            row += h * w; pos += (h > w ? h : w);
        }
    }
    a.n_seg = n_prefix + 1;
    a.rows = row;
    a.cos_out = cos; a.sin_out = sin;
    cudaError_t e = bdattn::launch_rope_tables(a, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_linear_attn_relu_fwd(const void* q, const void* k, const void* v, void* out, int dtype,
                                int batch, int num_heads, int head_dim, int n_tokens,
                                long long ld, long long batch_stride, float eps,
                                const float* sz_in, float w_in, float* sz_out,
                                bdattn_stream_t stream) {
    const char* op = "bdattn_linear_attn_relu_fwd";
    if (require_sm100(op)) return -1;
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr)
        return fail("%s: q/k/v/out must not be null", op);
    if (dtype != BDATTN_BF16)
        return fail("%s: dtype must be BF16 (the state sums n_tokens products and overflows FP16)", op);
    if (head_dim != 32)
        return fail("%s: head_dim must be 32 (got %d), as the reference's Sana attention requires", op,
                    head_dim);
    if (batch < 1 || num_heads < 1 || n_tokens < 1)
        return fail("%s: batch, num_heads and n_tokens must be >= 1", op);
    if (n_tokens % 8 != 0) return fail("%s: n_tokens must be a multiple of 8 (got %d)", op, n_tokens);
    if (ld < n_tokens || ld % 8 != 0 || batch_stride % 8 != 0 || !aligned16(q) || !aligned16(k) ||
        !aligned16(v) || !aligned16(out))
        return fail("%s: tensors must be 16-byte aligned, ld >= n_tokens, ld and batch_stride "
                    "multiples of 8 elements", op);
    bdattn::LinearAttnArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out;
    a.batch = batch; a.num_heads = num_heads; a.n_tokens = n_tokens;
    a.ld = ld; a.batch_stride = batch_stride > 0 ? batch_stride : static_cast<long long>(num_heads) * 32 * ld;
    a.eps = eps; a.sz_in = sz_in; a.w_in = w_in; a.sz_out = sz_out;
    const long long D = static_cast<long long>(num_heads) * 32;
    CUtensorMap tq, tk, tv, to;
    // output: one 32-token x 32-row piece per warp and store, 64-byte rows under the 64-byte swizzle
    if (make_map_3d(op, &to, out, true, n_tokens, D, batch, ld, a.batch_stride, 32, 32, 64)) return -1;
    if (make_map_3d(op, &tq, q, true, n_tokens, D, batch, ld, a.batch_stride, 32)) return -1;
    if (make_map_3d(op, &tk, k, true, n_tokens, D, batch, ld, a.batch_stride, 32)) return -1;
    if (make_map_3d(op, &tv, v, true, n_tokens, D, batch, ld, a.batch_stride, 32)) return -1;
    // Cluster size: spread one (batch, head) over several SMs while the grid
    // still fits the 148 SMs and every CTA keeps at least one 128-token chunk.
    const int chunks = (n_tokens + 127) / 128;
    int cs = 1;
    while (cs < 8 && static_cast<long long>(batch) * num_heads * cs * 2 <= 148 && chunks >= cs * 2) cs *= 2;
    // One CTA per SM (16 consumer warps, a ring of eight 16 KB items).  Splitting long
    // sequences once more so that two 8-warp CTAs share an SM was slower at every shape
    // tried (28.6 against 30.6 us at 4096 tokens, batch 2): it buys a cluster barrier
    // and a second reduction where the 16 warps of one CTA already hide the latencies.
    a.stages = 8;
    cudaError_t e = bdattn::launch_linear_attn(a, tq, tk, tv, to, cs, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_linear_fwd(const void* x, const void* w, const void* bias, void* y, int dtype, int M,
                      int N, int K, long long ldx, long long ldw, long long ldy,
                      bdattn_stream_t stream) {
    const char* op = "bdattn_linear_fwd";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: dtype must be BF16 or F16", op);
    bdattn::GemmLaunch L;
    std::memset(&L, 0, sizeof(L));
    L.bf16 = dtype == BDATTN_BF16;
    if (add_gemm_problem(op, L, 0, x, ldx, w, ldw, bias, y, ldy, M, N, K, 0, 0, 0)) return -1;
    finish_gemm_launch(L, 1);
    cudaError_t e = bdattn::launch_gemm(L, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_qkv_norm_rope_fwd(const bdattn_qkv_proj_params* p, bdattn_stream_t stream) {
    const char* op = "bdattn_qkv_norm_rope_fwd";
    if (p == nullptr) return fail("%s: params is null", op);
    if (require_sm100(op)) return -1;
    if (p->dtype != BDATTN_BF16 && p->dtype != BDATTN_F16) return fail("%s: dtype must be BF16 or F16", op);
    if (p->head_dim != 64 && p->head_dim != 128) return fail("%s: head_dim must be 64 or 128 (got %d)", op, p->head_dim);
    if (p->num_heads < 1 || p->rows < 1 || p->in_features < 1) return fail("%s: empty problem", op);
    if ((p->cos == nullptr) != (p->sin == nullptr)) return fail("%s: cos and sin must both be given", op);
    if (!aligned16(p->cos) || !aligned16(p->sin)) return fail("%s: cos and sin must be 16-byte aligned", op);
    if (p->gain_q != nullptr || p->gain_k != nullptr)
        if (p->gain_dtype != BDATTN_F32 && p->gain_dtype != p->dtype)
            return fail("%s: gain_dtype must be F32 or the tensor dtype", op);
    const int N = p->num_heads * p->head_dim;
    bdattn::GemmLaunch L;
    std::memset(&L, 0, sizeof(L));
    L.bf16 = p->dtype == BDATTN_BF16;
    const void* w[3] = {p->wq, p->wk, p->wv};
    const void* b[3] = {p->bq, p->bk, p->bv};
    void* out[3] = {p->q_out, p->k_out, p->v_out};
    const long long ld[3] = {p->q_ld > 0 ? p->q_ld : N, p->k_ld > 0 ? p->k_ld : N, p->v_ld > 0 ? p->v_ld : N};
    const void* gain[3] = {p->gain_q, p->gain_k, nullptr};
    int n = 0;
    for (int i = 0; i < 3; ++i) {
        if (w[i] == nullptr || out[i] == nullptr) continue;     // a projection may be left out
        if (add_gemm_problem(op, L, n, p->x, p->x_ld > 0 ? p->x_ld : p->in_features, w[i], p->in_features, b[i],
                             out[i], ld[i], p->rows, N, p->in_features, p->head_dim, p->head_dim, 0))
            return -1;
        bdattn::GemmProblem& g = L.args.p[n];
        g.norm_rope = 1;
        g.gain = gain[i];
        g.gain_is_f32 = p->gain_dtype == BDATTN_F32 ? 1 : 0;
        g.eps = p->eps;
        g.cos = i < 2 ? p->cos : nullptr;
        g.sin = i < 2 ? p->sin : nullptr;
        g.rope_row0 = p->rope_row0;
        ++n;
    }
    if (n == 0) return fail("%s: no projection requested", op);
    finish_gemm_launch(L, n);
    cudaError_t e = bdattn::launch_gemm(L, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_linear_geglu_fwd(const void* x, const void* w, const void* bias, void* y, int dtype,
                            int rows, int d_in, int d_out, bdattn_stream_t stream) {
    const char* op = "fused_linear_geglu";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: tensors must be FP16 or BF16", op);
    bdattn::GemmLaunch L;
    std::memset(&L, 0, sizeof(L));
    L.bf16 = dtype == BDATTN_BF16;
    if (add_gemm_problem(op, L, 0, x, d_in, w, d_in, bias, y, d_out, rows, d_out, d_in, 0, 0, d_out)) return -1;
    finish_gemm_launch(L, 1);
    cudaError_t e = bdattn::launch_gemm(L, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_add_inplace(void* y, const void* x, long long n, int dtype, bdattn_stream_t stream) {
    const char* op = "add_inplace_vec";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: tensors must be FP16 or BF16", op);
    if (y == nullptr || x == nullptr || n < 0) return fail("%s: bad arguments", op);
    if (n == 0) return 0;
    cudaError_t e = bdattn::launch_add_inplace(y, x, n, dtype == BDATTN_BF16, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_axpby_inplace(void* y, const void* x, long long n, float a, float b, int dtype,
                         bdattn_stream_t stream) {
    const char* op = "axpby_inplace";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: tensors must be FP16 or BF16", op);
    if (y == nullptr || n < 0) return fail("%s: bad arguments", op);
    if (x == nullptr && b != 0.0f) return fail("%s: x is null but b is not zero", op);
    if (n == 0 || (a == 1.0f && (x == nullptr || b == 0.0f))) return 0;
    cudaError_t e = bdattn::launch_axpby_inplace(y, x, n, a, b, dtype == BDATTN_BF16, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_add_row_bias(void* y, const void* bias, int rows, int cols, long long ld, int dtype,
                        bdattn_stream_t stream) {
    const char* op = "add_inplace_row_bias";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: tensors must be FP16 or BF16", op);
    if (y == nullptr || bias == nullptr || rows < 0 || cols < 0 || ld < cols) return fail("%s: bad arguments", op);
    if (rows == 0 || cols == 0) return 0;
    cudaError_t e = bdattn::launch_add_row_bias(y, bias, rows, cols, ld, dtype == BDATTN_BF16,
                                                reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

size_t bdattn_qkvo_workspace_bytes(int q_rows, int kv_rows, int num_heads, int head_dim) {
    if (q_rows < 0 || kv_rows < 0 || num_heads < 1 || head_dim < 1) return 0;
    const int pad = padded_head_dim(head_dim) ? padded_head_dim(head_dim) : head_dim;
    const size_t wq = static_cast<size_t>(q_rows) * num_heads * pad * 2;
    const size_t wkv = static_cast<size_t>(kv_rows) * num_heads * pad * 2;
    const size_t wo = static_cast<size_t>(q_rows) * num_heads * head_dim * 2;
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    return up(wq) + 2 * up(wkv) + up(wo);
}

int bdattn_project_kv(const void* ctx, int ctx_rows, int ctx_cols, long long ctx_ld, const void* wk,
                      const void* bk, const void* wv, const void* bv, void* k_out, void* v_out,
                      long long kv_ld, int inner_dim, int dtype, bdattn_stream_t stream) {
    const char* op = "flash_attention_project_kv";
    if (require_sm100(op)) return -1;
    if (dtype != BDATTN_BF16 && dtype != BDATTN_F16) return fail("%s: dtype must be BF16 or F16", op);
    bdattn::GemmLaunch L;
    std::memset(&L, 0, sizeof(L));
    L.bf16 = dtype == BDATTN_BF16;
    if (add_gemm_problem(op, L, 0, ctx, ctx_ld, wk, ctx_cols, bk, k_out, kv_ld, ctx_rows, inner_dim, ctx_cols, 0, 0, 0)) return -1;
    if (add_gemm_problem(op, L, 1, ctx, ctx_ld, wv, ctx_cols, bv, v_out, kv_ld, ctx_rows, inner_dim, ctx_cols, 0, 0, 0)) return -1;
    finish_gemm_launch(L, 2);
    cudaError_t e = bdattn::launch_gemm(L, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(op, e);
    return 0;
}

int bdattn_qkvo_fwd(const bdattn_qkvo_params* p, bdattn_stream_t stream) {
    if (p == nullptr) return fail("bdattn_qkvo_fwd: params is null");
    const bool cached = p->k_cached != nullptr || p->v_cached != nullptr;
    const char* op = cached ? "flash_attention_q_with_kv_cached_forward" : "flash_attention_qkvo_forward";
    if (require_sm100(op)) return -1;
    if (p->dtype != BDATTN_BF16 && p->dtype != BDATTN_F16) return fail("%s: dtype must be BF16 or F16", op);
    const bool bf16 = p->dtype == BDATTN_BF16;
    if (p->num_heads < 1 || p->inner_dim < 1 || p->inner_dim % p->num_heads != 0)
        return fail("%s: inner_dim must be a positive multiple of num_heads", op);
    const int nh = p->num_heads, C = p->inner_dim, hd = C / nh;
    if (hd % 8 != 0 || hd > 256) return fail("%s: head_dim must be a multiple of 8 up to 256 (got %d)", op, hd);
    if (p->x == nullptr || p->out == nullptr || p->wq == nullptr || p->wo == nullptr)
        return fail("%s: x, out, wq and wo must not be null", op);
    if (p->x_rows < 1) return fail("%s: x has no rows", op);
    if (cached && (p->k_cached == nullptr || p->v_cached == nullptr || p->kv_rows < 1))
        return fail("%s: k_cached, v_cached and kv_rows must all be given", op);
    if (!cached && (p->wk == nullptr || p->wv == nullptr)) return fail("%s: wk and wv must not be null", op);
    if (cached && (p->k_ld < C || p->v_ld < C || p->k_ld % 8 || p->v_ld % 8 || !aligned16(p->k_cached) ||
                   !aligned16(p->v_cached)))
        return fail("%s: cached K/V must be 16-byte aligned with ld >= inner_dim and a multiple of 8", op);
    const void* src = p->ctx != nullptr ? p->ctx : p->x;
    const int src_rows = p->ctx != nullptr ? p->ctx_rows : p->x_rows;
    const int src_cols = p->ctx != nullptr ? p->ctx_cols : p->x_cols;
    const long long src_ld = p->ctx != nullptr ? p->ctx_ld : p->x_ld;
    const int Lq = p->x_rows;
    const int Lk = cached ? p->kv_rows : src_rows;
    if (Lk < 1) return fail("%s: no key rows", op);
    const size_t need = bdattn_qkvo_workspace_bytes(Lq, Lk, nh, hd);
    if (p->workspace == nullptr || p->workspace_bytes < need)
        return fail("%s: workspace of %zu bytes needed (got %zu)", op, need, p->workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(p->workspace) & 255u) != 0) return fail("%s: workspace must be 256-byte aligned", op);
    const int pad = padded_head_dim(hd);
    const int P = pad ? pad : hd;
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    uint8_t* ws = static_cast<uint8_t*>(p->workspace);
    void* Qp = ws;
    void* Kp = ws + up(static_cast<size_t>(Lq) * nh * P * 2);
    void* Vp = static_cast<uint8_t*>(Kp) + up(static_cast<size_t>(Lk) * nh * P * 2);
    void* Op = static_cast<uint8_t*>(Vp) + up(static_cast<size_t>(Lk) * nh * P * 2);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const long long ldp = static_cast<long long>(nh) * P;

    // 1. projections into head-padded Q / K / V
    {
        bdattn::GemmLaunch L;
        std::memset(&L, 0, sizeof(L));
        L.bf16 = bf16;
        int n = 0;
        if (add_gemm_problem(op, L, n++, p->x, p->x_ld, p->wq, p->x_cols, p->bq, Qp, ldp, Lq, C, p->x_cols,
                             pad ? hd : 0, P, 0)) return -1;
        if (!cached) {
            if (add_gemm_problem(op, L, n++, src, src_ld, p->wk, src_cols, p->bk, Kp, ldp, Lk, C, src_cols,
                                 pad ? hd : 0, P, 0)) return -1;
            if (add_gemm_problem(op, L, n++, src, src_ld, p->wv, src_cols, p->bv, Vp, ldp, Lk, C, src_cols,
                                 pad ? hd : 0, P, 0)) return -1;
        }
        finish_gemm_launch(L, n);
        cudaError_t e = bdattn::launch_gemm(L, st);
        if (e != cudaSuccess) return cuda_fail(op, e);
    }
    const void* Kin = Kp;
    const void* Vin = Vp;
    long long k_ld = ldp, v_ld = ldp;
    if (cached) {
        if (P != hd) {
            cudaError_t e = bdattn::launch_pad_heads(p->k_cached, Kp, Lk, nh, hd, P, p->k_ld, st);
            if (e == cudaSuccess) e = bdattn::launch_pad_heads(p->v_cached, Vp, Lk, nh, hd, P, p->v_ld, st);
            if (e != cudaSuccess) return cuda_fail(op, e);
        } else {
            Kin = p->k_cached; Vin = p->v_cached; k_ld = p->k_ld; v_ld = p->v_ld;
        }
    }

    // 2. attention core
    const float scale = 1.0f / std::sqrt(static_cast<float>(hd));
    if (pad) {
        bdattn::SdpaLaunch L;
        std::memset(&L, 0, sizeof(L));
        for (int s = 0; s < 2; ++s) {
            if (make_map_heads(op, &L.tmQ[s], Qp, bf16, P, nh, Lq, 1, ldp, 0, 128)) return -1;
            if (make_map_heads(op, &L.tmK[s], Kin, bf16, P, nh, Lk, 1, k_ld, 0, 128)) return -1;
            if (make_map_heads(op, &L.tmV[s], Vin, bf16, P, nh, Lk, 1, v_ld, 0, 128)) return -1;
        }
        bdattn::SdpaDevArgs& a = L.args;
        a.q_rows[0] = Lq; a.kv_rows[0] = Lk;
        a.o[0] = Op; a.o_ld[0] = C; a.o_bs[0] = 0;
        a.q_ctas0 = (Lq + 255) / 256;
        a.kv_tiles0 = (Lk + 127) / 128;
        a.kv_tiles = a.kv_tiles0;
        a.mask_mode = p->causal ? 1 : 0;
        a.q_offset = Lk - Lq;
        a.hd_out = hd;
        a.kv_group = 1;
        a.key_mask = p->key_mask;
        a.scale_log2 = scale * 1.4426950408889634f;
        L.q_ctas = a.q_ctas0;
        L.num_heads = nh; L.batch = 1; L.head_dim = P; L.bf16 = bf16;
        cudaError_t e = bdattn::launch_sdpa_tc05(L, st);
        if (e != cudaSuccess) return cuda_fail(op, e);
    } else {
        bdattn::SdpaGeneralArgs g;
        std::memset(&g, 0, sizeof(g));
        g.q[0] = Qp; g.k[0] = Kin; g.v[0] = Vin; g.o[0] = Op;
        g.q_rows[0] = Lq; g.kv_rows[0] = Lk;
        g.q_ld[0] = ldp; g.k_ld[0] = k_ld; g.v_ld[0] = v_ld; g.o_ld[0] = C;
        g.mask_mode = p->causal ? 1 : 0;
        g.q_offset = Lk - Lq;
        g.head_dim = hd;
        g.kv_group = 1;
        g.key_mask = p->key_mask;
        g.scale = scale;
        cudaError_t e = bdattn::launch_sdpa_general(g, nh, 1, bf16, st);
        if (e != cudaSuccess) return cuda_fail(op, e);
    }

    // 3. output projection
    {
        const int out_cols = p->out_cols > 0 ? p->out_cols : C;
        bdattn::GemmLaunch L;
        std::memset(&L, 0, sizeof(L));
        L.bf16 = bf16;
        if (add_gemm_problem(op, L, 0, Op, C, p->wo, C, p->bo, p->out, p->out_ld > 0 ? p->out_ld : out_cols, Lq,
                             out_cols, C, 0, 0, 0)) return -1;
        finish_gemm_launch(L, 1);
        cudaError_t e = bdattn::launch_gemm(L, st);
        if (e != cudaSuccess) return cuda_fail(op, e);
    }
    return 0;
}

}  // extern "C"
