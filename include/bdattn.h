/* bdattn — C ABI of the B200 (sm_100a) denoiser-attention library.
 *
 * This is the boundary a brodiffusion build binds instead of the brotensor
 * attention operators and its own fused_transformer entry points.  Every
 * declaration cites the reference interface it replaces (path within the
 * brodiffusion source tree : line).
 *
 * Conventions (taken from the reference's own C ABI,
 * include/brodiffusion/qwenimage21_capi.h:32-37):
 *   - every function returns 0 on success and -1 on failure;
 *     bdattn_last_error() returns the calling thread's last message;
 *   - all tensor pointers are caller-owned DEVICE pointers on the current CUDA
 *     device; tensors are dense row-major 2-D (rows, cols) with an explicit
 *     row stride `ld` in elements; heads are column blocks (head h of an
 *     (L, nh*hd) tensor is columns [h*hd, (h+1)*hd));
 *   - work is enqueued on the given stream and the call returns without
 *     synchronising (include/brodiffusion/unet.h:50-51); no function
 *     allocates device memory: an operator that needs scratch takes it as an
 *     argument, with a bdattn_*_workspace_bytes() query beside it;
 *   - there is no CPU path: a call fails if no sm_100 device is current.
 */
#ifndef BDATTN_H_
#define BDATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* bdattn_stream_t; /* == cudaStream_t */

/* Element types; values follow brotensor::Dtype order as used by the callers
 * (FP32, FP16, BF16). */
enum { BDATTN_F32 = 0, BDATTN_F16 = 1, BDATTN_BF16 = 2 };

/* Attention visibility rules. */
enum {
    BDATTN_MASK_NONE = 0,
    /* key j visible to query i iff j <= i + (Lk - Lq): what
     * flash_attention_windowed_forward(window = 0) and causal = true compute
     * (src/dit/qwenimage21_forward.cpp:659-662). */
    BDATTN_MASK_CAUSAL = 1
};

/* Rotary pair conventions for bdattn_rmsnorm_rope. */
enum {
    BDATTN_ROPE_INTERLEAVED = 0, /* pair p = head elements (2p, 2p+1) */
    BDATTN_ROPE_HALF_SPLIT = 1   /* pair p = head elements (p, p + hd/2) */
};

/* Bits of the per-device status word (bdattn_device_status). */
enum { BDATTN_STATUS_WAIT_TIMEOUT = 1, BDATTN_STATUS_BAD_ARGS = 2 };

/* Library version (major*10000 + minor*100 + patch). */
int bdattn_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* bdattn_last_error(void);

/* Synchronises the current device and returns its status word: 0 when every
 * kernel ran to completion; a bit of BDATTN_STATUS_* when a kernel gave up a
 * bounded wait or rejected its arguments.  clear != 0 resets the word.
 * Replaces BRODIFFUSION_CUDA_CHECK(cudaGetLastError())
 * (include/brodiffusion/detail/cuda_check.cuh:13-21) for device-side
 * failures that do not fault. */
int bdattn_device_status(int* status, int clear);

/* ---------------------------------------------------------------- softmax
 * Multi-head softmax attention  O = softmax(Q K^T * scale [masks]) V.
 *
 * Replaces brotensor::flash_attention_forward (call sites
 * src/dit/common.cpp:194, src/dit/qwenimage21_forward.cpp:648,667,674,
 * src/dit/sana.cpp:623) and brotensor::flash_attention_windowed_forward
 * (src/dit/qwenimage21_forward.cpp:662).
 *
 * Queries/outputs and keys/values may each be given as ONE or TWO row
 * segments that are attended as if concatenated (segment 0 first).  That
 * removes the concat_rows/slice_rows copies of the Flux double-stream block
 * (src/dit/flux.cpp:491-494,514-516: text rows, then image rows) and the
 * k_full_/v_full_ copies of the Qwen-Image cached step
 * (src/dit/qwenimage21_forward.cpp:600-647: cached prefix rows, then fresh
 * rows).  `o_ld` lets the output land inside a wider row (the Flux
 * single-stream cat5_ buffer, src/dit/flux.cpp:626-632).
 *
 * key_scale / val_scale (optional, Lk floats each over the concatenated keys)
 * multiply K rows and V rows on the fly: the prefix K/V attenuation hook of
 * src/dit/qwenimage21_forward.cpp:606-645 without touching the cache.  The
 * tensor-core kernel scales the rows of the tiles it has staged in shared
 * memory and rounds them to the tensor dtype, which is what the reference's
 * scale_inplace on its k_full_ / v_full_ copies does; tiles whose factors are
 * all one are passed through untouched.
 *
 * head_dim 64 and 128 run on the tcgen05 tensor-core kernel; other head
 * dims (multiple of 8, <= 256) run on a general kernel.  dtype BF16 or F16.
 */
typedef struct bdattn_sdpa_params {
    int dtype;
    int batch;
    int num_heads;
    int head_dim;
    int n_q_seg;                 /* 1 or 2 */
    const void* q[2];
    void* o[2];
    int q_rows[2];
    long long q_ld[2];
    long long o_ld[2];
    long long q_batch_stride[2]; /* elements between batch items */
    long long o_batch_stride[2];
    int n_kv_seg;                /* 1 or 2 */
    const void* k[2];
    const void* v[2];
    int kv_rows[2];
    long long k_ld[2];
    long long v_ld[2];
    long long k_batch_stride[2];
    long long v_batch_stride[2];
    int mask_mode;               /* BDATTN_MASK_* */
    const float* key_mask;       /* Lk floats, 1 = valid, 0 = masked; or NULL */
    const float* key_scale;      /* Lk floats or NULL */
    const float* val_scale;      /* Lk floats or NULL */
    float softmax_scale;         /* 0 => 1/sqrt(head_dim) */
    /* Grouped-query attention (dit::gqa_attention_masked, src/dit/common.cpp:331-377):
     * K and V carry num_kv_heads heads (k_ld/v_ld >= num_kv_heads*head_dim) and
     * query head h reads K/V head h / (num_heads / num_kv_heads), so the widened
     * Krep / Vrep copies of the reference (common.cpp:361-375) are never made.
     * 0 or num_heads = plain multi-head attention; must divide num_heads. */
    int num_kv_heads;
    /* Optional per-head RMSNorm + RoPE of the QUERY rows inside the kernel (the
     * headnorm + rope_apply of Q in src/dit/flux.cpp:462-469,
     * src/dit/common.cpp:192 and src/dit/qwenimage21_forward.cpp:54-63,584):
     * every CTA normalises and rotates its own query tile in shared memory
     * before the first MMA, so the Q half of the bdattn_rmsnorm_rope pre-pass
     * and its HBM round trip disappear.  (K is not fused: every query-tile CTA
     * of a head would repeat that work.)
     *   q_gain[s]   head_dim gains of query segment s (q_gain_dtype: F32 or the
     *               tensor dtype), or NULL for no RMSNorm on that segment
     *   q_cos/q_sin FP32 (rows, head_dim/2) tables, interleaved pairs, or NULL;
     *               query row i of the concatenated segments uses table row
     *               q_rope_row0 + i
     * All NULL = disabled.  head_dim <= 128 only. */
    const void* q_gain[2];
    int q_gain_dtype;
    float q_eps;
    const float* q_cos;
    const float* q_sin;
    int q_rope_row0;
} bdattn_sdpa_params;

int bdattn_sdpa_fwd(const bdattn_sdpa_params* p, bdattn_stream_t stream);

/* Head-sharded attention with the all-gather of head outputs fused into the
 * kernel (no counterpart in the reference, which is single-device).  Rank g
 * of G computes its heads and p->o[] is ITS copy of the full (L, D) output,
 * offset to its own head columns (o_ld = D).  peer_o0[i] (and peer_o1[i] for
 * the second query segment) are the same location inside the copies that live
 * on the other GPUs, as pointers this process can store through (peer-mapped /
 * symmetric memory).  The epilogue writes every output vector to the local
 * copy and to all n_peers (<= 8) peer copies with plain 16-byte stores over
 * NVLink, so the transfer overlaps the attention of later tiles and no
 * staging or NCCL call is needed; the kernel never reads peer memory.  The caller orders the consumers: a cross-GPU barrier
 * after the call (all ranks' kernels complete) before any rank reads the
 * gathered tensor.  head_dim 64 or 128 only. */
int bdattn_sdpa_fwd_allgather(const bdattn_sdpa_params* p, void* const* peer_o0, void* const* peer_o1,
                              int n_peers, bdattn_stream_t stream);

/* The same gather through the NVSwitch.  mc_o0 (and mc_o1 for the second query
 * segment) is the MULTICAST address of the location p->o[] names: an address of
 * an NVLink multicast object to which every GPU of the group has bound its copy
 * of the output at the same offset (torch symmetric memory's multicast_ptr, or
 * cuMulticastCreate / cuMulticastBindMem / cuMemMap by the caller).  The epilogue
 * issues one multimem.st per 16-byte vector; the switch delivers it to every
 * copy, the caller's own included, so each GPU sends its head columns once
 * instead of once per peer and p->o[] itself is not stored to.  Ordering as
 * above: a cross-GPU barrier after the call before any rank reads.  The caller
 * keeps every rank of the group alive while a multicast object is bound. */
int bdattn_sdpa_fwd_allgather_multicast(const bdattn_sdpa_params* p, void* mc_o0, void* mc_o1,
                                        bdattn_stream_t stream);

/* ------------------------------------------------ several GPUs, one process
 * Set-up and completion for a caller that drives the GPUs of one node from one
 * process with one host thread per GPU (no counterpart in the reference, which
 * is single-device; conventions as above, after
 * include/brodiffusion/qwenimage21_capi.h:32-37: opaque handle, 0 / -1 returns,
 * bdattn_last_error()).
 *
 *   bdattn_mgpu_init     enables peer access between the listed devices (at most
 *                        BDATTN_MGPU_MAX, all different) and allocates, on each, a
 *                        small array of arrival counters.  This is the one call of
 *                        the library that allocates device memory; _destroy frees
 *                        it.  Call it once, from any thread, before the workers.
 *   bdattn_mgpu_sdpa_fwd_headsharded
 *                        rank r (its device current) computes ITS heads of the
 *                        attention p describes (p->num_heads = total_heads / n,
 *                        q/k/v pointing at that rank's head columns; p->o is
 *                        ignored) and stores them into the head columns
 *                        [r * num_heads * head_dim, ...) of EVERY replica:
 *                        replicas[g] is GPU g's caller-owned copy of the full
 *                        (batch, L, total_heads * head_dim) output, row stride
 *                        replica_ld, batch stride replica_batch_stride (elements).
 *                        This is bdattn_sdpa_fwd_allgather with the peer pointers
 *                        worked out by the library.
 *   bdattn_mgpu_barrier  enqueues, on rank r's stream, a kernel that tells every
 *                        peer that r has arrived and waits until every peer has
 *                        arrived too.  Once it has passed on a rank's stream, all
 *                        ranks' work enqueued before their own barrier call is
 *                        complete, so the local replica holds all heads.  The wait
 *                        is bounded: after timeout_ms (0 = 2000) the kernel sets
 *                        BDATTN_STATUS_WAIT_TIMEOUT in that GPU's status word and
 *                        returns normally; bdattn_device_status reports it and the
 *                        context stays usable.  Every rank must enqueue the same
 *                        number of barriers; a rank that skipped one catches up by
 *                        calling it, or the context is re-created.
 * Plain peer stores and local loads only: no TMA multicast, no multimem, no NVLS.
 */
#define BDATTN_MGPU_MAX 8
typedef struct bdattn_mgpu bdattn_mgpu;

int bdattn_mgpu_init(bdattn_mgpu** ctx, const int* devices, int n_gpus);

int bdattn_mgpu_destroy(bdattn_mgpu* ctx);

int bdattn_mgpu_size(const bdattn_mgpu* ctx);

int bdattn_mgpu_sdpa_fwd_headsharded(bdattn_mgpu* ctx, int rank, const bdattn_sdpa_params* p,
                                     void* const* replicas, long long replica_ld,
                                     long long replica_batch_stride, int total_heads,
                                     bdattn_stream_t stream);

int bdattn_mgpu_barrier(bdattn_mgpu* ctx, int rank, int timeout_ms, bdattn_stream_t stream);

/* Traced / steered attention on the device.
 *
 * Replaces the host round trip of dit::joint_attention_traced
 * (src/dit/common.cpp:198-329; include/brodiffusion/dit/common.h:117-129) and
 * brotensor::cross_attention_forward_with_attn (src/unet_blocks.cpp:282-290):
 *   - bias: optional FP32 (bias_rows, bias_cols) logit bias added to the
 *     scaled scores of queries [bias_row0, bias_row0 + bias_rows) against keys
 *     [0, bias_cols) before the softmax (for Flux: image rows x text keys,
 *     src/dit/common.cpp:259-281; for the U-Net: every row x every key);
 *   - attn_avg: optional FP32 output (map_rows, map_cols), the softmax of
 *     queries [map_row0, map_row0 + map_rows) over keys [0, map_cols),
 *     averaged over the heads — the block the callers keep
 *     (src/dit/flux.cpp:505-508) instead of the full (L, L) map.
 * Row indices count the concatenated query / key segments.  The attention
 * output goes to p->o as usual.  workspace: bdattn_sdpa_traced_workspace_bytes
 * bytes of device memory (per-row softmax statistics).  batch 1, head_dim <= 128.
 */
typedef struct bdattn_trace_params {
    const float* bias;
    int bias_row0;
    int bias_rows;
    int bias_cols;
    long long bias_ld;      /* 0 => bias_cols */
    float* attn_avg;
    int map_row0;
    int map_rows;
    int map_cols;
    long long map_ld;       /* 0 => map_cols */
    void* workspace;
    size_t workspace_bytes;
} bdattn_trace_params;

size_t bdattn_sdpa_traced_workspace_bytes(int num_heads, int q_rows_total);

int bdattn_sdpa_traced_fwd(const bdattn_sdpa_params* p, const bdattn_trace_params* t,
                           bdattn_stream_t stream);

/* ------------------------------------------------- per-head RMSNorm + RoPE
 * out = rope(rms_norm_heads(x) * gain).  Replaces the headnorm view +
 * brotensor::rms_norm_forward (src/dit/flux.cpp:462-469,
 * src/dit/qwenimage21_forward.cpp:54-63) followed by brotensor::rope_apply
 * (src/dit/common.cpp:192-193, src/dit/qwenimage21_forward.cpp:584-585) in
 * one pass over the tensor.
 *   x, out : (rows, num_heads*head_dim), dtype BF16/F16, may alias;
 *   gain   : head_dim values of gain_dtype (F32, or the tensor dtype), or
 *            NULL to skip the norm;
 *   cos, sin : FP32 (table_rows, head_dim/2) tables, or both NULL to skip
 *            the rotation; row r of x uses table row (rope_row0 + r).
 * Up to BDATTN_MAX_NORM_JOBS independent jobs run in one launch (the four
 * norms of a Flux double-stream block).
 */
#define BDATTN_MAX_NORM_JOBS 4
typedef struct bdattn_norm_rope_job {
    const void* x;
    void* out;
    int rows;
    long long x_ld;
    long long out_ld;
    const void* gain;
    int gain_dtype;
    const float* cos;
    const float* sin;
    int rope_row0;
} bdattn_norm_rope_job;

int bdattn_rmsnorm_rope(const bdattn_norm_rope_job* jobs, int n_jobs, int dtype, int num_heads,
                        int head_dim, float eps, int pair_mode, bdattn_stream_t stream);

/* ------------------------------------------------------- RoPE tables
 * FP32 cos/sin tables (rows, head_dim/2) built on the device, replacing the
 * host loops + upload the reference runs every forward.
 *
 * bdattn_rope_tables_flux replaces dit::build_axial_rope_tables
 * (src/dit/common.cpp:116-184, called at src/dit/flux.cpp:760): rows =
 * txt_len + hp*wp; text rows are the identity rotation; image token (i, j)
 * sits at axial position (0, i, j); axis a owns axes_dims[a]/2 pairs with
 * omega = theta^(-2p/axes_dims[a]).  Errors keep the reference's messages
 * ("build_axial_rope_tables: axes_dims_rope must sum to head_dim").
 *
 * bdattn_rope_tables_qwen replaces
 * QwenImage21Transformer2DModel::build_rope_tables_
 * (src/dit/qwenimage21_forward.cpp:124-200): a running position walks the
 * prefix segments and then the (hp, wp) target image; a text token sits at
 * (p, p, p); an image block freezes the frame axis at p, centres its grid on
 * zero and advances p by max(h, w).  bdattn_rope_rows_qwen returns the row
 * count of that table (host-only helper).
 */
typedef struct bdattn_rope_segment {
    int kind;      /* 0 = text (n_tokens), 1 = image (h x w) */
    int n_tokens;
    int h;
    int w;
} bdattn_rope_segment;

int bdattn_rope_tables_flux(int txt_len, int hp, int wp, int head_dim, const int* axes_dims,
                            int n_axes, float theta, float* cos, float* sin,
                            bdattn_stream_t stream);

int bdattn_rope_rows_qwen(const bdattn_rope_segment* prefix, int n_prefix, int hp, int wp);

int bdattn_rope_tables_qwen(const bdattn_rope_segment* prefix, int n_prefix, int hp, int wp,
                            int head_dim, const int* axes_dims3, float theta, float* cos,
                            float* sin, bdattn_stream_t stream);

/* ------------------------------------------------ ReLU linear attention
 * Sana self-attention core.  Replaces the op sequence of
 * SanaDenoiser::self_attention_ (src/dit/sana.cpp:521-586; FP32 statement of
 * the same math at 470-520):
 *   per head h:  [S; z] = [V_h; 1] relu(K_h)^T,
 *                out_h  = (S relu(Q_h)) / (z relu(Q_h) + eps).
 *   q, k, v, out : channel-major (num_heads*head_dim, n_tokens), row stride
 *                  ld, `batch` items batch_stride apart; head_dim == 32
 *                  (src/dit/sana.cpp:176-178);
 *   sz_in  : optional FP32 (batch, num_heads, head_dim+1, head_dim) state
 *            added with weight w_in before the query read (inject seam,
 *            src/dit/sana.cpp:550-559);
 *   sz_out : optional FP32 state output taken before injection (capture
 *            seam).
 * One thread-block cluster per (batch, head) reduces the state through
 * distributed shared memory, so the operator needs no scratch memory.
 */
int bdattn_linear_attn_relu_fwd(const void* q, const void* k, const void* v, void* out, int dtype,
                                int batch, int num_heads, int head_dim, int n_tokens,
                                long long ld, long long batch_stride, float eps,
                                const float* sz_in, float w_in, float* sz_out,
                                bdattn_stream_t stream);

/* -------------------------------------------------- SD1.5 attention block
 * Fused Q/K/V projection + multi-head attention + output projection.
 *
 * bdattn_qkvo_fwd replaces brotensor::flash_attention_qkvo_forward
 * (src/unet_blocks.cpp:264-271 self-attention, 320-327 cross-attention with
 * ctx) and, when k_cached / v_cached are given,
 * brotensor::flash_attention_q_with_kv_cached_forward
 * (src/unet_blocks.cpp:302-307).  bdattn_project_kv replaces
 * brotensor::flash_attention_project_kv (src/unet.cpp:476-480), which fills the
 * per-prompt cross-attention K/V cache.
 *   x (x_rows, x_cols); ctx (ctx_rows, ctx_cols) or NULL (keys from x);
 *   wq (inner_dim, x_cols); wk, wv (inner_dim, ctx_cols or x_cols);
 *   wo (out_cols, inner_dim); biases have one value per output feature, the
 *   tensor dtype, and may be NULL; out (x_rows, out_cols).
 * Weights are dense row-major (out_features, in_features).  Heads of 40 or
 * 80 columns are projected straight into a 64 / 128-wide padded layout in the
 * workspace so that the attention core runs on the tcgen05 kernel.
 * The workspace (device memory, 256-byte aligned, size from
 * bdattn_qkvo_workspace_bytes) holds Q, K, V and the attention output
 * between the three steps; the call does not allocate.
 */
typedef struct bdattn_qkvo_params {
    int dtype;
    int num_heads;
    int inner_dim;          /* num_heads * head_dim */
    int causal;
    const void* x;
    int x_rows;
    int x_cols;
    long long x_ld;
    const void* ctx;        /* NULL: self-attention */
    int ctx_rows;
    int ctx_cols;
    long long ctx_ld;
    const void* wq;
    const void* bq;
    const void* wk;
    const void* bk;
    const void* wv;
    const void* bv;
    const void* wo;
    const void* bo;
    const void* k_cached;   /* (kv_rows, inner_dim) pre-projected keys, or NULL */
    const void* v_cached;
    int kv_rows;
    long long k_ld;
    long long v_ld;
    const float* key_mask;  /* Lk floats, 1 = valid; or NULL */
    void* out;
    int out_cols;           /* 0 => inner_dim */
    long long out_ld;       /* 0 => out_cols */
    void* workspace;
    size_t workspace_bytes;
} bdattn_qkvo_params;

size_t bdattn_qkvo_workspace_bytes(int q_rows, int kv_rows, int num_heads, int head_dim);

int bdattn_qkvo_fwd(const bdattn_qkvo_params* p, bdattn_stream_t stream);

int bdattn_project_kv(const void* ctx, int ctx_rows, int ctx_cols, long long ctx_ld, const void* wk,
                      const void* bk, const void* wv, const void* bv, void* k_out, void* v_out,
                      long long kv_ld, int inner_dim, int dtype, bdattn_stream_t stream);

/* bdattn_qkvo_fwd_static has no counterpart in the reference.  It is
 * bdattn_qkvo_fwd for callers that are not able to hand over scratch memory
 * because they may not allocate any: a plugin inside a host application that
 * has given all device memory to its own pool and forbids cudaMalloc from
 * plugins, or a latency-critical loop where cudaMalloc / cudaFree are banned
 * because they synchronise the device.  The scratch is a fixed array inside
 * the library's device image instead: p->workspace and p->workspace_bytes are
 * ignored, inputs and outputs are still the caller's.
 *   - Capacity: bdattn_qkvo_static_capacity() bytes (16 MiB; every SD1.5
 *     attention call at 512 px fits, the largest needs 14.5 MiB).  A call
 *     whose bdattn_qkvo_workspace_bytes() exceeds it fails with a message
 *     that names both sizes.  Every GPU that loads the library keeps these
 *     16 MiB reserved until the process exits.
 *   - The call itself makes no cudaMalloc / cudaFree and uses no allocating
 *     library routine.  The first call on a device looks up the array's device
 *     address (once per device); make that first call before starting any
 *     stream capture.
 *   - All calls on a device share the one array and it keeps what the last
 *     call left in it.  Nothing in it has to start at zero: each call writes
 *     every byte it later reads (the projections also write the zero padding
 *     of the heads).  Two calls whose kernels overlap on the GPU (different
 *     streams, no ordering between them) race on the array: order them.
 *   - The array's address is looked up once per device and kept for the life
 *     of the process.  Do not use this entry point across cudaDeviceReset or
 *     after the device's primary context has been destroyed and re-created:
 *     the library's device image is reloaded then and the kept address is
 *     stale.
 */
size_t bdattn_qkvo_static_capacity(void);

int bdattn_qkvo_fwd_static(const bdattn_qkvo_params* p, bdattn_stream_t stream);

/* ------------------------------------------- linear layer and fused ops
 * bdattn_linear_fwd: Y(M, N) = X(M, K) W(N, K)^T + bias, the operation behind
 * the reference's lin_ / linear_batched helpers around attention
 * (src/dit/flux.cpp:471-484,519-525; include/brodiffusion/detail/compute.h:52-63).
 *
 * bdattn_linear_geglu_fwd replaces brodiffusion::fused_linear_geglu
 * (include/brodiffusion/fused_transformer.h:32-35,
 * src/fused_transformer.cu:319-358): Y(rows, d_out) = a * gelu_exact(g) with
 * [a | g] = X W^T + b, W (2*d_out, d_in), b (2*d_out); all tensors dense.
 *
 * bdattn_add_inplace replaces brodiffusion::add_inplace_vec
 * (fused_transformer.h:52, src/fused_transformer.cu:430-451): Y[i] += X[i].
 *
 * bdattn_add_row_bias replaces brodiffusion::add_inplace_row_bias
 * (fused_transformer.h:59-60, src/fused_transformer.cu:413-428):
 * Y[i, j] += bias[j].
 */
int bdattn_linear_fwd(const void* x, const void* w, const void* bias, void* y, int dtype, int M,
                      int N, int K, long long ldx, long long ldw, long long ldy,
                      bdattn_stream_t stream);

/* Q/K/V projections with the per-head RMSNorm and RoPE fused into the GEMM
 * epilogue: one launch replaces lin_(to_q), lin_(to_k), lin_(to_v)
 * (src/dit/flux.cpp:471-473,590-592, src/dit/qwenimage21_forward.cpp:579-581),
 * the two headnorm calls (flux.cpp:474-475, qwenimage21_forward.cpp:582-583)
 * and the two rope_apply calls (src/dit/common.cpp:192-193,
 * qwenimage21_forward.cpp:584-585) of one token stream.
 *   x (rows, in_features); wq/wk/wv (num_heads*head_dim, in_features), biases
 *   optional; gain_q / gain_k: head_dim values (gain_dtype F32 or the tensor
 *   dtype) or NULL; cos/sin FP32 (>= rope_row0 + rows, head_dim/2) or NULL;
 *   q_out, k_out receive rope(rmsnorm(x W^T + b) * gain), v_out the plain
 *   projection; a NULL weight or output skips that projection.
 * head_dim 64 or 128: each GEMM tile is one head, so the norm and the rotation
 * are local to the thread that holds a token's row of the accumulator. */
typedef struct bdattn_qkv_proj_params {
    int dtype;
    int num_heads;
    int head_dim;
    const void* x;
    int rows;
    int in_features;
    long long x_ld;        /* 0 => in_features */
    const void* wq;
    const void* wk;
    const void* wv;
    const void* bq;
    const void* bk;
    const void* bv;
    const void* gain_q;
    const void* gain_k;
    int gain_dtype;
    float eps;
    const float* cos;
    const float* sin;
    int rope_row0;
    void* q_out;
    void* k_out;
    void* v_out;
    long long q_ld;        /* 0 => num_heads * head_dim */
    long long k_ld;
    long long v_ld;
} bdattn_qkv_proj_params;

int bdattn_qkv_norm_rope_fwd(const bdattn_qkv_proj_params* p, bdattn_stream_t stream);

int bdattn_linear_geglu_fwd(const void* x, const void* w, const void* bias, void* y, int dtype,
                            int rows, int d_in, int d_out, bdattn_stream_t stream);

int bdattn_add_inplace(void* y, const void* x, long long n, int dtype, bdattn_stream_t stream);

int bdattn_add_row_bias(void* y, const void* bias, int rows, int cols, long long ld, int dtype,
                        bdattn_stream_t stream);

/* Y = a*Y + b*X over n dense elements, in place: the device side of the
 * prefix KV cache operations QwenImage21PrefixCache::scale_kv (brotensor
 * scale_inplace, x = NULL and b = 0) and ::blend_from (brotensor axpby_inplace
 * with a = 1 - alpha, b = alpha) of src/dit/qwenimage21_hooks.cpp:79-124, one
 * call per cached K or V tensor.  Products and sum are rounded to FP32
 * separately, the result once to the storage type.  Asynchronous on the
 * stream (the reference follows the loop with sync_all; the caller syncs). */
int bdattn_axpby_inplace(void* y, const void* x, long long n, float a, float b, int dtype,
                         bdattn_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* BDATTN_H_ */
