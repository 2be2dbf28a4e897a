// Internal launch interfaces shared by the C-ABI layer and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace bdattn {

// Device-side arguments of the softmax-attention kernels.
struct SdpaDevArgs {
    int q_rows[2];
    int kv_rows[2];
    void* o[2];
    long long o_ld[2];
    long long o_bs[2];
    int q_ctas0;    // CTAs covering query segment 0
    int kv_tiles0;  // 128-key tiles covering key segment 0
    int kv_tiles;   // key tiles in total
    int mask_mode;
    int q_offset;   // Lk - Lq
    int hd_out;     // columns stored per head
    int kv_group;   // query heads per K/V head (grouped-query attention), >= 1
    // Query-side RMSNorm + RoPE done by the kernel on its Q tiles (all null: off).
    int q_fused;
    const void* q_gain[2];   // per query segment, hd_out values, or null
    int q_gain_is_f32;
    float q_eps;
    const float* q_cos;      // (rows, hd_out / 2) FP32, or null
    const float* q_sin;
    int q_rope_row0;
    const float* key_mask;
    const float* key_scale;
    const float* val_scale;
    float scale_log2;  // softmax scale * log2(e)
    // Traced / steered attention (hooks path): FP32 logit bias added to the scaled
    // scores of queries [bias_row0, bias_row0 + bias_rows) x keys [0, bias_cols),
    // and per-row softmax statistics (reference maximum in log2 units, row sum)
    // written to lse[((batch * heads + head) * lq_total + query) * 2 + {0, 1}].
    const float* bias;
    int bias_row0, bias_rows, bias_cols;
    long long bias_ld;
    float bias_mul;     // 1 / softmax scale: the bias in raw-score units
    float* lse;
    int lq_total;
    // Fused all-gather: every output vector is also stored to the same offset of
    // these peer buffers (other GPUs' copies of the output tensor), per segment.
    int n_peers;
    void* o_peer[2][8];
    // The same through the NVSwitch: when set, o_mc[seg] is the multicast address of
    // o[seg] (one multimem.st per vector reaches every GPU's copy, this one's
    // included) and neither o[] nor o_peer[] is stored to.
    void* o_mc[2];
};

struct SdpaLaunch {
    CUtensorMap tmQ[2], tmK[2], tmV[2];
    SdpaDevArgs args;
    int q_ctas;
    int num_heads;
    int batch;
    int head_dim;
    bool bf16;
};

cudaError_t launch_sdpa_tc05(const SdpaLaunch& L, cudaStream_t stream);

// General kernel (any head_dim that is a multiple of 8 up to 256).
struct SdpaGeneralArgs {
    const void* q[2];
    const void* k[2];
    const void* v[2];
    void* o[2];
    int q_rows[2];
    int kv_rows[2];
    long long q_ld[2], k_ld[2], v_ld[2], o_ld[2];
    long long q_bs[2], k_bs[2], v_bs[2], o_bs[2];
    int mask_mode;
    int q_offset;
    int head_dim;
    int kv_group;   // query heads per K/V head, >= 1
    const float* key_mask;
    const float* key_scale;
    const float* val_scale;
    float scale;
};
cudaError_t launch_sdpa_general(const SdpaGeneralArgs& a, int num_heads, int batch, bool bf16,
                                cudaStream_t stream);

// Head-averaged attention map of a query-row range x leading key range.
struct AttnMapArgs {
    const void* q[2];
    const void* k[2];
    int q_rows[2], kv_rows[2];
    long long q_ld[2], k_ld[2];
    int num_heads, head_dim;
    float scale_log2;
    const float* lse;       // (heads, lq_total, 2)
    int lq_total;
    const float* bias;
    int bias_row0, bias_rows, bias_cols;
    long long bias_ld;
    float* map;             // (map_rows, map_cols) FP32
    int map_row0, map_rows, map_cols;
    long long map_ld;
    // The visibility rules the attention kernel applied, so that the map agrees
    // with the output: a masked key has weight 0, a scaled key a scaled score.
    int mask_mode;          // 1: key j visible to query i iff j <= i + q_offset
    int q_offset;
    const float* key_mask;  // Lk floats, 0 = masked; or null
    const float* key_scale; // Lk floats or null
};
cudaError_t launch_attn_map(const AttnMapArgs& a, bool bf16, cudaStream_t stream);

// Per-head RMSNorm + RoPE.
struct NormRopeJobDev {
    const void* x;
    void* out;
    int rows;
    long long x_ld;
    long long out_ld;
    const void* gain;
    int gain_is_f32;
    const float* cos;
    const float* sin;
    int rope_row0;
};
struct NormRopeArgs {
    NormRopeJobDev job[4];
    int n_jobs;
    int num_heads;
    int head_dim;
    float eps;
    int pair_mode;
};
cudaError_t launch_norm_rope(const NormRopeArgs& a, bool bf16, cudaStream_t stream);

// Sana ReLU linear attention.
struct LinearAttnArgs {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    int batch, num_heads, n_tokens;
    long long ld, batch_stride;
    float eps;
    const float* sz_in;
    float w_in;
    float* sz_out;
    int stages;   // ring items of 16 KB per CTA (3: two CTAs per SM, up to 8: one)
};
cudaError_t launch_linear_attn(const LinearAttnArgs& a, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                               const CUtensorMap& tmV, const CUtensorMap& tmO, int cluster_size,
                               cudaStream_t stream);

// Linear layers (tcgen05 GEMM), up to three problems per launch.
struct GemmProblem {
    int M, N, K;
    void* C;
    long long ldc;
    const void* bias;   // N values of the output dtype, or null
    int tiles_m, tiles_n;
    int n_tile;         // MMA N (multiple of 16, <= 128) = rows of the B box
    int n_step;         // weight rows between tile starts
    int n_valid;        // columns of a tile that carry results
    int c_step;         // output columns between tile starts
    int c_fill;         // output columns written per tile (zeros beyond n_valid)
    int geglu_offset;   // 0, or D_out
    // Per-head RMSNorm + RoPE epilogue (head tiles with n_tile == head_dim only):
    const void* gain;   // head_dim values, or null
    int gain_is_f32;
    float eps;
    const float* cos;   // (rows, head_dim / 2) tables, or null
    const float* sin;
    int rope_row0;
    int norm_rope;      // 1: run the per-head epilogue
};
struct GemmArgs {
    GemmProblem p[3];
    int n_tile_max;   // largest n_tile of the launch: sizes the shared-memory stages
    int any_geglu;
    int stages;
};
struct GemmLaunch {
    CUtensorMap tmA[3], tmB[3];
    CUtensorMap tmBw[3];   // weight maps with 256-row boxes (wide-tile kernel), valid where wide[i]
    bool wide[3];          // problem i can run as 128 x 256 tiles
    GemmArgs args;
    int n_problems;
    bool bf16;
};
cudaError_t launch_gemm_tc05(const GemmLaunch& L, cudaStream_t stream);
// Persistent 128 x 256-tile kernel; every problem of the launch must have wide[i] set.
cudaError_t launch_gemm_wide(const GemmLaunch& L, cudaStream_t stream);
int gemm_wide_tiles(const GemmLaunch& L);
// Picks the wide-tile kernel when every problem allows it and there is at least
// one wide tile per SM, the one-tile-per-CTA kernel otherwise.
cudaError_t launch_gemm(const GemmLaunch& L, cudaStream_t stream);

// Elementwise helpers.
cudaError_t launch_add_inplace(void* y, const void* x, long long n, bool bf16, cudaStream_t stream);
cudaError_t launch_axpby_inplace(void* y, const void* x, long long n, float a, float b, bool bf16,
                                 cudaStream_t stream);
cudaError_t launch_add_row_bias(void* y, const void* bias, long long rows, long long cols, long long ld,
                                bool bf16, cudaStream_t stream);
cudaError_t launch_pad_heads(const void* src, void* dst, int rows, int num_heads, int hd, int hd_pad,
                             long long src_ld, cudaStream_t stream);

// Device-side RoPE table build.
constexpr int kMaxRopeSegments = 64;
struct RopeTableArgs {
    int flux;      // 1: Flux rule (text identity, image (0, i, j)); 0: Qwen-Image running position
    int rows;
    int half;
    int n_axes;
    int axes[4];
    float theta;
    int n_seg;
    int seg_kind[kMaxRopeSegments];   // 0 text, 1 image
    int seg_row0[kMaxRopeSegments];
    int seg_pos0[kMaxRopeSegments];   // running position at the segment start
    int seg_h[kMaxRopeSegments];
    int seg_w[kMaxRopeSegments];
    float* cos_out;
    float* sin_out;
};
cudaError_t launch_rope_tables(const RopeTableArgs& a, cudaStream_t stream);

}  // namespace bdattn
