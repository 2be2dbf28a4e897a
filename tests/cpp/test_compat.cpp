// Host-mirror test in the style of the reference's own tests (plain
// executable, CHECK macro, exit code; tests/test_fused_parity.cpp,
// tests/test_flux_blocks.cpp): the brotensor / brodiffusion entry points of
// include/brotensor/ops.h, include/brodiffusion/dit/common.h and
// include/brodiffusion/fused_transformer.h against the CPU oracle.
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "brodiffusion/dit/common.h"
#include "brodiffusion/fused_transformer.h"

extern "C" {   // oracle/oracle.cpp (test infrastructure)
int bdo_flux_rope_tables(int, int, int, int, const int*, int, float, float*, float*);
void bdo_rope_apply(const float*, int, int, int, const float*, const float*, int, float*);
void bdo_sdpa(const float*, int, const float*, const float*, int, int, int, int, const int*, const int*,
              const float*, const float*, int, int, const int*, int, int, int, float*, float*);
void bdo_linear(const float*, const float*, const float*, int, int, int, int, float*);
void bdo_linear_geglu(const float*, const float*, const float*, int, int, int, int, float*);
}

namespace bt = brotensor;
namespace bd = brodiffusion;

static int g_failures = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("  CHECK failed: %s (line %d)\n", #cond, __LINE__); ++g_failures; } } while (0)

// Deterministic values in [-scale, scale] + bias, canonicalised to the storage
// type so both sides consume identical inputs (tests/test_fused_parity.cpp:50-62).
static std::vector<float> gen(std::size_t n, std::uint64_t seed, float scale, bool bf16, float bias = 0.0f) {
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<float> d(-1.0f, 1.0f);
    std::vector<float> out(n);
    for (auto& v : out) {
        const float x = d(rng) * scale + bias;
        v = bf16 ? bt::bf16_bits_to_fp32(bt::fp32_to_bf16_bits(x)) : __half2float(__float2half(x));
    }
    return out;
}
static bt::Tensor gpu_t(const std::vector<float>& v, int r, int c, bt::Dtype dt) {
    std::vector<std::uint16_t> bits(v.size());
    for (std::size_t i = 0; i < v.size(); ++i) {
        if (dt == bt::Dtype::BF16) bits[i] = bt::fp32_to_bf16_bits(v[i]);
        else { __half h = __float2half(v[i]); bits[i] = *reinterpret_cast<std::uint16_t*>(&h); }
    }
    return bt::Tensor::from_host_bits(bits.data(), r, c, dt);
}
static std::vector<float> download(const bt::Tensor& t) {
    const auto raw = t.to_host_bytes();
    std::vector<float> out(t.size());
    if (t.dtype == bt::Dtype::FP32) { std::memcpy(out.data(), raw.data(), raw.size()); return out; }
    const auto* b = reinterpret_cast<const std::uint16_t*>(raw.data());
    for (std::size_t i = 0; i < out.size(); ++i) {
        if (t.dtype == bt::Dtype::BF16) out[i] = bt::bf16_bits_to_fp32(b[i]);
        else { __half h; *reinterpret_cast<std::uint16_t*>(&h) = b[i]; out[i] = __half2float(h); }
    }
    return out;
}
static void expect_parity(const char* label, const std::vector<float>& ref, const std::vector<float>& got,
                          float tol_rel, float tol_abs) {
    float err = 0, mag = 0; int bad = 0;
    CHECK(ref.size() == got.size());
    for (std::size_t i = 0; i < std::min(ref.size(), got.size()); ++i) {
        if (!std::isfinite(got[i])) { ++bad; continue; }
        err = std::max(err, std::fabs(ref[i] - got[i]));
        mag = std::max(mag, std::fabs(ref[i]));
    }
    const float bound = tol_rel * mag + tol_abs;
    std::printf("  %-34s err=%.5f ref=%.4f bound=%.5f%s\n", label, err, mag, bound, err <= bound ? "" : "  <-- OVER");
    CHECK(bad == 0); CHECK(mag > 0.0f); CHECK(err <= bound);
}

static void test_joint_attention(int txt, int hp, int wp, int nh, int hd, const std::vector<int>& axes, const char* label) {
    const int L = txt + hp * wp, D = nh * hd;
    const auto q = gen((std::size_t)L * D, 1, 1.0f, true), k = gen((std::size_t)L * D, 2, 1.0f, true),
               v = gen((std::size_t)L * D, 3, 1.0f, true);
    bd::dit::RopeTables tab = bd::dit::build_axial_rope_tables(txt, hp, wp, hd, axes);
    bt::Tensor Q = gpu_t(q, L, D, bt::Dtype::BF16), K = gpu_t(k, L, D, bt::Dtype::BF16), V = gpu_t(v, L, D, bt::Dtype::BF16);
    bt::Tensor out, out2, Qr, Kr;
    bd::dit::joint_attention(Q, K, V, tab.cos, tab.sin, hd, nh, out, Qr, Kr);
    bd::dit::joint_attention(Q, K, V, tab.cos, tab.sin, hd, nh, out2, Qr, Kr);
    const auto got = download(out), got2 = download(out2);
    CHECK(got == got2);   // two forwards are bit-identical (tests/test_flux_blocks.cpp determinism checks)
    // host path: same statements as dit::joint_attention_traced (src/dit/common.cpp:198-305)
    std::vector<float> cos((std::size_t)L * hd / 2), sin(cos.size()), qr(q.size()), kr(k.size()), ref(q.size());
    bdo_flux_rope_tables(txt, hp, wp, hd, axes.data(), (int)axes.size(), 10000.f, cos.data(), sin.data());
    bdo_rope_apply(q.data(), L, nh, hd, cos.data(), sin.data(), 0, qr.data());
    bdo_rope_apply(k.data(), L, nh, hd, cos.data(), sin.data(), 0, kr.data());
    bdo_sdpa(qr.data(), L, kr.data(), v.data(), L, nh, hd, 0, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, L, 1, 0,
             ref.data(), nullptr);
    // BF16 bound of the reference's fused-vs-traced check (tests/test_flux_blocks.cpp:283-300)
    expect_parity(label, ref, got, 0.0f, 1e-2f);
}

// dit::gqa_attention_masked (src/dit/common.cpp:331-377): the oracle widens the
// K/V heads as the reference does and runs plain attention on the result.
static void test_gqa(int L, int nq, int nkv, int hd, bool with_rope, bool with_mask, const char* label) {
    const int Dq = nq * hd, Dkv = nkv * hd, group = nq / nkv;
    const auto q = gen((std::size_t)L * Dq, 8101 + L, 1.0f, true), k = gen((std::size_t)L * Dkv, 8102 + L, 1.0f, true),
               v = gen((std::size_t)L * Dkv, 8103 + L, 1.0f, true);
    const std::vector<int> axes = hd == 128 ? std::vector<int>{16, 56, 56} : std::vector<int>{8, 28, 28};
    std::vector<float> rcos((std::size_t)L * hd / 2), rsin(rcos.size());
    // text rows rotate by the identity in the Flux tables; use image rows to exercise RoPE
    bdo_flux_rope_tables(0, 1, L, hd, axes.data(), 3, 10000.f, rcos.data(), rsin.data());
    std::vector<float> mask(L, 1.0f);
    if (with_mask) for (int i = 0; i < L; i += 3) mask[i] = 0.0f;
    std::vector<float> qr = q, kr = k;
    if (with_rope) {
        bdo_rope_apply(q.data(), L, nq, hd, rcos.data(), rsin.data(), 0, qr.data());
        bdo_rope_apply(k.data(), L, nkv, hd, rcos.data(), rsin.data(), 0, kr.data());
        for (auto& x : qr) x = bt::bf16_bits_to_fp32(bt::fp32_to_bf16_bits(x));
        for (auto& x : kr) x = bt::bf16_bits_to_fp32(bt::fp32_to_bf16_bits(x));
    }
    std::vector<float> krep((std::size_t)L * Dq), vrep(krep.size()), ref(krep.size());
    for (int r = 0; r < L; ++r)
        for (int h = 0; h < nq; ++h)
            for (int d = 0; d < hd; ++d) {
                krep[(std::size_t)r * Dq + h * hd + d] = kr[(std::size_t)r * Dkv + (h / group) * hd + d];
                vrep[(std::size_t)r * Dq + h * hd + d] = v[(std::size_t)r * Dkv + (h / group) * hd + d];
            }
    bdo_sdpa(qr.data(), L, krep.data(), vrep.data(), L, nq, hd, 0, nullptr, nullptr,
             with_mask ? mask.data() : nullptr, nullptr, 0, 0, nullptr, L, 1, 0, ref.data(), nullptr);

    bt::Tensor Q = gpu_t(q, L, Dq, bt::Dtype::BF16), K = gpu_t(k, L, Dkv, bt::Dtype::BF16),
               V = gpu_t(v, L, Dkv, bt::Dtype::BF16);
    bd::dit::RopeTables tab = bd::dit::build_axial_rope_tables(0, 1, L, hd, axes);
    float* d_mask = nullptr;
    CHECK(cudaMalloc(&d_mask, sizeof(float) * L) == cudaSuccess);
    CHECK(cudaMemcpy(d_mask, mask.data(), sizeof(float) * L, cudaMemcpyHostToDevice) == cudaSuccess);
    bt::Tensor out, Qr, Kr, Krep, Vrep;
    bd::dit::gqa_attention_masked(Q, K, V, with_rope ? &tab.cos : nullptr, with_rope ? &tab.sin : nullptr, hd, nq, nkv,
                                  with_mask ? d_mask : nullptr, out, Qr, Kr, Krep, Vrep);
    bt::sync_all();
    CHECK(Krep.data == nullptr && Vrep.data == nullptr);   // no widened copies
    expect_parity(label, ref, download(out), 0.0f, 1e-2f);
    cudaFree(d_mask);
}

static void test_geglu(int B, int D_in, int D_out, const char* label) {
    const auto x = gen((std::size_t)B * D_in, 21, 1.0f, false), w = gen((std::size_t)2 * D_out * D_in, 22, 0.1f, false),
               b = gen((std::size_t)2 * D_out, 23, 0.2f, false);
    bt::Tensor X = gpu_t(x, B, D_in, bt::Dtype::FP16), W = gpu_t(w, 2 * D_out, D_in, bt::Dtype::FP16),
               Bt = gpu_t(b, 2 * D_out, 1, bt::Dtype::FP16), Y;
    bd::fused_linear_geglu(X, W, Bt, Y);
    std::vector<float> ref((std::size_t)B * D_out);
    bdo_linear_geglu(x.data(), w.data(), b.data(), B, D_in, D_out, 0, ref.data());
    expect_parity(label, ref, download(Y), 0.01f, 0.008f);
}

static void test_adds() {
    for (auto rc : {std::pair<int, int>{10, 37}, {64, 64}}) {
        const auto y0 = gen((std::size_t)rc.first * rc.second, 31, 1.0f, false), x = gen(y0.size(), 32, 1.0f, false);
        bt::Tensor Y = gpu_t(y0, rc.first, rc.second, bt::Dtype::FP16), X = gpu_t(x, rc.first, rc.second, bt::Dtype::FP16);
        bd::add_inplace_vec(Y, X);
        std::vector<float> ref(y0.size());
        for (std::size_t i = 0; i < ref.size(); ++i) ref[i] = y0[i] + x[i];
        expect_parity("add_inplace_vec", ref, download(Y), 0.005f, 0.003f);
    }
    for (auto rc : {std::pair<int, int>{13, 29}, {48, 80}}) {
        const auto y0 = gen((std::size_t)rc.first * rc.second, 41, 1.0f, false), bias = gen(rc.second, 42, 1.0f, false);
        bt::Tensor Y = gpu_t(y0, rc.first, rc.second, bt::Dtype::FP16), Bs = gpu_t(bias, rc.second, 1, bt::Dtype::FP16);
        bd::add_inplace_row_bias(Y, Bs);
        std::vector<float> ref(y0.size());
        for (int i = 0; i < rc.first; ++i) for (int j = 0; j < rc.second; ++j) ref[(std::size_t)i * rc.second + j] = y0[(std::size_t)i * rc.second + j] + bias[j];
        expect_parity("add_inplace_row_bias", ref, download(Y), 0.005f, 0.003f);
    }
}

// QwenImage21PrefixCache::scale_kv / blend_from on one cached tensor
// (src/dit/qwenimage21_hooks.cpp:79-124): scale_inplace, then axpby_inplace.
static void test_prefix_cache_ops() {
    const int rows = 256, cols = 96;
    const auto y0 = gen((std::size_t)rows * cols, 61, 1.0f, true), x = gen(y0.size(), 62, 1.0f, true);
    bt::Tensor Y = gpu_t(y0, rows, cols, bt::Dtype::BF16), X = gpu_t(x, rows, cols, bt::Dtype::BF16);
    bt::scale_inplace(Y, 0.75f);
    bt::axpby_inplace(Y, X, 1.0f - 0.3f, 0.3f);
    std::vector<float> ref(y0.size());
    for (std::size_t i = 0; i < ref.size(); ++i) {
        const float s = bt::bf16_bits_to_fp32(bt::fp32_to_bf16_bits(0.75f * y0[i]));
        const volatile float p1 = (1.0f - 0.3f) * s, p2 = 0.3f * x[i];   // no contraction into an FMA
        ref[i] = bt::bf16_bits_to_fp32(bt::fp32_to_bf16_bits(p1 + p2));
    }
    const auto got = download(Y);
    CHECK(got == ref);   // products and sum rounded separately: bit-exact
}

static void test_unet_attention() {
    // SD1.5-shaped block, smaller token count: (512, 320), 8 heads x 40, ctx (77, 768)
    const int L = 512, C = 320, nh = 8, Lc = 77, Cc = 768;
    const auto x = gen((std::size_t)L * C, 51, 1.0f, false), ctx = gen((std::size_t)Lc * Cc, 52, 1.0f, false);
    const auto wq = gen((std::size_t)C * C, 53, 0.05f, false), wo = gen((std::size_t)C * C, 54, 0.05f, false),
               wk = gen((std::size_t)C * Cc, 55, 0.05f, false), wv = gen((std::size_t)C * Cc, 56, 0.05f, false),
               bo = gen(C, 57, 0.1f, false);
    bt::Tensor X = gpu_t(x, L, C, bt::Dtype::FP16), Ctx = gpu_t(ctx, Lc, Cc, bt::Dtype::FP16);
    bt::Tensor Wq = gpu_t(wq, C, C, bt::Dtype::FP16), Wo = gpu_t(wo, C, C, bt::Dtype::FP16),
               Wk = gpu_t(wk, C, Cc, bt::Dtype::FP16), Wv = gpu_t(wv, C, Cc, bt::Dtype::FP16), Bo = gpu_t(bo, C, 1, bt::Dtype::FP16);
    bt::Tensor out, K, V, out_c;
    bt::flash_attention_qkvo_forward(X, &Ctx, Wq, nullptr, Wk, nullptr, Wv, nullptr, Wo, &Bo, nullptr, nh, false, out);
    bt::flash_attention_project_kv(Ctx, Wk, nullptr, Wv, nullptr, K, V);
    bt::flash_attention_q_with_kv_cached_forward(X, K, V, Wq, nullptr, Wo, &Bo, nullptr, nh, false, out_c);
    std::vector<float> q((std::size_t)L * C), kk((std::size_t)Lc * C), vv(kk.size()), o(q.size()), ref(q.size());
    bdo_linear(x.data(), wq.data(), nullptr, L, C, C, 0, q.data());
    bdo_linear(ctx.data(), wk.data(), nullptr, Lc, C, Cc, 0, kk.data());
    bdo_linear(ctx.data(), wv.data(), nullptr, Lc, C, Cc, 0, vv.data());
    bdo_sdpa(q.data(), L, kk.data(), vv.data(), Lc, nh, C / nh, 0, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, L, 1, 0, o.data(), nullptr);
    bdo_linear(o.data(), wo.data(), bo.data(), L, C, C, 0, ref.data());
    // trace-vs-fast bound of the reference's U-Net test (tests/test_unet.cpp:379-409): 0.05
    expect_parity("cross-attn qkvo", ref, download(out), 0.0f, 0.05f);
    expect_parity("cross-attn cached K/V", ref, download(out_c), 0.0f, 0.05f);
}

// dit::joint_attention_traced (src/dit/common.cpp:198-329): output, head-averaged
// (L, L) map and the image->text logit bias, against the oracle's statement of the
// same host loop.  Bounds: BF16 output 1e-2 (tests/test_flux_blocks.cpp:283-300);
// map rows are non-negative and sum to one (tests/test_flux_blocks.cpp:268-281).
static void test_joint_attention_traced(int txt, int hp, int wp, int nh, int hd, const std::vector<int>& axes, const char* label) {
    const int L = txt + hp * wp, D = nh * hd, img = hp * wp;
    const auto q = gen((std::size_t)L * D, 71, 1.0f, true), k = gen((std::size_t)L * D, 72, 1.0f, true),
               v = gen((std::size_t)L * D, 73, 1.0f, true);
    std::vector<float> bias((std::size_t)img * txt, 0.0f);
    for (int r = 0; r < img; ++r) bias[(std::size_t)r * txt + 1] = 1.5f;     // steer every image row to text token 1
    bd::dit::RopeTables tab = bd::dit::build_axial_rope_tables(txt, hp, wp, hd, axes);
    bt::Tensor Q = gpu_t(q, L, D, bt::Dtype::BF16), K = gpu_t(k, L, D, bt::Dtype::BF16), V = gpu_t(v, L, D, bt::Dtype::BF16);
    bt::Tensor B = bt::Tensor::from_host(bias.data(), img, txt);
    bt::Tensor out, avg, out0, avg0, Qr, Kr;
    bd::dit::joint_attention_traced(Q, K, V, tab.cos, tab.sin, hd, nh, out, avg, Qr, Kr, txt, &B);
    bd::dit::joint_attention_traced(Q, K, V, tab.cos, tab.sin, hd, nh, out0, avg0, Qr, Kr);
    std::vector<float> cos((std::size_t)L * hd / 2), sin(cos.size()), qr(q.size()), kr(k.size()), ref(q.size()),
        ref_avg((std::size_t)L * L);
    bdo_flux_rope_tables(txt, hp, wp, hd, axes.data(), (int)axes.size(), 10000.f, cos.data(), sin.data());
    bdo_rope_apply(q.data(), L, nh, hd, cos.data(), sin.data(), 0, qr.data());
    bdo_rope_apply(k.data(), L, nh, hd, cos.data(), sin.data(), 0, kr.data());
    bdo_sdpa(qr.data(), L, kr.data(), v.data(), L, nh, hd, 0, nullptr, nullptr, nullptr, bias.data(), txt, txt, nullptr, L, 1, 0,
             ref.data(), ref_avg.data());
    expect_parity(label, ref, download(out), 0.0f, 1e-2f);
    const auto m = download(avg), m0 = download(avg0);
    expect_parity("  head-averaged map", ref_avg, m, 0.0f, 5e-3f);
    float worst = 0.0f, steered = 0.0f, plain = 0.0f; bool neg = false;
    for (int r = 0; r < L; ++r) {
        float sum = 0.0f;
        for (int c = 0; c < L; ++c) { sum += m[(std::size_t)r * L + c]; neg = neg || m[(std::size_t)r * L + c] < 0.0f; }
        worst = std::max(worst, std::fabs(sum - 1.0f));
        if (r >= txt) { steered += m[(std::size_t)r * L + 1]; plain += m0[(std::size_t)r * L + 1]; }
    }
    CHECK(!neg); CHECK(worst < 2e-2f);
    CHECK(steered > plain);                 // the bias moves weight onto the steered text token
    bool threw = false;
    bt::Tensor bad = bt::Tensor::from_host(bias.data(), 1, txt);
    try { bd::dit::joint_attention_traced(Q, K, V, tab.cos, tab.sin, hd, nh, out, avg, Qr, Kr, txt, &bad); }
    catch (const std::runtime_error& e) { threw = std::string(e.what()).find("image_text_bias must be (img_len, txt_len)") != std::string::npos; }
    CHECK(threw);
}

// brotensor::cross_attention_forward_with_attn (src/unet_blocks.cpp:282-290): the
// traced SD1.5 cross-attention; the output bias is added afterwards by the caller.
static void test_unet_traced_attention() {
    const int L = 256, C = 320, nh = 8, Lc = 77, Cc = 768;
    const auto x = gen((std::size_t)L * C, 81, 1.0f, false), ctx = gen((std::size_t)Lc * Cc, 82, 1.0f, false);
    const auto wq = gen((std::size_t)C * C, 83, 0.05f, false), wo = gen((std::size_t)C * C, 84, 0.05f, false),
               wk = gen((std::size_t)C * Cc, 85, 0.05f, false), wv = gen((std::size_t)C * Cc, 86, 0.05f, false),
               lb = gen((std::size_t)L * Lc, 87, 0.5f, false);
    bt::Tensor X = gpu_t(x, L, C, bt::Dtype::FP16), Ctx = gpu_t(ctx, Lc, Cc, bt::Dtype::FP16);
    bt::Tensor Wq = gpu_t(wq, C, C, bt::Dtype::FP16), Wo = gpu_t(wo, C, C, bt::Dtype::FP16),
               Wk = gpu_t(wk, C, Cc, bt::Dtype::FP16), Wv = gpu_t(wv, C, Cc, bt::Dtype::FP16);
    bt::Tensor LB = bt::Tensor::from_host(lb.data(), L, Lc);
    bt::Tensor out, avg;
    bt::cross_attention_forward_with_attn(X, Ctx, Wq, Wk, Wv, Wo, nullptr, &LB, nh, out, avg);
    std::vector<float> q((std::size_t)L * C), kk((std::size_t)Lc * C), vv(kk.size()), o(q.size()), ref(q.size()),
        ref_avg((std::size_t)L * Lc);
    bdo_linear(x.data(), wq.data(), nullptr, L, C, C, 0, q.data());
    bdo_linear(ctx.data(), wk.data(), nullptr, Lc, C, Cc, 0, kk.data());
    bdo_linear(ctx.data(), wv.data(), nullptr, Lc, C, Cc, 0, vv.data());
    bdo_sdpa(q.data(), L, kk.data(), vv.data(), Lc, nh, C / nh, 0, nullptr, nullptr, nullptr, lb.data(), 0, Lc, nullptr, L, 1, 0,
             o.data(), ref_avg.data());
    bdo_linear(o.data(), wo.data(), nullptr, L, C, C, 0, ref.data());
    expect_parity("traced cross-attn output", ref, download(out), 0.0f, 0.05f);   // tests/test_unet.cpp:379-409
    const auto m = download(avg);
    expect_parity("traced cross-attn map", ref_avg, m, 0.0f, 1e-2f);
    float worst = 0.0f;
    for (int r = 0; r < L; ++r) { float sum = 0.0f; for (int c = 0; c < Lc; ++c) sum += m[(std::size_t)r * Lc + c]; worst = std::max(worst, std::fabs(sum - 1.0f)); }
    CHECK(worst < 0.05f);                                                          // tests/test_unet.cpp:487-500
}

// brotensor::matmul_abt as Sana calls it (src/dit/sana.cpp:441-443):
// q (D, N) = W (D, D) . x_mod (N, D)^T, channel-major output, no bias.
static void test_matmul_abt(int D, int N, const char* label) {
    const auto w = gen((std::size_t)D * D, 91, 0.02f, true), x = gen((std::size_t)N * D, 92, 1.0f, true);
    bt::Tensor W = gpu_t(w, D, D, bt::Dtype::BF16), X = gpu_t(x, N, D, bt::Dtype::BF16), Cm;
    bt::matmul_abt(W, X, Cm, 1, D, N, D, 0, 0, 0, nullptr, 0);
    CHECK(Cm.rows == D && Cm.cols == N);
    std::vector<float> ref((std::size_t)D * N);
    bdo_linear(w.data(), x.data(), nullptr, D, N, D, 0, ref.data());     // rows of W against rows of x_mod
    expect_parity(label, ref, download(Cm), 0.01f, 0.004f);
}

static void test_refusals() {
    bt::Tensor cpu; cpu.device = bt::Device::cpu(); cpu.rows = 4; cpu.cols = 8; cpu.dtype = bt::Dtype::FP16;
    bt::Tensor y;
    bool threw = false;
    try { bd::fused_linear_geglu(cpu, cpu, cpu, y); } catch (const std::runtime_error& e) { threw = std::string(e.what()).find("fused_linear_geglu:") == 0; }
    CHECK(threw);
    // FP32 tensors are refused, as in src/fused_transformer.cu:323-326
    std::vector<float> z(64, 0.f);
    bt::Tensor f32 = bt::Tensor::from_host(z.data(), 8, 8), b32 = bt::Tensor::from_host(z.data(), 8, 1);
    threw = false;
    try { bd::fused_linear_geglu(f32, f32, b32, y); } catch (const std::runtime_error& e) { threw = std::string(e.what()).find("fused_linear_geglu:") == 0; }
    CHECK(threw);
    threw = false;
    try { bd::dit::build_axial_rope_tables(1, 2, 2, 8, {2, 2, 2}); } catch (const std::runtime_error& e) {
        threw = std::string(e.what()) == "build_axial_rope_tables: axes_dims_rope must sum to head_dim";
    }
    CHECK(threw);
}

int main() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { std::printf("test_compat: no GPU\n"); return 2; }
    try {
        std::printf("test_compat: host mirror over libbdattn\n");
        test_joint_attention(3, 4, 4, 2, 8, {2, 2, 4}, "joint_attention tiny (2x8)");       // tests/test_flux_blocks.cpp:480-507
        test_joint_attention(40, 16, 16, 4, 128, {16, 56, 56}, "joint_attention 4x128");
        test_gqa(200, 8, 2, 128, true, true, "gqa 8q/2kv x128 rope+mask");
        test_gqa(150, 6, 3, 64, false, false, "gqa 6q/3kv x64");
        test_geglu(40, 64, 48, "geglu B40 64->48");
        test_geglu(128, 128, 96, "geglu B128 128->96");
        test_adds();
        test_prefix_cache_ops();
        test_unet_attention();
        test_joint_attention_traced(3, 4, 4, 2, 8, {2, 2, 4}, "joint_attention_traced tiny (2x8)");   // tests/test_flux_blocks.cpp:480-507
        test_joint_attention_traced(24, 12, 10, 4, 128, {16, 56, 56}, "joint_attention_traced 4x128");
        test_unet_traced_attention();
        test_matmul_abt(2240, 256, "matmul_abt Sana 2240 x 256 tokens");
        test_refusals();
        int status = 0;
        CHECK(bdattn_device_status(&status, 1) == 0 && status == 0);
    } catch (const std::exception& e) {
        std::printf("test_compat: exception: %s\n", e.what());
        ++g_failures;
    }
    std::printf("test_compat: %s (%d failure%s)\n", g_failures ? "FAILED" : "ok", g_failures, g_failures == 1 ? "" : "s");
    return g_failures ? 1 : 0;
}
