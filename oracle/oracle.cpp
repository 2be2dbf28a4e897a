// CPU oracle for the denoiser-attention hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++ with no dependencies, the arithmetic of the
// brodiffusion attention path so that the CUDA kernels can be checked against
// it.  It is never linked into, imported by, or called from the product
// library; only the test-suite, the smoke check and the bench's CPU-baseline
// leg load it.
//
// PARITY PIN STATUS
//   * softmax attention core  : follows brodiffusion's own host loop
//     dit::joint_attention_traced (src/dit/common.cpp:246-305) statement by
//     statement (double scores, stable softmax, float P.V accumulation).
//     PINNED: that source file is compiled unmodified (Makefile target
//     _ref/libref.so, host-only brotensor stand-in in ref_stub/) and
//     tests/test_oracle_pin.py holds bdo_sdpa to it: head-averaged maps
//     bit-identical, outputs within one FP32 ulp; its outputs on seeded inputs
//     are committed as tests/golden/ref_pin.npz.
//   * Flux RoPE tables        : follow src/dit/common.cpp:116-184.  PINNED the
//     same way, bit-identical.
//   * Qwen-Image RoPE tables  : follow src/dit/qwenimage21_forward.cpp:136-196
//     (a member function of the model class; not compilable on its own).
//   * ReLU linear attention   : follows src/dit/sana.cpp:470-520.
//   * SD1.5 attention block   : follows src/unet_blocks.cpp:253-330.
//   * GEGLU                   : follows src/fused_transformer.cu:89-92,275-282.
//   * rms_norm_forward and rope_apply live in the external brotensor library
//     (fetched by the reference at an unpinned revision; source not
//     available).  They are restated from their standard definitions and the
//     reference's call sites: "parity unpinned" for those two ops.  The rotary
//     pair convention is therefore a runtime switch (interleaved by default).
//   The reference's tests hold no golden numbers for this path (they are all
//   relational), so the absolute values are cross-checked against an
//   independent PyTorch FP32 CPU implementation in tests/golden/.
//
// All tensors are dense row-major float32 on the host.  Heads are column
// blocks: head h of an (L, nh*hd) tensor is columns [h*hd, (h+1)*hd).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

int resolve_threads(int n) {
    if (n > 0) return n;
    unsigned hc = std::thread::hardware_concurrency();
    return hc == 0 ? 1 : static_cast<int>(hc);
}

// Dynamic row-parallel loop: fn(i) for i in [0, n).
template <class F>
void parallel_for(int n, int nthreads, F fn) {
    nthreads = std::min(resolve_threads(nthreads), std::max(n, 1));
    if (nthreads <= 1) {
        for (int i = 0; i < n; ++i) fn(i);
        return;
    }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    pool.reserve(static_cast<std::size_t>(nthreads));
    for (int t = 0; t < nthreads; ++t) {
        pool.emplace_back([&] {
            for (;;) {
                int i = next.fetch_add(1);
                if (i >= n) break;
                fn(i);
            }
        });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

int bdo_hardware_threads(void) { return resolve_threads(0); }

// ---------------------------------------------------------------------------
// Flux axial RoPE tables.  src/dit/common.cpp:116-184.
// cos/sin are (txt_len + hp*wp, head_dim/2).  Text rows are the identity
// rotation; image token (i, j) sits at axial position (0, i, j); axis a owns
// the pair range [off_a, off_a + axes[a]/2) with omega = theta^(-2p/axes[a]).
// Returns the row count, or -1 on a bad argument.
int bdo_flux_rope_tables(int txt_len, int hp, int wp, int head_dim,
                         const int* axes, int n_axes, float theta,
                         float* cos_out, float* sin_out) {
    if (head_dim % 2 != 0) return -1;
    int sum = 0;
    for (int a = 0; a < n_axes; ++a) sum += axes[a];
    if (sum != head_dim) return -1;
    const int half = head_dim / 2;
    const int L = txt_len + hp * wp;
    for (std::size_t i = 0; i < static_cast<std::size_t>(L) * half; ++i) {
        cos_out[i] = 1.0f;
        sin_out[i] = 0.0f;
    }
    std::vector<int> off(static_cast<std::size_t>(n_axes));
    {
        int o = 0;
        for (int a = 0; a < n_axes; ++a) { off[a] = o; o += axes[a] / 2; }
    }
    for (int i = 0; i < hp; ++i) {
        for (int j = 0; j < wp; ++j) {
            const std::size_t row = static_cast<std::size_t>(txt_len) +
                                    static_cast<std::size_t>(i) * wp + j;
            const int pos[3] = {0, i, j};
            for (int a = 0; a < n_axes && a < 3; ++a) {
                const int cnt = axes[a] / 2;
                for (int p = 0; p < cnt; ++p) {
                    const double omega =
                        1.0 / std::pow(static_cast<double>(theta),
                                       (2.0 * p) / static_cast<double>(axes[a]));
                    const double ang = static_cast<double>(pos[a]) * omega;
                    const std::size_t idx = row * half + off[a] + p;
                    cos_out[idx] = static_cast<float>(std::cos(ang));
                    sin_out[idx] = static_cast<float>(std::sin(ang));
                }
            }
        }
    }
    return L;
}

// ---------------------------------------------------------------------------
// Qwen-Image 3-axis RoPE tables.  src/dit/qwenimage21_forward.cpp:136-196.
// A running position p walks the sequence: a text token sits at (p, p, p) and
// advances p; an image block freezes the frame axis at p, centres its h/w
// grid on zero (first index -(n - n/2)), then advances p by max(h, w).  The
// prefix segments are followed by the (hp, wp) target image.
// seg_kind: 0 = text (seg_n tokens), 1 = image (seg_h x seg_w tokens).
// Pass cos_out == nullptr to only count rows.  Returns the row count.
int bdo_qwen_rope_tables(const int* seg_kind, const int* seg_n,
                         const int* seg_h, const int* seg_w, int n_seg,
                         int hp, int wp, int head_dim, const int* axes3,
                         float theta, float* cos_out, float* sin_out) {
    const int half = head_dim / 2;
    std::vector<int> ax[3];
    int pos = 0;
    auto add_text = [&](int n) {
        for (int i = 0; i < n; ++i) {
            ax[0].push_back(pos); ax[1].push_back(pos); ax[2].push_back(pos);
            ++pos;
        }
    };
    auto add_image = [&](int h, int w) {
        const int frame = pos;
        const int h0 = -(h - h / 2);
        const int w0 = -(w - w / 2);
        for (int i = 0; i < h; ++i)
            for (int j = 0; j < w; ++j) {
                ax[0].push_back(frame);
                ax[1].push_back(h0 + i);
                ax[2].push_back(w0 + j);
            }
        pos += (h > w ? h : w);
    };
    for (int s = 0; s < n_seg; ++s) {
        if (seg_kind[s] == 0) add_text(seg_n[s]);
        else add_image(seg_h[s], seg_w[s]);
    }
    add_image(hp, wp);
    const int L = static_cast<int>(ax[0].size());
    if (cos_out == nullptr || sin_out == nullptr) return L;
    if (axes3[0] / 2 + axes3[1] / 2 + axes3[2] / 2 != half) return -1;

    std::vector<double> freqs(static_cast<std::size_t>(half));
    std::vector<int> pair_axis(static_cast<std::size_t>(half));
    {
        int o = 0;
        for (int a = 0; a < 3; ++a) {
            const int dim = axes3[a];
            for (int p = 0; p < dim / 2; ++p) {
                freqs[o + p] = std::pow(static_cast<double>(theta),
                                        -2.0 * static_cast<double>(p) /
                                            static_cast<double>(dim));
                pair_axis[o + p] = a;
            }
            o += dim / 2;
        }
    }
    for (int r = 0; r < L; ++r) {
        for (int p = 0; p < half; ++p) {
            const double ang =
                static_cast<double>(ax[pair_axis[p]][r]) * freqs[p];
            cos_out[static_cast<std::size_t>(r) * half + p] =
                static_cast<float>(std::cos(ang));
            sin_out[static_cast<std::size_t>(r) * half + p] =
                static_cast<float>(std::sin(ang));
        }
    }
    return L;
}

// ---------------------------------------------------------------------------
// Per-head RMSNorm: the (L, nh*hd) tensor is viewed as (L*nh, hd) and each
// row is scaled by rsqrt(mean(x^2) + eps) * gain[d].  Call sites:
// src/dit/flux.cpp:462-469, src/dit/qwenimage21_forward.cpp:54-63.  Sum of
// squares accumulates in FP32 as the reference's comment at
// src/dit/qwenimage21.cpp:335-337 states.  (brotensor op: parity unpinned.)
void bdo_rms_norm_heads(const float* x, int L, int nh, int hd,
                        const float* gain, float eps, float* out) {
    const std::size_t rows = static_cast<std::size_t>(L) * nh;
    for (std::size_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hd;
        float ss = 0.0f;
        for (int d = 0; d < hd; ++d) ss += xr[d] * xr[d];
        const float inv = 1.0f / std::sqrt(ss / static_cast<float>(hd) + eps);
        for (int d = 0; d < hd; ++d) out[r * hd + d] = xr[d] * inv * gain[d];
    }
}

// ---------------------------------------------------------------------------
// Rotary embedding: table row r, column p rotates pair p of every head of
// token r.  Call sites: src/dit/common.cpp:192-193.
// pair_mode 0: pair p = elements (2p, 2p+1) of the head (interleaved);
// pair_mode 1: pair p = elements (p, p + hd/2) (half-split).
// (brotensor op: parity unpinned; interleaved is the Flux/Qwen convention of
// the upstream Python models the reference states parity with.)
void bdo_rope_apply(const float* x, int L, int nh, int hd, const float* cos_t,
                    const float* sin_t, int pair_mode, float* out) {
    const int half = hd / 2;
    for (int r = 0; r < L; ++r) {
        const float* cr = cos_t + static_cast<std::size_t>(r) * half;
        const float* sr = sin_t + static_cast<std::size_t>(r) * half;
        for (int h = 0; h < nh; ++h) {
            const std::size_t base =
                (static_cast<std::size_t>(r) * nh + h) * hd;
            for (int p = 0; p < half; ++p) {
                const int i0 = pair_mode == 0 ? 2 * p : p;
                const int i1 = pair_mode == 0 ? 2 * p + 1 : p + half;
                const float a = x[base + i0];
                const float b = x[base + i1];
                out[base + i0] = a * cr[p] - b * sr[p];
                out[base + i1] = a * sr[p] + b * cr[p];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Softmax attention core.  src/dit/common.cpp:246-305.
//   q (Lq, nh*hd), k/v (Lk, nh*hd), out (n_rows, nh*hd).
//   scale = 1/sqrt(hd); scores and softmax in double; inv = denom>0 ? 1/denom
//   : 0; P.V accumulated in float with float(p) * v.
// Visibility of key j for query i (absolute query index i in [0, Lq)):
//   mask_mode 0: every key;
//   mask_mode 1: causal with q_offset = Lk - Lq: j <= i + (Lk - Lq)
//                (src/dit/qwenimage21_forward.cpp:659-662);
//   mask_mode 2: block-causal from per-token segment tables (Lq == Lk):
//                j <= i, or seg_id[i] == seg_id[j] and that segment is an
//                image (include/brodiffusion/dit/qwenimage21.h:31-33).
//   key_mask (Lk floats, 1 = valid, 0 = masked) may be null.
//   bias (Lq, bias_cols) is added to the scaled score of keys j < bias_cols
//   for queries i >= bias_row0, row (i - bias_row0) of the bias
//   (src/dit/common.cpp:259-281); may be null.
//   rows / n_rows: compute only these query rows (null = all Lq rows).
//   attn_avg: optional (n_rows, Lk) head-averaged softmax map.
//   precise = 1: the arithmetic above (parity oracle).
//   precise = 0: float dot products and float exp (the timed CPU baseline).
void bdo_sdpa(const float* q, int Lq, const float* k, const float* v, int Lk,
              int nh, int hd, int mask_mode, const int* seg_id,
              const int* seg_is_image, const float* key_mask,
              const float* bias, int bias_row0, int bias_cols, const int* rows,
              int n_rows, int precise, int nthreads, float* out,
              float* attn_avg) {
    const int D = nh * hd;
    if (rows == nullptr) n_rows = Lq;
    const double scale = 1.0 / std::sqrt(static_cast<double>(hd));
    const float scale_f = static_cast<float>(scale);
    const int q_offset = Lk - Lq;
    std::vector<double> avg;
    if (attn_avg != nullptr)
        avg.assign(static_cast<std::size_t>(n_rows) * Lk, 0.0);

    parallel_for(n_rows, nthreads, [&](int ri) {
        const int qi = rows ? rows[ri] : ri;
        std::vector<double> s(static_cast<std::size_t>(Lk));
        std::vector<float> sf(precise ? 0 : static_cast<std::size_t>(Lk));
        std::vector<unsigned char> vis(static_cast<std::size_t>(Lk));
        for (int kk = 0; kk < Lk; ++kk) {
            bool ok = true;
            if (mask_mode == 1) ok = kk <= qi + q_offset;
            else if (mask_mode == 2)
                ok = kk <= qi || (seg_id[qi] == seg_id[kk] &&
                                  seg_is_image[seg_id[qi]] != 0);
            if (key_mask != nullptr && key_mask[kk] == 0.0f) ok = false;
            vis[kk] = ok ? 1 : 0;
        }
        const float* brow = (bias != nullptr && qi >= bias_row0)
                                ? bias + static_cast<std::size_t>(qi - bias_row0) * bias_cols
                                : nullptr;
        for (int h = 0; h < nh; ++h) {
            const int hd0 = h * hd;
            const float* qrow = q + static_cast<std::size_t>(qi) * D + hd0;
            float* orow = out + static_cast<std::size_t>(ri) * D + hd0;
            for (int d = 0; d < hd; ++d) orow[d] = 0.0f;
            if (precise) {
                double smax = -std::numeric_limits<double>::infinity();
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) continue;
                    const float* krow = k + static_cast<std::size_t>(kk) * D + hd0;
                    double dot = 0.0;
                    for (int d = 0; d < hd; ++d)
                        dot += static_cast<double>(qrow[d]) *
                               static_cast<double>(krow[d]);
                    double sc = dot * scale;
                    if (brow != nullptr && kk < bias_cols)
                        sc += static_cast<double>(brow[kk]);
                    s[kk] = sc;
                    if (sc > smax) smax = sc;
                }
                double denom = 0.0;
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) { s[kk] = 0.0; continue; }
                    const double e = std::exp(s[kk] - smax);
                    s[kk] = e;
                    denom += e;
                }
                const double inv = (denom > 0.0) ? (1.0 / denom) : 0.0;
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) continue;
                    const double p = s[kk] * inv;
                    if (attn_avg != nullptr)
                        avg[static_cast<std::size_t>(ri) * Lk + kk] += p;
                    const float pf = static_cast<float>(p);
                    const float* vrow = v + static_cast<std::size_t>(kk) * D + hd0;
                    for (int d = 0; d < hd; ++d) orow[d] += pf * vrow[d];
                }
            } else {
                float smax = -std::numeric_limits<float>::infinity();
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) continue;
                    const float* krow = k + static_cast<std::size_t>(kk) * D + hd0;
                    float dot = 0.0f;
                    for (int d = 0; d < hd; ++d) dot += qrow[d] * krow[d];
                    float sc = dot * scale_f;
                    if (brow != nullptr && kk < bias_cols) sc += brow[kk];
                    sf[kk] = sc;
                    if (sc > smax) smax = sc;
                }
                float denom = 0.0f;
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) { sf[kk] = 0.0f; continue; }
                    const float e = std::exp(sf[kk] - smax);
                    sf[kk] = e;
                    denom += e;
                }
                const float inv = (denom > 0.0f) ? (1.0f / denom) : 0.0f;
                for (int kk = 0; kk < Lk; ++kk) {
                    if (!vis[kk]) continue;
                    const float pf = sf[kk] * inv;
                    const float* vrow = v + static_cast<std::size_t>(kk) * D + hd0;
                    for (int d = 0; d < hd; ++d) orow[d] += pf * vrow[d];
                }
            }
        }
    });
    if (attn_avg != nullptr) {
        const float inv_h = 1.0f / static_cast<float>(nh);
        for (std::size_t i = 0; i < avg.size(); ++i)
            attn_avg[i] = static_cast<float>(avg[i]) * inv_h;
    }
}

// ---------------------------------------------------------------------------
// Y(M, N) = X(M, K) . W(N, K)^T + b(N)   (bias may be null).  The reference's
// linear layers store weights as (out_features, in_features)
// (src/unet_blocks.cpp:264-271 passes Wq (C, C), Wk (C, ctx_dim)).
void bdo_linear(const float* x, const float* w, const float* b, int M, int N,
                int K, int nthreads, float* y) {
    parallel_for(M, nthreads, [&](int m) {
        const float* xr = x + static_cast<std::size_t>(m) * K;
        for (int n = 0; n < N; ++n) {
            const float* wr = w + static_cast<std::size_t>(n) * K;
            double acc = 0.0;
            for (int kk = 0; kk < K; ++kk)
                acc += static_cast<double>(xr[kk]) * static_cast<double>(wr[kk]);
            if (b != nullptr) acc += static_cast<double>(b[n]);
            y[static_cast<std::size_t>(m) * N + n] = static_cast<float>(acc);
        }
    });
}

// ---------------------------------------------------------------------------
// Sana ReLU linear attention core, FP32 per-head path.
// src/dit/sana.cpp:470-520.  q, k, v, out are channel-major (D, N): row c is
// channel c over the N tokens; head h owns rows [h*hd, (h+1)*hd).
//   [S_h; z_h] = [V_h; 1] . relu(K_h)^T          ((hd+1) x hd)
//   hid        = [S_h; z_h] . relu(Q_h)          ((hd+1) x N)
//   out_h      = hid[:hd] / (hid[hd] + eps)
// sz_in  (nh, hd+1, hd), optional: added with weight w_in before the query
//        read (the reference-attention inject seam, sana.cpp:502-508).
// sz_out (nh, hd+1, hd), optional: receives [S; z] before injection
//        (the capture seam, sana.cpp:495-501).
void bdo_sana_linear_attn(const float* q, const float* k, const float* v,
                          int nh, int hd, int N, float eps,
                          const float* sz_in, float w_in, float* sz_out,
                          int nthreads, float* out) {
    parallel_for(nh, nthreads, [&](int h) {
        const std::size_t base = static_cast<std::size_t>(h) * hd * N;
        const float* Q = q + base;
        const float* K = k + base;
        const float* V = v + base;
        std::vector<float> sz(static_cast<std::size_t>(hd + 1) * hd, 0.0f);
        for (int i = 0; i <= hd; ++i) {
            for (int j = 0; j < hd; ++j) {
                float acc = 0.0f;
                const float* kr = K + static_cast<std::size_t>(j) * N;
                if (i < hd) {
                    const float* vr = V + static_cast<std::size_t>(i) * N;
                    for (int n = 0; n < N; ++n)
                        acc += vr[n] * std::max(kr[n], 0.0f);
                } else {
                    for (int n = 0; n < N; ++n) acc += std::max(kr[n], 0.0f);
                }
                sz[static_cast<std::size_t>(i) * hd + j] = acc;
            }
        }
        const std::size_t hh = static_cast<std::size_t>(hd + 1) * hd;
        if (sz_out != nullptr)
            std::memcpy(sz_out + h * hh, sz.data(), hh * sizeof(float));
        if (sz_in != nullptr)
            for (std::size_t i = 0; i < hh; ++i) sz[i] += w_in * sz_in[h * hh + i];
        std::vector<float> rq(static_cast<std::size_t>(hd));
        for (int n = 0; n < N; ++n) {
            for (int j = 0; j < hd; ++j)
                rq[j] = std::max(Q[static_cast<std::size_t>(j) * N + n], 0.0f);
            float den = 0.0f;
            for (int j = 0; j < hd; ++j)
                den += sz[static_cast<std::size_t>(hd) * hd + j] * rq[j];
            const float rec = 1.0f / (den + eps);
            for (int i = 0; i < hd; ++i) {
                float num = 0.0f;
                for (int j = 0; j < hd; ++j)
                    num += sz[static_cast<std::size_t>(i) * hd + j] * rq[j];
                out[base + static_cast<std::size_t>(i) * N + n] = num * rec;
            }
        }
    });
}

// ---------------------------------------------------------------------------
// Fused FF1 + exact GEGLU.  src/fused_transformer.cu:89-92,275-282.
//   T = X(B, D_in) . W(2*D_out, D_in)^T + b;  Y = T[:, :D_out] *
//   gelu_exact(T[:, D_out:]),  gelu_exact(g) = 0.5 g (1 + erf(g / sqrt 2)).
void bdo_linear_geglu(const float* x, const float* w, const float* b, int B,
                      int D_in, int D_out, int nthreads, float* y) {
    parallel_for(B, nthreads, [&](int m) {
        const float* xr = x + static_cast<std::size_t>(m) * D_in;
        for (int n = 0; n < D_out; ++n) {
            const float* wv = w + static_cast<std::size_t>(n) * D_in;
            const float* wg = w + static_cast<std::size_t>(n + D_out) * D_in;
            double val = 0.0, gate = 0.0;
            for (int kk = 0; kk < D_in; ++kk) {
                val += static_cast<double>(xr[kk]) * wv[kk];
                gate += static_cast<double>(xr[kk]) * wg[kk];
            }
            if (b != nullptr) { val += b[n]; gate += b[n + D_out]; }
            const double g = 0.5 * gate * (1.0 + std::erf(gate * 0.7071067811865475));
            y[static_cast<std::size_t>(m) * D_out + n] = static_cast<float>(val * g);
        }
    });
}

}  // extern "C"
