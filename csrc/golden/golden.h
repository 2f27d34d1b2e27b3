// f32 CPU golden ops: the numerical oracle (and timed CPU baseline) for every GLM op.
// Plain loops over row-major float buffers; no threading, no SIMD intrinsics, so that the
// result is the same on every host.  Semantics follow the reference's CpuBackend
// (crates/ferrite-kernel/src/cpu.rs:82-808), its MHC helpers
// (crates/ferrite-exec/src/mhc.rs:19-213) and its DCP model (crates/ferrite-kernel/src/dcp.rs:49-174).
#pragma once
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>
#include <algorithm>

namespace golden {

constexpr float kF32Eps = 1.1920929e-07f;

inline float sigmoid(float x) { return 1.f / (1.f + std::exp(-x)); }

// out[n,out_f] = x[n,in_f] . w[out_f,in_f]^T
inline void matmul(const float* x, const float* w, float* out, int n, int in_f, int out_f) {
    for (int i = 0; i < n; ++i)
        for (int o = 0; o < out_f; ++o) {
            float acc = 0.f;
            const float* xr = x + (size_t)i * in_f;
            const float* wr = w + (size_t)o * in_f;
            for (int k = 0; k < in_f; ++k) acc += xr[k] * wr[k];
            out[(size_t)i * out_f + o] = acc;
        }
}

inline void rmsnorm(const float* x, const float* w, float* out, int n, int d, float eps) {
    for (int i = 0; i < n; ++i) {
        const float* r = x + (size_t)i * d;
        float ss = 0.f;
        for (int j = 0; j < d; ++j) ss += r[j] * r[j];
        const float inv = 1.f / std::sqrt(ss / d + eps);
        for (int j = 0; j < d; ++j) out[(size_t)i * d + j] = r[j] * inv * w[j];
    }
}

// rows of length d: o * rsqrt(mean o^2 + eps) * w * sigmoid(gate)
inline void gated_rmsnorm(const float* o, const float* gate, const float* w, float* out, int rows, int d, float eps) {
    for (int i = 0; i < rows; ++i) {
        const float* r = o + (size_t)i * d;
        float ss = 0.f;
        for (int j = 0; j < d; ++j) ss += r[j] * r[j];
        const float inv = 1.f / std::sqrt(ss / d + eps);
        for (int j = 0; j < d; ++j) out[(size_t)i * d + j] = r[j] * inv * w[j] * sigmoid(gate[(size_t)i * d + j]);
    }
}

inline void swiglu_limited(const float* gate, const float* up, float* out, size_t n, float limit) {
    for (size_t i = 0; i < n; ++i) {
        const float g = std::min(gate[i], limit);
        const float u = std::max(std::min(up[i], limit), -limit);
        out[i] = g / (1.f + std::exp(-g)) * u;
    }
}

// x [n,ch], w [ch,k], state [ch,k-1] oldest first -> out [n,ch], state_out [ch,k-1]
inline void causal_conv1d(const float* x, const float* w, const float* state, float* out, float* state_out,
                          int n, int ch, int k) {
    const int hist = k - 1;
    std::vector<float> stream(hist + n);
    for (int c = 0; c < ch; ++c) {
        for (int h = 0; h < hist; ++h) stream[h] = state[(size_t)c * hist + h];
        for (int t = 0; t < n; ++t) stream[hist + t] = x[(size_t)t * ch + c];
        for (int t = 0; t < n; ++t) {
            float acc = 0.f;
            for (int i = 0; i < k; ++i) acc += w[(size_t)c * k + i] * stream[t + i];
            out[(size_t)t * ch + c] = acc;
        }
        for (int h = 0; h < hist; ++h) state_out[(size_t)c * hist + h] = stream[n + h];
    }
}

// q,k [n,h,dk]; v [n,h,dv]; beta [n,h]; g [n,h,dk] log-decay; state [h,dk,dv] (updated in place)
inline void gdn_recurrent(const float* q, const float* k, const float* v, const float* beta, const float* g,
                          float* state, float* out, int n, int h, int dk, int dv) {
    std::vector<float> u(dv);
    for (int t = 0; t < n; ++t)
        for (int hd = 0; hd < h; ++hd) {
            float* S = state + (size_t)hd * dk * dv;
            const float* qh = q + ((size_t)t * h + hd) * dk;
            const float* kh = k + ((size_t)t * h + hd) * dk;
            const float* vh = v + ((size_t)t * h + hd) * dv;
            const float* gh = g + ((size_t)t * h + hd) * dk;
            const float bt = beta[(size_t)t * h + hd];
            for (int i = 0; i < dk; ++i) {
                const float dec = std::exp(gh[i]);
                for (int j = 0; j < dv; ++j) S[(size_t)i * dv + j] *= dec;
            }
            for (int j = 0; j < dv; ++j) {
                float a = 0.f;
                for (int i = 0; i < dk; ++i) a += kh[i] * S[(size_t)i * dv + j];
                u[j] = a;
            }
            for (int i = 0; i < dk; ++i)
                for (int j = 0; j < dv; ++j) S[(size_t)i * dv + j] += bt * kh[i] * (vh[j] - u[j]);
            for (int j = 0; j < dv; ++j) {
                float a = 0.f;
                for (int i = 0; i < dk; ++i) a += qh[i] * S[(size_t)i * dv + j];
                out[((size_t)t * h + hd) * dv + j] = a;
            }
        }
}

// q_idx [n,H*D]; keys [t,D]; w [n,H]; idx out [n,topk] (-1 = invisible); ties to the lower index
inline void indexer_topk(const float* q_idx, const float* keys, const float* w, int n, int H, int D, int t,
                         int topk, int ctx0, int64_t* idx) {
    const float inv = 1.f / std::sqrt((float)D);
    std::vector<std::pair<float, int>> sc(t);
    for (int i = 0; i < n; ++i) {
        const int jmax = std::min(ctx0 + i + 1, t);
        for (int j = 0; j < t; ++j) {
            if (j >= jmax) { sc[j] = {-std::numeric_limits<float>::infinity(), j}; continue; }
            float s = 0.f;
            for (int hh = 0; hh < H; ++hh) {
                float dot = 0.f;
                for (int l = 0; l < D; ++l) dot += q_idx[((size_t)i * H + hh) * D + l] * keys[(size_t)j * D + l];
                s += w[(size_t)i * H + hh] * std::max(dot, 0.f);
            }
            sc[j] = {s * inv, j};
        }
        std::stable_sort(sc.begin(), sc.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
        for (int r = 0; r < topk; ++r)
            idx[(size_t)i * topk + r] = std::isinf(sc[r].first) && sc[r].first < 0 ? -1 : sc[r].second;
    }
}

// q [n,h,d]; k [t,h,d]; v [t,h,dv]; idx [n,W] (-1 skip, repeats count once) -> out [n,h,dv];
// optional lse [n,h] = max + log(denominator); an empty set gives zeros and lse = -inf.
inline void sparse_mla_attn(const float* q, const float* k, const float* v, const int64_t* idx, float* out,
                            float* lse, int n, int h, int d, int dv, int t, int W) {
    const float scale = 1.f / std::sqrt((float)d);
    std::vector<int> sel;
    std::vector<float> s;
    for (int i = 0; i < n; ++i) {
        sel.clear();
        for (int c = 0; c < W; ++c) {
            const int64_t j = idx[(size_t)i * W + c];
            if (j < 0 || j >= t) continue;
            if (std::find(sel.begin(), sel.end(), (int)j) == sel.end()) sel.push_back((int)j);
        }
        for (int hd = 0; hd < h; ++hd) {
            float* o = out + ((size_t)i * h + hd) * dv;
            for (int l = 0; l < dv; ++l) o[l] = 0.f;
            if (sel.empty()) { if (lse) lse[(size_t)i * h + hd] = -std::numeric_limits<float>::infinity(); continue; }
            s.resize(sel.size());
            float mx = -std::numeric_limits<float>::infinity();
            for (size_t c = 0; c < sel.size(); ++c) {
                float a = 0.f;
                for (int l = 0; l < d; ++l) a += q[((size_t)i * h + hd) * d + l] * k[((size_t)sel[c] * h + hd) * d + l];
                s[c] = a * scale;
                mx = std::max(mx, s[c]);
            }
            float den = 0.f;
            for (auto& x : s) { x = std::exp(x - mx); den += x; }
            den += kF32Eps;
            for (size_t c = 0; c < sel.size(); ++c) {
                const float wgt = s[c] / den;
                for (int l = 0; l < dv; ++l) o[l] += wgt * v[((size_t)sel[c] * h + hd) * dv + l];
            }
            if (lse) lse[(size_t)i * h + hd] = mx + std::log(den);
        }
    }
}

// outs [S][n*h][dv], lses [S][n*h] -> merged [n*h][dv]
inline void lse_merge(const float* outs, const float* lses, float* merged, int S, int rows, int dv) {
    for (int r = 0; r < rows; ++r) {
        float m = -std::numeric_limits<float>::infinity();
        for (int s = 0; s < S; ++s) m = std::max(m, lses[(size_t)s * rows + r]);
        if (std::isinf(m)) m = 0.f;
        float den = 0.f;
        for (int l = 0; l < dv; ++l) merged[(size_t)r * dv + l] = 0.f;
        for (int s = 0; s < S; ++s) {
            const float wgt = std::exp(lses[(size_t)s * rows + r] - m);
            den += wgt;
            for (int l = 0; l < dv; ++l) merged[(size_t)r * dv + l] += wgt * outs[((size_t)s * rows + r) * dv + l];
        }
        den = std::max(den, 1e-38f);
        for (int l = 0; l < dv; ++l) merged[(size_t)r * dv + l] /= den;
    }
}

inline void moe_route(const float* logits, const float* bias, int n, int E, int topk, float scaling, float* wts,
                      int64_t* ids) {
    std::vector<float> sg(E);
    std::vector<std::pair<float, int>> sc(E);
    for (int i = 0; i < n; ++i) {
        for (int e = 0; e < E; ++e) { sg[e] = sigmoid(logits[(size_t)i * E + e]); sc[e] = {sg[e] + bias[e], e}; }
        std::stable_sort(sc.begin(), sc.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
        float sum = 0.f;
        for (int r = 0; r < topk; ++r) sum += sg[sc[r].second];
        for (int r = 0; r < topk; ++r) {
            ids[(size_t)i * topk + r] = sc[r].second;
            wts[(size_t)i * topk + r] = sg[sc[r].second] / (sum + kF32Eps) * scaling;
        }
    }
}

// R [T,n,H]; fn [mix,n*H]; scale [3]; base [mix] -> x [T,H], post [T,n], comb [T,n,n]
inline void hc_pre(const float* R, const float* fn, const float* scale, const float* base, float* x, float* post,
                   float* comb, int T, int n, int H, float rms_eps, float hc_eps, int iters) {
    const int mix = (2 + n) * n, D = n * H;
    std::vector<float> mixes(mix);
    for (int t = 0; t < T; ++t) {
        const float* r = R + (size_t)t * D;
        float ss = 0.f;
        for (int j = 0; j < D; ++j) ss += r[j] * r[j];
        const float rr = 1.f / std::sqrt(ss / D + rms_eps);
        for (int m = 0; m < mix; ++m) {
            float a = 0.f;
            for (int j = 0; j < D; ++j) a += fn[(size_t)m * D + j] * r[j];
            mixes[m] = a * rr;
        }
        for (int j = 0; j < H; ++j) x[(size_t)t * H + j] = 0.f;
        for (int i = 0; i < n; ++i) {
            const float pre = sigmoid(mixes[i] * scale[0] + base[i]) + hc_eps;
            for (int j = 0; j < H; ++j) x[(size_t)t * H + j] += pre * r[(size_t)i * H + j];
            post[(size_t)t * n + i] = 2.f * sigmoid(mixes[n + i] * scale[1] + base[n + i]);
        }
        float* c = comb + (size_t)t * n * n;
        for (int i = 0; i < n * n; ++i) c[i] = mixes[2 * n + i] * scale[2] + base[2 * n + i];
        for (int i = 0; i < n; ++i) {
            float mx = -std::numeric_limits<float>::infinity(), den = 0.f;
            for (int k = 0; k < n; ++k) mx = std::max(mx, c[i * n + k]);
            for (int k = 0; k < n; ++k) { c[i * n + k] = std::exp(c[i * n + k] - mx); den += c[i * n + k]; }
            for (int k = 0; k < n; ++k) c[i * n + k] = c[i * n + k] / den + hc_eps;
        }
        auto col_norm = [&]() {
            for (int k = 0; k < n; ++k) {
                float s = 0.f;
                for (int i = 0; i < n; ++i) s += c[i * n + k];
                for (int i = 0; i < n; ++i) c[i * n + k] /= (s + hc_eps);
            }
        };
        col_norm();
        for (int it = 1; it < iters; ++it) {
            for (int i = 0; i < n; ++i) {
                float s = 0.f;
                for (int k = 0; k < n; ++k) s += c[i * n + k];
                for (int k = 0; k < n; ++k) c[i * n + k] /= (s + hc_eps);
            }
            col_norm();
        }
    }
}

// R'[t][i] = post[t][i]*y[t] + sum_k comb[t][k][i] R[t][k]
inline void hc_post(const float* y, const float* R, const float* post, const float* comb, float* out, int T, int n, int H) {
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < H; ++j) {
                float a = post[(size_t)t * n + i] * y[(size_t)t * H + j];
                for (int k = 0; k < n; ++k) a += comb[((size_t)t * n + k) * n + i] * R[((size_t)t * n + k) * H + j];
                out[((size_t)t * n + i) * H + j] = a;
            }
}

inline int64_t argmax_first(const float* x, int n) {
    int64_t b = 0;
    for (int i = 1; i < n; ++i) if (x[i] > x[b]) b = i;
    return b;
}

inline int spec_accept(const int64_t* drafts, int nd, const int64_t* judges, int nj, bool anchor_in_block) {
    int m = 0;
    const int lim = std::min(nd, nj);
    while (m < lim && drafts[m] == judges[m]) ++m;
    return anchor_in_block ? m + 1 : m;
}

}  // namespace golden
