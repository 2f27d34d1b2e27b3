// f32 CPU golden ops of the DSV41 family (C++): low-precision codecs and the ops whose semantics are
// easy to get subtly wrong (sink attention, sqrt-softplus routing with selection-only bias, candidate
// blocks).  They mirror ferrite_b200/ops/quant.py and ferrite_b200/models/dsv41_ref.py and are tested
// against them; reference: crates/ferrite-models/src/dsv41/{quant,ops}.rs.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <vector>

namespace golden_d4 {

inline float pow2_ceil(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    int e = (int)((b >> 23) & 0xff) + ((b & 0x7fffffu) ? 1 : 0);
    e = std::min(std::max(e, 0), 254);
    const uint32_t o = (uint32_t)e << 23;
    float r;
    std::memcpy(&r, &o, 4);
    return r;
}

// nearest e4m3 (round to nearest even, saturating at 448), returned as f32
inline float e4m3_round(float v) {
    if (std::isnan(v)) return v;
    const float a = std::min(std::fabs(v), 448.f);
    if (a == 0.f) return std::copysign(0.f, v);
    int e;
    std::frexp(a, &e);                       // a = m * 2^e, m in [0.5, 1)
    int exp = std::max(e - 1, -6);           // normal exponents -6..8, subnormals share 2^-6
    const float q = std::ldexp(1.f, exp - 3);   // spacing: 3 mantissa bits
    float r = std::nearbyint(a / q) * q;     // default rounding mode: to nearest even
    r = std::min(r, 448.f);
    return std::copysign(r, v);
}

inline float e2m1_round(float v) {
    const float a = std::min(std::fabs(v), 6.f);
    float r;
    if (a <= 0.25f) r = 0.f;
    else if (a < 0.75f) r = 0.5f;
    else if (a <= 1.25f) r = 1.f;
    else if (a < 1.75f) r = 1.5f;
    else if (a <= 2.5f) r = 2.f;
    else if (a < 3.5f) r = 3.f;
    else if (a <= 5.f) r = 4.f;
    else r = 6.f;
    return std::copysign(r, v);
}

// e4m3 values with a power-of-two scale per `block` consecutive values (in place round trip)
inline void fp8_act_roundtrip(float* x, size_t n, int block) {
    const float inv448 = 1.f / 448.f;
    for (size_t b0 = 0; b0 < n; b0 += block) {
        float amax = 1e-4f;
        for (int i = 0; i < block; ++i) amax = std::max(amax, std::fabs(x[b0 + i]));
        const float s = pow2_ceil(amax * inv448);
        for (int i = 0; i < block; ++i) x[b0 + i] = e4m3_round(x[b0 + i] / s) * s;
    }
}

// e2m1 values with a ue8m0 scale per block, or (e4m3_scale) an e4m3 scale with the 6 * 2^-9 floor
inline void fp4_act_roundtrip(float* x, size_t n, int block, bool e4m3_scale) {
    const float inv6 = 1.f / 6.f;
    for (size_t b0 = 0; b0 < n; b0 += block) {
        float amax = 0.f;
        for (int i = 0; i < block; ++i) amax = std::max(amax, std::fabs(x[b0 + i]));
        float s;
        if (e4m3_scale) s = e4m3_round(std::max(amax, 6.f * 0.001953125f) / 6.f);
        else s = pow2_ceil(std::max(amax, 6.f * 1.17549435e-38f) * inv6);
        for (int i = 0; i < block; ++i) x[b0 + i] = e2m1_round(x[b0 + i] / s) * s;
    }
}

// q [H][d] against gathered kv [n][d] with a per-head sink logit: max over real keys only, the sink
// joins the denominator, no keys -> zeros.
inline void sparse_attn_sink(const float* q, const float* kv, const float* sink, float* out, int H, int d, int n, float scale) {
    std::vector<float> s(std::max(n, 1));
    for (int h = 0; h < H; ++h) {
        float* o = out + (size_t)h * d;
        std::fill(o, o + d, 0.f);
        if (n == 0) continue;
        float m = -std::numeric_limits<float>::infinity();
        for (int t = 0; t < n; ++t) {
            float acc = 0.f;
            for (int j = 0; j < d; ++j) acc += q[(size_t)h * d + j] * kv[(size_t)t * d + j];
            s[t] = acc * scale;
            m = std::max(m, s[t]);
        }
        float den = std::exp(sink[h] - m);
        for (int t = 0; t < n; ++t) { s[t] = std::exp(s[t] - m); den += s[t]; }
        for (int t = 0; t < n; ++t)
            for (int j = 0; j < d; ++j) o[j] += s[t] * kv[(size_t)t * d + j];
        for (int j = 0; j < d; ++j) o[j] /= den;
    }
}

// scores = sqrt(softplus(logits)); selection by scores + bias (ties to the lower index); weights from the
// raw scores, normalised over the selection (+1e-20), times route_scale.
inline void route_sqrtsoftplus(const float* logits, const float* bias, int n, int E, int topk, float route_scale,
                               int64_t* idx, float* wts) {
    std::vector<float> sc(E), sel(E);
    for (int r = 0; r < n; ++r) {
        for (int e = 0; e < E; ++e) {
            const float x = logits[(size_t)r * E + e];
            const float sp = x > 20.f ? x : std::log1p(std::exp(x));
            sc[e] = std::sqrt(sp);
            sel[e] = sc[e] + bias[e];
        }
        float sum = 0.f;
        for (int k = 0; k < topk; ++k) {
            int best = 0;
            for (int e = 1; e < E; ++e)
                if (sel[e] > sel[best]) best = e;
            idx[(size_t)r * topk + k] = best;
            wts[(size_t)r * topk + k] = sc[best];
            sum += sc[best];
            sel[best] = -std::numeric_limits<float>::infinity();
        }
        for (int k = 0; k < topk; ++k) {
            float w = wts[(size_t)r * topk + k];
            if (topk > 1) w = w / (sum + 1e-20f);
            wts[(size_t)r * topk + k] = w * route_scale;
        }
    }
}

// keep[j] = 1 for positions inside the `topk_blocks` best blocks (block score = max over `bs` positions
// below clen; the block of the newest visible position is pinned); ties to the lower block index.
inline void candidate_blocks(const float* score, int n_pos, int clen, int topk_blocks, int bs, uint8_t* keep) {
    std::fill(keep, keep + n_pos, 0);
    const int nb = (n_pos + bs - 1) / bs;
    std::vector<float> bscore(nb, -std::numeric_limits<float>::infinity());
    for (int j = 0; j < n_pos && j < clen; ++j) bscore[j / bs] = std::max(bscore[j / bs], score[j]);
    if (clen > 0) bscore[(clen - 1) / bs] = std::numeric_limits<float>::infinity();
    std::vector<int> order(nb);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return bscore[a] > bscore[b]; });
    for (int k = 0; k < std::min(topk_blocks, nb); ++k) {
        const int b = order[k];
        if (bscore[b] == -std::numeric_limits<float>::infinity()) continue;
        for (int j = b * bs; j < std::min(n_pos, (b + 1) * bs); ++j) keep[j] = 1;
    }
}

}  // namespace golden_d4
