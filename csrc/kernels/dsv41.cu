// Kernels of the DSV41 family (sliding-window + compressed-KV latent attention with an indexer,
// sqrt-softplus MoE with fp4 experts, offset hyper-connections, engram n-gram memory).
//
// Storage choices (all device-side, the golden model only defines values):
//   * window KV: ring of `cap` rows per slot, row of position p at p % cap, cap >= window +
//     rows of one forward, so that a multi-row forward (verify, chunked prefill) never
//     overwrites a row that an earlier row of the same forward still sees, and rejected rows
//     are simply overwritten later; values are e4m3-per-32 round trips held as bf16 (exact);
//   * compressor input ring: the raw (kv, score) rows of the last `depth` positions, so a
//     group is pooled from positions, not from a mutable partial state (no rollback needed);
//   * compressed KV / index keys: one row per group j at index j, e2m1 round trips held as
//     bf16 (exact: 1 + 3 mantissa bits).
// Reference kernels replaced: kernels/cuda/dsv41/*.cu (`rmsnorm_*`, `apply_rope*`, `ring_*`,
// `win_kv_quant_rt`, `compress_*`, `indexer_score*`, `candidate_blocks`, `indexer_topk`,
// `sparse_attn_pf`, `route_*`, `expert_gemv_fp4_*`, `engram_*`, `hc_*`), semantics of
// ref_inference/model.py and ref_inference/kernel.py.
#include <cuda_fp4.h>

#include <cooperative_groups.h>

#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

constexpr int kMaxMixD4 = 24;  // (2 + hc) * hc for hc = 4; accumulator rows are kMaxMixD4 + 1 wide

// ---- codecs ------------------------------------------------------------------------------------
__device__ __forceinline__ float pow2_ceil(float x) {  // 2^ceil(log2 x), x > 0 normal
    const uint32_t b = __float_as_uint(x);
    const int e = (int)((b >> 23) & 0xff) + ((b & 0x7fffffu) ? 1 : 0);
    return __uint_as_float((uint32_t)min(max(e, 0), 254) << 23);
}
__device__ __forceinline__ float e4m3_rt(float v) {  // nearest e4m3 (saturating), as f32
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float e2m1_rt(float v) {  // nearest e2m1 (ties to even code, saturating), as f32
    const float a = fminf(fabsf(v), 6.f);
    float r;
    if (a <= 0.25f) r = 0.f;
    else if (a < 0.75f) r = 0.5f;
    else if (a <= 1.25f) r = 1.f;
    else if (a < 1.75f) r = 1.5f;
    else if (a <= 2.5f) r = 2.f;
    else if (a < 3.5f) r = 3.f;
    else if (a <= 5.f) r = 4.f;
    else r = 6.f;
    return copysignf(r, v);
}
// Scale of one 32-value block whose |max| is amax: e4m3 values with a power-of-two scale.
__device__ __forceinline__ float fp8_block_scale(float amax) { return pow2_ceil(fmaxf(amax, 1e-4f) * (1.f / 448.f)); }

// ---- activation quantisation: e4m3 per 32 with power-of-two scales, round trip ----------------
// One warp per 32-value block.  xq may alias x.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const float* __restrict__ x, int ldx, float* __restrict__ xq, int ldq, SplitBuf osp, int n, int K) {
    PDL_PROLOGUE();
    const int lane = threadIdx.x & 31;
    const int nb = K / 32;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n * nb) return;
    const int r = w / nb, b = w % nb;
    const float v = x[(size_t)r * ldx + b * 32 + lane];
    const float s = fp8_block_scale(warp_max(fabsf(v)));
    const float q = e4m3_rt(v / s) * s;
    if (xq) xq[(size_t)r * ldq + b * 32 + lane] = q;
    split_store(osp, r, b * 32 + lane, q);
}

// ---- offset hyper-connection front -------------------------------------------------------------
// acc [n][25]: the 24 mix dots of the CURRENT stream R plus its sum of squares (cleared here).
// Computes this site's (pre, post, comb); `pre` is only stored (the NEXT site contracts with
// it), the contraction uses pre_in, the coefficients of the previous site.
//   xn = rmsnorm(sum_i pre_in[i] R_i) * ln_w ; optionally also xq = the e4m3-per-32 round trip of xn
// Block = C contraction warps + one coefficient warp.  All warps first sum the per-tile partial dots; then
// the contraction warps (which only need the PREVIOUS site's `pre`) and the coefficient warp (sigmoids +
// Sinkhorn, a serial chain of ~40 divisions) run side by side; the contraction warps meet on a named
// barrier of their own.  A thread owns up to two float4 columns, loaded before the first barrier.
__global__ void __launch_bounds__(1024)
hc_pre_offset_kernel(const float* __restrict__ R, float* __restrict__ acc, const float* __restrict__ scale,
                     const float* __restrict__ base, const float* __restrict__ ln_w, const float* __restrict__ pre_in,
                     float* __restrict__ pre_out, float* __restrict__ post_out, float* __restrict__ comb_out,
                     float* __restrict__ xn_out, float* __restrict__ xc_out, int H, float rms_eps, float hc_eps, int iters,
                     SplitBuf osp, const float* __restrict__ part, int* __restrict__ part_n, int part_ld,
                     float* __restrict__ xq_out, SplitBuf qsp) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    const int n = 4;
    const int r = blockIdx.x;
    const float* row = R + (size_t)r * n * H;
    const int nct = blockDim.x - 32;              // contraction threads
    const bool coef_warp = (int)threadIdx.x >= nct;
    // residual loads first: they are in flight while the partial dots are summed
    float4 v[2][4], lw[2];
    bool act[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int j = (threadIdx.x + c * nct) * 4;
        act[c] = !coef_warp && j < H;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            v[c][k] = act[c] ? *reinterpret_cast<const float4*>(row + (size_t)k * H + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        lw[c] = act[c] ? *reinterpret_cast<const float4*>(ln_w + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (acc && part_n) {
        // per-tile partial mix dots left by a fused GEMV epilogue: one warp per dot sums the tiles
        const int nt = part_n[r];
        if (nt > 0) {
            const int lane = threadIdx.x & 31;
            for (int o = threadIdx.x >> 5; o <= kMaxMixD4; o += blockDim.x >> 5) {
                const float* pp = part + ((size_t)r * (kMaxMixD4 + 1) + o) * part_ld;
                float sum = 0.f;
                for (int i = lane; i < nt; i += 32) sum += pp[i];
                sum = warp_sum(sum);
                if (lane == 0) acc[(size_t)r * (kMaxMixD4 + 1) + o] += sum;
            }
            __syncthreads();
            if (threadIdx.x == 0) part_n[r] = 0;
        }
    }
    if (coef_warp) {
        if (!acc) return;
        float* a = acc + (size_t)r * (kMaxMixD4 + 1);
        const int lane = threadIdx.x & 31;
        const float rr = rsqrtf(a[kMaxMixD4] / (float)(n * H) + rms_eps);
        if (lane < n) {
            pre_out[(size_t)r * n + lane] = sigmoidf_(a[lane] * rr * scale[0] + base[lane]) + hc_eps;
            post_out[(size_t)r * n + lane] = 2.f * sigmoidf_(a[n + lane] * rr * scale[1] + base[n + lane]);
        }
        float c = 0.f;
        const bool on = lane < n * n;
        if (on) c = a[2 * n + lane] * rr * scale[2] + base[2 * n + lane];
        float mx = on ? c : -INFINITY;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float e = on ? __expf(c - mx) : 0.f;
        float den = e + __shfl_xor_sync(0xffffffffu, e, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        c = on ? e / den + hc_eps : 0.f;
        float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        c = c / (cs + hc_eps);
        for (int it = 1; it < iters; ++it) {
            float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            c = c / (rs + hc_eps);
            cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            c = c / (cs + hc_eps);
        }
        if (on) comb_out[(size_t)r * n * n + lane] = c;
        __syncwarp();
        if (lane <= kMaxMixD4) a[lane] = 0.f;
        return;
    }
    const float p0 = pre_in[r * n + 0], p1 = pre_in[r * n + 1], p2 = pre_in[r * n + 2], p3 = pre_in[r * n + 3];
    float4 x[2];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        x[c].x = p0 * v[c][0].x + p1 * v[c][1].x + p2 * v[c][2].x + p3 * v[c][3].x;
        x[c].y = p0 * v[c][0].y + p1 * v[c][1].y + p2 * v[c][2].y + p3 * v[c][3].y;
        x[c].z = p0 * v[c][0].z + p1 * v[c][1].z + p2 * v[c][2].z + p3 * v[c][3].z;
        x[c].w = p0 * v[c][0].w + p1 * v[c][1].w + p2 * v[c][2].w + p3 * v[c][3].w;
        if (act[c]) ss += x[c].x * x[c].x + x[c].y * x[c].y + x[c].z * x[c].z + x[c].w * x[c].w;
    }
    // sum over the contraction warps only (named barrier 1; the coefficient warp never joins it)
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    asm volatile("bar.sync 1, %0;" ::"r"(nct) : "memory");
    float tot = 0.f;
    for (int w = 0; w < (nct >> 5); ++w) tot += red[w];
    const float inv = rsqrtf(tot / H + rms_eps);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int j = (threadIdx.x + c * nct) * 4;
        float4 o;   // zeros in inactive threads (their x and ln_w are zero)
        o.x = x[c].x * inv * lw[c].x; o.y = x[c].y * inv * lw[c].y; o.z = x[c].z * inv * lw[c].z; o.w = x[c].w * inv * lw[c].w;
        if (act[c]) {
            if (xc_out) *reinterpret_cast<float4*>(xc_out + (size_t)r * H + j) = x[c];
            *reinterpret_cast<float4*>(xn_out + (size_t)r * H + j) = o;
            split_store(osp, r, j, o.x); split_store(osp, r, j + 1, o.y);
            split_store(osp, r, j + 2, o.z); split_store(osp, r, j + 3, o.w);
        }
        if (xq_out || qsp.base) {
            // e4m3-per-32 round trip of the normed row (what the next projections consume): a 32-value block is the
            // four values of eight consecutive threads; whole warps run the shuffles, only live threads store
            float am = fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w)));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
            const float sc = fp8_block_scale(am);
            float4 q;
            q.x = e4m3_rt(o.x / sc) * sc; q.y = e4m3_rt(o.y / sc) * sc; q.z = e4m3_rt(o.z / sc) * sc; q.w = e4m3_rt(o.w / sc) * sc;
            if (act[c]) {
                if (xq_out) *reinterpret_cast<float4*>(xq_out + (size_t)r * H + j) = q;
                split_store(qsp, r, j, q.x); split_store(qsp, r, j + 1, q.y);
                split_store(qsp, r, j + 2, q.z); split_store(qsp, r, j + 3, q.w);
            }
        }
    }
}

// ---- RoPE on the last `rd` dims of each head (adjacent pairs), in place -------------------------
// position of row r = meta[r].pos (+ pos_off); optional fp4-per-32 round trip of the whole head
// afterwards (the indexer's q).
__global__ void __launch_bounds__(128)
rope_heads_kernel(float* __restrict__ x, int ld, int heads, int hd, int rd, const float* __restrict__ freqs,
                  const RowMeta* __restrict__ meta, int pos_off, int inverse, int fp4_rt, SplitBuf osp) {
    PDL_PROLOGUE();
    const int r = blockIdx.y, h = blockIdx.x;
    float* v = x + (size_t)r * ld + (size_t)h * hd;
    const float pos = (float)(meta[r].pos + pos_off);
    for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * freqs[i], &sn, &cs);
        if (inverse) sn = -sn;
        float* p = v + (hd - rd) + 2 * i;
        const float a = p[0], b = p[1];
        p[0] = a * cs - b * sn;
        p[1] = a * sn + b * cs;
    }
    if (fp4_rt) {
        __syncthreads();
        const int lane = threadIdx.x & 31;
        for (int b = threadIdx.x >> 5; b < hd / 32; b += blockDim.x >> 5) {
            const float t = v[b * 32 + lane];
            const float s = pow2_ceil(fmaxf(warp_max(fabsf(t)), 6.f * 1.17549435e-38f) * (1.f / 6.f));
            const float q = e2m1_rt(t / s) * s;
            v[b * 32 + lane] = q;
            split_store(osp, r, h * hd + b * 32 + lane, q);
        }
    }
}

// ---- KV row: rmsnorm -> rope -> e4m3/32 round trip -> ring (bf16) and/or plain rows --------------
__device__ __forceinline__ void kv_append_body(float* sh, const float* __restrict__ kv, int ld, const float* __restrict__ norm_w,
                                               const float* __restrict__ freqs, const RowMeta* __restrict__ meta,
                                               __nv_bfloat16* __restrict__ ring, int cap, float* __restrict__ rows_out,
                                               int hd, int rd, float eps, int pos_off) {
    float* red = sh;
    float* v = sh + 32;
    const int r = blockIdx.x;
    const RowMeta m = meta[r];
    float ss = 0.f;
    for (int j = threadIdx.x; j < hd; j += blockDim.x) {
        const float t = kv[(size_t)r * ld + j];
        v[j] = t;
        ss += t * t;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / hd + eps);
    for (int j = threadIdx.x; j < hd; j += blockDim.x) v[j] = v[j] * inv * norm_w[j];
    __syncthreads();
    const int p = m.pos + pos_off;
    for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) {
        float sn, cs;
        sincosf((float)p * freqs[i], &sn, &cs);
        float* q = v + (hd - rd) + 2 * i;
        const float a = q[0], b = q[1];
        q[0] = a * cs - b * sn;
        q[1] = a * sn + b * cs;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    for (int b = threadIdx.x >> 5; b < hd / 32; b += blockDim.x >> 5) {
        const float t = v[b * 32 + lane];
        const float s = fp8_block_scale(warp_max(fabsf(t)));
        const float q = e4m3_rt(t / s) * s;
        if (ring) ring[((size_t)m.slot * cap + (p % cap)) * hd + b * 32 + lane] = __float2bfloat16_rn(q);
        if (rows_out) rows_out[(size_t)r * hd + b * 32 + lane] = q;
    }
}

__global__ void __launch_bounds__(128)
kv_append_kernel(const float* __restrict__ kv, int ld, const float* __restrict__ norm_w, const float* __restrict__ freqs,
                 const RowMeta* __restrict__ meta, __nv_bfloat16* __restrict__ ring, int cap, float* __restrict__ rows_out,
                 int hd, int rd, float eps, int pos_off) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    kv_append_body(sh, kv, ld, norm_w, freqs, meta, ring, cap, rows_out, hd, rd, eps, pos_off);
}

// ---- compressor ------------------------------------------------------------------------------------
// Phase 1: every row stores its raw (kv, score) at position % depth of the input ring.
// Phase 2: a row whose position completes a group pools the group's `ratio` positions with a
// per-channel softmax over the scores, RMS-normalises, and writes lat[r] (pre-RoPE) with
// flag[r] = 1; other rows get flag 0.  ratio == 1: lat = rmsnorm(kv), no ring.
__global__ void __launch_bounds__(512)
compress_kernel(const float* __restrict__ kv, const float* __restrict__ sc, int ld, const RowMeta* __restrict__ meta,
                float* __restrict__ ring_kv, float* __restrict__ ring_sc, int depth, const float* __restrict__ norm_w,
                float* __restrict__ lat, int* __restrict__ flag, int n, int hd, int ratio, float eps) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    if (ratio > 1) {
        for (int r = 0; r < n; ++r) {
            const RowMeta m = meta[r];
            const size_t o = ((size_t)m.slot * depth + (m.pos % depth)) * hd;
            for (int j = threadIdx.x; j < hd; j += blockDim.x) {
                ring_kv[o + j] = kv[(size_t)r * ld + j];
                ring_sc[o + j] = sc[(size_t)r * ld + j];
            }
        }
        __syncthreads();
    }
    for (int r = 0; r < n; ++r) {
        const RowMeta m = meta[r];
        const bool done = ((m.pos + 1) % ratio) == 0;
        if (threadIdx.x == 0) flag[r] = done ? 1 : 0;
        if (!done) continue;  // block-uniform
        float ss = 0.f;
        for (int j = threadIdx.x; j < hd; j += blockDim.x) {
            float v;
            if (ratio == 1) {
                v = kv[(size_t)r * ld + j];
            } else {
                float mx = -INFINITY;
                for (int i = 0; i < ratio; ++i)
                    mx = fmaxf(mx, ring_sc[((size_t)m.slot * depth + ((m.pos - i) % depth)) * hd + j]);
                float den = 0.f, num = 0.f;
                for (int i = ratio - 1; i >= 0; --i) {
                    const size_t o = ((size_t)m.slot * depth + ((m.pos - i) % depth)) * hd + j;
                    const float e = __expf(ring_sc[o] - mx);
                    den += e;
                    num += e * ring_kv[o];
                }
                v = num / den;
            }
            lat[(size_t)r * hd + j] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / hd + eps);
        for (int j = threadIdx.x; j < hd; j += blockDim.x) lat[(size_t)r * hd + j] *= inv * norm_w[j];
        __syncthreads();
    }
}

// Finished latents -> compressed-KV cache: rope at position (group * ratio), e2m1 per 16 with an
// e4m3 scale, row j = pos / ratio of the slot's cache.  Rows with flag 0 are skipped.
__global__ void __launch_bounds__(128)
latent_store_kernel(const float* __restrict__ lat, const int* __restrict__ flag, const RowMeta* __restrict__ meta,
                    const float* __restrict__ freqs, __nv_bfloat16* __restrict__ cache, int cap, int hd, int rd, int ratio) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* v = sh;
    const int r = blockIdx.x;
    if (!flag[r]) return;
    const RowMeta m = meta[r];
    const int j = m.pos / ratio;
    if (j >= cap) return;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) v[i] = lat[(size_t)r * hd + i];
    __syncthreads();
    const float p = (float)(j * ratio);
    for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(p * freqs[i], &sn, &cs);
        float* q = v + (hd - rd) + 2 * i;
        const float a = q[0], b = q[1];
        q[0] = a * cs - b * sn;
        q[1] = a * sn + b * cs;
    }
    __syncthreads();
    // 16-value groups: half-warps
    const int lane = threadIdx.x & 31, half = lane >> 4;
    for (int g = (threadIdx.x >> 5) * 2 + half; g < hd / 16; g += (blockDim.x >> 5) * 2) {
        const float t = v[g * 16 + (lane & 15)];
        float am = fabsf(t);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        const float s = e4m3_rt(fmaxf(am, 6.f * 0.001953125f) * (1.f / 6.f));
        cache[((size_t)m.slot * cap + j) * hd + g * 16 + (lane & 15)] = __float2bfloat16_rn(e2m1_rt(t / s) * s);
    }
}

// Index keys: kraw [n, id] = wk . latent (pre-RoPE latent) -> rmsnorm -> rope(group * ratio) ->
// e2m1 per 32 with power-of-two scales -> k cache row pos / ratio.
__global__ void __launch_bounds__(128)
index_k_store_kernel(const float* __restrict__ kraw, int ld, const int* __restrict__ flag, const RowMeta* __restrict__ meta,
                     const float* __restrict__ norm_w, const float* __restrict__ freqs, __nv_bfloat16* __restrict__ cache,
                     int cap, int id, int rd, int ratio, float eps) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* red = sh;
    float* v = sh + 32;
    const int r = blockIdx.x;
    if (!flag[r]) return;
    const RowMeta m = meta[r];
    const int j = m.pos / ratio;
    if (j >= cap) return;
    float ss = 0.f;
    for (int i = threadIdx.x; i < id; i += blockDim.x) {
        const float t = kraw[(size_t)r * ld + i];
        v[i] = t;
        ss += t * t;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / id + eps);
    for (int i = threadIdx.x; i < id; i += blockDim.x) v[i] = v[i] * inv * norm_w[i];
    __syncthreads();
    const float p = (float)(j * ratio);
    for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(p * freqs[i], &sn, &cs);
        float* q = v + (id - rd) + 2 * i;
        const float a = q[0], b = q[1];
        q[0] = a * cs - b * sn;
        q[1] = a * sn + b * cs;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    for (int b = threadIdx.x >> 5; b < id / 32; b += blockDim.x >> 5) {
        const float t = v[b * 32 + lane];
        const float s = pow2_ceil(fmaxf(warp_max(fabsf(t)), 6.f * 1.17549435e-38f) * (1.f / 6.f));
        cache[((size_t)m.slot * cap + j) * id + b * 32 + lane] = __float2bfloat16_rn(e2m1_rt(t / s) * s);
    }
}

}  // namespace

namespace {

// ---- indexer ------------------------------------------------------------------------------------
// score[r][j] = sum_h relu(q[r][h] . k[j]) * w[r][h] for j < clen(r) = (pos + 1) / ratio, -inf beyond,
// over this rank's heads (the caller all-reduces across ranks).  One lane per head, keys
// broadcast from shared memory; q rows padded by one float against bank conflicts.
__global__ void __launch_bounds__(256)
index_score_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ w, int ldw,
                   const __nv_bfloat16* __restrict__ kc, int cap, const RowMeta* __restrict__ meta,
                   float* __restrict__ score, int lds, int heads, int id, int ratio, float wscale) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* qs = sh;                          // [heads][id + 1]
    float* ks = sh + heads * (id + 1);       // [8 warps][id]
    const int r = blockIdx.y;
    const RowMeta m = meta[r];
    const int clen = (m.pos + 1) / ratio;
    const int per = (blockDim.x >> 5) * 4;
    const int j0 = blockIdx.x * per;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (j0 >= min(cap, lds)) return;
    if (j0 >= clen) {  // whole block beyond the visible range
        for (int j = j0 + threadIdx.x; j < min(j0 + per, lds); j += blockDim.x) score[(size_t)r * lds + j] = -INFINITY;
        return;
    }
    for (int i = threadIdx.x; i < heads * id; i += blockDim.x) qs[(i / id) * (id + 1) + (i % id)] = q[(size_t)r * ldq + i];
    __syncthreads();
    const float wh = lane < heads ? w[(size_t)r * ldw + lane] * wscale : 0.f;
    float* kw = ks + warp * id;
    for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + warp * 4 + jj;
        if (j >= lds) break;
        if (j >= clen) { if (lane == 0) score[(size_t)r * lds + j] = -INFINITY; continue; }
        __syncwarp();
        for (int e = lane; e < id; e += 32) kw[e] = __bfloat162float(kc[((size_t)m.slot * cap + j) * id + e]);
        __syncwarp();
        float acc = 0.f;
        for (int h = lane; h < heads; h += 32) {   // heads <= 32 in every shipped config; loop keeps it general
            float d = 0.f;
            const float* qh = qs + h * (id + 1);
            for (int e = 0; e < id; ++e) d = fmaf(qh[e], kw[e], d);
            const float whh = (h == lane) ? wh : w[(size_t)r * ldw + h] * wscale;
            acc += fmaxf(d, 0.f) * whh;
        }
        acc = warp_sum(acc);
        if (lane == 0) score[(size_t)r * lds + j] = acc;
    }
}

__device__ __forceinline__ uint32_t ordered_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Block-wide exclusive scan of one int per thread (blockDim.x <= 1024); returns the exclusive
// prefix and writes the block total to *total.
__device__ __forceinline__ int block_excl_scan(int v, int* wsum, int* total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += t;
    }
    __syncthreads();
    if (lane == 31) wsum[wid] = x;
    __syncthreads();
    if (wid == 0) {
        int s = lane < nw ? wsum[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += t;
        }
        wsum[lane] = s;  // inclusive warp totals
    }
    __syncthreads();
    const int base = wid ? wsum[wid - 1] : 0;
    *total = wsum[nw - 1];
    return base + x - v;
}

// Top-k of each row by (score descending, index ascending), emitted in index order, -1 padded.
// len(r) = ceil(((pos + 1) / ratio) / div); entries whose mask byte is 0 count as -inf.
// Four 8-bit radix passes find the k-th key, one ordered pass emits.
__global__ void __launch_bounds__(1024)
topk_sorted_kernel(const float* __restrict__ score, int lds, const uint8_t* __restrict__ mask, int ldm,
                   const RowMeta* __restrict__ meta, int ratio, int div, int k, int* __restrict__ out, int ldo) {
    PDL_PROLOGUE();
    __shared__ int hist[256];
    __shared__ int wsum[32];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need, s_written, s_eq_taken;
    const int r = blockIdx.x;
    const int clen = (meta[r].pos + 1) / ratio;
    const int len = min((clen + div - 1) / div, lds);
    const float* sc = score + (size_t)r * lds;
    const uint8_t* mk = mask ? mask + (size_t)r * ldm : nullptr;
    int* o = out + (size_t)r * ldo;
    const int kk = min(k, len);
    auto key_at = [&](int j) -> uint32_t {
        const float v = (mk && !mk[j]) ? -INFINITY : sc[j];
        return ordered_key(v);
    };
    uint32_t T = 0;
    int need_eq = 0;
    if (kk < len) {
        // k-th largest key: walk the digits from the top
        if (threadIdx.x == 0) { s_prefix = 0; s_need = kk; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix;
            const uint32_t pmask = pass ? (0xffffffffu << (shift + 8)) : 0u;
            for (int j = threadIdx.x; j < len; j += blockDim.x) {
                const uint32_t key = key_at(j);
                if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int need = s_need, d = 255;
                for (; d > 0; --d) {
                    if (hist[d] >= need) break;
                    need -= hist[d];
                }
                s_need = need;
                s_prefix = prefix | ((uint32_t)d << shift);
            }
            __syncthreads();
        }
        T = s_prefix;
        need_eq = s_need;  // how many entries equal to T are taken (the lowest indices)
    }
    if (threadIdx.x == 0) { s_written = 0; s_eq_taken = 0; }
    __syncthreads();
    for (int j0 = 0; j0 < len; j0 += blockDim.x) {
        const int j = j0 + threadIdx.x;
        int gt = 0, eq = 0;
        if (j < len) {
            if (kk >= len) gt = 1;
            else {
                const uint32_t key = key_at(j);
                gt = key > T;
                eq = key == T;
            }
        }
        int tot_eq, tot_sel;
        const int eq_before = block_excl_scan(eq, wsum, &tot_eq) + s_eq_taken;
        const int sel = gt || (eq && eq_before < need_eq);
        __syncthreads();
        const int pos = block_excl_scan(sel, wsum, &tot_sel) + s_written;
        if (sel && pos < ldo) o[pos] = j;
        __syncthreads();
        if (threadIdx.x == 0) { s_written += tot_sel; s_eq_taken += tot_eq; }
        __syncthreads();
    }
    for (int i = s_written + threadIdx.x; i < min(k, ldo); i += blockDim.x) o[i] = -1;
}

// Block scores for the candidate level: max over each `bs` positions below clen, the block
// holding the newest visible position pinned to +inf.
__global__ void __launch_bounds__(256)
block_max_kernel(const float* __restrict__ score, int lds, const RowMeta* __restrict__ meta, int ratio, int bs,
                 float* __restrict__ out, int ldo) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int clen = (meta[r].pos + 1) / ratio;
    const int nb = (clen + bs - 1) / bs;
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= ldo) return;
    float v = -INFINITY;
    if (b < nb) {
        for (int i = 0; i < bs; ++i) {
            const int j = b * bs + i;
            if (j < clen && j < lds) v = fmaxf(v, score[(size_t)r * lds + j]);
        }
        if (b == (clen - 1) / bs) v = INFINITY;
    }
    out[(size_t)r * ldo + b] = v;
}

// mask[r][j] = 1 for positions inside the selected blocks (mask is cleared by the caller).
__global__ void __launch_bounds__(256)
cand_mask_kernel(const int* __restrict__ blk, int ldb, int kb, int bs, uint8_t* __restrict__ mask, int ldm) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= kb * bs) return;
    const int b = blk[(size_t)r * ldb + t / bs];
    if (b < 0) return;
    const int j = b * bs + t % bs;
    if (j < ldm) mask[(size_t)r * ldm + j] = 1;
}

// ---- sparse attention with a sink ----------------------------------------------------------------
// One CTA per (row, tile of 8 heads), one warp per head.  Keys: the row's window positions from
// the ring, the selected compressed rows, then `n_extra` plain rows (a draft block's own KV).
// Lane i of a warp owns elements {2i + 64j, 2i + 1 + 64j}: adjacent pairs (the RoPE pairs) and
// conflict-free 4-byte reads of a staged bf16 key.  q is rotated on load, the output gets the
// inverse rotation; softmax runs online with max over the real keys only, the sink logit
// joins the denominator at the end, a row without keys yields zeros.
constexpr int kAttnTile = 8;
constexpr int kAttnStage = 48;   // keys staged per pass (48 KB of shared memory at head_dim 512)
// CL: launched as clusters of kAttnCluster CTAs along the split axis.  The CTAs of a cluster exchange their partials
// through distributed shared memory (CTA c merges head c of the tile: the merge of a cluster runs on eight SMs side by
// side) and global memory only sees one partial per cluster; one CTA merging all splits of eight heads is bound by one
// SM's L2 bandwidth (32 splits x 8 heads x 2 KB).
constexpr int kAttnCluster = 8;
template <int NJ, bool CL>  // NJ = head_dim / 64
__global__ void __launch_bounds__(256)
sparse_attn_kernel(const float* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ ring, int cap, int window,
                   const __nv_bfloat16* __restrict__ comp, int ccap, const int* __restrict__ idx, int ldi, int ktop,
                   const float* __restrict__ extra, int n_extra, const float* __restrict__ sink,
                   const float* __restrict__ freqs, int rd, const RowMeta* __restrict__ meta, int pos_off, int win_mode,
                   float scale, int heads, int nsplit, float* __restrict__ o_part, float* __restrict__ ml_part,
                   unsigned* __restrict__ ticket, float* __restrict__ out, int ldo, SplitBuf osp) {
    PDL_PROLOGUE();
    constexpr int HD = NJ * 64;
    extern __shared__ __align__(16) uint32_t ktile[];   // [kAttnStage][HD / 2] staged bf16 keys
    __shared__ int kvalid[kAttnStage];
    __shared__ int s_last;
    const int r = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x * 8 + warp;
    const bool hv = h < heads;
    const RowMeta m = meta[r];
    const int pos = m.pos + pos_off;          // position of the query (RoPE)
    const int wpos = win_mode ? m.ctx0 - 1 : m.pos;  // newest window position visible to the query (mode 1: the
                                                     // rows of a draft block all see the window up to the block's start)
    const int nw = min(wpos + 1, window);
    const int L = max(nw, 0) + ktop + n_extra;
    // rotation factors of this lane's pairs
    float cs[NJ], sn[NJ];
    float qv[NJ][2];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = 2 * lane + 64 * j;
        cs[j] = 1.f; sn[j] = 0.f;
        if (e >= HD - rd) sincosf((float)pos * freqs[(e - (HD - rd)) >> 1], &sn[j], &cs[j]);
        const float a = hv ? q[(size_t)r * ldq + (size_t)h * HD + e] : 0.f;
        const float b = hv ? q[(size_t)r * ldq + (size_t)h * HD + e + 1] : 0.f;
        qv[j][0] = (a * cs[j] - b * sn[j]) * scale;
        qv[j][1] = (a * sn[j] + b * cs[j]) * scale;
    }
    float mx = -1e30f, den = 0.f;
    float ov[NJ][2];
#pragma unroll
    for (int j = 0; j < NJ; ++j) ov[j][0] = ov[j][1] = 0.f;
    // this CTA's share of the key list (split-K over blockIdx.z).  The share is staged in passes of up to kAttnStage
    // keys: every warp issues the 16-byte loads of its keys back to back, so a pass costs one memory latency, and
    // the 8-key tiles of the pass are then consumed from shared memory.
    const int sp = blockIdx.z;
    const int per = ((L + nsplit - 1) / nsplit + kAttnTile - 1) / kAttnTile * kAttnTile;
    const int k_lo = sp * per, k_hi = min(L, k_lo + per);
    for (int base = k_lo; base < k_hi; base += kAttnStage) {
        const int cnt = min(kAttnStage, k_hi - base);
        const int cnt8 = (cnt + kAttnTile - 1) / kAttnTile * kAttnTile;
        __syncthreads();
        // Lane u < KPW resolves the source of key (warp + 8u) of this pass (the index loads of a warp's keys go out
        // together); the warp then issues the 16-byte loads of ALL its keys before the first store, so a pass costs
        // one index latency plus one key latency however many keys a warp stages.
        constexpr int KPW = kAttnStage / 8;            // keys per warp and pass
        constexpr int VW = (HD / 8 + 31) / 32;         // 16-byte words per lane and key
        const __nv_bfloat16* my_src = nullptr;
        const float* my_srcf = nullptr;
        {
            const int t = warp + 8 * lane, i = base + t;
            if (lane < KPW && t < cnt) {
                if (i < nw) {
                    const int p = wpos - nw + 1 + i;
                    my_src = ring + ((size_t)m.slot * cap + (p % cap)) * HD;
                } else if (i < nw + ktop) {
                    const int c = idx[(size_t)r * ldi + (i - nw)];
                    if (c >= 0 && c < ccap) my_src = comp + ((size_t)m.slot * ccap + c) * HD;
                } else {
                    my_srcf = extra + (size_t)(i - nw - ktop) * HD;
                }
            }
        }
        uint4 kv[KPW][VW];
        unsigned long long sp[KPW];
#pragma unroll
        for (int u = 0; u < KPW; ++u) {
            sp[u] = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_src, u);
#pragma unroll
            for (int w = 0; w < VW; ++w) {
                kv[u][w] = make_uint4(0u, 0u, 0u, 0u);   // a masked key must not feed NaN into 0 * k
                if (sp[u] && lane + 32 * w < HD / 8) kv[u][w] = __ldg(reinterpret_cast<const uint4*>(sp[u]) + lane + 32 * w);
            }
        }
#pragma unroll
        for (int u = 0; u < KPW; ++u) {
            const int t = warp + 8 * u;
            const unsigned long long sf = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_srcf, u);
            if (t >= cnt8) continue;
            uint32_t* dst = ktile + (size_t)t * (HD / 2);
            if (lane == 0) kvalid[t] = (sp[u] || sf) ? 1 : 0;
            if (sf) {   // a draft block's own row, kept in f32
                const float* srcf = reinterpret_cast<const float*>(sf);
                for (int e = lane; e < HD / 2; e += 32) {
                    const __nv_bfloat162 v = __floats2bfloat162_rn(srcf[2 * e], srcf[2 * e + 1]);
                    dst[e] = *reinterpret_cast<const uint32_t*>(&v);
                }
            } else {
#pragma unroll
                for (int w = 0; w < VW; ++w)
                    if (lane + 32 * w < HD / 8) reinterpret_cast<uint4*>(dst)[lane + 32 * w] = kv[u][w];
            }
        }
        __syncthreads();
        for (int t0 = 0; t0 < cnt; t0 += kAttnTile) {
            const uint32_t* kt = ktile + (size_t)t0 * (HD / 2);
            float sc[kAttnTile];
            float tmax = -INFINITY;
#pragma unroll
            for (int t = 0; t < kAttnTile; ++t) {
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const uint32_t kw = kt[t * (HD / 2) + lane + 32 * j];
                    d = fmaf(qv[j][0], bf16lo(kw), d);
                    d = fmaf(qv[j][1], bf16hi(kw), d);
                }
                sc[t] = d;
            }
#pragma unroll
            for (int t = 0; t < kAttnTile; ++t) {
                sc[t] = warp_sum(sc[t]);
                if (!kvalid[t0 + t] || t0 + t >= cnt) sc[t] = -INFINITY;
                tmax = fmaxf(tmax, sc[t]);
            }
            const float mnew = fmaxf(mx, tmax);
            const float resc = __expf(mx - mnew);
            den *= resc;
#pragma unroll
            for (int j = 0; j < NJ; ++j) { ov[j][0] *= resc; ov[j][1] *= resc; }
#pragma unroll
            for (int t = 0; t < kAttnTile; ++t) {
                const float p = __expf(sc[t] - mnew);  // exp(-inf) = 0 for masked keys
                den += p;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const uint32_t kw = kt[t * (HD / 2) + lane + 32 * j];
                    ov[j][0] = fmaf(p, bf16lo(kw), ov[j][0]);
                    ov[j][1] = fmaf(p, bf16hi(kw), ov[j][1]);
                }
            }
            mx = mnew;
        }
    }
    // un-normalised partial of this split: o (already rotated keys), running max and denominator
    if constexpr (CL) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        constexpr int PS = HD + 8;                            // floats per staged partial: o, max, denominator
        float* ps = reinterpret_cast<float*>(ktile);          // [8 heads][PS]: this CTA's partials
        float* ps2 = ps + 8 * PS;                             // [8 CTAs][PS]: the cluster's partials of MY head
        __syncthreads();                                      // the key tile is no longer read
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            *reinterpret_cast<float2*>(ps + warp * PS + 2 * lane + 64 * j) = make_float2(ov[j][0], ov[j][1]);
        if (lane == 0) { ps[warp * PS + HD] = mx; ps[warp * PS + HD + 1] = den; }
        cluster.sync();
        const int cr = (int)cluster.block_rank();             // head of the tile that this CTA merges
        {
            const float* rp = cluster.map_shared_rank(ps, warp) + cr * PS;   // CTA `warp`'s partial of head cr
            float2 po[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) po[j] = *reinterpret_cast<const float2*>(rp + 2 * lane + 64 * j);
            const float pm = rp[HD], pd = rp[HD + 1];
#pragma unroll
            for (int j = 0; j < NJ; ++j) *reinterpret_cast<float2*>(ps2 + warp * PS + 2 * lane + 64 * j) = po[j];
            if (lane == 0) { ps2[warp * PS + HD] = pm; ps2[warp * PS + HD + 1] = pd; }
        }
        __syncthreads();
        const int hc = blockIdx.x * 8 + cr;
        const int nparts = nsplit / kAttnCluster;
        if (hc < heads) {
            float Mc = -1e30f;
#pragma unroll
            for (int w = 0; w < kAttnCluster; ++w) Mc = fmaxf(Mc, ps2[w * PS + HD]);
            float wgt[kAttnCluster], dc = 0.f;
#pragma unroll
            for (int w = 0; w < kAttnCluster; ++w) { wgt[w] = __expf(ps2[w * PS + HD] - Mc); dc = fmaf(ps2[w * PS + HD + 1], wgt[w], dc); }
            const size_t pi = ((size_t)r * heads + hc) * nparts + sp / kAttnCluster;
            for (int e2 = threadIdx.x; e2 < HD / 2; e2 += 256) {
                float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int w = 0; w < kAttnCluster; ++w) {
                    const float2 v = *reinterpret_cast<const float2*>(ps2 + w * PS + 2 * e2);
                    acc.x = fmaf(v.x, wgt[w], acc.x);
                    acc.y = fmaf(v.y, wgt[w], acc.y);
                }
                *reinterpret_cast<float2*>(o_part + pi * HD + 2 * e2) = acc;
            }
            if (threadIdx.x == 0) { ml_part[pi * 2] = Mc; ml_part[pi * 2 + 1] = dc; }
        }
        cluster.sync();                                       // nobody leaves while its partials may still be read
        nsplit = nparts;                                      // what the final merge below sees
    }
    const size_t p0 = ((size_t)r * heads + h) * nsplit;
    if (!CL && hv) {
        const size_t pi = p0 + sp;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = 2 * lane + 64 * j;
            *reinterpret_cast<float2*>(o_part + pi * HD + e) = make_float2(ov[j][0], ov[j][1]);
        }
        if (lane == 0) { ml_part[pi * 2] = mx; ml_part[pi * 2 + 1] = den; }
    }
    if (!ticket) return;   // the partials are merged by a second kernel
    // The CTA that finishes a (row, head tile) last merges its splits: max-shifted sum, the sink logit joins the
    // denominator, the output gets the inverse rotation (this lane's factors are the ones computed above).
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* tk = ticket + (size_t)r * gridDim.x + blockIdx.x;
        const unsigned t = atomicAdd(tk, 1u);
        s_last = (t == gridDim.z - 1u) ? 1 : 0;
        if (s_last) *tk = 0u;   // every CTA of the group has taken its ticket
    }
    __syncthreads();
    if (!s_last || !hv) return;
    __threadfence();
    // lane s holds split s's (max, denominator): one round trip for all of them; the partial outputs then come in
    // groups of four splits whose loads are all issued before the first is used (a split per iteration would pay one
    // L2 latency per split)
    float2 mlv = make_float2(-1e30f, 0.f);
    if (lane < nsplit) mlv = __ldcg(reinterpret_cast<const float2*>(ml_part + (p0 + lane) * 2));
    const float M = warp_max(mlv.x);
    const float wl = lane < nsplit ? __expf(mlv.x - M) : 0.f;
    const float dsum = __expf(sink[h] - M) + warp_sum(mlv.y * wl);
    float a[NJ], b[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) a[j] = b[j] = 0.f;
    for (int s0 = 0; s0 < nsplit; s0 += 4) {
        float2 o[4][NJ];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int s = min(s0 + u, nsplit - 1);
#pragma unroll
            for (int j = 0; j < NJ; ++j)
                o[u][j] = __ldcg(reinterpret_cast<const float2*>(o_part + (p0 + s) * HD + 2 * lane + 64 * j));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float w = s0 + u < nsplit ? __shfl_sync(0xffffffffu, wl, (s0 + u) & 31) : 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                a[j] = fmaf(o[u][j].x, w, a[j]);
                b[j] = fmaf(o[u][j].y, w, b[j]);
            }
        }
    }
    const float inv = 1.f / dsum;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = 2 * lane + 64 * j;
        const float x = a[j] * inv, y = b[j] * inv;
        const float x0 = x * cs[j] + y * sn[j], x1 = -x * sn[j] + y * cs[j];   // inverse rotation (identity where cs = 1, sn = 0)
        float* o = out + (size_t)r * ldo + (size_t)h * HD + e;
        o[0] = x0;
        o[1] = x1;
        split_store(osp, r, h * HD + e, x0);
        split_store(osp, r, h * HD + e + 1, x1);
    }
}

// Merge of the split-K partials: max-shifted sum, the sink logit joins the denominator, the output gets
// the inverse rotation.  grid (heads, rows), 128 threads, one adjacent pair per thread step.
__global__ void __launch_bounds__(128)
sparse_attn_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, const float* __restrict__ sink,
                         const float* __restrict__ freqs, int rd, const RowMeta* __restrict__ meta, int pos_off, int heads,
                         int hd, int nsplit, float* __restrict__ out, int ldo, SplitBuf osp) {
    PDL_PROLOGUE();
    const int h = blockIdx.x, r = blockIdx.y;
    const size_t p0 = ((size_t)r * heads + h) * nsplit;
    float M = -1e30f;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml_part[(p0 + s) * 2]);
    float den = __expf(sink[h] - M);
    for (int s = 0; s < nsplit; ++s) den += ml_part[(p0 + s) * 2 + 1] * __expf(ml_part[(p0 + s) * 2] - M);
    const float inv = 1.f / den;
    const float pos = (float)(meta[r].pos + pos_off);
    for (int e = 2 * threadIdx.x; e < hd; e += 2 * blockDim.x) {
        float a = 0.f, b = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float w = __expf(ml_part[(p0 + s) * 2] - M);
            a = fmaf(o_part[(p0 + s) * hd + e], w, a);
            b = fmaf(o_part[(p0 + s) * hd + e + 1], w, b);
        }
        a *= inv; b *= inv;
        float x0 = a, x1 = b;
        if (e >= hd - rd) {
            float sn, cs;
            sincosf(pos * freqs[(e - (hd - rd)) >> 1], &sn, &cs);
            x0 = a * cs + b * sn;    // inverse rotation
            x1 = -a * sn + b * cs;
        }
        float* o = out + (size_t)r * ldo + (size_t)h * hd + e;
        o[0] = x0;
        o[1] = x1;
        split_store(osp, r, h * hd + e, x0);
        split_store(osp, r, h * hd + e + 1, x1);
    }
}

}  // namespace

namespace {

// ---- MoE route: sqrt(softplus) scores, bias only for selection, normalised, scaled -------------
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, const float* __restrict__ bias_vl,
             const uint8_t* __restrict__ is_image, int E, int topk, float route_scale, int* __restrict__ idx,
             float* __restrict__ wts) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* sc = sh;        // E scores
    float* sel = sh + E;   // E selection values
    __shared__ float red[32];
    __shared__ int s_best;
    const int r = blockIdx.x;
    const float* b = (bias_vl && is_image && is_image[r]) ? bias_vl : bias;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float x = logits[(size_t)r * ld + e];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        const float s = sqrtf(sp);
        sc[e] = s;
        sel[e] = s + b[e];
    }
    __syncthreads();
    float wsum = 0.f;
    for (int k = 0; k < topk; ++k) {
        float best = -INFINITY;
        int bi = E;
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const float v = sel[e];
            if (v > best || (v == best && e < bi)) { best = v; bi = e; }
        }
        // block argmax with the lower index winning ties
        const float bm = block_max(best, red);
        int cand = (best == bm) ? bi : E;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __syncthreads();
        if (threadIdx.x == 0) s_best = E;
        __syncthreads();
        if ((threadIdx.x & 31) == 0) atomicMin(&s_best, cand);
        __syncthreads();
        const int e = s_best;
        if (threadIdx.x == 0) {
            idx[(size_t)r * topk + k] = e;
            wts[(size_t)r * topk + k] = sc[e];
            sel[e] = -INFINITY;
        }
        wsum += sc[e];
        __syncthreads();
    }
    if (threadIdx.x < topk) {
        float w = wts[(size_t)r * topk + threadIdx.x];
        if (topk > 1) w = w / (wsum + 1e-20f);
        wts[(size_t)r * topk + threadIdx.x] = w * route_scale;
    }
}

// ---- fp4 experts ---------------------------------------------------------------------------------
// Weights: e2m1 packed two per byte (even k in the low nibble) with one ue8m0 byte per 32 values
// of K, per row.  Activations arrive already e4m3-per-32 round-tripped (f32).
__device__ __forceinline__ void fp4x8_to_f32(uint32_t p, float* o) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((p >> (8 * i)) & 0xffu), __NV_E2M1);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ float ue8m0_f32(uint8_t b) { return __uint_as_float((uint32_t)b << 23); }

// Activations sit in shared memory "chunk-transposed": value k of a row of K is at
// xs[(k % 16) * (K / 16 + 1) + k / 16], so the 32 lanes of a warp, which work on 32 different 16-value
// chunks, read 32 consecutive words (no bank conflicts; a lane-major layout would be 16-way conflicted).
__device__ __forceinline__ float fp4x16_dot(uint2 p, const float* __restrict__ xs, int c, int stride) {
    float v[16];
    fp4x8_to_f32(p.x, v);
    fp4x8_to_f32(p.y, v + 8);
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) d = fmaf(v[i], xs[i * stride + c], d);
    return d;
}
__device__ __forceinline__ void stage_transposed(float* __restrict__ xs, const float* __restrict__ x, int K) {
    const int stride = K / 16 + 1;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[(k & 15) * stride + (k >> 4)] = x[k];
}

// dot of one packed fp4 row (K values, scales per 32) with x (shared memory, chunk-transposed); whole
// warp.  Four 8-byte loads are in flight per lane before the first is consumed.
__device__ __forceinline__ float fp4_row_dot(const uint8_t* __restrict__ wrow, const uint8_t* __restrict__ srow,
                                             const float* __restrict__ xs, int K, int lane) {
    float acc = 0.f;
    const int nc = K / 16, stride = nc + 1;
    int c = lane;
    for (; c + 96 < nc; c += 128) {
        uint2 p[4];
        uint8_t sc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            p[u] = *reinterpret_cast<const uint2*>(wrow + (size_t)(c + 32 * u) * 8);
            sc[u] = srow[(c + 32 * u) >> 1];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) acc = fmaf(fp4x16_dot(p[u], xs, c + 32 * u, stride), ue8m0_f32(sc[u]), acc);
    }
    for (; c < nc; c += 32) {
        const uint2 p = *reinterpret_cast<const uint2*>(wrow + (size_t)c * 8);
        acc = fmaf(fp4x16_dot(p, xs, c, stride), ue8m0_f32(srow[c >> 1]), acc);
    }
    return warp_sum(acc);
}

// h[r][s][i] = silu(min(gate, lim)) * clamp(up, +-lim) * w[r][s]; gate/up rows i of expert idx[r][s].
// w13 [E][2][I][K/2], s13 [E][2][I][K/32].  grid (ceil(I/8), topk, rows), 8 warps = 8 rows i.
__global__ void __launch_bounds__(256)
expert_gate_up_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ idx, const float* __restrict__ wts,
                      const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13, float* __restrict__ h,
                      int topk, int I, int K, float lim) {
    PDL_PROLOGUE();
    extern __shared__ float xs[];
    const int r = blockIdx.z, s = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    stage_transposed(xs, x + (size_t)r * ldx, K);
    __syncthreads();
    const int i = blockIdx.x * 8 + warp;
    if (i >= I) return;
    const int e = idx[(size_t)r * topk + s];
    const size_t wrow = (size_t)K / 2, srow = (size_t)K / 32;
    const uint8_t* wg = w13 + ((size_t)e * 2 * I + i) * wrow;
    const uint8_t* wu = w13 + ((size_t)e * 2 * I + I + i) * wrow;
    const uint8_t* sg = s13 + ((size_t)e * 2 * I + i) * srow;
    const uint8_t* su = s13 + ((size_t)e * 2 * I + I + i) * srow;
    float g = fp4_row_dot(wg, sg, xs, K, lane);
    float u = fp4_row_dot(wu, su, xs, K, lane);
    if (lane == 0) {
        if (lim > 0.f) { u = fminf(fmaxf(u, -lim), lim); g = fminf(g, lim); }
        h[((size_t)r * topk + s) * I + i] = siluf_(g) * u * wts[(size_t)r * topk + s];
    }
}

// y[r][c] (+)= sum_s w2[idx[r][s]][c] . hq[r][s]   (hq already e4m3 round-tripped).
// w2 [E][D][I/2], s2 [E][D][I/32].  grid (ceil(D/8), rows).
__global__ void __launch_bounds__(256)
expert_down_kernel(const float* __restrict__ hq, const int* __restrict__ idx, const uint8_t* __restrict__ w2,
                   const uint8_t* __restrict__ s2, float* __restrict__ y, int ldy, int topk, int I, int D, int accumulate) {
    PDL_PROLOGUE();
    extern __shared__ float hs[];  // [topk] chunk-transposed rows of I values
    const int r = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hstride = 16 * (I / 16 + 1);
    for (int s = 0; s < topk; ++s) stage_transposed(hs + (size_t)s * hstride, hq + ((size_t)r * topk + s) * I, I);
    __syncthreads();
    const int c = blockIdx.x * 8 + warp;
    if (c >= D) return;
    // lanes walk the flattened (slot, 16-value chunk) list so that short rows still fill the warp
    const int nc = I / 16, items = topk * nc;
    float acc = 0.f;
    for (int it = lane; it < items; it += 128) {
        uint2 p[4];
        float sc[4];
        const float* xp[4];
        int xc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = it + 32 * u;
            p[u] = make_uint2(0u, 0u);
            sc[u] = 0.f;
            xp[u] = hs;
            xc[u] = 0;
            if (j < items) {
                const int s = j / nc, ch = j % nc;
                const int e = idx[(size_t)r * topk + s];
                p[u] = *reinterpret_cast<const uint2*>(w2 + ((size_t)e * D + c) * (I / 2) + (size_t)ch * 8);
                sc[u] = ue8m0_f32(s2[((size_t)e * D + c) * (I / 32) + (ch >> 1)]);
                xp[u] = hs + (size_t)s * hstride;
                xc[u] = ch;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) acc = fmaf(fp4x16_dot(p[u], xp[u], xc[u], nc + 1), sc[u], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        float* o = y + (size_t)r * ldy + c;
        *o = accumulate ? *o + acc : acc;
    }
}

// SwiGLU with clamps on a fused [gate | up] row (shared expert): out = silu(min(g, lim)) * clamp(u).
__global__ void __launch_bounds__(256)
swiglu_clamp_kernel(const float* __restrict__ gu, int ld, float* __restrict__ out, int ldo, int n, int I, float lim) {
    PDL_PROLOGUE();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n * I) return;
    const int r = t / I, i = t % I;
    float g = gu[(size_t)r * ld + i], u = gu[(size_t)r * ld + I + i];
    if (lim > 0.f) { u = fminf(fmaxf(u, -lim), lim); g = fminf(g, lim); }
    out[(size_t)r * ldo + i] = siluf_(g) * u;
}

// RMSNorm of a row slice followed by the e4m3-per-32 round trip (the q-lora vector on its way to wq_b):
// out = rt(x * rsqrt(mean x^2 + eps) * w).  One CTA per row, a warp per 32-value block.
__device__ __forceinline__ void rmsnorm_quant_body(float* red, const float* __restrict__ x, int ldx, const float* __restrict__ w,
                                                   float* __restrict__ out, int ldo, int K, float eps, SplitBuf osp) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = x + (size_t)r * ldx;
    float ss = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) { const float v = row[k]; ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / K + eps);
    for (int b = warp; b < K / 32; b += blockDim.x >> 5) {
        const int k = b * 32 + lane;
        const float v = row[k] * inv * w[k];
        const float s = fp8_block_scale(warp_max(fabsf(v)));
        const float q = e4m3_rt(v / s) * s;
        out[(size_t)r * ldo + k] = q;
        split_store(osp, r, k, q);
    }
}

__global__ void __launch_bounds__(256)
rmsnorm_quant_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, float* __restrict__ out, int ldo,
                     int K, float eps, SplitBuf osp) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    rmsnorm_quant_body(red, x, ldx, w, out, ldo, K, eps, osp);
}

// The two consumers of the fused q-lora | kv projection in one launch, grid (rows, 2): CTA (r, 0) normalises and
// quantises the q-lora slice of row r (rmsnorm_quant), CTA (r, 1) normalises, rotates, quantises and stores its kv
// slice (kv_append).  Neither depends on the other; apart they cost a launch each on the decode critical path.
__global__ void __launch_bounds__(256)
qnorm_kv_append_kernel(const float* __restrict__ qa, int ld, int ql, const float* __restrict__ q_w, float* __restrict__ q_out,
                       int ldo, float eps, SplitBuf osp, const float* __restrict__ kv_w, const float* __restrict__ freqs,
                       const RowMeta* __restrict__ meta, __nv_bfloat16* __restrict__ ring, int cap,
                       float* __restrict__ rows_out, int hd, int rd, int pos_off) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    if (blockIdx.y == 0) rmsnorm_quant_body(sh, qa, ld, q_w, q_out, ldo, ql, eps, osp);
    else kv_append_body(sh, qa + ql, ld, kv_w, freqs, meta, ring, cap, rows_out, hd, rd, eps, pos_off);
}

// Shared expert: SwiGLU with clamps, then the e4m3-per-32 round trip of the result (f32 + split planes).
// One warp per 32-value block.
__device__ __forceinline__ void swiglu_clamp_quant_body(const float* __restrict__ gu, int ld, float* __restrict__ out, int ldo,
                                                        int n, int I, float lim, SplitBuf osp, int block) {
    const int lane = threadIdx.x & 31;
    const int nb = I / 32;
    const int w = block * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n * nb) return;
    const int r = w / nb, i = (w % nb) * 32 + lane;
    float g = gu[(size_t)r * ld + i], u = gu[(size_t)r * ld + I + i];
    if (lim > 0.f) { u = fminf(fmaxf(u, -lim), lim); g = fminf(g, lim); }
    const float v = siluf_(g) * u;
    const float s = fp8_block_scale(warp_max(fabsf(v)));
    const float q = e4m3_rt(v / s) * s;
    out[(size_t)r * ldo + i] = q;
    split_store(osp, r, i, q);
}

__global__ void __launch_bounds__(256)
swiglu_clamp_quant_kernel(const float* __restrict__ gu, int ld, float* __restrict__ out, int ldo, int n, int I, float lim,
                          SplitBuf osp) {
    PDL_PROLOGUE();
    swiglu_clamp_quant_body(gu, ld, out, ldo, n, I, lim, osp, (int)blockIdx.x);
}

// ---- MoE route without block-wide barriers in the pick loop ---------------------------------------
// The same selection as route_kernel (sqrt(softplus) scores, bias only for the selection, ties to the lower
// expert, weights of the picks normalised in pick order).  The whole block computes the scores (shared memory),
// then ONE warp picks: lane l holds experts l, l + 32, ... (E <= 32 * kRouteSlots) as order-preserving 32-bit
// keys; a pick is a register scan, a warp-wide integer maximum, and a warp-wide minimum over the indices that
// hold it (two redux instructions).  The block-wide form takes six barriers per pick.
constexpr int kRouteSlots = 12;
__device__ __forceinline__ void route_row_block_d4(const float* __restrict__ lrow, const float* __restrict__ b, int E, int topk,
                                                   float route_scale, int* __restrict__ idx_row, float* __restrict__ wts_row,
                                                   uint32_t* u_s, float* sc_s) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float x = lrow[e];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        const float v = sqrtf(sp);
        const float sv = v + b[e];
        uint32_t u = __float_as_uint(sv);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // order-preserving map of finite and infinite floats
        if (sv != sv) u = 1u;                             // NaN: below every number; 0 = not (or no longer) a candidate
        sc_s[e] = v;
        u_s[e] = u;
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    float sc[kRouteSlots];
    uint32_t u[kRouteSlots];
#pragma unroll
    for (int j = 0; j < kRouteSlots; ++j) {
        const int e = lane + 32 * j;
        sc[j] = e < E ? sc_s[e] : 0.f;
        u[j] = e < E ? u_s[e] : 0u;
    }
    float wsum = 0.f, my_w = 0.f;
    int my_e = 0;
    for (int k = 0; k < topk; ++k) {
        uint32_t m[kRouteSlots / 2];
#pragma unroll
        for (int j = 0; j < kRouteSlots / 2; ++j) m[j] = max(u[2 * j], u[2 * j + 1]);
        const uint32_t lm = max(max(max(m[0], m[1]), max(m[2], m[3])), max(m[4], m[5]));
        const uint32_t gm = __reduce_max_sync(0xffffffffu, lm);
        uint32_t ce = 0xffffffffu;
#pragma unroll
        for (int j = kRouteSlots - 1; j >= 0; --j) ce = (u[j] == gm) ? (uint32_t)(lane + 32 * j) : ce;   // lowest j last
        const int e = (int)__reduce_min_sync(0xffffffffu, ce);
        const int jw = e >> 5, lw = e & 31;
        float mine = 0.f;
#pragma unroll
        for (int j = 0; j < kRouteSlots; ++j) {
            if (j == jw) {
                mine = sc[j];
                if (lane == lw) u[j] = 0u;
            }
        }
        const float s_e = __shfl_sync(0xffffffffu, mine, lw);
        if (lane == k) { my_e = e; my_w = s_e; }
        wsum += s_e;
    }
    if (lane < topk) {
        float w = my_w;
        if (topk > 1) w = w / (wsum + 1e-20f);
        idx_row[lane] = my_e;
        wts_row[lane] = w * route_scale;
    }
}

// Routing of the rows and the shared expert's SwiGLU + quantiser in ONE launch: the two belong to independent
// chains (router logits / shared gate | up, themselves one two-problem GEMV launch) that meet again only at the
// down projections.  Blocks [0, n) route (a block per row), the others run swiglu_clamp_quant.
__global__ void __launch_bounds__(256)
route_swiglu_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, const float* __restrict__ bias_vl,
                    const uint8_t* __restrict__ is_image, int n, int E, int topk, float route_scale, int* __restrict__ idx,
                    float* __restrict__ wts, const float* __restrict__ gu, int ldgu, float* __restrict__ out, int ldo, int I,
                    float lim, SplitBuf osp) {
    PDL_PROLOGUE();
    __shared__ uint32_t u_s[32 * kRouteSlots];
    __shared__ float sc_s[32 * kRouteSlots];
    const int rb = n;
    if ((int)blockIdx.x < rb) {
        const int r = blockIdx.x;
        const float* b = (bias_vl && is_image && is_image[r]) ? bias_vl : bias;
        route_row_block_d4(logits + (size_t)r * ld, b, E, topk, route_scale, idx + (size_t)r * topk, wts + (size_t)r * topk,
                           u_s, sc_s);
        return;
    }
    if (gu) swiglu_clamp_quant_body(gu, ldgu, out, ldo, n, I, lim, osp, (int)blockIdx.x - rb);
}

// ---- engram --------------------------------------------------------------------------------------
// Phase 1 stores each row's compressed token id (DEAD = -1 for masked rows) at its position of
// the slot's history; phase 2 hashes the 2..G-grams ending at each row.
__global__ void __launch_bounds__(256)
engram_hash_kernel(const int* __restrict__ ids, const uint8_t* __restrict__ dead, const RowMeta* __restrict__ meta,
                   const int* __restrict__ token_map, int* __restrict__ hist, int hist_cap,
                   const long long* __restrict__ mult, const long long* __restrict__ primes,
                   const long long* __restrict__ offs, int pad_id, int n, int L, int G, int heads,
                   long long* __restrict__ out) {
    PDL_PROLOGUE();
    for (int r = threadIdx.x; r < n; r += blockDim.x) {
        const RowMeta m = meta[r];
        if (m.pos < hist_cap) hist[(size_t)m.slot * hist_cap + m.pos] = (dead && dead[r]) ? -1 : token_map[ids[r]];
    }
    __syncthreads();
    const int cols = (G - 1) * heads;
    for (int t = threadIdx.x; t < n * L * cols; t += blockDim.x) {
        const int r = t / (L * cols), l = (t / cols) % L, c = t % cols;
        const int g = c / heads;  // uses look-backs 0 .. g + 1
        const RowMeta m = meta[r];
        long long rolling = 0;
        bool blocked = false;
        for (int shift = 0; shift <= g + 1; ++shift) {
            const int p = m.pos - shift;
            int tok = pad_id;
            if (p < 0) blocked = true;
            else {
                const int src = hist[(size_t)m.slot * hist_cap + min(p, hist_cap - 1)];
                if (src < 0) blocked = true;
                if (!blocked) tok = src;
            }
            const long long prod = (long long)tok * mult[l * G + shift];
            rolling = shift == 0 ? prod : (rolling ^ prod);
        }
        long long md = rolling % primes[l * cols + c];
        out[((size_t)r * L + l) * cols + c] = md + offs[l * cols + c];
    }
}

// Gather `cols` table rows (e4m3 with ue8m0 per 32) of layer index l; rows outside
// [row_lo, row_hi) contribute zeros (another rank owns them).  out [n][cols * hd] f32.
__global__ void __launch_bounds__(256)
engram_gather_kernel(const long long* __restrict__ hash, int L, int l, int cols, const uint8_t* __restrict__ table,
                     const uint8_t* __restrict__ scale, long long row_lo, long long row_hi, int hd,
                     float* __restrict__ out) {
    PDL_PROLOGUE();
    const int r = blockIdx.y, c = blockIdx.x;
    const long long id = hash[((size_t)r * L + l) * cols + c];
    float* o = out + ((size_t)r * cols + c) * hd;
    const bool mine = id >= row_lo && id < row_hi;
    const size_t loc = (size_t)(id - row_lo);
    for (int j = threadIdx.x; j < hd; j += blockDim.x) {
        float v = 0.f;
        if (mine) {
            const __half_raw hr = __nv_cvt_fp8_to_halfraw(table[loc * hd + j], __NV_E4M3);
            v = __half2float(*reinterpret_cast<const __half*>(&hr)) * ue8m0_f32(scale[loc * (hd / 32) + j / 32]);
        }
        o[j] = v;
    }
}

// R[r][i] += gate_i * value; gate_i = sigmoid(sign(d) sqrt(max(|d|, 1e-6))),
// d = sum(R_i * qk_i * key_i) * rstd(R_i) * rstd(key_i) / sqrt(D).  kv [n][(hc + 1) * D].
__global__ void __launch_bounds__(256)
engram_apply_kernel(float* __restrict__ R, const float* __restrict__ kv, const float* __restrict__ qk,
                    const uint8_t* __restrict__ dead, int hc, int D, float eps) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    const int r = blockIdx.y, i = blockIdx.x;
    if (dead && dead[r]) return;
    float* h = R + ((size_t)r * hc + i) * D;
    const float* key = kv + (size_t)r * (hc + 1) * D + (size_t)i * D;
    const float* val = kv + (size_t)r * (hc + 1) * D + (size_t)hc * D;
    const float* w = qk + (size_t)i * D;
    float hh = 0.f, kk = 0.f, dt = 0.f;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        const float a = h[j], b = key[j];
        hh += a * a;
        kk += b * b;
        dt += a * w[j] * b;
    }
    hh = block_sum(hh, red);
    kk = block_sum(kk, red);
    dt = block_sum(dt, red);
    const float d = dt * rsqrtf(hh / D + eps) * rsqrtf(kk / D + eps) * rsqrtf((float)D);
    const float g = sigmoidf_(copysignf(sqrtf(fmaxf(fabsf(d), 1e-6f)), d));
    for (int j = threadIdx.x; j < D; j += blockDim.x) h[j] += g * val[j];
}

// ---- small helpers -------------------------------------------------------------------------------
// out[r][col0 + j] = mean_i R[r][i][j]
__global__ void __launch_bounds__(256)
copy_mean_kernel(const float* __restrict__ R, float* __restrict__ out, int ldo, int col0, int hc, int D) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= D) return;
    float s = 0.f;
    for (int i = 0; i < hc; ++i) s += R[((size_t)r * hc + i) * D + j];
    out[(size_t)r * ldo + col0 + j] = s / hc;
}

// x[j] = table[id][j] (bf16 table), id read from device memory.
__global__ void __launch_bounds__(256)
gather_row_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ id, int D, int vocab,
                  float* __restrict__ out, SplitBuf osp) {
    PDL_PROLOGUE();
    const int t = min(max(id[0], 0), vocab - 1);
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < D; j += gridDim.x * blockDim.x) {
        const float v = __bfloat162float(table[(size_t)t * D + j]);
        out[j] = v;
        split_store(osp, 0, j, v);
    }
}

// plain f32-weight GEMV (compressor projections): out[r][n] = sum_k x[r][k] W[n][k]; warp per n.
__global__ void __launch_bounds__(256)
gemv_f32w_kernel(const float* __restrict__ W, const float* __restrict__ x, int ldx, float* __restrict__ out, int ldo,
                 int m, int N, int K) {
    PDL_PROLOGUE();
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    const float* wrow = W + (size_t)n * K;
    for (int k0 = lane * 4; k0 < K; k0 += 512) {   // four independent 16-byte weight loads in flight per lane
        float4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + 128 * u;
            w[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < K) {
                const uint4 t = ldg_nc_v4(wrow + k);
                w[u] = make_float4(__uint_as_float(t.x), __uint_as_float(t.y), __uint_as_float(t.z), __uint_as_float(t.w));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + 128 * u;
            if (k >= K) break;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < m) {
                    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)r * ldx + k);
                    acc[r] += w[u].x * v.x + w[u].y * v.y + w[u].z * v.z + w[u].w * v.w;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < m) out[(size_t)r * ldo + n] = v;
    }
}

}  // namespace

// ---- C ABI ------------------------------------------------------------------------------------------
static inline SplitBuf mk_split(void* base, int64_t ld, int64_t plane, int64_t mask) {
    return SplitBuf{(uint16_t*)base, (int)ld, (int)plane, (int)mask};
}

FB_API int fb_d4_quant_rows(const float* x, int64_t ldx, float* xq, int64_t ldq, int64_t n, int64_t K, void* s_base,
                            int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (K % 32) return (int)cudaErrorInvalidValue;
    const int64_t warps = n * (K / 32);
    FB_LAUNCH((quant_rows_kernel), (warps + 7) / 8, 256, 0, st, x, (int)ldx, xq, (int)ldq,
              mk_split(s_base, s_ld, s_plane, s_mask), (int)n, (int)K);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_hc_pre(const float* R, float* acc, const float* scale, const float* base, const float* ln_w,
                        const float* pre_in, float* pre_out, float* post_out, float* comb_out, float* xn_out,
                        float* xc_out, int64_t n, int64_t H, int64_t mult, float rms_eps, float hc_eps, int64_t iters,
                        void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, const float* part, int* part_n,
                        int64_t part_ld, float* xq_out, void* q_base, int64_t q_ld, int64_t q_plane, int64_t q_mask,
                        cudaStream_t st) {
    if (mult != 4 || (part_n && n > 64) || (H % 4)) return (int)cudaErrorInvalidValue;
    if ((xq_out || q_base) && (H % 32)) return (int)cudaErrorInvalidValue;   // whole quantisation blocks
    const int nct = (int)(((H / 4 + 1) / 2 + 31) / 32 * 32);   // two float4 columns per contraction thread
    if (nct + 32 > 1024) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((hc_pre_offset_kernel), n, nct + 32, 0, st, R, acc, scale, base, ln_w, pre_in, pre_out, post_out, comb_out,
              xn_out, xc_out, (int)H, rms_eps, hc_eps, (int)iters, mk_split(s_base, s_ld, s_plane, s_mask), part, part_n,
              (int)part_ld, xq_out, mk_split(q_base, q_ld, q_plane, q_mask));
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_rope_heads(float* x, int64_t ld, int64_t n, int64_t heads, int64_t hd, int64_t rd, const float* freqs,
                            const void* meta, int64_t pos_off, int64_t inverse, int64_t fp4_rt, void* s_base,
                            int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (hd % 32 || rd % 2) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((rope_heads_kernel), dim3((unsigned)heads, (unsigned)n), 128, 0, st, x, (int)ld, (int)heads, (int)hd, (int)rd,
              freqs, (const RowMeta*)meta, (int)pos_off, (int)inverse, (int)fp4_rt, mk_split(s_base, s_ld, s_plane, s_mask));
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_kv_append(const float* kv, int64_t ld, const float* norm_w, const float* freqs, const void* meta,
                           void* ring, int64_t cap, float* rows_out, int64_t n, int64_t hd, int64_t rd, float eps,
                           int64_t pos_off, cudaStream_t st) {
    if (hd % 32) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((kv_append_kernel), n, 128, (32 + hd) * sizeof(float), st, kv, (int)ld, norm_w, freqs, (const RowMeta*)meta,
              (__nv_bfloat16*)ring, (int)cap, rows_out, (int)hd, (int)rd, eps, (int)pos_off);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_compress(const float* kv, const float* sc, int64_t ld, const void* meta, float* ring_kv, float* ring_sc,
                          int64_t depth, const float* norm_w, float* lat, int* flag, int64_t n, int64_t hd,
                          int64_t ratio, float eps, cudaStream_t st) {
    if (ratio > 1 && depth < ratio + n) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((compress_kernel), 1, 512, 0, st, kv, sc, (int)ld, (const RowMeta*)meta, ring_kv, ring_sc, (int)depth, norm_w,
              lat, flag, (int)n, (int)hd, (int)ratio, eps);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_latent_store(const float* lat, const int* flag, const void* meta, const float* freqs, void* cache,
                              int64_t cap, int64_t n, int64_t hd, int64_t rd, int64_t ratio, cudaStream_t st) {
    if (hd % 16) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((latent_store_kernel), n, 128, hd * sizeof(float), st, lat, flag, (const RowMeta*)meta, freqs,
              (__nv_bfloat16*)cache, (int)cap, (int)hd, (int)rd, (int)ratio);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_index_k_store(const float* kraw, int64_t ld, const int* flag, const void* meta, const float* norm_w,
                               const float* freqs, void* cache, int64_t cap, int64_t n, int64_t id, int64_t rd,
                               int64_t ratio, float eps, cudaStream_t st) {
    if (id % 32) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((index_k_store_kernel), n, 128, (32 + id) * sizeof(float), st, kraw, (int)ld, flag, (const RowMeta*)meta,
              norm_w, freqs, (__nv_bfloat16*)cache, (int)cap, (int)id, (int)rd, (int)ratio, eps);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_index_score(const float* q, int64_t ldq, const float* w, int64_t ldw, const void* kc, int64_t cap,
                             const void* meta, float* score, int64_t lds, int64_t n, int64_t heads, int64_t id,
                             int64_t ratio, float wscale, cudaStream_t st) {
    const size_t sm = ((size_t)heads * (id + 1) + 8 * id) * sizeof(float);
    if (sm > 48 * 1024) cudaFuncSetAttribute(index_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    const int64_t len = lds < cap ? lds : cap;
    FB_LAUNCH((index_score_kernel), dim3((unsigned)((len + 31) / 32), (unsigned)n), 256, sm, st, q, (int)ldq, w, (int)ldw,
              (const __nv_bfloat16*)kc, (int)cap, (const RowMeta*)meta, score, (int)lds, (int)heads, (int)id, (int)ratio, wscale);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_topk_sorted(const float* score, int64_t lds, const uint8_t* mask, int64_t ldm, const void* meta,
                             int64_t ratio, int64_t div, int64_t k, int* out, int64_t ldo, int64_t n, cudaStream_t st) {
    FB_LAUNCH((topk_sorted_kernel), n, 1024, 0, st, score, (int)lds, mask, (int)ldm, (const RowMeta*)meta, (int)ratio,
              (int)div, (int)k, out, (int)ldo);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_block_max(const float* score, int64_t lds, const void* meta, int64_t ratio, int64_t bs, float* out,
                           int64_t ldo, int64_t n, cudaStream_t st) {
    FB_LAUNCH((block_max_kernel), dim3((unsigned)((ldo + 255) / 256), (unsigned)n), 256, 0, st, score, (int)lds,
              (const RowMeta*)meta, (int)ratio, (int)bs, out, (int)ldo);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_cand_mask(const int* blk, int64_t ldb, int64_t kb, int64_t bs, uint8_t* mask, int64_t ldm, int64_t n,
                           cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(mask, 0, (size_t)n * ldm, st);
    if (e != cudaSuccess) return (int)e;
    FB_LAUNCH((cand_mask_kernel), dim3((unsigned)((kb * bs + 255) / 256), (unsigned)n), 256, 0, st, blk, (int)ldb, (int)kb,
              (int)bs, mask, (int)ldm);
    return FB_LAUNCH_CHECK();
}

template <int NJ>
static int launch_attn(const float* q, int ldq, const void* ring, int cap, int window, const void* comp, int ccap,
                       const int* idx, int ldi, int ktop, const float* extra, int n_extra, const float* sink,
                       const float* freqs, int rd, const void* meta, int pos_off, int win_mode, float scale, int heads,
                       int nsplit, float* o_part, float* ml_part, int n, unsigned* ticket, float* out, int ldo, SplitBuf osp,
                       cudaStream_t st) {
    constexpr int kSm = kAttnStage * NJ * 64 * 2;
    static_assert(2 * 8 * (NJ * 64 + 8) * 4 <= kSm, "the cluster merge stages its partials in the key tile");
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(sparse_attn_kernel<NJ, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSm);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(sparse_attn_kernel<NJ, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSm);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const dim3 grid((unsigned)((heads + 7) / 8), (unsigned)n, (unsigned)nsplit);
    if (ticket && nsplit % kAttnCluster == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = kSm;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = kAttnCluster;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_fb_pdl ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, sparse_attn_kernel<NJ, true>, q, ldq, (const __nv_bfloat16*)ring, cap, window,
                                       (const __nv_bfloat16*)comp, ccap, idx, ldi, ktop, extra, n_extra, sink, freqs, rd,
                                       (const RowMeta*)meta, pos_off, win_mode, scale, heads, nsplit, o_part, ml_part, ticket,
                                       out, ldo, osp);
    }
    FB_LAUNCH((sparse_attn_kernel<NJ, false>), grid, 256, kSm, st, q, ldq,
              (const __nv_bfloat16*)ring, cap, window, (const __nv_bfloat16*)comp, ccap, idx, ldi, ktop, extra, n_extra, sink,
              freqs, rd, (const RowMeta*)meta, pos_off, win_mode, scale, heads, nsplit, o_part, ml_part, ticket, out, ldo, osp);
    return FB_LAUNCH_CHECK();
}

// q [n][heads*hd] un-rotated; out gets the inverse rotation.  idx may be null (ktop = 0), extra may be null.
// o_part: scratch of n * heads * nsplit * hd floats, ml_part: n * heads * nsplit * 2 floats.  ticket: null (a second
// kernel merges the splits) or n * ceil(heads / 8) zero-initialised words, left at zero (the last CTA of a group merges).
FB_API int fb_d4_sparse_attn(const float* q, int64_t ldq, const void* ring, int64_t cap, int64_t window, const void* comp,
                             int64_t ccap, const int* idx, int64_t ldi, int64_t ktop, const float* extra, int64_t n_extra,
                             const float* sink, const float* freqs, int64_t rd, const void* meta, int64_t pos_off,
                             int64_t win_mode, float scale, int64_t heads, int64_t hd, float* out, int64_t ldo, int64_t n,
                             int64_t nsplit, float* o_part, float* ml_part, void* s_base, int64_t s_ld, int64_t s_plane,
                             int64_t s_mask, void* ticket, cudaStream_t st) {
    const SplitBuf osp = mk_split(s_base, s_ld, s_plane, s_mask);
    if (!idx) ktop = 0;
    if (!extra) n_extra = 0;
    if (nsplit < 1 || !o_part || !ml_part || (ticket && nsplit > 32)) return (int)cudaErrorInvalidValue;   // the merging warp keeps one split per lane
    int rc;
#define D4_ATTN(NJ) launch_attn<NJ>(q, (int)ldq, ring, (int)cap, (int)window, comp, (int)ccap, idx, (int)ldi, (int)ktop, extra, \
                                    (int)n_extra, sink, freqs, (int)rd, meta, (int)pos_off, (int)win_mode, scale, (int)heads, \
                                    (int)nsplit, o_part, ml_part, (int)n, (unsigned*)ticket, out, (int)ldo, osp, st)
    switch (hd) {
        case 64: rc = D4_ATTN(1); break;
        case 128: rc = D4_ATTN(2); break;
        case 256: rc = D4_ATTN(4); break;
        case 512: rc = D4_ATTN(8); break;
        default: return (int)cudaErrorInvalidValue;
    }
#undef D4_ATTN
    if (rc || ticket) return rc;   // with a ticket buffer the last CTA of every (row, head tile) has merged the splits
    FB_LAUNCH((sparse_attn_merge_kernel), dim3((unsigned)heads, (unsigned)n), 128, 0, st, o_part, ml_part, sink, freqs, (int)rd,
              (const RowMeta*)meta, (int)pos_off, (int)heads, (int)hd, (int)nsplit, out, (int)ldo, osp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_route(const float* logits, int64_t ld, const float* bias, const float* bias_vl, const uint8_t* is_image,
                       int64_t n, int64_t E, int64_t topk, float route_scale, int* idx, float* wts, cudaStream_t st) {
    if (topk > 32) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((route_kernel), n, 128, 2 * E * sizeof(float), st, logits, (int)ld, bias, bias_vl, is_image, (int)E, (int)topk,
              route_scale, idx, wts);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_expert_gate_up(const float* x, int64_t ldx, const int* idx, const float* wts, const void* w13,
                                const void* s13, float* h, int64_t n, int64_t topk, int64_t I, int64_t K, float lim,
                                cudaStream_t st) {
    if (K % 32) return (int)cudaErrorInvalidValue;
    const size_t sm = 16 * (K / 16 + 1) * sizeof(float);
    if (sm > 48 * 1024) cudaFuncSetAttribute(expert_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    FB_LAUNCH((expert_gate_up_kernel), dim3((unsigned)((I + 7) / 8), (unsigned)topk, (unsigned)n), 256, sm, st, x, (int)ldx, idx,
              wts, (const uint8_t*)w13, (const uint8_t*)s13, h, (int)topk, (int)I, (int)K, lim);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_expert_down(const float* hq, const int* idx, const void* w2, const void* s2, float* y, int64_t ldy,
                             int64_t n, int64_t topk, int64_t I, int64_t D, int64_t accumulate, cudaStream_t st) {
    if (I % 32) return (int)cudaErrorInvalidValue;
    const size_t sm = (size_t)topk * 16 * (I / 16 + 1) * sizeof(float);
    if (sm > 48 * 1024) cudaFuncSetAttribute(expert_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    FB_LAUNCH((expert_down_kernel), dim3((unsigned)((D + 7) / 8), (unsigned)n), 256, sm, st, hq, idx, (const uint8_t*)w2,
              (const uint8_t*)s2, y, (int)ldy, (int)topk, (int)I, (int)D, (int)accumulate);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_swiglu_clamp(const float* gu, int64_t ld, float* out, int64_t ldo, int64_t n, int64_t I, float lim,
                              cudaStream_t st) {
    FB_LAUNCH((swiglu_clamp_kernel), (n * I + 255) / 256, 256, 0, st, gu, (int)ld, out, (int)ldo, (int)n, (int)I, lim);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_rmsnorm_quant(const float* x, int64_t ldx, const float* w, float* out, int64_t ldo, int64_t n, int64_t K,
                               float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (K % 32) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((rmsnorm_quant_kernel), n, 256, 0, st, x, (int)ldx, w, out, (int)ldo, (int)K, eps,
              mk_split(s_base, s_ld, s_plane, s_mask));
    return FB_LAUNCH_CHECK();
}

// qa [n][ld]: columns [0, ql) the q-lora vector, [ql, ql + hd) the raw kv row.  q_out / split planes as
// fb_d4_rmsnorm_quant, ring / rows_out as fb_d4_kv_append.
FB_API int fb_d4_qnorm_kv_append(const float* qa, int64_t ld, int64_t ql, const float* q_w, float* q_out, int64_t ldo,
                                 float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, const float* kv_w,
                                 const float* freqs, const void* meta, void* ring, int64_t cap, float* rows_out, int64_t n,
                                 int64_t hd, int64_t rd, int64_t pos_off, cudaStream_t st) {
    if ((ql % 32) || (hd % 32)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((qnorm_kv_append_kernel), dim3((unsigned)n, 2u), 256, (32 + hd) * sizeof(float), st, qa, (int)ld, (int)ql, q_w,
              q_out, (int)ldo, eps, mk_split(s_base, s_ld, s_plane, s_mask), kv_w, freqs, (const RowMeta*)meta,
              (__nv_bfloat16*)ring, (int)cap, rows_out, (int)hd, (int)rd, (int)pos_off);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_swiglu_clamp_quant(const float* gu, int64_t ld, float* out, int64_t ldo, int64_t n, int64_t I, float lim,
                                    void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (I % 32) return (int)cudaErrorInvalidValue;
    const int64_t warps = n * (I / 32);
    FB_LAUNCH((swiglu_clamp_quant_kernel), (warps + 7) / 8, 256, 0, st, gu, (int)ld, out, (int)ldo, (int)n, (int)I, lim,
              mk_split(s_base, s_ld, s_plane, s_mask));
    return FB_LAUNCH_CHECK();
}

// fb_d4_route and fb_d4_swiglu_clamp_quant (gu may be null: routing only) in one launch; E <= 384, topk <= 32.
FB_API int fb_d4_route_swiglu(const float* logits, int64_t ld, const float* bias, const float* bias_vl, const uint8_t* is_image,
                              int64_t n, int64_t E, int64_t topk, float route_scale, int* idx, float* wts, const float* gu,
                              int64_t ldgu, float* out, int64_t ldo, int64_t I, float lim, void* s_base, int64_t s_ld,
                              int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (topk > 32 || topk > E || E > 32 * kRouteSlots || (gu && (I % 32))) return (int)cudaErrorInvalidValue;
    const int64_t rb = n, sb = gu ? (n * (I / 32) + 7) / 8 : 0;
    FB_LAUNCH((route_swiglu_kernel), (unsigned)(rb + sb), 256, 0, st, logits, (int)ld, bias, bias_vl, is_image, (int)n, (int)E,
              (int)topk, route_scale, idx, wts, gu, (int)ldgu, out, (int)ldo, (int)I, lim, mk_split(s_base, s_ld, s_plane, s_mask));
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_engram_hash(const int* ids, const uint8_t* dead, const void* meta, const int* token_map, int* hist,
                             int64_t hist_cap, const long long* mult, const long long* primes, const long long* offs,
                             int64_t pad_id, int64_t n, int64_t L, int64_t G, int64_t heads, long long* out, cudaStream_t st) {
    FB_LAUNCH((engram_hash_kernel), 1, 256, 0, st, ids, dead, (const RowMeta*)meta, token_map, hist, (int)hist_cap, mult, primes,
              offs, (int)pad_id, (int)n, (int)L, (int)G, (int)heads, out);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_engram_gather(const long long* hash, int64_t L, int64_t l, int64_t cols, const void* table,
                               const void* scale, int64_t row_lo, int64_t row_hi, int64_t hd, float* out, int64_t n,
                               cudaStream_t st) {
    FB_LAUNCH((engram_gather_kernel), dim3((unsigned)cols, (unsigned)n), 256, 0, st, hash, (int)L, (int)l, (int)cols,
              (const uint8_t*)table, (const uint8_t*)scale, (long long)row_lo, (long long)row_hi, (int)hd, out);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_engram_apply(float* R, const float* kv, const float* qk, const uint8_t* dead, int64_t n, int64_t hc,
                              int64_t D, float eps, cudaStream_t st) {
    FB_LAUNCH((engram_apply_kernel), dim3((unsigned)hc, (unsigned)n), 256, 0, st, R, kv, qk, dead, (int)hc, (int)D, eps);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_copy_mean(const float* R, float* out, int64_t ldo, int64_t col0, int64_t n, int64_t hc, int64_t D,
                           cudaStream_t st) {
    FB_LAUNCH((copy_mean_kernel), dim3((unsigned)((D + 255) / 256), (unsigned)n), 256, 0, st, R, out, (int)ldo, (int)col0,
              (int)hc, (int)D);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_gather_row(const void* table, const int* id, int64_t D, int64_t vocab, float* out, void* s_base,
                            int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    FB_LAUNCH((gather_row_kernel), (D + 255) / 256, 256, 0, st, (const __nv_bfloat16*)table, id, (int)D, (int)vocab, out,
              mk_split(s_base, s_ld, s_plane, s_mask));
    return FB_LAUNCH_CHECK();
}

FB_API int fb_d4_gemv_f32w(const float* W, const float* x, int64_t ldx, float* out, int64_t ldo, int64_t m, int64_t N,
                           int64_t K, cudaStream_t st) {
    if (m > 8 || (K % 4) || (ldx % 4)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((gemv_f32w_kernel), (N + 7) / 8, 256, 0, st, W, x, (int)ldx, out, (int)ldo, (int)m, (int)N, (int)K);
    return FB_LAUNCH_CHECK();
}
