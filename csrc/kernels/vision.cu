// ViT support kernels: bidirectional attention with 2-D rotary embedding, bias / GELU / residual
// epilogue, f32 -> bf16 packing and the aligner's zero-padded r x r unfold.  The linear layers are
// the tcgen05 GEMM of gemm_tc.cu.  Replaces kernels/cuda/dsv41_vision.cu of the reference.
#include "common.cuh"

namespace {

// One CTA = 8 query rows of one head (one warp each).  Keys / values are staged 32 at a time in
// shared memory already rotated; every lane scores one key (full dot over head_dim, q broadcast from
// shared memory), softmax runs online per tile, and P.V lets every lane own head_dim / 32 outputs.
// qkv [n][3 * H * hd] (q | k | v blocks); ang [n][hd / 2]: rotation angle of pair (i, i + hd / 2).
template <int HD>
__global__ void __launch_bounds__(256)
vit_attention_kernel(const float* __restrict__ qkv, const float* __restrict__ ang, float* __restrict__ out, int n, int H,
                     float scale) {
    PDL_PROLOGUE();
    constexpr int HALF = HD / 2, DPL = HD / 32;
    __shared__ float ks[32][HD + 1];
    __shared__ float vs[32][HD + 1];
    __shared__ float qs[8][HD];
    const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qi = blockIdx.x * 8 + warp;
    const int D3 = 3 * H * HD;
    if (qi < n) {
        for (int i = lane; i < HALF; i += 32) {
            float sn, cs;
            sincosf(ang[(size_t)qi * HALF + i], &sn, &cs);
            const float a = qkv[(size_t)qi * D3 + h * HD + i], b = qkv[(size_t)qi * D3 + h * HD + HALF + i];
            qs[warp][i] = (a * cs - b * sn) * scale;
            qs[warp][HALF + i] = (b * cs + a * sn) * scale;
        }
    }
    float mx = -1e30f, den = 0.f, o[DPL];
#pragma unroll
    for (int d = 0; d < DPL; ++d) o[d] = 0.f;
    for (int t0 = 0; t0 < n; t0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * HALF; i += blockDim.x) {
            const int t = i / HALF, c = i % HALF, key = t0 + t;
            float ka = 0.f, kb = 0.f, va = 0.f, vb = 0.f;
            if (key < n) {
                float sn, cs;
                sincosf(ang[(size_t)key * HALF + c], &sn, &cs);
                const float a = qkv[(size_t)key * D3 + (H + h) * HD + c], b = qkv[(size_t)key * D3 + (H + h) * HD + HALF + c];
                ka = a * cs - b * sn;
                kb = b * cs + a * sn;
                va = qkv[(size_t)key * D3 + (2 * H + h) * HD + c];
                vb = qkv[(size_t)key * D3 + (2 * H + h) * HD + HALF + c];
            }
            ks[t][c] = ka; ks[t][HALF + c] = kb;
            vs[t][c] = va; vs[t][HALF + c] = vb;
        }
        __syncthreads();
        if (qi >= n) continue;
        float s = -INFINITY;
        if (t0 + lane < n) {
            s = 0.f;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) s = fmaf(qs[warp][d], ks[lane][d], s);
        }
        const float mnew = fmaxf(mx, warp_max(s));
        const float resc = __expf(mx - mnew);
        const float p = __expf(s - mnew);
        den = den * resc + warp_sum(p);
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] *= resc;
        for (int t = 0; t < 32; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
#pragma unroll
            for (int d = 0; d < DPL; ++d) o[d] = fmaf(pt, vs[t][lane + 32 * d], o[d]);
        }
        mx = mnew;
    }
    if (qi < n) {
#pragma unroll
        for (int d = 0; d < DPL; ++d) out[(size_t)qi * H * HD + h * HD + lane + 32 * d] = o[d] / den;
    }
}

// out = act(x + bias) + res   (bias / res optional; act: 0 none, 1 exact GELU); out may alias x or res.
__global__ void __launch_bounds__(256)
vit_bias_act_kernel(const float* x, const float* __restrict__ bias, const float* res, float* out, int n, int D, int act) {
    PDL_PROLOGUE();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n * D) return;
    float v = x[i] + (bias ? bias[i % D] : 0.f);
    if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    if (res) v += res[i];
    out[i] = v;
}

__global__ void __launch_bounds__(256)
vit_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, size_t n) {
    PDL_PROLOGUE();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}

// x [n_h][n_w][C] -> out [ceil(n_h / r) * ceil(n_w / r)][C * r * r] with feature index c * r * r + dy * r + dx
// (zero beyond the image), bf16.
__global__ void __launch_bounds__(256)
vit_unfold_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, int n_h, int n_w, int C, int r) {
    PDL_PROLOGUE();
    const int lw = (n_w + r - 1) / r;
    const int cell = blockIdx.x, cy = cell / lw, cx = cell % lw;
    const int F = C * r * r;
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
        const int c = f / (r * r), dy = (f / r) % r, dx = f % r;
        const int y = cy * r + dy, xx = cx * r + dx;
        const float v = (y < n_h && xx < n_w) ? x[((size_t)y * n_w + xx) * C + c] : 0.f;
        out[(size_t)cell * F + f] = __float2bfloat16_rn(v);
    }
}

}  // namespace

FB_API int fb_vit_attention(const float* qkv, const float* ang, float* out, int64_t n, int64_t H, int64_t hd, float scale,
                            cudaStream_t st) {
    dim3 grid((unsigned)((n + 7) / 8), (unsigned)H);
    if (hd == 64) FB_LAUNCH((vit_attention_kernel<64>), grid, 256, 0, st, qkv, ang, out, (int)n, (int)H, scale);
    else if (hd == 32) FB_LAUNCH((vit_attention_kernel<32>), grid, 256, 0, st, qkv, ang, out, (int)n, (int)H, scale);
    else return (int)cudaErrorInvalidValue;
    return FB_LAUNCH_CHECK();
}

FB_API int fb_vit_bias_act(const float* x, const float* bias, const float* res, float* out, int64_t n, int64_t D,
                           int64_t act, cudaStream_t st) {
    FB_LAUNCH((vit_bias_act_kernel), (n * D + 255) / 256, 256, 0, st, x, bias, res, out, (int)n, (int)D, (int)act);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_vit_to_bf16(const float* x, void* out, int64_t n, cudaStream_t st) {
    FB_LAUNCH((vit_to_bf16_kernel), (n + 255) / 256, 256, 0, st, x, (__nv_bfloat16*)out, (size_t)n);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_vit_unfold(const float* x, void* out, int64_t n_h, int64_t n_w, int64_t C, int64_t r, cudaStream_t st) {
    const int64_t cells = ((n_h + r - 1) / r) * ((n_w + r - 1) / r);
    FB_LAUNCH((vit_unfold_kernel), cells, 256, 0, st, x, (__nv_bfloat16*)out, (int)n_h, (int)n_w, (int)C, (int)r);
    return FB_LAUNCH_CHECK();
}
