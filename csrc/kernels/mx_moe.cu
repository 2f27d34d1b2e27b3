// Glue of the block-scaled grouped expert path (csrc/kernels/mx_gemm.cu) for prefill-sized and batched row counts:
//
//   fb_mx_sort          (row, slot) pairs -> position in an expert-sorted list; per-expert counts, the GEMM's tile
//                       list and the routing weight of every sorted position, one CTA
//   fb_mx_quant_scatter rows -> e4m3 bytes + ue8m0 scale bytes per 32 values, written to every sorted position of
//                       the row (the "dispatch" of a one-rank expert layer)
//   fb_mx_swiglu_quant  gate | up accumulators of the sorted rows -> routing weight * SwiGLU, quantised again
//   fb_mx_combine       y[row] (+)= sum over the row's slots, in slot order, of the down projection's sorted rows
//
// Quantisation is the model's: scale = 2^ceil(log2(amax / 448)) with amax floored at 1e-4, values rounded to e4m3
// (ops/quant.py::fp8_act_quant).  Replaces the reference's route_group / moe_align + act_quant kernels
// (kernels/cuda/dsv41_route.cu, dsv41_moe_align.cu) for this path.
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

struct MxTile { int expert, row0, nrows, pad; };

constexpr int kMaxExperts = 512;

// One CTA.  ids [npairs] expert per (row, slot) pair (-1 or outside [e_lo, e_lo + E): not on this rank).
__global__ void __launch_bounds__(1024)
mx_sort_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int npairs, int e_lo, int E, int bn,
               int* __restrict__ pos, float* __restrict__ wts_sorted, int* __restrict__ counts, int* __restrict__ offsets,
               MxTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
    PDL_PROLOGUE();
    __shared__ int hist[kMaxExperts], start[kMaxExperts + 1], cursor[kMaxExperts];
    for (int e = threadIdx.x; e < E; e += blockDim.x) { hist[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
        const int le = ids[p] - e_lo;
        if (le >= 0 && le < E) atomicAdd(&hist[le], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, t = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = off;
            offsets[e] = off;
            counts[e] = hist[e];
            for (int r = 0; r < hist[e]; r += bn) {
                if (t < max_tiles) tiles[t] = MxTile{e, off + r, min(bn, hist[e] - r), 0};
                ++t;
            }
            off += hist[e];
        }
        start[E] = off;
        offsets[E] = off;
        *n_tiles = min(t, max_tiles);
    }
    __syncthreads();
    // the order inside an expert's segment follows the atomics; every row's result is independent of it
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) {
        const int le = ids[p] - e_lo;
        int q = -1;
        if (le >= 0 && le < E) {
            q = start[le] + atomicAdd(&cursor[le], 1);
            wts_sorted[q] = wts ? wts[p] : 1.f;
        }
        pos[p] = q;
    }
}

__device__ __forceinline__ float pow2_ceil_scale(float amax) {
    // 2^ceil(log2(amax / 448)), exactly: exponent + (mantissa != 0)
    const float v = fmaxf(amax, 1e-4f) * (1.f / 448.f);
    const uint32_t b = __float_as_uint(v);
    int e = (int)((b >> 23) & 0xffu) + ((b & 0x7fffffu) ? 1 : 0);
    e = min(max(e, 0), 254);
    return __uint_as_float((uint32_t)e << 23);
}

// One warp per (row, 32-value block): lane j owns value j.
__global__ void __launch_bounds__(256)
mx_quant_scatter_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ pos, int topk, int n, int K,
                        uint8_t* __restrict__ x8, uint8_t* __restrict__ sf, int ld_sf) {
    PDL_PROLOGUE();
    const int nb = K / 32;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n * nb) return;
    const int r = w / nb, b = w % nb;
    const float v = x[(size_t)r * ldx + b * 32 + lane];
    const float s = pow2_ceil_scale(warp_max(fabsf(v)));
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v / s, __NV_SATFINITE, __NV_E4M3);
    const uint8_t sb = (uint8_t)(__float_as_uint(s) >> 23);
    for (int k = 0; k < topk; ++k) {
        const int p = pos[r * topk + k];
        if (p < 0) continue;
        x8[(size_t)p * K + b * 32 + lane] = q;
        if (lane == 0) sf[(size_t)p * ld_sf + b] = sb;
        if (b == nb - 1 && lane > 0 && nb + lane - 1 < ld_sf) sf[(size_t)p * ld_sf + nb + lane - 1] = 127;   // pad
    }
}

// h [m, ldh] = [gate (I) | up (I)] of sorted row p -> a = wts[p] * silu(min(g, L)) * clamp(u, -L, L), quantised.
__global__ void __launch_bounds__(256)
mx_swiglu_quant_kernel(const float* __restrict__ h, int ldh, const float* __restrict__ wts, const int* __restrict__ m_ptr,
                       int I, float limit, uint8_t* __restrict__ a8, uint8_t* __restrict__ sf, int ld_sf) {
    PDL_PROLOGUE();
    const int nb = I / 32;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= *m_ptr * nb) return;
    const int p = w / nb, b = w % nb;
    const float g = fminf(h[(size_t)p * ldh + b * 32 + lane], limit);
    const float u = fminf(fmaxf(h[(size_t)p * ldh + I + b * 32 + lane], -limit), limit);
    const float v = siluf_(g) * u * wts[p];
    const float s = pow2_ceil_scale(warp_max(fabsf(v)));
    a8[(size_t)p * I + b * 32 + lane] = __nv_cvt_float_to_fp8(v / s, __NV_SATFINITE, __NV_E4M3);
    if (lane == 0) sf[(size_t)p * ld_sf + b] = (uint8_t)(__float_as_uint(s) >> 23);
    if (b == nb - 1 && lane > 0 && nb + lane - 1 < ld_sf) sf[(size_t)p * ld_sf + nb + lane - 1] = 127;
}

__global__ void __launch_bounds__(256)
mx_combine_kernel(const float* __restrict__ ypair, int ldy, const int* __restrict__ pos, int topk, float* __restrict__ y,
                  int ldo, int D, int accumulate) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= D) return;
    float4 a = accumulate ? *reinterpret_cast<const float4*>(y + (size_t)r * ldo + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < topk; ++k) {
        const int p = pos[r * topk + k];
        if (p < 0) continue;
        const float4 v = *reinterpret_cast<const float4*>(ypair + (size_t)p * ldy + c);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    *reinterpret_cast<float4*>(y + (size_t)r * ldo + c) = a;
}

}  // namespace

// pos [npairs], wts_sorted [npairs], counts [E], offsets [E + 1], tiles [max_tiles] x 4 ints, n_tiles [1].
FB_API int fb_mx_sort(const int* ids, const float* wts, int64_t npairs, int64_t e_lo, int64_t E, int64_t bn, int* pos,
                      float* wts_sorted, int* counts, int* offsets, void* tiles, int* n_tiles, int64_t max_tiles,
                      cudaStream_t st) {
    if (E > kMaxExperts || npairs < 1) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((mx_sort_kernel), 1, 1024, 0, st, ids, wts, (int)npairs, (int)e_lo, (int)E, (int)bn, pos, wts_sorted, counts,
              offsets, (MxTile*)tiles, n_tiles, (int)max_tiles);
    return FB_LAUNCH_CHECK();
}

// x [n, ldx] f32 -> for every pair (r, k) with pos >= 0: x8[pos] (K bytes), sf[pos] (ld_sf bytes: K / 32 scales, rest 127).
FB_API int fb_mx_quant_scatter(const float* x, int64_t ldx, const int* pos, int64_t topk, int64_t n, int64_t K, void* x8,
                               void* sf, int64_t ld_sf, cudaStream_t st) {
    if ((K % 32) || ld_sf < K / 32 || ld_sf - K / 32 > 31) return (int)cudaErrorInvalidValue;
    const int64_t warps = n * (K / 32);
    FB_LAUNCH((mx_quant_scatter_kernel), (warps + 7) / 8, 256, 0, st, x, (int)ldx, pos, (int)topk, (int)n, (int)K,
              (uint8_t*)x8, (uint8_t*)sf, (int)ld_sf);
    return FB_LAUNCH_CHECK();
}

// m_ptr: device int, number of sorted rows (offsets[E]); max_m bounds the grid.
FB_API int fb_mx_swiglu_quant(const float* h, int64_t ldh, const float* wts_sorted, const int* m_ptr, int64_t max_m,
                              int64_t I, float limit, void* a8, void* sf, int64_t ld_sf, cudaStream_t st) {
    if ((I % 32) || ld_sf < I / 32 || ld_sf - I / 32 > 31) return (int)cudaErrorInvalidValue;
    const int64_t warps = max_m * (I / 32);
    FB_LAUNCH((mx_swiglu_quant_kernel), (warps + 7) / 8, 256, 0, st, h, (int)ldh, wts_sorted, m_ptr, (int)I, limit,
              (uint8_t*)a8, (uint8_t*)sf, (int)ld_sf);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_mx_combine(const float* ypair, int64_t ldy, const int* pos, int64_t topk, float* y, int64_t ldo, int64_t n,
                         int64_t D, int64_t accumulate, cudaStream_t st) {
    if ((D % 4) || (ldy % 4) || (ldo % 4)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((mx_combine_kernel), dim3((unsigned)((D / 4 + 255) / 256), (unsigned)n), 256, 0, st, ypair, (int)ldy, pos,
              (int)topk, y, (int)ldo, (int)D, (int)accumulate);
    return FB_LAUNCH_CHECK();
}
