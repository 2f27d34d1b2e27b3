// Expert-grouped MoE for prefill-sized row counts.
//
// With more than a handful of rows, many (row, slot) pairs select the same expert.  The per-pair
// kernels of moe.cu would stream that expert's weights once per pair; here pairs are first grouped by
// expert (up to 8 per group = the 8 activation columns of one mma.sync tile), so that a group streams
// its expert's gate/up and down weights once:
//   fb_moe_group        counting sort of the pairs by local expert -> groups of <= 8 pairs
//   fb_moe_gate_up_grp  per group: gate/up tile . 8 activation columns, SwiGLU * routing weight
//   fb_moe_down_grp     per group: down tile . 8 activation columns -> per-pair outputs
//   fb_moe_sum_pairs    y[row] (+)= sum of the row's local-expert pair outputs (fixed slot order)
// Values do not depend on how pairs were packed into groups (MMA columns are independent), so the
// result is deterministic although the packing uses atomics.
// Reference counterpart: moe_sort_assignments + the batched expert kernels
// (kernels/cuda/ferrite_kernels.cu:3548-3963, 4021-).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

constexpr int kMaxLocalExperts = 512;

// Single CTA.  g_pairs [max_groups][8] (pair index or -1), g_expert [max_groups], n_groups [1].
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int n_pairs, int e_lo, int e_cnt, int* __restrict__ g_pairs,
                 int* __restrict__ g_expert, int* __restrict__ n_groups, int max_groups) {
    PDL_PROLOGUE();
    __shared__ int count[kMaxLocalExperts];
    __shared__ int gstart[kMaxLocalExperts];
    __shared__ int fill[kMaxLocalExperts];
    for (int e = threadIdx.x; e < e_cnt; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    for (int i = threadIdx.x; i < max_groups * 8; i += blockDim.x) g_pairs[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int le = ids[p] - e_lo;
        if (le >= 0 && le < e_cnt) atomicAdd(&count[le], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int g = 0;
        for (int e = 0; e < e_cnt; ++e) {
            gstart[e] = g;
            const int ng = (count[e] + 7) >> 3;
            for (int k = 0; k < ng; ++k) g_expert[g + k] = e;
            g += ng;
        }
        *n_groups = g;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int le = ids[p] - e_lo;
        if (le >= 0 && le < e_cnt) {
            const int pos = atomicAdd(&fill[le], 1);
            g_pairs[(size_t)(gstart[le] + (pos >> 3)) * 8 + (pos & 7)] = p;
        }
    }
}

// Activation fragment of MMA column g = pair g of the group (f16 hi plane), zero for an empty column.
__device__ __forceinline__ void load_xfrag_gather(const uint16_t* __restrict__ hi, int ld, int row, int k0, uint32_t (&xh)[16]) {
    if (row >= 0) {
        const uint4* ph = reinterpret_cast<const uint4*>(hi + (size_t)row * ld + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 a = __ldg(ph + i);
            xh[4 * i] = a.x; xh[4 * i + 1] = a.y; xh[4 * i + 2] = a.z; xh[4 * i + 3] = a.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) xh[i] = 0u;
    }
}

constexpr int kGuWarps = 4;
// grid (I / 16, max_groups).  W13 [e_cnt][2I][H] e4m3, S13 [e_cnt][2I/128][H/128].
__global__ void __launch_bounds__(kGuWarps * 32)
moe_gate_up_grp_kernel(const uint8_t* __restrict__ W13, const float* __restrict__ S13, const uint16_t* __restrict__ xhi,
                       int ldx, const float* __restrict__ wts, const int* __restrict__ g_pairs,
                       const int* __restrict__ g_expert, const int* __restrict__ n_groups, SplitBuf asplit, int topk,
                       int I, int H, float limit) {
    PDL_PROLOGUE();
    __shared__ float red[kGuWarps][2][32][4];
    const int grp = blockIdx.y;
    if (grp >= *n_groups) return;
    const int le = g_expert[grp];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int i0 = blockIdx.x * 16;
    const int my_pair = g_pairs[(size_t)grp * 8 + g];          // the pair in MMA column g
    const int my_row = my_pair >= 0 ? my_pair / topk : -1;
    const int kb_n = H >> 7;
    const int nb = (2 * I + 127) >> 7;
    const uint8_t* W = W13 + (size_t)le * 2 * I * H;
    const float* S = S13 + (size_t)le * nb * kb_n;
    const uint8_t* wa[2];
    const uint8_t* wb[2];
    int rowblk[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int base = q * I;
        wa[q] = W + (size_t)(base + min(i0 + g, I - 1)) * H + t * 32;
        wb[q] = W + (size_t)(base + min(i0 + g + 8, I - 1)) * H + t * 32;
        rowblk[q] = (base + i0) >> 7;
    }
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    WFrag fa[2], fb[2];   // alternate roles: no register copies per k-block
    auto fetch = [&](WFrag (&f)[2], int kb) {
#pragma unroll
        for (int q = 0; q < 2; ++q) f[q] = load_wfrag(wa[q] + (size_t)kb * 128, wb[q] + (size_t)kb * 128);
    };
    auto compute = [&](const WFrag (&f)[2], int kb) {
        uint32_t xh[16];
        load_xfrag_gather(xhi, ldx, my_row, kb * 128 + t * 32, xh);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            mma_wfrag_fp8<false>(d, f[q], xh, xh);
            const float sc = __ldg(S + (size_t)rowblk[q] * kb_n + kb);
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[q][c] = fmaf(d[c], sc, acc[q][c]);
        }
    };
    int kb = warp;
    if (kb < kb_n) fetch(fa, kb);
    while (kb < kb_n) {
        const int k1 = kb + kGuWarps;
        if (k1 < kb_n) fetch(fb, k1);
        compute(fa, kb);
        if (k1 >= kb_n) break;
        const int k2 = k1 + kGuWarps;
        if (k2 < kb_n) fetch(fa, k2);
        compute(fb, k1);
        kb = k2;
    }
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][q][lane][c] = acc[q][c];
    __syncthreads();
    {   // 16 tile rows x 8 columns: D element (row j, col) sits in lane (j & 7) * 4 + (col >> 1), reg (j >> 3) * 2 + (col & 1)
        const int j = threadIdx.x & 15, col = threadIdx.x >> 4;
        const int pair = g_pairs[(size_t)grp * 8 + col];
        if (pair >= 0 && i0 + j < I) {
            const int l = (j & 7) * 4 + (col >> 1), c = (j >> 3) * 2 + (col & 1);
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < kGuWarps; ++w) { gsum += red[w][0][l][c]; usum += red[w][1][l][c]; }
            const float gc = fminf(gsum, limit);
            const float uc = fminf(fmaxf(usum, -limit), limit);
            split_store(asplit, pair, i0 + j, siluf_(gc) * uc * wts[pair]);
        }
    }
}

// grid (H / 32, max_groups), 256 threads = two groups of four warps; a group owns 16 output rows and its warps
// split K (512 contiguous bytes of a weight row per step of the group).  W2 [e_cnt][H][I], S2 [e_cnt][H/128][I/128];
// act: f16 hi plane [pairs][lda]; ypair [pairs][H].  Two fragment buffers alternate (no register copies).
__global__ void __launch_bounds__(256, 3)
moe_down_grp_kernel(const uint8_t* __restrict__ W2, const float* __restrict__ S2, const uint16_t* __restrict__ ahi, int lda,
                    const int* __restrict__ g_pairs, const int* __restrict__ g_expert, const int* __restrict__ n_groups,
                    float* __restrict__ ypair, int I, int H) {
    PDL_PROLOGUE();
    __shared__ float red[8][32][4];
    const int grp = blockIdx.y;
    if (grp >= *n_groups) return;
    const int le = g_expert[grp];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int half = warp >> 2, wk = warp & 3;
    const int c0 = (blockIdx.x * 2 + half) * 16;
    const int kb_n = I >> 7;
    const int nb = (H + 127) >> 7;
    const int my_pair = g_pairs[(size_t)grp * 8 + g];
    const uint8_t* W = W2 + (size_t)le * H * I;
    const size_t ra = (size_t)min(c0 + g, H - 1) * I + t * 32, rb = (size_t)min(c0 + g + 8, H - 1) * I + t * 32;
    const float* S = S2 + (size_t)le * nb * kb_n + (size_t)(min(c0, H - 1) >> 7) * kb_n;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    WFrag fa, fb;
    auto compute = [&](const WFrag& f, int kb) {
        uint32_t xh[16];
        load_xfrag_gather(ahi, lda, my_pair, kb * 128 + t * 32, xh);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        mma_wfrag_fp8<false>(d, f, xh, xh);
        const float sc = __ldg(S + kb);
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] = fmaf(d[c], sc, acc[c]);
    };
    int kb = wk;
    if (kb < kb_n) fa = load_wfrag(W + ra + (size_t)kb * 128, W + rb + (size_t)kb * 128);
    while (kb < kb_n) {
        const int k1 = kb + 4;
        if (k1 < kb_n) fb = load_wfrag(W + ra + (size_t)k1 * 128, W + rb + (size_t)k1 * 128);
        compute(fa, kb);
        if (k1 >= kb_n) break;
        const int k2 = k1 + 4;
        if (k2 < kb_n) fa = load_wfrag(W + ra + (size_t)k2 * 128, W + rb + (size_t)k2 * 128);
        compute(fb, k1);
        kb = k2;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][lane][c] = acc[c];
    __syncthreads();
    {   // thread -> (tile of the CTA, tile row j, column): sums the four warps of its tile
        const int th = threadIdx.x >> 7, j = threadIdx.x & 15, col = (threadIdx.x >> 4) & 7;
        const int row = (blockIdx.x * 2 + th) * 16 + j;
        const int pair = g_pairs[(size_t)grp * 8 + col];
        if (pair >= 0 && row < H) {
            const int l = (j & 7) * 4 + (col >> 1), c = (j >> 3) * 2 + (col & 1);
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) v += red[th * 4 + w][l][c];
            ypair[(size_t)pair * H + row] = v;
        }
    }
}

// y[r][c] (+)= sum over the row's slots with a local expert of ypair[r * topk + s][c], in slot order.
__global__ void __launch_bounds__(256)
moe_sum_pairs_kernel(const float* __restrict__ ypair, const int* __restrict__ ids, float* __restrict__ y, int ldy, int topk,
                     int H, int e_lo, int e_cnt, int accumulate) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= H) return;
    float4 acc = accumulate ? *reinterpret_cast<const float4*>(y + (size_t)r * ldy + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < topk; ++s) {
        const int le = ids[r * topk + s] - e_lo;
        if (le < 0 || le >= e_cnt) continue;
        const float4 v = *reinterpret_cast<const float4*>(ypair + (size_t)(r * topk + s) * H + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(y + (size_t)r * ldy + c) = acc;
}

}  // namespace

FB_API int fb_moe_group(const int* ids, int64_t n_pairs, int64_t e_lo, int64_t e_cnt, int* g_pairs, int* g_expert,
                        int* n_groups, int64_t max_groups, cudaStream_t st) {
    if (e_cnt > kMaxLocalExperts) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((moe_group_kernel), 1, 1024, 0, st, ids, (int)n_pairs, (int)e_lo, (int)e_cnt, g_pairs, g_expert, n_groups,
              (int)max_groups);
    return FB_LAUNCH_CHECK();
}

// xs: split activation planes of the rows (the f16 hi plane is read); as_*: split output planes per pair.
FB_API int fb_moe_gate_up_grp(const void* W13, const float* S13, const void* xs, int64_t xs_ld, int64_t xs_plane,
                              const float* wts, const int* g_pairs, const int* g_expert, const int* n_groups,
                              void* as_base, int64_t as_ld, int64_t as_plane, int64_t max_groups, int64_t topk, int64_t I,
                              int64_t H, float limit, cudaStream_t st) {
    if ((H % 128) || (xs_ld % 8)) return (int)cudaErrorInvalidValue;
    const uint16_t* hi = (const uint16_t*)xs + 2 * xs_plane;
    SplitBuf asp{(uint16_t*)as_base, (int)as_ld, (int)as_plane, 2};
    dim3 grid((unsigned)((I + 15) / 16), (unsigned)max_groups);
    FB_LAUNCH((moe_gate_up_grp_kernel), grid, kGuWarps * 32, 0, st, (const uint8_t*)W13, S13, hi, (int)xs_ld, wts, g_pairs,
              g_expert, n_groups, asp, (int)topk, (int)I, (int)H, limit);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_moe_down_grp(const void* W2, const float* S2, const void* as_base, int64_t as_ld, int64_t as_plane,
                           const int* g_pairs, const int* g_expert, const int* n_groups, float* ypair,
                           int64_t max_groups, int64_t I, int64_t H, cudaStream_t st) {
    if ((I % 128) || (as_ld % 8)) return (int)cudaErrorInvalidValue;
    const uint16_t* hi = (const uint16_t*)as_base + 2 * as_plane;
    dim3 grid((unsigned)((H + 31) / 32), (unsigned)max_groups);
    FB_LAUNCH((moe_down_grp_kernel), grid, 256, 0, st, (const uint8_t*)W2, S2, hi, (int)as_ld, g_pairs, g_expert, n_groups, ypair,
              (int)I, (int)H);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_moe_sum_pairs(const float* ypair, const int* ids, float* y, int64_t ldy, int64_t n, int64_t topk, int64_t H,
                            int64_t e_lo, int64_t e_cnt, int64_t accumulate, cudaStream_t st) {
    if (H % 4) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)((H / 4 + 255) / 256), (unsigned)n);
    FB_LAUNCH((moe_sum_pairs_kernel), grid, 256, 0, st, ypair, ids, y, (int)ldy, (int)topk, (int)H, (int)e_lo, (int)e_cnt,
              (int)accumulate);
    return FB_LAUNCH_CHECK();
}
