// Weight-stationary multi-row GEMV family for decode (1..8 activation rows).
//
//   out[m, n] (+)= sum_k x[m, k] * W[n, k]        W bf16 or fp8-e4m3 with 128x128 block scales
//
// Decode at 1..8 rows is bound by streaming W from HBM once; every activation row rides on
// the same weight stream (the reference measured 4.45x for 6 verify rows because its forms
// re-stream per row: AGENTS.md:110-120).  One warp owns R consecutive weight rows so that an
// x fragment fetched from L1 is reused R times (L1/shared bandwidth, not HBM, is what a
// naive multi-row GEMV runs out of on B200), lanes stride over K with 16-byte loads, and the
// weight loads bypass L1 so the activations stay resident there.
//
// Replaces the reference's gemv_bf16_v2/_mrows/_nt, gemv_tri, gemv_fp8_v2 and the DSV41
// gemm_fp8_gemv/mrows families (kernels/cuda/ferrite_kernels.cu:3016-3785,10650-11275).
#include "common.cuh"
#include "mma_gemv.cuh"

int g_fb_l2_ahead = 2;   // measured on the GLM decode step: 0 -> 12.09-12.13 ms, 2 -> 12.00, 3 -> 12.08, 5 -> 12.27
FB_API int fb_set_l2_ahead(int n) { g_fb_l2_ahead = n; return 0; }

namespace {

constexpr int kWarps = 8;

template <int M, int R, bool FP8>
__global__ void __launch_bounds__(kWarps * 32)
gemv_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales,
            const float* __restrict__ x, int ldx, float* __restrict__ out, int ldo,
            int mrows, int N, int K, int group_rows, int accumulate) {
    PDL_PROLOGUE();
    constexpr int VEC = FP8 ? 16 : 8;          // elements per 16-byte load
    constexpr int ESZ = FP8 ? 1 : 2;
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int n0 = gw * R;
    if (n0 >= N) return;
    const float* xg = x + (group_rows > 0 ? (size_t)(n0 / group_rows) * K : 0);
    const int kblocks = (K + 127) >> 7;

    float acc[M][R];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[m][r] = 0.f;

    const uint8_t* wrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int n = min(n0 + r, N - 1);
        wrow[r] = W + (size_t)n * K * ESZ;
    }

#pragma unroll 2
    for (int k = lane * VEC; k < K; k += 32 * VEC) {
        uint4 wv[R];
#pragma unroll
        for (int r = 0; r < R; ++r) wv[r] = ldg_nc_v4(wrow[r] + (size_t)k * ESZ);
        float xv[M][VEC];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m < mrows) {
#pragma unroll
                for (int v = 0; v < VEC; v += 4) {
                    float4 t = __ldg(reinterpret_cast<const float4*>(xg + (size_t)m * ldx + k + v));
                    xv[m][v] = t.x; xv[m][v + 1] = t.y; xv[m][v + 2] = t.z; xv[m][v + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) xv[m][v] = 0.f;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float wf[VEC];
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv[r]);
            if (FP8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) e4m3x4_to_f32(pw[i], &wf[4 * i]);
                const float sc = __ldg(scales + (size_t)(min(n0 + r, N - 1) >> 7) * kblocks + (k >> 7));
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float p = 0.f;
#pragma unroll
                    for (int v = 0; v < VEC; ++v) p = fmaf(wf[v], xv[m][v], p);
                    acc[m][r] = fmaf(p, sc, acc[m][r]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) { wf[2 * i] = bf16lo(pw[i]); wf[2 * i + 1] = bf16hi(pw[i]); }
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[m][r] = fmaf(wf[v], xv[m][v], acc[m][r]);
            }
        }
    }

#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float v = warp_sum(acc[m][r]);
            if (lane == 0 && m < mrows && n0 + r < N) {
                float* o = out + (size_t)m * ldo + n0 + r;
                *o = accumulate ? (*o + v) : v;
            }
        }
}


// Split-K form for K >= 1024: a CTA owns RB consecutive weight rows, its 8 warps take
// interleaved 512-byte slabs of K, and an x fragment is reused for all RB rows.  There are
// N/RB CTAs whatever K is, so mid-size matrices (N = 4096) still fill 148 SMs, and every lane
// keeps RB 16-byte weight loads in flight per step.
template <int M, int RB, bool FP8>
__global__ void __launch_bounds__(kWarps * 32)
gemv_splitk_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales,
                   const float* __restrict__ x, int ldx, float* __restrict__ out, int ldo,
                   int mrows, int N, int K, int accumulate) {
    PDL_PROLOGUE();
    constexpr int VEC = FP8 ? 16 : 8;
    constexpr int ESZ = FP8 ? 1 : 2;
    __shared__ float red[kWarps][M * RB];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = blockIdx.x * RB;
    const int kblocks = (K + 127) >> 7;
    float acc[M][RB];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[m][r] = 0.f;
    const uint8_t* wrow[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) wrow[r] = W + (size_t)min(n0 + r, N - 1) * K * ESZ;
    const float* srow = FP8 ? scales + (size_t)(n0 >> 7) * kblocks : nullptr;

#pragma unroll 2
    for (int k = (warp * 32 + lane) * VEC; k < K; k += kWarps * 32 * VEC) {
        uint4 wv[RB];
#pragma unroll
        for (int r = 0; r < RB; ++r) wv[r] = ldg_nc_v4(wrow[r] + (size_t)k * ESZ);
        float xv[M][VEC];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m < mrows) {
#pragma unroll
                for (int v = 0; v < VEC; v += 4) {
                    float4 t = __ldg(reinterpret_cast<const float4*>(x + (size_t)m * ldx + k + v));
                    xv[m][v] = t.x; xv[m][v + 1] = t.y; xv[m][v + 2] = t.z; xv[m][v + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) xv[m][v] = 0.f;
            }
        }
        float sc = 1.f;
        if (FP8) sc = __ldg(srow + (k >> 7));
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            float wf[VEC];
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv[r]);
            if (FP8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) e4m3x4_to_f32(pw[i], &wf[4 * i]);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float p = 0.f;
#pragma unroll
                    for (int v = 0; v < VEC; ++v) p = fmaf(wf[v], xv[m][v], p);
                    acc[m][r] = fmaf(p, sc, acc[m][r]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) { wf[2 * i] = bf16lo(pw[i]); wf[2 * i + 1] = bf16hi(pw[i]); }
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[m][r] = fmaf(wf[v], xv[m][v], acc[m][r]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const float v = warp_sum(acc[m][r]);
            if (lane == 0) red[warp][m * RB + r] = v;
        }
    __syncthreads();
    if (threadIdx.x < M * RB) {
        const int m = threadIdx.x / RB, r = threadIdx.x % RB;
        if (m < mrows && n0 + r < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) v += red[w][threadIdx.x];
            float* o = out + (size_t)m * ldo + n0 + r;
            *o = accumulate ? (*o + v) : v;
        }
    }
}

template <int M, int RB, bool FP8>
int launch_sk(const void* W, const float* scales, const float* x, int ldx, float* out, int ldo, int mrows,
              int N, int K, int accumulate, cudaStream_t st) {
    dim3 grid((N + RB - 1) / RB), block(kWarps * 32);
    FB_LAUNCH((gemv_splitk_kernel<M, RB, FP8>), grid, block, 0, st, static_cast<const uint8_t*>(W), scales, x, ldx, out, ldo,
                                                            mrows, N, K, accumulate);
    return FB_LAUNCH_CHECK();
}

template <int M, bool FP8>
int launch_sk_rb(const void* W, const float* scales, const float* x, int ldx, float* out, int ldo, int mrows,
                 int N, int K, int accumulate, cudaStream_t st) {
    if (N >= 2368) return launch_sk<M, 8, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
    if (N >= 592) return launch_sk<M, 4, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
    return launch_sk<M, 2, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
}


// ---- MoE routing as the tail of the router GEMV ---------------------------------------------
// The router logits are the first E outputs of the [router | shared gate | shared up] GEMV.  The CTAs that own
// those outputs take a ticket when their tile is stored; the last of them routes every row (one warp per row)
// while the rest of the grid is still streaming the shared expert's rows, so routing costs no launch and no time.
//   s = sigmoid(logit); top-k of (s + bias), ties to the lower index; w = s_sel / (sum s_sel + eps_f32) * scaling
struct RouteTail {
    const float* bias;   // [E]   (null: no routing)
    int* ids;            // [m][topk]
    float* wts;          // [m][topk]
    unsigned* ticket;
    int E, topk;
    float scaling;
};

__device__ __forceinline__ uint32_t route_okey(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kRouteKeys = 12;   // experts per lane: E <= 384

__device__ __noinline__ void route_row_warp(const float* __restrict__ logits, const RouteTail& rt, int row, int lane) {
    unsigned long long key[kRouteKeys];
    float sig[kRouteKeys], lg[kRouteKeys], bs[kRouteKeys];
#pragma unroll
    for (int i = 0; i < kRouteKeys; ++i) {   // every load in flight before the first use (L2 reads: other CTAs wrote them)
        const int e = lane + 32 * i;
        lg[i] = e < rt.E ? __ldcg(logits + e) : 0.f;
        bs[i] = e < rt.E ? __ldg(rt.bias + e) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < kRouteKeys; ++i) {
        const int e = lane + 32 * i;
        key[i] = 0ull;
        sig[i] = 0.f;
        if (e < rt.E) {
            const float sv = 1.f / (1.f + expf(-lg[i]));
            sig[i] = sv;
            key[i] = ((unsigned long long)route_okey(sv + bs[i]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)e);
        }
    }
    float my_s = 0.f;
    int my_id = 0;
    for (int k = 0; k < rt.topk; ++k) {
        unsigned long long best = 0ull;
#pragma unroll
        for (int i = 0; i < kRouteKeys; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
            best = t > best ? t : best;
        }
        const int e = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        float cand = 0.f;
#pragma unroll
        for (int i = 0; i < kRouteKeys; ++i)
            if (key[i] == best) { cand = sig[i]; key[i] = 0ull; }
        const float sv = __shfl_sync(0xffffffffu, cand, e & 31);
        if (lane == k) { my_s = sv; my_id = e; }
    }
    float sum = 0.f;
    for (int k = 0; k < rt.topk; ++k) sum += __shfl_sync(0xffffffffu, my_s, k);
    const float inv = rt.scaling / (sum + 1.1920929e-07f);
    if (lane < rt.topk) {
        rt.ids[(size_t)row * rt.topk + lane] = my_id;
        rt.wts[(size_t)row * rt.topk + lane] = my_s * inv;
    }
}

// ---- tensor-core form (see mma_gemv.cuh) ---------------------------------------------------
// A CTA owns 16*RT weight rows; its NW warps take interleaved k-blocks (64 bf16 / 128 e4m3
// elements) with the next block's weight loads in flight while the current block is
// multiplied; partial D tiles are summed across warps through shared memory.
// tile_x: the CTA's row tile (blockIdx.x of a one-problem launch).
template <int RT, int NW, bool FP8>
__device__ __forceinline__ void gemv_mma_body(const uint8_t* __restrict__ W, const float* __restrict__ scales,
                                              const uint16_t* __restrict__ xhi, const uint16_t* __restrict__ xlo, int ldx,
                                              float* __restrict__ out, int ldo, int mrows, int N, int K, int group_rows,
                                              int accumulate, SplitBuf osplit, int l2_ahead, RouteTail rt, int tile_x) {
    pdl_launch();  // weights are constant: the first k-block is fetched before pdl_wait()
    constexpr int KB = FP8 ? 128 : 64;
    constexpr int XW = FP8 ? 16 : 8;
    __shared__ float red[NW][RT][32][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = tile_x * 16 * RT;
    const int nkb = K / KB;
    const int kblocks = (K + 127) >> 7;
    // blockIdx.y walks 8-row windows of the activations: prefill-sized row counts take one launch, every
    // window streams the weights again (from L2 after the first)
    const int r0 = blockIdx.y * 8;
    xhi += (size_t)r0 * ldx;
    xlo += (size_t)r0 * ldx;
    mrows = min(8, mrows - r0);
    if (group_rows > 0) { const size_t go = (size_t)(n0 / group_rows) * K; xhi += go; xlo += go; }
    float acc[RT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
    const uint8_t* wa[RT];
    const uint8_t* wb[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const size_t esz = FP8 ? 1 : 2;
        wa[r] = W + (size_t)min(n0 + r * 16 + g, N - 1) * K * esz + (size_t)t * 32;
        wb[r] = W + (size_t)min(n0 + r * 16 + g + 8, N - 1) * K * esz + (size_t)t * 32;
    }
    // two fragment sets alternate roles (one is loaded while the other is multiplied): no register copies per k-block
    WFrag fa[RT], fb[RT];
    auto fetch = [&](WFrag (&f)[RT], int kb) {
#pragma unroll
        for (int r = 0; r < RT; ++r) f[r] = load_wfrag(wa[r] + (size_t)kb * 128, wb[r] + (size_t)kb * 128);
        const int kp = kb + (l2_ahead - 1) * NW;   // read-ahead into L2, one lane per 128-byte line
        if (l2_ahead > 1 && kp < nkb && t == 0) {
#pragma unroll
            for (int r = 0; r < RT; ++r) { prefetch_l2(wa[r] + (size_t)kp * 128); prefetch_l2(wb[r] + (size_t)kp * 128); }
        }
    };
    auto compute = [&](const WFrag (&f)[RT], int kb) {
        uint32_t xh[XW], xl[XW];
        load_xfrag<XW, !FP8>(xhi, xlo, ldx, g, mrows, kb * KB + t * (KB / 4), xh, xl);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (FP8) {
                float d[4] = {0.f, 0.f, 0.f, 0.f};
                mma_wfrag_fp8<false>(d, f[r], reinterpret_cast<const uint32_t(&)[16]>(xh), reinterpret_cast<const uint32_t(&)[16]>(xl));
                const float sc = __ldg(scales + (size_t)((n0 + r * 16) >> 7) * kblocks + kb);
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(d[c], sc, acc[r][c]);
            } else {
                mma_wfrag_bf16(acc[r], f[r], reinterpret_cast<const uint32_t(&)[8]>(xh), reinterpret_cast<const uint32_t(&)[8]>(xl));
            }
        }
    };
    if (warp < nkb) fetch(fa, warp);
    pdl_wait();
    for (int kb = warp; kb < nkb;) {
        const int k1 = kb + NW;
        if (k1 < nkb) fetch(fb, k1);
        compute(fa, kb);
        if (k1 >= nkb) break;
        const int k2 = k1 + NW;
        if (k2 < nkb) fetch(fa, k2);
        compute(fb, k1);
        kb = k2;
    }
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][r][lane][c] = acc[r][c];
    __syncthreads();
    for (int idx = threadIdx.x; idx < RT * 128; idx += NW * 32) {
        const int r = idx >> 7, l = (idx & 127) >> 2, c = idx & 3;
        const int row = n0 + r * 16 + (l >> 2) + 8 * (c >> 1);
        const int col = 2 * (l & 3) + (c & 1);
        if (col < mrows && row < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) v += red[w][r][l][c];
            float* o = out + (size_t)(r0 + col) * ldo + row;
            if (accumulate) v += *o;
            *o = v;
            split_store(osplit, r0 + col, row, v);
        }
    }
    if (rt.bias != nullptr && n0 < rt.E && blockIdx.y == 0) {
        __shared__ int s_route;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const unsigned owners = (unsigned)((rt.E + 16 * RT - 1) / (16 * RT));
            s_route = atomicAdd(rt.ticket, 1u) == owners - 1u;
            if (s_route) *rt.ticket = 0u;
        }
        __syncthreads();
        if (s_route) {
            __threadfence();
            for (int row = warp; row < mrows; row += NW) route_row_warp(out + (size_t)row * ldo, rt, row, lane);
        }
    }
}

template <int RT, int NW, bool FP8>
__global__ void __launch_bounds__(NW * 32, (NW >= 16 ? 2 : (RT >= 2 ? 2 : 4)))
gemv_mma_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales,
                const uint16_t* __restrict__ xhi, const uint16_t* __restrict__ xlo, int ldx,
                float* __restrict__ out, int ldo, int mrows, int N, int K, int group_rows, int accumulate,
                SplitBuf osplit, int l2_ahead, RouteTail rt) {
    gemv_mma_body<RT, NW, FP8>(W, scales, xhi, xlo, ldx, out, ldo, mrows, N, K, group_rows, accumulate, osplit, l2_ahead, rt,
                               (int)blockIdx.x);
}

// Two independent bf16 problems over the same rows in ONE launch (e.g. router logits from the un-quantised input and
// the shared expert's gate | up from the quantised one): CTAs [0, tiles_a) work on problem a, the rest on problem b.
// Apart, the smaller problem is a launch of a few dozen CTAs on the decode critical path.
struct GemvProb {
    const uint8_t* W;
    const uint16_t* xhi;
    const uint16_t* xlo;
    int ldx;
    float* out;
    int ldo, N, K;
};
template <int NW>
__global__ void __launch_bounds__(NW * 32, (NW >= 16 ? 2 : 4))
gemv_mma_dual_kernel(GemvProb a, GemvProb b, int tiles_a, int mrows, int l2_ahead) {
    const bool second = (int)blockIdx.x >= tiles_a;
    const GemvProb p = second ? b : a;
    gemv_mma_body<1, NW, false>(p.W, nullptr, p.xhi, p.xlo, p.ldx, p.out, p.ldo, mrows, p.N, p.K, 0, 0,
                                SplitBuf{nullptr, 0, 0, 0}, l2_ahead, RouteTail{}, (int)blockIdx.x - (second ? tiles_a : 0));
}

template <bool FP8>
int launch_mma(const void* W, const float* scales, const uint16_t* xs, int ldx, int plane, float* out, int ldo,
               int mrows, int N, int K, int group_rows, int accumulate, SplitBuf osplit, cudaStream_t st,
               RouteTail rt = RouteTail{}) {
    const uint16_t* hi = xs + (FP8 ? 2 * (size_t)plane : 0);
    const uint16_t* lo = hi + plane;
    const uint8_t* w8 = static_cast<const uint8_t*>(W);
    constexpr int KB = FP8 ? 128 : 64;
    const int nkb = K / KB;
    if (N >= 9472 && (group_rows == 0 || group_rows % 32 == 0)) {
        FB_LAUNCH((gemv_mma_kernel<2, 8, FP8>), dim3((unsigned)((N + 31) / 32), (unsigned)((mrows + 7) / 8)), 256, 0, st, w8, scales, hi, lo, ldx, out, ldo, mrows, N, K, group_rows, accumulate, osplit, g_fb_l2_ahead, rt);
    } else if (nkb >= 64 && N <= 8192) {  // few row tiles, long rows: split K over 16 warps
        FB_LAUNCH((gemv_mma_kernel<1, 16, FP8>), dim3((unsigned)((N + 15) / 16), (unsigned)((mrows + 7) / 8)), 512, 0, st, w8, scales, hi, lo, ldx, out, ldo, mrows, N, K, group_rows, accumulate, osplit, g_fb_l2_ahead, rt);
    } else if (nkb >= 8) {
        FB_LAUNCH((gemv_mma_kernel<1, 8, FP8>), dim3((unsigned)((N + 15) / 16), (unsigned)((mrows + 7) / 8)), 256, 0, st, w8, scales, hi, lo, ldx, out, ldo, mrows, N, K, group_rows, accumulate, osplit, g_fb_l2_ahead, rt);
    } else {
        FB_LAUNCH((gemv_mma_kernel<1, 2, FP8>), dim3((unsigned)((N + 15) / 16), (unsigned)((mrows + 7) / 8)), 64, 0, st, w8, scales, hi, lo, ldx, out, ldo, mrows, N, K, group_rows, accumulate, osplit, g_fb_l2_ahead, rt);
    }
    return FB_LAUNCH_CHECK();
}

template <int M, bool FP8>
int launch_r(const void* W, const float* scales, const float* x, int ldx, float* out, int ldo,
             int mrows, int N, int K, int group_rows, int accumulate, cudaStream_t st) {
    // Pick R so that there are enough warps to fill 148 SMs; large matrices amortise x reads.
    int R = (N >= 9472) ? 4 : (N >= 4736 ? 2 : 1);
    if (group_rows > 0) while (R > 1 && (group_rows % R)) R >>= 1;
    const int warps = (N + R - 1) / R;
    dim3 grid((warps + kWarps - 1) / kWarps), block(kWarps * 32);
    const uint8_t* w8 = static_cast<const uint8_t*>(W);
    if (R == 4) FB_LAUNCH((gemv_kernel<M, 4, FP8>), grid, block, 0, st, w8, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate);
    else if (R == 2) FB_LAUNCH((gemv_kernel<M, 2, FP8>), grid, block, 0, st, w8, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate);
    else FB_LAUNCH((gemv_kernel<M, 1, FP8>), grid, block, 0, st, w8, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate);
    return FB_LAUNCH_CHECK();
}

template <bool FP8>
int launch_m(const void* W, const float* scales, const float* x, int ldx, float* out, int ldo,
             int mrows, int N, int K, int group_rows, int accumulate, cudaStream_t st) {
    if (group_rows == 0 && K >= 1024) {
        switch (mrows) {
            case 1: return launch_sk_rb<1, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
            case 2: return launch_sk_rb<2, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
            case 3: return launch_sk_rb<3, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
            case 4: return launch_sk_rb<4, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
            default: return launch_sk<8, 4, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, accumulate, st);
        }
    }
    if (mrows <= 1) return launch_r<1, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate, st);
    if (mrows <= 2) return launch_r<2, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate, st);
    if (mrows <= 4) return launch_r<4, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate, st);
    return launch_r<8, FP8>(W, scales, x, ldx, out, ldo, mrows, N, K, group_rows, accumulate, st);
}

}  // namespace

// W [N,K] bf16; x [m,K] f32 (row stride ldx); out [m,N] f32 (row stride ldo); m <= 8.
// K % 8 == 0, ldx % 4 == 0.  group_rows > 0 makes it block-diagonal: weight rows
// [g*group_rows, (g+1)*group_rows) read x[:, g*K : (g+1)*K].
FB_API int fb_gemv_bf16(const void* W, const float* x, int64_t ldx, float* out, int64_t ldo,
                        int64_t m, int64_t N, int64_t K, int64_t group_rows, int64_t accumulate,
                        cudaStream_t st) {
    if (m < 1 || m > 8 || (K % 8) || (ldx % 4)) return (int)cudaErrorInvalidValue;
    return launch_m<false>(W, nullptr, x, (int)ldx, out, (int)ldo, (int)m, (int)N, (int)K, (int)group_rows, (int)accumulate, st);
}

// W [N,K] e4m3 with scales [ceil(N/128), ceil(K/128)] f32; K % 16 == 0.
FB_API int fb_gemv_fp8(const void* W, const float* scales, const float* x, int64_t ldx, float* out,
                       int64_t ldo, int64_t m, int64_t N, int64_t K, int64_t group_rows,
                       int64_t accumulate, cudaStream_t st) {
    if (m < 1 || m > 8 || (K % 16) || (ldx % 4)) return (int)cudaErrorInvalidValue;
    return launch_m<true>(W, scales, x, (int)ldx, out, (int)ldo, (int)m, (int)N, (int)K, (int)group_rows, (int)accumulate, st);
}

// Tensor-core forms.  xs is a split-activation buffer (planes bf16 hi/lo, f16 hi/lo of
// `xs_plane` elements, row stride xs_ld); bf16 weights read planes 0/1, e4m3 weights read
// planes 2/3.  K must be a multiple of 64 (bf16) / 128 (e4m3); m <= 8.  When os_base is
// given the result is also written in split form (os_mask picks the plane pairs).
FB_API int fb_gemv_mma_bf16(const void* W, const void* xs, int64_t xs_ld, int64_t xs_plane, float* out,
                            int64_t ldo, int64_t m, int64_t N, int64_t K, int64_t group_rows, int64_t accumulate,
                            void* os_base, int64_t os_ld, int64_t os_plane, int64_t os_mask, cudaStream_t st) {
    if (m < 1 || m > 8 * 65535 || (K % 64) || (xs_ld % 8) || (group_rows % 16)) return (int)cudaErrorInvalidValue;
    SplitBuf os{(uint16_t*)os_base, (int)os_ld, (int)os_plane, (int)os_mask};
    return launch_mma<false>(W, nullptr, (const uint16_t*)xs, (int)xs_ld, (int)xs_plane, out, (int)ldo, (int)m, (int)N,
                             (int)K, (int)group_rows, (int)accumulate, os, st);
}

// out_a[m][N_a] = x_a . W_a^T and out_b[m][N_b] = x_b . W_b^T in one launch (bf16 weights, split-plane activations as
// in fb_gemv_mma_bf16; plain stores, no groups).  K_a, K_b multiples of 64.
FB_API int fb_gemv_mma_bf16_dual(const void* Wa, const void* xa, int64_t xa_ld, int64_t xa_plane, float* out_a, int64_t ldo_a,
                                 int64_t Na, int64_t Ka, const void* Wb, const void* xb, int64_t xb_ld, int64_t xb_plane,
                                 float* out_b, int64_t ldo_b, int64_t Nb, int64_t Kb, int64_t m, cudaStream_t st) {
    if (m < 1 || m > 8 * 65535 || (Ka % 64) || (Kb % 64) || (xa_ld % 8) || (xb_ld % 8) || Na < 1 || Nb < 1)
        return (int)cudaErrorInvalidValue;
    const uint16_t* ha = (const uint16_t*)xa;
    const uint16_t* hb = (const uint16_t*)xb;
    GemvProb a{(const uint8_t*)Wa, ha, ha + xa_plane, (int)xa_ld, out_a, (int)ldo_a, (int)Na, (int)Ka};
    GemvProb b{(const uint8_t*)Wb, hb, hb + xb_plane, (int)xb_ld, out_b, (int)ldo_b, (int)Nb, (int)Kb};
    const int ta = (int)((Na + 15) / 16), tb = (int)((Nb + 15) / 16);
    const dim3 grid((unsigned)(ta + tb), (unsigned)((m + 7) / 8));
    if (Ka / 64 >= 64 && Kb / 64 >= 64) {
        FB_LAUNCH((gemv_mma_dual_kernel<16>), grid, 512, 0, st, a, b, ta, (int)m, g_fb_l2_ahead);
    } else {
        FB_LAUNCH((gemv_mma_dual_kernel<8>), grid, 256, 0, st, a, b, ta, (int)m, g_fb_l2_ahead);
    }
    return FB_LAUNCH_CHECK();
}

// fb_gemv_mma_bf16 for the MoE router matrix [E router rows | shared gate | shared up]: the launch also routes the
// rows (ids / wts [m][topk]) from its first E outputs; E <= 384, m <= 8; ticket: one zeroed counter.
FB_API int fb_gemv_mma_bf16_route(const void* W, const void* xs, int64_t xs_ld, int64_t xs_plane, float* out,
                                  int64_t ldo, int64_t m, int64_t N, int64_t K, const float* bias, int* ids, float* wts,
                                  void* ticket, int64_t E, int64_t topk, float scaling, cudaStream_t st) {
    if (m < 1 || m > 8 || (K % 64) || (xs_ld % 8) || E > 32 * kRouteKeys || E > N || topk > 32 || !bias || !ids || !wts || !ticket)
        return (int)cudaErrorInvalidValue;
    RouteTail rt{bias, ids, wts, (unsigned*)ticket, (int)E, (int)topk, scaling};
    return launch_mma<false>(W, nullptr, (const uint16_t*)xs, (int)xs_ld, (int)xs_plane, out, (int)ldo, (int)m, (int)N,
                             (int)K, 0, 0, SplitBuf{nullptr, 0, 0, 0}, st, rt);
}

FB_API int fb_gemv_mma_fp8(const void* W, const float* scales, const void* xs, int64_t xs_ld, int64_t xs_plane,
                           float* out, int64_t ldo, int64_t m, int64_t N, int64_t K, int64_t accumulate,
                           void* os_base, int64_t os_ld, int64_t os_plane, int64_t os_mask, cudaStream_t st) {
    if (m < 1 || m > 8 * 65535 || (K % 128) || (xs_ld % 8)) return (int)cudaErrorInvalidValue;
    SplitBuf os{(uint16_t*)os_base, (int)os_ld, (int)os_plane, (int)os_mask};
    return launch_mma<true>(W, scales, (const uint16_t*)xs, (int)xs_ld, (int)xs_plane, out, (int)ldo, (int)m, (int)N,
                            (int)K, 0, (int)accumulate, os, st);
}

namespace {
__global__ void split_rows_kernel(const float* __restrict__ x, int ldx, SplitBuf s, int K) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < K) split_store(s, r, k, x[(size_t)r * ldx + k]);
}
}  // namespace

// Stand-alone f32 -> split conversion (producers normally emit the split form themselves).
FB_API int fb_split_rows(const float* x, int64_t ldx, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask,
                         int64_t m, int64_t K, cudaStream_t st) {
    SplitBuf s{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    FB_LAUNCH((split_rows_kernel), dim3((unsigned)((K + 255) / 256), (unsigned)m), 256, 0, st, x, (int)ldx, s, (int)K);
    return FB_LAUNCH_CHECK();
}
