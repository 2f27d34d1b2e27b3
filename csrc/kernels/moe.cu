// MoE decode path: sigmoid noaux-tc routing and W8A16 fp8 expert GEMVs.
//
//   s = sigmoid(logits); choose top-k of (s + bias), ties to the lower index;
//   w = s_sel / (sum s_sel + eps_f32) * scaling                      (cpu.rs:528-572)
//   y = sum_slot w_slot * down_e(silu(min(gate_e x, L)) * clamp(up_e x, +-L))
// Expert weights stay e4m3 with 128x128 block scales in HBM and are dequantised in
// registers; activations are f32.  gate/up of an expert are one [2I, H] matrix (gate rows
// first) so a warp streams the two rows of an output pair together and applies SwiGLU in
// its epilogue; the down kernel folds the routing weights and the sum over slots, so no
// per-slot buffer is reduced afterwards.  Replaces moe_route, router_gemm_route_fused,
// moe_fused_act(_fp8), moe_fused_down_sum(_fp8), moe_weighted_sum, swiglu/swiglu2
// (kernels/cuda/ferrite_kernels.cu:392-421,1207-1300,2977,4021-4499).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

__device__ __forceinline__ uint32_t okey(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// E <= 384: the block computes the sigmoids and the order-preserving selection keys into shared memory, then ONE warp
// picks: lane l holds experts l, l + 32, ... in registers, a pick is a register scan, a warp-wide integer maximum and a
// warp-wide minimum over the indices that hold it (two redux instructions) instead of three block barriers and a serial
// scan by thread 0.  Same picks, same pick order, same sums as the general form below.
constexpr int kFastSlots = 12;
__device__ __forceinline__ void moe_route_row_fast(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                                   int* __restrict__ ids, float* __restrict__ wts, int E, int topk,
                                                   float scaling, int r) {
    __shared__ uint32_t u_s[32 * kFastSlots];
    __shared__ float sig_s[32 * kFastSlots];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float s = 1.f / (1.f + expf(-logits[(size_t)r * ld + e]));
        sig_s[e] = s;
        u_s[e] = okey(s + bias[e]);   // > 0 for every number; 0 marks "not (or no longer) a candidate"
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    uint32_t u[kFastSlots];
    float sg[kFastSlots];
#pragma unroll
    for (int j = 0; j < kFastSlots; ++j) {
        const int e = lane + 32 * j;
        u[j] = e < E ? u_s[e] : 0u;
        sg[j] = e < E ? sig_s[e] : 0.f;
    }
    float sum = 0.f, my_s = 0.f;
    int my_e = 0;
    for (int k = 0; k < topk; ++k) {
        uint32_t m[kFastSlots / 2];
#pragma unroll
        for (int j = 0; j < kFastSlots / 2; ++j) m[j] = max(u[2 * j], u[2 * j + 1]);
        const uint32_t gm = __reduce_max_sync(0xffffffffu, max(max(max(m[0], m[1]), max(m[2], m[3])), max(m[4], m[5])));
        uint32_t ce = 0xffffffffu;
#pragma unroll
        for (int j = kFastSlots - 1; j >= 0; --j) ce = (u[j] == gm) ? (uint32_t)(lane + 32 * j) : ce;   // lowest index last
        const int e = (int)__reduce_min_sync(0xffffffffu, ce);
        const int jw = e >> 5, lw = e & 31;
        float mine = 0.f;
#pragma unroll
        for (int j = 0; j < kFastSlots; ++j) {
            if (j == jw) {
                mine = sg[j];
                if (lane == lw) u[j] = 0u;
            }
        }
        const float sv = __shfl_sync(0xffffffffu, mine, lw);
        if (lane == k) { my_s = sv; my_e = e; }
        sum += sv;
    }
    if (lane < topk) {
        const float inv = scaling / (sum + 1.1920929e-07f);
        ids[(size_t)r * topk + lane] = my_e;
        wts[(size_t)r * topk + lane] = my_s * inv;
    }
}

// One block (256 threads) per row; E <= 1024.
__device__ __forceinline__ void moe_route_row(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                              int* __restrict__ ids, float* __restrict__ wts, int E, int topk, float scaling, int r) {
    __shared__ unsigned long long wbest[8];
    __shared__ unsigned long long s_pick;
    __shared__ float s_sig[1024];
    __shared__ float s_sel[32];
    unsigned long long key[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x + i * 256;
        key[i] = 0ull;
        if (e < E) {
            const float s = 1.f / (1.f + expf(-logits[(size_t)r * ld + e]));
            s_sig[e] = s;
            key[i] = ((unsigned long long)okey(s + bias[e]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)e);
        }
    }
    __syncthreads();
    for (int k = 0; k < topk; ++k) {
        unsigned long long best = 0ull;
#pragma unroll
        for (int i = 0; i < 4; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
            best = t > best ? t : best;
        }
        if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = 0ull;
            for (int w = 0; w < 8; ++w) b = wbest[w] > b ? wbest[w] : b;
            s_pick = b;
            const int e = (int)(0xffffffffu - (uint32_t)(b & 0xffffffffull));
            ids[(size_t)r * topk + k] = e;
            s_sel[k] = s_sig[e];
        }
        __syncthreads();
        const unsigned long long pick = s_pick;
#pragma unroll
        for (int i = 0; i < 4; ++i) if (key[i] == pick) key[i] = 0ull;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float sum = 0.f;
        for (int k = 0; k < topk; ++k) sum += s_sel[k];
        const float inv = scaling / (sum + 1.1920929e-07f);
        for (int k = 0; k < topk; ++k) wts[(size_t)r * topk + k] = s_sel[k] * inv;
    }
}

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int* __restrict__ ids,
                 float* __restrict__ wts, int E, int topk, float scaling) {
    PDL_PROLOGUE();
    if (E <= 32 * kFastSlots && topk <= E) moe_route_row_fast(logits, ld, bias, ids, wts, E, topk, scaling, blockIdx.x);
    else moe_route_row(logits, ld, bias, ids, wts, E, topk, scaling, blockIdx.x);
}


// act[r][s][i] = swiglu(gate_i . x_r, up_i . x_r) for expert ids[r][s]; one warp owns IPW pairs.
template <int IPW>
__global__ void __launch_bounds__(256)
moe_gate_up_fp8_kernel(const uint8_t* __restrict__ W13, const float* __restrict__ S13,
                       const float* __restrict__ x, int ldx, const int* __restrict__ ids,
                       float* __restrict__ act, int topk, int I, int H, int e_lo, int e_cnt, float limit) {
    PDL_PROLOGUE();
    const int pair = blockIdx.y;  // r * topk + s
    const int r = pair / topk;
    const int le = ids[pair] - e_lo;
    const int lane = threadIdx.x & 31;
    const int i0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * IPW;
    if (i0 >= I) return;
    float* dst = act + (size_t)pair * I;
    if (le < 0 || le >= e_cnt) {  // expert lives on another rank: contributes nothing here
        if (lane == 0) for (int j = 0; j < IPW && i0 + j < I; ++j) dst[i0 + j] = 0.f;
        return;
    }
    const int kb = (H + 127) >> 7;
    const int nb = (2 * I + 127) >> 7;
    const uint8_t* W = W13 + (size_t)le * 2 * I * H;
    const float* S = S13 + (size_t)le * nb * kb;
    const float* xr = x + (size_t)r * ldx;
    float ag[IPW], au[IPW];
#pragma unroll
    for (int j = 0; j < IPW; ++j) { ag[j] = 0.f; au[j] = 0.f; }
#pragma unroll 2
    for (int k = lane * 16; k < H; k += 512) {
        uint4 wg[IPW], wu[IPW];
#pragma unroll
        for (int j = 0; j < IPW; ++j) {
            const int i = min(i0 + j, I - 1);
            wg[j] = ldg_nc_v4(W + (size_t)i * H + k);
            wu[j] = ldg_nc_v4(W + (size_t)(I + i) * H + k);
        }
        float xv[16];
#pragma unroll
        for (int v = 0; v < 16; v += 4) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(xr + k + v));
            xv[v] = t.x; xv[v + 1] = t.y; xv[v + 2] = t.z; xv[v + 3] = t.w;
        }
#pragma unroll
        for (int j = 0; j < IPW; ++j) {
            const int i = min(i0 + j, I - 1);
            float wf[16];
            const uint32_t* pg = reinterpret_cast<const uint32_t*>(&wg[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) e4m3x4_to_f32(pg[q], &wf[4 * q]);
            float p = 0.f;
#pragma unroll
            for (int v = 0; v < 16; ++v) p = fmaf(wf[v], xv[v], p);
            ag[j] = fmaf(p, __ldg(S + (size_t)(i >> 7) * kb + (k >> 7)), ag[j]);
            const uint32_t* pu = reinterpret_cast<const uint32_t*>(&wu[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) e4m3x4_to_f32(pu[q], &wf[4 * q]);
            p = 0.f;
#pragma unroll
            for (int v = 0; v < 16; ++v) p = fmaf(wf[v], xv[v], p);
            au[j] = fmaf(p, __ldg(S + (size_t)((I + i) >> 7) * kb + (k >> 7)), au[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < IPW; ++j) {
        const float g = warp_sum(ag[j]), u = warp_sum(au[j]);
        if (lane == 0 && i0 + j < I) {
            const float gc = fminf(g, limit);
            const float uc = fminf(fmaxf(u, -limit), limit);
            dst[i0 + j] = siluf_(gc) * uc;
        }
    }
}

// out[r][c] (+)= sum_s wts[r][s] * (W2[e_s][c][:] . act[r][s][:]); one warp owns CPW columns,
// lanes stride over the flattened (slot, 16-element chunk) space.
template <int CPW>
__global__ void __launch_bounds__(256)
moe_down_fp8_kernel(const uint8_t* __restrict__ W2, const float* __restrict__ S2,
                    const float* __restrict__ act, const int* __restrict__ ids,
                    const float* __restrict__ wts, float* __restrict__ out, int ldo, int topk, int I, int H,
                    int e_lo, int e_cnt, int accumulate) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int c0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * CPW;
    if (c0 >= H) return;
    const int cpr = I >> 4;  // 16-element chunks per weight row
    const int kb = (I + 127) >> 7;
    const int nb = (H + 127) >> 7;
    float acc[CPW];
#pragma unroll
    for (int j = 0; j < CPW; ++j) acc[j] = 0.f;
    const int items = topk * cpr;
#pragma unroll 2
    for (int it = lane; it < items; it += 32) {
        const int s = it / cpr, ck = it % cpr;
        const int le = ids[(size_t)r * topk + s] - e_lo;
        if (le < 0 || le >= e_cnt) continue;
        const float wt = wts[(size_t)r * topk + s];
        const uint8_t* W = W2 + (size_t)le * H * I;
        const float* S = S2 + (size_t)le * nb * kb;
        const int k = ck * 16;
        uint4 wv[CPW];
#pragma unroll
        for (int j = 0; j < CPW; ++j) wv[j] = ldg_nc_v4(W + (size_t)min(c0 + j, H - 1) * I + k);
        const float* a = act + ((size_t)r * topk + s) * I + k;
        float xv[16];
#pragma unroll
        for (int v = 0; v < 16; v += 4) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(a + v));
            xv[v] = t.x; xv[v + 1] = t.y; xv[v + 2] = t.z; xv[v + 3] = t.w;
        }
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            float wf[16];
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wv[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) e4m3x4_to_f32(pw[q], &wf[4 * q]);
            float p = 0.f;
#pragma unroll
            for (int v = 0; v < 16; ++v) p = fmaf(wf[v], xv[v], p);
            acc[j] = fmaf(p * wt, __ldg(S + (size_t)(min(c0 + j, H - 1) >> 7) * kb + (k >> 7)), acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < CPW; ++j) {
        const float v = warp_sum(acc[j]);
        if (lane == 0 && c0 + j < H) {
            float* o = out + (size_t)r * ldo + c0 + j;
            *o = accumulate ? (*o + v) : v;
        }
    }
}


// ---- tensor-core forms (see mma_gemv.cuh) --------------------------------------------------
// gate/up: a CTA owns 16 gate rows and the matching 16 up rows of one (row, slot) pair's
// expert; activations sit in MMA column 0.  The epilogue applies SwiGLU, multiplies by the
// routing weight (so the down kernel is a plain sum over slots) and writes the result in
// f16 split form for the down kernel.
constexpr int kGuWarps = 4;
__global__ void __launch_bounds__(kGuWarps * 32)
moe_gate_up_mma_kernel(const uint8_t* __restrict__ W13, const float* __restrict__ S13,
                       const uint16_t* __restrict__ xhi, const uint16_t* __restrict__ xlo, int ldx,
                       const int* __restrict__ ids, const float* __restrict__ wts, SplitBuf asplit,
                       int topk, int I, int H, int e_lo, int e_cnt, float limit) {
    PDL_PROLOGUE();
    __shared__ float red[kGuWarps][2][32][4];
    const int pair = blockIdx.y;
    const int r = pair / topk;
    const int le = ids[pair] - e_lo;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int i0 = blockIdx.x * 16;
    if (le < 0 || le >= e_cnt) {
        if (threadIdx.x < 16 && i0 + threadIdx.x < I) split_store(asplit, pair, i0 + threadIdx.x, 0.f);
        return;
    }
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
    const uint16_t* xh_row = xhi + (size_t)r * ldx;
    const uint16_t* xl_row = xlo + (size_t)r * ldx;
    // two fragment sets alternate roles (load one while the other is multiplied): no register copies per k-block
    WFrag fa[2], fb[2];
    auto fetch = [&](WFrag (&f)[2], int kb) {
#pragma unroll
        for (int q = 0; q < 2; ++q) f[q] = load_wfrag(wa[q] + (size_t)kb * 128, wb[q] + (size_t)kb * 128);
    };
    auto compute = [&](const WFrag (&f)[2], int kb) {
        uint32_t xh[16], xl[16];
        load_xfrag<16, false>(xh_row, xl_row, 0, g, 1, kb * 128 + t * 32, xh, xl);  // column 0 only
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            mma_wfrag_fp8<false>(d, f[q], xh, xl);
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
    if (threadIdx.x < 16 && i0 + threadIdx.x < I) {
        const int j = threadIdx.x;           // row of the tile
        const int l = (j & 7) * 4, c = (j >> 3) * 2;  // lane with t == 0, column 0
        float gsum = 0.f, usum = 0.f;
#pragma unroll
        for (int w = 0; w < kGuWarps; ++w) { gsum += red[w][0][l][c]; usum += red[w][1][l][c]; }
        const float gc = fminf(gsum, limit);
        const float uc = fminf(fmaxf(usum, -limit), limit);
        split_store(asplit, pair, i0 + j, siluf_(gc) * uc * wts[pair]);
    }
}

// down: a CTA owns 16 output columns of one row; warps walk the (slot, k-block) items.
// act comes pre-multiplied by the routing weights, in f16 split form.
__global__ void __launch_bounds__(256, 3)
moe_down_mma_kernel(const uint8_t* __restrict__ W2, const float* __restrict__ S2,
                    const uint16_t* __restrict__ ahi, const uint16_t* __restrict__ alo, int lda,
                    const int* __restrict__ ids, float* __restrict__ out, int ldo, int topk, int I, int H,
                    int e_lo, int e_cnt, int accumulate, SplitBuf osplit) {
    PDL_PROLOGUE();
    __shared__ float red[8][32][4];
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int c0 = blockIdx.x * 16;
    const int kb_n = I >> 7;
    const int nb = (H + 127) >> 7;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const size_t ra = (size_t)min(c0 + g, H - 1) * I + t * 32, rb = (size_t)min(c0 + g + 8, H - 1) * I + t * 32;
    // Items are (slot, k-block) pairs; warp w takes items w, w + 8, ...  The coordinates advance incrementally (no
    // division per item) and the two fragment buffers alternate roles (no register copies): the kernel issues about
    // as many instructions per weight byte as the memory system can hide, so the bookkeeping is kept minimal.
    struct Item { int s, kb, le; float sc; };
    auto advance = [&](Item& q) { q.kb += 8; while (q.kb >= kb_n) { q.kb -= kb_n; ++q.s; } };
    auto fetch = [&](Item& q, WFrag& f) {   // loads the item's weights and block scale; le = -1: not a local expert
        q.le = -1;
        if (q.s >= topk) return;
        const int le = ids[r * topk + q.s] - e_lo;
        if (le < 0 || le >= e_cnt) return;
        const uint8_t* W = W2 + (size_t)le * H * I + (size_t)q.kb * 128;
        f = load_wfrag(W + ra, W + rb);
        q.sc = __ldg(S2 + (size_t)le * nb * kb_n + (size_t)(c0 >> 7) * kb_n + q.kb);
        q.le = le;
    };
    auto compute = [&](const Item& q, const WFrag& f) {
        if (q.le < 0) return;  // warp-uniform
        const int pair = r * topk + q.s;
        uint32_t xh[16], xl[16];
        load_xfrag<16, false>(ahi + (size_t)pair * lda, alo + (size_t)pair * lda, 0, g, 1, q.kb * 128 + t * 32, xh, xl);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        mma_wfrag_fp8<false>(d, f, xh, xl);
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] = fmaf(d[c], q.sc, acc[c]);
    };
    WFrag fa, fb;
    Item qa{warp / kb_n, warp % kb_n, -1, 0.f}, qb;
    fetch(qa, fa);
    while (qa.s < topk) {
        qb = qa; advance(qb); fetch(qb, fb);
        compute(qa, fa);
        if (qb.s >= topk) break;
        qa = qb; advance(qa); fetch(qa, fa);
        compute(qb, fb);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][lane][c] = acc[c];
    __syncthreads();
    if (threadIdx.x < 16 && c0 + threadIdx.x < H) {
        const int j = threadIdx.x;
        const int l = (j & 7) * 4, c = (j >> 3) * 2;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][l][c];
        float* o = out + (size_t)r * ldo + c0 + j;
        if (accumulate) v += *o;
        *o = v;
        split_store(osplit, r, c0 + j, v);
    }
}

__global__ void swiglu_kernel(const float* __restrict__ gu, int ld, float* __restrict__ act, int I, float limit,
                              SplitBuf asplit) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const float g = fminf(gu[(size_t)r * ld + i], limit);
    const float u = fminf(fmaxf(gu[(size_t)r * ld + I + i], -limit), limit);
    const float v = siluf_(g) * u;
    if (act) act[(size_t)r * I + i] = v;
    split_store(asplit, r, i, v);
}

// Route and the shared expert's SwiGLU in one launch: both read the row of [router logits | shared gate | shared up]
// that one GEMV produced.  grid (1 + ceil(I / 256), rows): block x == 0 routes, the others apply the SwiGLU.
__global__ void __launch_bounds__(256)
moe_route_swiglu_kernel(const float* __restrict__ lg, int ld, const float* __restrict__ bias, int* __restrict__ ids,
                        float* __restrict__ wts, int E, int topk, float scaling, float* __restrict__ act, int I, float limit,
                        SplitBuf asplit) {
    PDL_PROLOGUE();
    if (blockIdx.x == 0) {
        if (E <= 32 * kFastSlots && topk <= E) moe_route_row_fast(lg, ld, bias, ids, wts, E, topk, scaling, blockIdx.y);
        else moe_route_row(lg, ld, bias, ids, wts, E, topk, scaling, blockIdx.y);
        return;
    }
    const int r = blockIdx.y;
    const int i = (blockIdx.x - 1) * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const float* gu = lg + E;
    const float g = fminf(gu[(size_t)r * ld + i], limit);
    const float u = fminf(fmaxf(gu[(size_t)r * ld + I + i], -limit), limit);
    const float v = siluf_(g) * u;
    if (act) act[(size_t)r * I + i] = v;
    split_store(asplit, r, i, v);
}

}  // namespace

// lg [n, ld] = [E router logits | I shared gate | I shared up] per row; act / split planes get the shared SwiGLU.
FB_API int fb_moe_route_swiglu(const float* lg, int64_t ld, const float* bias, int* ids, float* wts, int64_t n, int64_t E,
                               int64_t topk, float scaling, float* act, void* s_base, int64_t s_ld, int64_t s_plane,
                               int64_t s_mask, int64_t I, float limit, cudaStream_t st) {
    if (E > 1024 || topk > 32) return (int)cudaErrorInvalidValue;
    SplitBuf sp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    FB_LAUNCH((moe_route_swiglu_kernel), dim3((unsigned)(1 + (I + 255) / 256), (unsigned)n), 256, 0, st, lg, (int)ld, bias, ids,
              wts, (int)E, (int)topk, scaling, act, (int)I, limit, sp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_moe_route(const float* logits, int64_t ld, const float* bias, int* ids, float* wts, int64_t n,
                        int64_t E, int64_t topk, float scaling, cudaStream_t st) {
    if (E > 1024 || topk > 32) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((moe_route_kernel), n, 256, 0, st, logits, (int)ld, bias, ids, wts, (int)E, (int)topk, scaling);
    return FB_LAUNCH_CHECK();
}

// W13 [E_loc, 2I, H] e4m3 (gate rows then up rows), S13 [E_loc, ceil(2I/128), ceil(H/128)];
// act [n, topk, I].  Experts outside [e_lo, e_lo+e_cnt) produce zeros.
FB_API int fb_moe_gate_up_fp8(const void* W13, const float* S13, const float* x, int64_t ldx, const int* ids,
                              float* act, int64_t n, int64_t topk, int64_t I, int64_t H, int64_t e_lo,
                              int64_t e_cnt, float limit, cudaStream_t st) {
    if (H % 16) return (int)cudaErrorInvalidValue;
    const int64_t pairs = n * topk;
    const int ipw = (I * pairs >= 148 * 8 * 8) ? 4 : ((I * pairs >= 148 * 8 * 4) ? 2 : 1);
    dim3 grid((unsigned)((I + 8 * ipw - 1) / (8 * ipw)), (unsigned)pairs);
#define GU_ARGS (const uint8_t*)W13, S13, x, (int)ldx, ids, act, (int)topk, (int)I, (int)H, (int)e_lo, (int)e_cnt, limit
    if (ipw == 4) FB_LAUNCH((moe_gate_up_fp8_kernel<4>), grid, 256, 0, st, GU_ARGS);
    else if (ipw == 2) FB_LAUNCH((moe_gate_up_fp8_kernel<2>), grid, 256, 0, st, GU_ARGS);
    else FB_LAUNCH((moe_gate_up_fp8_kernel<1>), grid, 256, 0, st, GU_ARGS);
#undef GU_ARGS
    return FB_LAUNCH_CHECK();
}

// W2 [E_loc, H, I] e4m3, S2 [E_loc, ceil(H/128), ceil(I/128)]; out [n, H].
FB_API int fb_moe_down_fp8(const void* W2, const float* S2, const float* act, const int* ids, const float* wts,
                           float* out, int64_t ldo, int64_t n, int64_t topk, int64_t I, int64_t H,
                           int64_t e_lo, int64_t e_cnt, int64_t accumulate, cudaStream_t st) {
    if (I % 16) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)((H + 31) / 32), (unsigned)n);
    FB_LAUNCH((moe_down_fp8_kernel<4>), grid, 256, 0, st, (const uint8_t*)W2, S2, act, ids, wts, out, (int)ldo, (int)topk,
                                                  (int)I, (int)H, (int)e_lo, (int)e_cnt, (int)accumulate);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_swiglu(const float* gu, int64_t ld, float* act, int64_t n, int64_t I, float limit, cudaStream_t st) {
    SplitBuf none{nullptr, 0, 0, 0};
    FB_LAUNCH((swiglu_kernel), dim3((unsigned)((I + 255) / 256), (unsigned)n), 256, 0, st, gu, (int)ld, act, (int)I, limit, none);
    return FB_LAUNCH_CHECK();
}

// act (f32, optional) and/or its split form (row stride s_ld).
FB_API int fb_swiglu_split(const float* gu, int64_t ld, float* act, void* s_base, int64_t s_ld, int64_t s_plane,
                           int64_t s_mask, int64_t n, int64_t I, float limit, cudaStream_t st) {
    SplitBuf sp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    FB_LAUNCH((swiglu_kernel), dim3((unsigned)((I + 255) / 256), (unsigned)n), 256, 0, st, gu, (int)ld, act, (int)I, limit, sp);
    return FB_LAUNCH_CHECK();
}

// Tensor-core expert kernels.  xs: split activations (f16 planes 2/3 are read), one row per
// token.  as: split buffer of n*topk rows x I (f16 planes) that carries
// swiglu(gate, up) * routing weight from gate_up to down.  H % 128 == 0 and I % 128 == 0.
FB_API int fb_moe_gate_up_mma(const void* W13, const float* S13, const void* xs, int64_t xs_ld, int64_t xs_plane,
                              const int* ids, const float* wts, void* as_base, int64_t as_ld, int64_t as_plane,
                              int64_t n, int64_t topk, int64_t I, int64_t H, int64_t e_lo, int64_t e_cnt,
                              float limit, cudaStream_t st) {
    if ((H % 128) || (xs_ld % 8)) return (int)cudaErrorInvalidValue;
    const uint16_t* hi = (const uint16_t*)xs + 2 * xs_plane;
    SplitBuf asp{(uint16_t*)as_base, (int)as_ld, (int)as_plane, 2};
    dim3 grid((unsigned)((I + 15) / 16), (unsigned)(n * topk));
    FB_LAUNCH((moe_gate_up_mma_kernel), grid, kGuWarps * 32, 0, st, (const uint8_t*)W13, S13, hi, hi + xs_plane, (int)xs_ld, ids, wts, asp,
                                                 (int)topk, (int)I, (int)H, (int)e_lo, (int)e_cnt, limit);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_moe_down_mma(const void* W2, const float* S2, const void* as_base, int64_t as_ld, int64_t as_plane,
                           const int* ids, float* out, int64_t ldo, int64_t n, int64_t topk, int64_t I, int64_t H,
                           int64_t e_lo, int64_t e_cnt, int64_t accumulate, void* os_base, int64_t os_ld,
                           int64_t os_plane, int64_t os_mask, cudaStream_t st) {
    if ((I % 128) || (as_ld % 8)) return (int)cudaErrorInvalidValue;
    const uint16_t* hi = (const uint16_t*)as_base + 2 * as_plane;
    SplitBuf os{(uint16_t*)os_base, (int)os_ld, (int)os_plane, (int)os_mask};
    dim3 grid((unsigned)((H + 15) / 16), (unsigned)n);
    FB_LAUNCH((moe_down_mma_kernel), grid, 256, 0, st, (const uint8_t*)W2, S2, hi, hi + as_plane, (int)as_ld, ids, out, (int)ldo,
                                              (int)topk, (int)I, (int)H, (int)e_lo, (int)e_cnt, (int)accumulate, os);
    return FB_LAUNCH_CHECK();
}
