// DSV41 routed experts on the tensor cores for decode-sized row counts: e2m1 weights with one ue8m0
// scale per 32 values of K, activations e4m3-per-32 round-tripped (so their f16 copy is exact).
//
// out[16 weight rows x 8] tiles with mma.sync.m16n8k16 (f16 inputs, f32 accumulation): the WEIGHTS are
// the A operand, the activation row is column 0 of the B operand.  e2m1 converts exactly to f16 (one
// cvt per two values); the power-of-two block scale cannot be folded into an f16 operand without range
// limits, so each 32-value block is multiplied into a fresh accumulator (two MMAs) that is then scaled
// per weight row and added to the running sum.  All four lanes of a quad must therefore work on the
// SAME scale block in one MMA, while a lane wants one 16-byte load per row and 128-value k-block.  Both
// hold with a load-time repack of the weight bytes ("quad-interleaved", fb_d4_fp4_repack): inside every
// 64-byte group of a row (128 values = 4 scale blocks x 4 words), word (block b, position q) moves to
// (position q, block b).  Lane q of a quad then reads 16 bytes = its 8 values of each of the 4 blocks.
//
// gate/up:  grid (I / 8, topk, rows): 8 intermediate channels of one (row, slot) pair (gate rows in the upper
//           half of the MMA tile, up rows in the lower half); the warps split K, partial tiles meet in shared
//           memory, the epilogue applies the clamped SwiGLU and the routing weight.
// down:     grid (D / 16, rows): 16 output channels; the warps split the (slot, k-block) list.
// Replaces the reference's `expert_gemv_fp4_*` decode kernels (kernels/cuda/dsv41_kernels.cu).
#include <cuda_fp8.h>
#include <cuda_fp4.h>

#include "mma_gemv.cuh"

namespace {

__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float ue8m0_of(uint32_t word, int b) { return __uint_as_float(((word >> (8 * b)) & 0xffu) << 23); }

// One k-block (128 values) of one 16-row weight tile against the activation fragment: acc[0..1] belong to
// weight row g, acc[2..3] to row g + 8 (columns 2q, 2q + 1 of the activation operand).
//   wa / wb : the lane's 16 repacked bytes of rows g / g + 8;  sa / sb : the 4 scale bytes of the k-block
//   x       : the lane's activation fragment, x[b] = 8 f16 values of scale block b
__device__ __forceinline__ void mma_block_fp4(float (&acc)[4], const uint4& wa, const uint4& wb, uint32_t sa, uint32_t sb,
                                              const uint4 (&x)[4], int nb = 4) {
    const uint32_t A[4] = {wa.x, wa.y, wa.z, wa.w};
    const uint32_t B[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= nb) break;   // warp-uniform: a 64-value tail has two blocks
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        mma_f16_16816(d, e2m1x2_to_f16x2(A[b]), e2m1x2_to_f16x2(B[b]), e2m1x2_to_f16x2(A[b] >> 8), e2m1x2_to_f16x2(B[b] >> 8),
                      x[b].x, x[b].y);
        mma_f16_16816(d, e2m1x2_to_f16x2(A[b] >> 16), e2m1x2_to_f16x2(B[b] >> 16), e2m1x2_to_f16x2(A[b] >> 24),
                      e2m1x2_to_f16x2(B[b] >> 24), x[b].z, x[b].w);
        const float fa = ue8m0_of(sa, b), fb = ue8m0_of(sb, b);
        acc[0] = fmaf(d[0], fa, acc[0]);
        acc[1] = fmaf(d[1], fa, acc[1]);
        acc[2] = fmaf(d[2], fb, acc[2]);
        acc[3] = fmaf(d[3], fb, acc[3]);
    }
}

// The lane's activation fragment of a k-block: row pointer `xr` (f16), only column-0 lanes (g == 0) load.
__device__ __forceinline__ void load_x_fp4(uint4 (&x)[4], const uint16_t* __restrict__ xr, int k0, int g, int tq, int nb = 4) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        x[b] = make_uint4(0u, 0u, 0u, 0u);
        if (g == 0 && b < nb) x[b] = __ldg(reinterpret_cast<const uint4*>(xr + k0 + b * 32 + tq * 8));
    }
}

// The same fragment from f32 rows that are not quantised yet: the e4m3-per-32 round trip (power-of-two block scale)
// happens here.  The 32 values of scale block b sit in the four column-0 lanes (lanes 0..3, 8 values each), so the
// block maximum is two shuffles; the round-tripped values are exact in f16.  All lanes of the warp must call.
__device__ __forceinline__ void load_x_f32_quant(uint4 (&x)[4], const float* __restrict__ xr, int k0, int g, int tq, int nb = 4) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
        if (g == 0 && b < nb) {
            const float4* p = reinterpret_cast<const float4*>(xr + k0 + b * 32 + tq * 8);
            lo = __ldg(p);
            hi = __ldg(p + 1);
        }
        float am = fmaxf(fmaxf(fmaxf(fabsf(lo.x), fabsf(lo.y)), fmaxf(fabsf(lo.z), fabsf(lo.w))),
                         fmaxf(fmaxf(fabsf(hi.x), fabsf(hi.y)), fmaxf(fabsf(hi.z), fabsf(hi.w))));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        // 2^ceil(log2(amax / 448)), amax clamped from below as in the stand-alone quantiser
        const float tt = fmaxf(am, 1e-4f) * (1.f / 448.f);
        const uint32_t tb = __float_as_uint(tt);
        const int ex = (int)((tb >> 23) & 0xff) + ((tb & 0x7fffffu) ? 1 : 0);
        const float sc = __uint_as_float((uint32_t)min(max(ex, 0), 254) << 23);
        const float inv = 1.f / sc;   // a power of two: exact
        auto rt2 = [&](float a, float c) -> uint32_t {
            // e4m3 (saturating) and back: two values per conversion
            const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(make_float2(a * inv, c * inv), __NV_SATFINITE, __NV_E4M3);
            const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(q, __NV_E4M3);
            const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&h), __float2half2_rn(sc));
            return *reinterpret_cast<const uint32_t*>(&r);
        };
        x[b] = make_uint4(rt2(lo.x, lo.y), rt2(lo.z, lo.w), rt2(hi.x, hi.y), rt2(hi.z, hi.w));
    }
}

struct Fp4Frag { uint4 wa, wb; uint32_t sa, sb; };
__device__ __forceinline__ Fp4Frag load_fp4(const uint8_t* __restrict__ wa, const uint8_t* __restrict__ wb,
                                            const uint8_t* __restrict__ sa, const uint8_t* __restrict__ sb, int kb, int tq) {
    Fp4Frag f;
    f.wa = ldg_nc_v4(wa + (size_t)kb * 64 + tq * 16);
    f.wb = ldg_nc_v4(wb + (size_t)kb * 64 + tq * 16);
    // scale rows are only 2-byte aligned when K / 32 is not a multiple of 4
    const uint16_t* pa = reinterpret_cast<const uint16_t*>(sa + (size_t)kb * 4);
    const uint16_t* pb = reinterpret_cast<const uint16_t*>(sb + (size_t)kb * 4);
    f.sa = (uint32_t)__ldg(pa) | ((uint32_t)__ldg(pa + 1) << 16);
    f.sb = (uint32_t)__ldg(pb) | ((uint32_t)__ldg(pb + 1) << 16);
    return f;
}
// The 64-value tail of a row whose length is an odd multiple of 64: 8 bytes per lane, two scale bytes.
__device__ __forceinline__ Fp4Frag load_fp4_tail(const uint8_t* __restrict__ wa, const uint8_t* __restrict__ wb,
                                                 const uint8_t* __restrict__ sa, const uint8_t* __restrict__ sb, int kb, int tq) {
    Fp4Frag f;
    const uint2 a = __ldg(reinterpret_cast<const uint2*>(wa + (size_t)kb * 64 + tq * 8));
    const uint2 b = __ldg(reinterpret_cast<const uint2*>(wb + (size_t)kb * 64 + tq * 8));
    f.wa = make_uint4(a.x, a.y, 0u, 0u);
    f.wb = make_uint4(b.x, b.y, 0u, 0u);
    f.sa = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sa + (size_t)kb * 4));
    f.sb = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sb + (size_t)kb * 4));
    return f;
}

constexpr int kNW = 8;

// One 16-row MMA tile holds 8 intermediate channels: rows 0..7 are their GATE rows, rows 8..15 their UP rows,
// so a thread's accumulators d[0] / d[2] are the gate and up value of the same channel and the SwiGLU needs
// no exchange.  Small tiles keep the grid large at tensor-parallel slice sizes (I = 320: 240 CTAs) and the
// register count low enough for a two-deep prefetch of the weight fragments.
__global__ void __launch_bounds__(kNW * 32)
expert_gate_up_mma_kernel(const uint16_t* __restrict__ xh, int ldx, const int* __restrict__ idx, const float* __restrict__ wts,
                          const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13, float* __restrict__ h, int topk,
                          int I, int K, float lim) {
    pdl_launch();
    __shared__ float red[kNW][2][8];
    const int r = blockIdx.z, s = blockIdx.y, i0 = blockIdx.x * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int nkb = K >> 7;
    const size_t wrow = (size_t)K / 2, srow = (size_t)K / 32;
    pdl_wait();
    const int e = idx[(size_t)r * topk + s];
    const int ri = min(i0 + g, I - 1);
    const uint8_t* wg = w13 + ((size_t)e * 2 * I + ri) * wrow;       // gate row
    const uint8_t* wu = wg + (size_t)I * wrow;                       // up row
    const uint8_t* sg = s13 + ((size_t)e * 2 * I + ri) * srow;
    const uint8_t* su = sg + (size_t)I * srow;
    const uint16_t* xr = xh + (size_t)r * ldx;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // two fragment buffers alternate roles (one loads while the other is multiplied): no register copies
    Fp4Frag fa, fb;
    auto compute = [&](const Fp4Frag& f, int kb) {
        uint4 x[4];
        load_x_fp4(x, xr, kb * 128, g, tq);
        mma_block_fp4(acc, f.wa, f.wb, f.sa, f.sb, x);
    };
    int kb = warp;
    if (kb < nkb) fa = load_fp4(wg, wu, sg, su, kb, tq);
    while (kb < nkb) {
        const int k1 = kb + kNW;
        if (k1 < nkb) fb = load_fp4(wg, wu, sg, su, k1, tq);
        compute(fa, kb);
        if (k1 >= nkb) break;
        const int k2 = k1 + kNW;
        if (k2 < nkb) fa = load_fp4(wg, wu, sg, su, k2, tq);
        compute(fb, k1);
        kb = k2;
    }
    if (tq == 0) { red[warp][0][g] = acc[0]; red[warp][1][g] = acc[2]; }   // column 0: gate (row g), up (row g + 8)
    __syncthreads();
    if (threadIdx.x < 8 && i0 + threadIdx.x < I) {
        float gv = 0.f, uv = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) { gv += red[w][0][threadIdx.x]; uv += red[w][1][threadIdx.x]; }
        if (lim > 0.f) { uv = fminf(fmaxf(uv, -lim), lim); gv = fminf(gv, lim); }
        h[((size_t)r * topk + s) * I + i0 + threadIdx.x] = gv / (1.f + __expf(-gv)) * uv * wts[(size_t)r * topk + s];
    }
}

// QF: `hh` holds f32 rows that are quantised on load (no separate quantiser launch before this kernel).
template <bool QF>
__global__ void __launch_bounds__(kNW * 32)
expert_down_mma_kernel(const void* __restrict__ hh, const int* __restrict__ idx, const uint8_t* __restrict__ w2,
                       const uint8_t* __restrict__ s2, float* __restrict__ y, int ldy, int topk, int I, int D, int accumulate) {
    pdl_launch();
    __shared__ float red[kNW][16];
    const int r = blockIdx.y, c0 = blockIdx.x * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int nfull = I >> 7, nkb = (I + 127) >> 7;   // a slot's last k-block may hold 64 values
    const size_t wrow = (size_t)I / 2, srow = (size_t)I / 32;
    const int ra = min(c0 + g, D - 1), rb = min(c0 + g + 8, D - 1);
    pdl_wait();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // items are (slot, k-block) pairs; coordinates advance incrementally (no division per item), two fragment
    // buffers alternate roles
    struct Item { int s, kb; };
    auto advance = [&](Item& q) { q.kb += kNW; while (q.kb >= nkb) { q.kb -= nkb; ++q.s; } };
    auto fetch = [&](const Item& q, Fp4Frag& f) {
        if (q.s >= topk) return;
        const int e = idx[(size_t)r * topk + q.s];
        const uint8_t* wb = w2 + (size_t)e * D * wrow;
        const uint8_t* sb = s2 + (size_t)e * D * srow;
        f = q.kb < nfull ? load_fp4(wb + ra * wrow, wb + rb * wrow, sb + ra * srow, sb + rb * srow, q.kb, tq)
                         : load_fp4_tail(wb + ra * wrow, wb + rb * wrow, sb + ra * srow, sb + rb * srow, q.kb, tq);
    };
    auto compute = [&](const Item& q, const Fp4Frag& f) {
        const int nb = q.kb < nfull ? 4 : 2;
        uint4 x[4];
        if constexpr (QF) load_x_f32_quant(x, static_cast<const float*>(hh) + ((size_t)r * topk + q.s) * I, q.kb * 128, g, tq, nb);
        else load_x_fp4(x, static_cast<const uint16_t*>(hh) + ((size_t)r * topk + q.s) * I, q.kb * 128, g, tq, nb);
        mma_block_fp4(acc, f.wa, f.wb, f.sa, f.sb, x, nb);
    };
    Fp4Frag fa, fb;
    Item qa{warp / nkb, warp % nkb}, qb;
    fetch(qa, fa);
    while (qa.s < topk) {
        qb = qa; advance(qb); fetch(qb, fb);
        compute(qa, fa);
        if (qb.s >= topk) break;
        qa = qb; advance(qa); fetch(qa, fa);
        compute(qb, fb);
    }
    if (tq == 0) { red[warp][g] = acc[0]; red[warp][g + 8] = acc[2]; }
    __syncthreads();
    if (threadIdx.x < 16 && c0 + threadIdx.x < D) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) v += red[w][threadIdx.x];
        float* o = y + (size_t)r * ldy + c0 + threadIdx.x;
        *o = accumulate ? *o + v : v;
    }
}

// In place, per row: inside every 64-byte group the 4 x 4 matrix of 32-bit words is transposed; a
// 32-byte tail (rows that are an odd multiple of 64 values) is a 2 x 4 matrix: word (block b, position
// q) moves to q * 2 + b.  One thread per group.
__global__ void __launch_bounds__(256)
fp4_repack_kernel(uint8_t* __restrict__ w, size_t rows, int row_bytes, int inverse) {
    const int gpr = (row_bytes + 63) / 64;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * gpr) return;
    const size_t row = i / gpr;
    const int grp = (int)(i % gpr);
    uint8_t* base = w + row * row_bytes + (size_t)grp * 64;
    if (grp * 64 + 64 <= row_bytes) {
        uint4* p = reinterpret_cast<uint4*>(base);
        const uint4 a = p[0], b = p[1], c = p[2], d = p[3];
        p[0] = make_uint4(a.x, b.x, c.x, d.x);
        p[1] = make_uint4(a.y, b.y, c.y, d.y);
        p[2] = make_uint4(a.z, b.z, c.z, d.z);
        p[3] = make_uint4(a.w, b.w, c.w, d.w);
    } else {
        uint4* p = reinterpret_cast<uint4*>(base);
        const uint4 a = p[0], b = p[1];
        if (!inverse) {
            p[0] = make_uint4(a.x, b.x, a.y, b.y);
            p[1] = make_uint4(a.z, b.z, a.w, b.w);
        } else {
            p[0] = make_uint4(a.x, a.z, b.x, b.z);
            p[1] = make_uint4(a.y, a.w, b.y, b.w);
        }
    }
}

}  // namespace

// Quad-interleave packed e2m1 rows in place; inverse != 0 restores the original bytes.
// row_bytes (= K / 2) must be a multiple of 32; 16-byte aligned base.
FB_API int fb_d4_fp4_repack(void* w, int64_t rows, int64_t row_bytes, int64_t inverse, cudaStream_t st) {
    if ((row_bytes % 32) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
    const size_t groups = (size_t)rows * ((row_bytes + 63) / 64);
    if (!groups) return 0;
    FB_LAUNCH((fp4_repack_kernel), (unsigned)((groups + 255) / 256), 256, 0, st, (uint8_t*)w, (size_t)rows, (int)row_bytes,
              (int)inverse);
    return FB_LAUNCH_CHECK();
}

// xh: f16 plane of the e4m3-round-tripped input rows (row stride ldx elements); w13 [E][2][I][K/2]
// quad-interleaved, s13 [E][2][I][K/32]; h [rows][topk][I] f32.  K % 128 == 0.
FB_API int fb_d4_expert_gate_up_mma(const void* xh, int64_t ldx, const int* idx, const float* wts, const void* w13,
                                    const void* s13, float* h, int64_t n, int64_t topk, int64_t I, int64_t K, float lim,
                                    cudaStream_t st) {
    if ((K % 128) || (ldx % 8) || ((uintptr_t)xh & 15)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((expert_gate_up_mma_kernel), dim3((unsigned)((I + 7) / 8), (unsigned)topk, (unsigned)n), kNW * 32, 0, st,
              (const uint16_t*)xh, (int)ldx, idx, wts, (const uint8_t*)w13, (const uint8_t*)s13, h, (int)topk, (int)I, (int)K, lim);
    return FB_LAUNCH_CHECK();
}

// hh: f16 plane of the e4m3-round-tripped h [rows][topk][I]; w2 [E][D][I/2] quad-interleaved, s2 [E][D][I/32].
// I % 64 == 0.
FB_API int fb_d4_expert_down_mma(const void* hh, const int* idx, const void* w2, const void* s2, float* y, int64_t ldy,
                                 int64_t n, int64_t topk, int64_t I, int64_t D, int64_t accumulate, cudaStream_t st) {
    if ((I % 64) || ((uintptr_t)hh & 15)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((expert_down_mma_kernel<false>), dim3((unsigned)((D + 15) / 16), (unsigned)n), kNW * 32, 0, st, hh, idx,
              (const uint8_t*)w2, (const uint8_t*)s2, y, (int)ldy, (int)topk, (int)I, (int)D, (int)accumulate);
    return FB_LAUNCH_CHECK();
}

// The same with h [rows][topk][I] in f32, NOT yet quantised: every CTA applies the e4m3-per-32 round trip to the
// blocks it loads (the result equals fb_d4_quant_rows followed by fb_d4_expert_down_mma, one launch fewer).
FB_API int fb_d4_expert_down_mma_f32(const float* h, const int* idx, const void* w2, const void* s2, float* y, int64_t ldy,
                                     int64_t n, int64_t topk, int64_t I, int64_t D, int64_t accumulate, cudaStream_t st) {
    if ((I % 64) || ((uintptr_t)h & 15)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((expert_down_mma_kernel<true>), dim3((unsigned)((D + 15) / 16), (unsigned)n), kNW * 32, 0, st, (const void*)h, idx,
              (const uint8_t*)w2, (const uint8_t*)s2, y, (int)ldy, (int)topk, (int)I, (int)D, (int)accumulate);
    return FB_LAUNCH_CHECK();
}
