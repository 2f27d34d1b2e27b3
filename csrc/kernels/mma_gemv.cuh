// Tensor-core core for weight-streaming GEMVs with 1..8 activation rows.
//
// out[m][n] = sum_k x[m][k] W[n][k] is computed as D[16 weight rows x 8 act rows] with
// mma.sync.m16n8k16: the WEIGHTS are the A operand (16 rows), the activations are the B
// operand padded to 8 columns ("swapAB"), so the cost per weight byte does not depend on
// the number of activation rows and the kernels stay HBM-bound at 1..8 rows.  A dot
// product is invariant under a permutation of k applied to both operands, so a lane loads
// 16 CONTIGUOUS 16-bit weights of one row (two 16-byte loads, 128 B per row per quad) and
// treats them as the k-slots its A fragments need; the activation fragment uses the same
// permutation.  Activations are read in "split" form: x = hi + lo with hi, lo both 16-bit
// (bf16 for bf16 weights, f16 for fp8 weights, which convert exactly to f16), two MMAs per
// fragment, which keeps ~16 mantissa bits of the f32 activations.
#pragma once
#include "common.cuh"

// Split-activation buffer: four planes of `plane` 16-bit elements each,
//   0: bf16 hi   1: bf16 lo   2: f16 hi   3: f16 lo ;  element (row, col) at row*ld + col.
struct SplitBuf {
    uint16_t* base;
    int ld;
    int plane;
    int mask;  // producers write plane pair 0/1 if (mask & 1), pair 2/3 if (mask & 2)
};

__device__ __forceinline__ void split_store(const SplitBuf& s, int row, int col, float v) {
    if (!s.base) return;
    const size_t i = (size_t)row * s.ld + col;
    if (s.mask & 1) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
        s.base[i] = __bfloat16_as_ushort(h);
        s.base[(size_t)s.plane + i] = __bfloat16_as_ushort(l);
    }
    if (s.mask & 2) {
        const __half h = __float2half_rn(v);
        const __half l = __float2half_rn(v - __half2float(h));
        s.base[2 * (size_t)s.plane + i] = __half_as_ushort(h);
        s.base[3 * (size_t)s.plane + i] = __half_as_ushort(l);
    }
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two e4m3 bytes -> packed f16x2 (exact).
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Activation fragment of one lane for a k-block: WORDS 32-bit words of hi and of lo
// (2 elements per word), taken from activation row g = lane >> 2 at element offset k0.
// Rows >= mrows read as zero.
template <int WORDS, bool LO = true>
__device__ __forceinline__ void load_xfrag(const uint16_t* __restrict__ hi, const uint16_t* __restrict__ lo, int ld,
                                           int g, int mrows, int k0, uint32_t (&xh)[WORDS], uint32_t (&xl)[WORDS]) {
    if (g < mrows) {
        const uint4* ph = reinterpret_cast<const uint4*>(hi + (size_t)g * ld + k0);
        const uint4* pl = reinterpret_cast<const uint4*>(lo + (size_t)g * ld + k0);
#pragma unroll
        for (int i = 0; i < WORDS / 4; ++i) {
            const uint4 a = __ldg(ph + i);
            xh[4 * i] = a.x; xh[4 * i + 1] = a.y; xh[4 * i + 2] = a.z; xh[4 * i + 3] = a.w;
            if (LO) {
                const uint4 b = __ldg(pl + i);
                xl[4 * i] = b.x; xl[4 * i + 1] = b.y; xl[4 * i + 2] = b.z; xl[4 * i + 3] = b.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < WORDS; ++i) { xh[i] = 0u; xl[i] = 0u; }
    }
}

// Weights of one lane for one k-block of one 16-row tile: 32 bytes of row (tile + g) and of
// row (tile + g + 8).  Kept separate from the MMAs so that the next block's loads can be
// issued before the current block's math (software pipelining).
struct WFrag { uint4 a0, a1, b0, b1; };

// Register-free read-ahead: asks L2 for a 128-byte line that a later k-block will load.  The weight-streaming
// kernels keep one k-block per warp in flight in registers; lines requested two or three k-blocks ahead are in L2
// by the time they are loaded, which shortens the latency each warp has to cover.
extern int g_fb_l2_ahead;   // host: read-ahead distance in units of the warp's k-block stride; 0 disables (fb_set_l2_ahead)
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ WFrag load_wfrag(const uint8_t* wa, const uint8_t* wb) {
    WFrag f;
    f.a0 = ldg_nc_v4(wa); f.a1 = ldg_nc_v4(wa + 16);
    f.b0 = ldg_nc_v4(wb); f.b1 = ldg_nc_v4(wb + 16);
    return f;
}

// bf16 weights, k-block = 64 elements: the lane's 16 elements of each row feed 4 MMAs (x2
// for the hi and lo activation halves).  d accumulates D[16 x 8].
__device__ __forceinline__ void mma_wfrag_bf16(float (&d)[4], const WFrag& f, const uint32_t (&xh)[8],
                                               const uint32_t (&xl)[8]) {
    const uint32_t A[8] = {f.a0.x, f.a0.y, f.a0.z, f.a0.w, f.a1.x, f.a1.y, f.a1.z, f.a1.w};
    const uint32_t B[8] = {f.b0.x, f.b0.y, f.b0.z, f.b0.w, f.b1.x, f.b1.y, f.b1.z, f.b1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        mma_bf16_16816(d, A[2 * j], B[2 * j], A[2 * j + 1], B[2 * j + 1], xh[2 * j], xh[2 * j + 1]);
        mma_bf16_16816(d, A[2 * j], B[2 * j], A[2 * j + 1], B[2 * j + 1], xl[2 * j], xl[2 * j + 1]);
    }
}

// e4m3 weights, k-block = 128 elements (one scale block): the lane's 32 bytes of each row
// feed 8 MMAs.  d receives the UNSCALED block sum.  LO adds the low activation half (8 more
// MMAs); the f16 high half alone keeps 11 mantissa bits, and the legacy tensor pipe is the
// co-bottleneck of the fp8 kernels, so the expert and dense-FFN kernels run hi-only.
template <bool LO>
__device__ __forceinline__ void mma_wfrag_fp8(float (&d)[4], const WFrag& f, const uint32_t (&xh)[16],
                                              const uint32_t (&xl)[16]) {
    const uint32_t A[8] = {f.a0.x, f.a0.y, f.a0.z, f.a0.w, f.a1.x, f.a1.y, f.a1.z, f.a1.w};
    const uint32_t B[8] = {f.b0.x, f.b0.y, f.b0.z, f.b0.w, f.b1.x, f.b1.y, f.b1.z, f.b1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // 32-bit word j holds 4 e4m3 = elements 4j..4j+3 -> two f16x2 words (slots 2t.., 2t+8..)
        const uint32_t a_lo = e4m3x2_to_f16x2((uint16_t)(A[j] & 0xffffu)), a_hi = e4m3x2_to_f16x2((uint16_t)(A[j] >> 16));
        const uint32_t b_lo = e4m3x2_to_f16x2((uint16_t)(B[j] & 0xffffu)), b_hi = e4m3x2_to_f16x2((uint16_t)(B[j] >> 16));
        mma_f16_16816(d, a_lo, b_lo, a_hi, b_hi, xh[2 * j], xh[2 * j + 1]);
        if (LO) mma_f16_16816(d, a_lo, b_lo, a_hi, b_hi, xl[2 * j], xl[2 * j + 1]);
    }
}
