// Expert-grouped W8A16 GEMM on the 5th-generation tensor cores for prefill-sized row counts:
//
//   out[p, n] = sum_k  (e4m3 W[e(p)][n, k] * S[e(p)][n / 128][k / 128])  *  x[p, k]        x: bf16 rows sorted by expert
//
// GLM-5.3-Flash's routed experts keep their checkpoint format in HBM (e4m3 values, one f32 scale per 128 x 128 block)
// and bf16 activations.  tcgen05.mma takes both operands from shared memory in ONE type, so the weight tile is
// widened on the way: a TMA box of raw e4m3 bytes [128 rows x 64 B] lands in a staging buffer, eight expander warps
// turn it into bf16 (value * block scale, rounded once) in the 128-byte-swizzled K-major layout, and the MMA warp
// issues kind::f16 MMAs against the activation tile that TMA delivered in that layout directly.  The weights are the
// UMMA A operand (128 weight rows per CTA = the TMEM lanes), the rows of one expert are the B operand (UMMA N = BN),
// the accumulator D[128 x BN] f32 stays in tensor memory over the whole K loop.  HBM traffic stays one byte per
// weight; every expert's weights stream once per call however many rows it has.
//
// Warp roles (320 threads): warp 0 producer (TMA, no cluster multicast), warp 1 MMA issuer, warps 2..9 expanders,
// warps 2..5 epilogue (tcgen05.ld of their TMEM lane quarter, masked stores).  Every mbarrier wait has a clock
// budget; on expiry the kernel reports FB_TIMEOUT, skips its stores and still releases its tensor memory.
//
// Replaces the mma.sync grouped kernels (moe_grouped.cu: 8 pairs per tile, about 60 TFLOP/s at 1024 rows) for row
// counts of 64 and more; counterpart of the reference's e4m3 expert GEMMs (kernels/cuda/dsv41_experts_mxf4.cu:6770,
// 7171 e4m3_gemm(_grouped)) and of its cuBLAS prefill path (crates/ferrite-kernel/src/cuda.rs:2268-2396).
#include <cuda_fp8.h>

#include "tc_common.cuh"

namespace {

constexpr int kTileW = 128;     // weight rows per CTA (UMMA M)
constexpr int kBK = 64;         // values per stage: one 128-byte bf16 swizzle atom
constexpr int kFwThreads = 320;
constexpr int kConvWarps = 8;

template <int BN>
struct FwCfg {
    static constexpr int kStages = BN <= 64 ? 3 : 4;        // BN <= 64: two CTAs per SM
    static constexpr int kABytes = kTileW * kBK * 2;         // expanded bf16 weights, 16 KB
    static constexpr int kRawBytes = kTileW * kBK;           // e4m3 bytes, 8 KB
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = (kABytes + kBBytes + kRawBytes + 1023) / 1024 * 1024;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 + 256;
};

struct FwTile { int expert, row0, nrows, pad; };

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Two e4m3 bytes -> bf16x2 of (value * scale).
__device__ __forceinline__ uint32_t e4m3x2_scaled_bf16x2(uint32_t two, float s) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two & 0xffffu), __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * s, f.y * s);
    return *reinterpret_cast<const uint32_t*>(&b);
}

template <int BN>
__global__ void __launch_bounds__(kFwThreads, (BN <= 64 ? 2 : 1))
fp8w_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const float* __restrict__ scales, const FwTile* __restrict__ tiles, const int* __restrict__ n_tiles,
                 float* __restrict__ out, int ldo, int m_total, int N, int K, int* __restrict__ status) {
    using C = FwCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_g = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t bars = base + C::kStages * C::kStageBytes;
    auto raw_full = [&](int s) { return bars + 8u * s; };
    auto conv_full = [&](int s) { return bars + 8u * (C::kStages + s); };
    auto empty = [&](int s) { return bars + 8u * (2 * C::kStages + s); };
    const uint32_t accum_bar = bars + 8u * (3 * C::kStages);
    const uint32_t tmem_slot = accum_bar + 8u;
    __shared__ int s_fail;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileW;
    pdl_launch();
    pdl_wait();   // the tile list is written by the kernel before this one
    if ((int)blockIdx.y >= *n_tiles) return;
    const FwTile tl = tiles[blockIdx.y];
    const int nkb = K / kBK;
    auto a_off = [&](int s) { return (uint32_t)(s * C::kStageBytes); };
    auto b_off = [&](int s) { return a_off(s) + C::kABytes; };
    auto raw_off = [&](int s) { return b_off(s) + C::kBBytes; };

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < C::kStages; ++s) {
            tc::mbar_init(raw_full(s), 1);
            tc::mbar_init(conv_full(s), kConvWarps);
            tc::mbar_init(empty(s), 1);
        }
        tc::mbar_init(accum_bar, 1);
        tc::mbar_fence_init();
        tc::prefetch_tmap(&tmap_w);
        tc::prefetch_tmap(&tmap_x);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, C::kTmemCols);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % C::kStages;
                if (kb >= C::kStages && !tc::mbar_wait(empty(s), ((kb / C::kStages) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
                tc::mbar_expect_tx(raw_full(s), C::kRawBytes + C::kBBytes);
                tc::tma_load_2d(base + raw_off(s), &tmap_w, kb * kBK, tl.expert * N + n0, raw_full(s));
                tc::tma_load_2d(base + b_off(s), &tmap_x, kb * kBK, tl.row0, raw_full(s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::umma_idesc_bf16(kTileW, BN < 16 ? 16 : BN);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % C::kStages;
                if (!tc::mbar_wait(conv_full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                tc::tc_fence_after();
                const uint64_t ad = tc::umma_desc_sw128(base + a_off(s)), bd = tc::umma_desc_sw128(base + b_off(s));
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)
                    tc::umma_bf16(tmem_base, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
                tc::umma_commit(empty(s));
            }
            tc::umma_commit(accum_bar);
        }
    } else {
        const int ct = threadIdx.x - 64;   // 0..255
        // block scales of this CTA's 128 weight rows: one f32 per 128-value k-block
        const float* srow = scales + ((size_t)tl.expert * (N / kTileW) + blockIdx.x) * (K / 128);
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % C::kStages;
            const float sc = __ldg(srow + (kb >> 1));   // in flight before the wait
            if (!tc::mbar_wait(raw_full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; }
            if (ok) {
                // 512 units of 16 e4m3 bytes per stage; consecutive threads take consecutive units; a unit becomes two
                // 16-byte chunks of bf16 at their swizzled place in its 128-byte row
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int q = ct + 256 * u;
                    const int row = q >> 2, c16 = q & 3;
                    const uint4 p = *reinterpret_cast<const uint4*>(base_g + raw_off(s) + q * 16);
                    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
                    uint32_t o[8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o[2 * j] = e4m3x2_scaled_bf16x2(w[j], sc);
                        o[2 * j + 1] = e4m3x2_scaled_bf16x2(w[j] >> 16, sc);
                    }
                    uint8_t* arow = base_g + a_off(s) + row * 128;
                    const int c0 = c16 * 2;
                    *reinterpret_cast<uint4*>(arow + (((c0) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(arow + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(conv_full(s));
        }
        if (warp < 6) {
            const int q = warp & 3;
            const bool done = tc::mbar_wait(accum_bar, 0, 4000000000ll);
            tc::tc_fence_after();
            if (!done) atomicExch(&s_fail, 1);
            const bool go = __shfl_sync(0xffffffffu, (done && s_fail == 0) ? 1 : 0, 0) != 0;
            if (go) {
                const int n = n0 + q * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < BN; c += 8) {
                    float v[8];
                    tc::tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                    if (n < N) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = c + i;
                            if (r < tl.nrows && tl.row0 + r < m_total) out[(size_t)(tl.row0 + r) * ldo + n] = v[i];
                        }
                    }
                }
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && s_fail) { status[0] = FB_TIMEOUT; status[1] = blockIdx.x; status[2] = blockIdx.y; status[3] = nkb; }
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

int make_tmap_u8_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p)
            return (int)cudaErrorNotSupported;
        fn = (EncodeFn)p;
    }
    if (((uintptr_t)base & 15) || (cols & 15) || (box_cols & 15)) return (int)cudaErrorInvalidValue;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN>
int launch_fw(const CUtensorMap& tw, const CUtensorMap& tx, const float* scales, const FwTile* tiles, const int* n_tiles,
              int max_tiles, float* out, int ldo, int m_total, int N, int K, int* status, cudaStream_t st) {
    auto k = fp8w_gemm_kernel<BN>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FwCfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid(N / kTileW, max_tiles);
    FB_LAUNCH((k), grid, kFwThreads, FwCfg<BN>::kSmem, st, tw, tx, scales, tiles, n_tiles, out, ldo, m_total, N, K, status);
    return FB_LAUNCH_CHECK();
}

// dst[pos[r * topk + k]] = src[r] (bf16 rows) for every pair with pos >= 0: the rows of an expert become contiguous.
__global__ void __launch_bounds__(256)
scatter_rows_bf16_kernel(const uint16_t* __restrict__ src, int ld, const int* __restrict__ pos, int topk, int K,
                         uint16_t* __restrict__ dst) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= K) return;
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + c);
    for (int k = 0; k < topk; ++k) {
        const int p = pos[r * topk + k];
        if (p >= 0) *reinterpret_cast<uint4*>(dst + (size_t)p * K + c) = v;
    }
}

// h [m, ldh] = [gate (I) | up (I)] of sorted row p -> act[p] = bf16(wts[p] * silu(min(g, L)) * clamp(u, -L, L)).
__global__ void __launch_bounds__(256)
swiglu_rows_bf16_kernel(const float* __restrict__ h, int ldh, const float* __restrict__ wts, const int* __restrict__ m_ptr,
                        int I, float limit, __nv_bfloat16* __restrict__ act) {
    PDL_PROLOGUE();
    const int p = blockIdx.y;
    if (p >= *m_ptr) return;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= I) return;
    const float4 g = *reinterpret_cast<const float4*>(h + (size_t)p * ldh + i);
    const float4 u = *reinterpret_cast<const float4*>(h + (size_t)p * ldh + I + i);
    const float w = wts[p];
    const float ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w};
    __nv_bfloat16 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = __float2bfloat16_rn(siluf_(fminf(ga[j], limit)) * fminf(fmaxf(ua[j], -limit), limit) * w);
    *reinterpret_cast<uint2*>(act + (size_t)p * I + i) = *reinterpret_cast<const uint2*>(o);
}

}  // namespace

// W      [E * N, K] e4m3, scales [E][N / 128][K / 128] f32; N % 128 == 0, K % 128 == 0
// X      [m_total, K] bf16 rows sorted by expert
// tiles  [max_tiles] of (expert, first row, rows, 0) with n_tiles on the device (fb_mx_sort builds both)
// out    [m_total, N] f32 (row stride ldo); bn: rows per tile, one of 32 / 64 / 128 / 256
FB_API int fb_fp8w_gemm_grouped(const void* W, const float* scales, const void* X, const void* tiles, const int* n_tiles,
                                int64_t max_tiles, float* out, int64_t ldo, int64_t m_total, int64_t E, int64_t N, int64_t K,
                                int64_t bn, int* status, cudaStream_t st) {
    if ((N % kTileW) || (K % 128) || m_total < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    int rc = make_tmap_u8_rows(&tw, W, (uint64_t)(E * N), (uint64_t)K, kTileW, kBK);
    if (rc) return rc;
    rc = fb_make_tmap_2d(&tx, X, (uint64_t)m_total, (uint64_t)K, (uint32_t)bn, kBK, 2);
    if (rc) return rc;
#define FW_ARGS tw, tx, scales, (const FwTile*)tiles, n_tiles, (int)max_tiles, out, (int)ldo, (int)m_total, (int)N, (int)K, status, st
    switch (bn) {
        case 32: return launch_fw<32>(FW_ARGS);
        case 64: return launch_fw<64>(FW_ARGS);
        case 128: return launch_fw<128>(FW_ARGS);
        case 256: return launch_fw<256>(FW_ARGS);
        default: return (int)cudaErrorInvalidValue;
    }
#undef FW_ARGS
}

FB_API int fb_scatter_rows_bf16(const void* src, int64_t ld, const int* pos, int64_t topk, int64_t n, int64_t K, void* dst,
                                cudaStream_t st) {
    if ((K % 8) || (ld % 8)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((scatter_rows_bf16_kernel), dim3((unsigned)((K / 8 + 255) / 256), (unsigned)n), 256, 0, st, (const uint16_t*)src,
              (int)ld, pos, (int)topk, (int)K, (uint16_t*)dst);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_swiglu_rows_bf16(const float* h, int64_t ldh, const float* wts_sorted, const int* m_ptr, int64_t max_m, int64_t I,
                               float limit, void* act, cudaStream_t st) {
    if ((I % 4) || (ldh % 4)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((swiglu_rows_bf16_kernel), dim3((unsigned)((I / 4 + 255) / 256), (unsigned)max_m), 256, 0, st, h, (int)ldh,
              wts_sorted, m_ptr, (int)I, limit, (__nv_bfloat16*)act);
    return FB_LAUNCH_CHECK();
}
