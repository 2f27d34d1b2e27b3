// Prefill GEMM on the 5th-generation tensor cores: out[m, n] = sum_k x[m, k] * W[n, k].
//
// The weight matrix is the A operand ("swapAB"): one CTA owns a 128-row weight tile
// (UMMA M = 128) and a BN-row activation tile (UMMA N = BN <= 256), so decode-sized and
// prefill-sized activation counts share one kernel and the accumulator D[128 x BN] f32 lives
// in tensor memory.  Both operands are bf16, K-major, brought in by TMA as 64-column boxes
// (128-byte rows, 128-byte swizzle) through a multi-stage shared-memory ring:
//   warp 0 (one lane)  : producer  - waits for a free stage, arms its mbarrier with the byte
//                        count, issues the two tensor copies (no cluster multicast);
//   warp 1 (one lane)  : MMA issuer - waits for a full stage, issues 4 tcgen05.mma (K = 16
//                        each) on shared-memory descriptors, commits to the stage's "empty"
//                        barrier; commits to the accumulator barrier after the last k-block;
//   warps 2..5         : epilogue  - wait for the accumulator, tcgen05.ld their 32-lane
//                        quarter of TMEM and store out[m0 + col][n0 + lane] (coalesced in n).
// Every mbarrier wait has a clock budget; on expiry the kernel writes FB_TIMEOUT to the
// status word, skips its stores and still releases TMEM.
// Replaces the reference's cuBLAS prefill path (crates/ferrite-kernel/src/cuda.rs:2268-2396)
// and its mma.sync batched GEMMs (kernels/cuda/ferrite_kernels.cu:3548-3963).
#include "tc_common.cuh"

namespace {

constexpr int kTileW = 128;  // weight rows per CTA (UMMA M)
constexpr int kBK = 64;      // bf16 elements per k-block = 128 bytes
constexpr int kThreads = 192;

template <int BN>
struct Cfg {
    static constexpr int kStages = BN >= 256 ? 4 : 6;
    static constexpr int kABytes = kTileW * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               float* __restrict__ out, int ldo, int M, int N, int K, int accumulate, int* __restrict__ status) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;  // SW128 tiles need 1024-byte alignment
    const uint32_t bars = base + C::kStages * C::kStageBytes;         // full[S], empty[S], accum, tmem slot
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (C::kStages + s); };
    const uint32_t accum_bar = bars + 8u * (2 * C::kStages);
    const uint32_t tmem_slot = accum_bar + 8u;
    __shared__ int s_fail;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileW;
    const int m0 = blockIdx.y * BN;
    const int nkb = (K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < C::kStages; ++s) { tc::mbar_init(full(s), 1); tc::mbar_init(empty(s), 1); }
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
    pdl_launch();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---- producer ----
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % C::kStages;
            if (kb >= C::kStages && !tc::mbar_wait(empty(s), ((kb / C::kStages) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
            const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
            tc::mbar_expect_tx(full(s), C::kStageBytes);
            tc::tma_load_2d(a, &tmap_w, kb * kBK, n0, full(s));
            tc::tma_load_2d(b, &tmap_x, kb * kBK, m0, full(s));
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = tc::umma_idesc_bf16(kTileW, BN < 16 ? 16 : BN);
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % C::kStages;
            if (!tc::mbar_wait(full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
            tc::tc_fence_after();
            const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
            const uint64_t ad = tc::umma_desc_sw128(a), bd = tc::umma_desc_sw128(b);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)  // 32 bytes (two 16-byte units) per K = 16 step inside the swizzle atom
                tc::umma_bf16(tmem_base, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
            tc::umma_commit(empty(s));
        }
        tc::umma_commit(accum_bar);
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch TMEM lanes 32*(w % 4) .. +31 ----
        const int q = warp & 3;
        const bool ok = tc::mbar_wait(accum_bar, 0, 4000000000ll);
        tc::tc_fence_after();
        if (!ok) atomicExch(&s_fail, 1);
        const bool go = __shfl_sync(0xffffffffu, (ok && s_fail == 0) ? 1 : 0, 0) != 0;  // warp-uniform
        if (go) {
            const int n = n0 + q * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                float v[8];
                tc::tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                if (n < N) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int m = m0 + c + i;
                        if (m < M) {
                            float* o = out + (size_t)m * ldo + n;
                            *o = accumulate ? (*o + v[i]) : v[i];
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

template <int BN>
int launch_tc(const CUtensorMap& tw, const CUtensorMap& tx, float* out, int ldo, int M, int N, int K, int accumulate,
              int* status, cudaStream_t st) {
    auto k = gemm_tc_kernel<BN>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid((N + kTileW - 1) / kTileW, (M + BN - 1) / BN);
    FB_LAUNCH((k), grid, kThreads, Cfg<BN>::kSmem, st, tw, tx, out, ldo, M, N, K, accumulate, status);
    return FB_LAUNCH_CHECK();
}

}  // namespace

// W [N, K] bf16 row-major, x [M, K] bf16 row-major (row stride ldx elements), out [M, N] f32.
// K % 8 == 0, ldx % 8 == 0, 16-byte aligned bases.  status: int[4] device buffer.
FB_API int fb_gemm_tc_bf16(const void* W, const void* x, int64_t ldx, float* out, int64_t ldo, int64_t M, int64_t N,
                           int64_t K, int64_t accumulate, int* status, cudaStream_t st) {
    if ((K % 8) || (ldx % 8) || M < 1) return (int)cudaErrorInvalidValue;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap tw, tx;
    int rc = fb_make_tmap_2d(&tw, W, (uint64_t)N, (uint64_t)K, kTileW, kBK, 2);
    if (rc) return rc;
    // the activation tensor is described with its row stride as the inner extent
    {
        typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p)
            return (int)cudaErrorNotSupported;
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
        cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)bn};
        cuuint32_t estr[2] = {1, 1};
        if (((uintptr_t)x & 15)) return (int)cudaErrorInvalidValue;
        CUresult r = ((EncodeFn)p)(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    switch (bn) {
        case 16: return launch_tc<16>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, status, st);
        case 32: return launch_tc<32>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, status, st);
        case 64: return launch_tc<64>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, status, st);
        case 128: return launch_tc<128>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, status, st);
        default: return launch_tc<256>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, status, st);
    }
}
