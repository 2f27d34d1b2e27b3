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
    static constexpr int kAccCols = BN < 32 ? 32 : BN;
    static constexpr int kTmemCols = 2 * kAccCols;           // two accumulators: the epilogue of a tile overlaps the next tile's MMAs
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

// Persistent: CTA c walks the tiles c, c + grid, c + 2 grid, ...; tile t = (weight tile t / MT, row tile t % MT), so the
// CTAs that run side by side share a weight tile (read from HBM once, then from L2) and the activations stay in L2.
// The shared-memory ring and both accumulators run across tile boundaries: while the epilogue warps drain tile i out
// of one accumulator, the MMA warp is already filling the other with tile i + 1.
template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               float* __restrict__ out, int ldo, int M, int N, int K, int accumulate, int group_rows,
               int* __restrict__ status) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;  // SW128 tiles need 1024-byte alignment
    const uint32_t bars = base + C::kStages * C::kStageBytes;         // full[S], empty[S], acc_full[2], acc_empty[2], slot
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (C::kStages + s); };
    auto acc_full = [&](int s) { return bars + 8u * (2 * C::kStages + s); };
    auto acc_empty = [&](int s) { return bars + 8u * (2 * C::kStages + 2 + s); };
    const uint32_t tmem_slot = bars + 8u * (2 * C::kStages + 4);
    __shared__ int s_fail;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (K + kBK - 1) / kBK;
    const int MT = (M + BN - 1) / BN, NT = (N + kTileW - 1) / kTileW;
    const int total = MT * NT;

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < C::kStages; ++s) { tc::mbar_init(full(s), 1); tc::mbar_init(empty(s), 1); }
        for (int s = 0; s < 2; ++s) { tc::mbar_init(acc_full(s), 1); tc::mbar_init(acc_empty(s), 4); }
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
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const int n0 = (t / MT) * kTileW, m0 = (t % MT) * BN;
            const int xk0 = group_rows > 0 ? (n0 / group_rows) * K : 0;   // block-diagonal: group g reads x columns [g K, (g + 1) K)
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % C::kStages;
                if (it >= C::kStages && !tc::mbar_wait(empty(s), ((it / C::kStages) - 1) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
                tc::mbar_expect_tx(full(s), C::kStageBytes);
                tc::tma_load_2d(a, &tmap_w, kb * kBK, n0, full(s));
                tc::tma_load_2d(b, &tmap_x, xk0 + kb * kBK, m0, full(s));
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: tile i of this CTA accumulates into accumulator i & 1 ----
        constexpr uint32_t idesc = tc::umma_idesc_bf16(kTileW, BN < 16 ? 16 : BN);
        int it = 0, ti = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++ti) {
            const int slot = ti & 1;
            if (ti >= 2 && !tc::mbar_wait(acc_empty(slot), ((ti >> 1) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
            tc::tc_fence_after();
            const uint32_t d = tmem_base + (uint32_t)(slot * C::kAccCols);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % C::kStages;
                if (!tc::mbar_wait(full(s), (it / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                tc::tc_fence_after();
                const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
                const uint64_t ad = tc::umma_desc_sw128(a), bd = tc::umma_desc_sw128(b);
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)  // 32 bytes (two 16-byte units) per K = 16 step inside the swizzle atom
                    tc::umma_bf16(d, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
                tc::umma_commit(empty(s));
            }
            if (ok) tc::umma_commit(acc_full(slot));
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch TMEM lanes 32*(w % 4) .. +31 ----
        const int q = warp & 3;
        int ti = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++ti) {
            const int slot = ti & 1;
            const int n0 = (t / MT) * kTileW, m0 = (t % MT) * BN;
            bool ok = tc::mbar_wait(acc_full(slot), (ti >> 1) & 1, 4000000000ll);
            ok = __shfl_sync(0xffffffffu, (ok && s_fail == 0) ? 1 : 0, 0) != 0;  // warp-uniform
            if (!ok) { atomicExch(&s_fail, 1); break; }
            tc::tc_fence_after();
            const int n = n0 + q * 32 + lane;
            const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * C::kAccCols);
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                if (m0 + c >= M) break;
                float v[8];
                tc::tmem_ld8(ta + (uint32_t)c, v);
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
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(slot)) : "memory");
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && s_fail) { status[0] = FB_TIMEOUT; status[1] = blockIdx.x; status[2] = total; status[3] = nkb; }
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int BN>
int launch_tc(const CUtensorMap& tw, const CUtensorMap& tx, float* out, int ldo, int M, int N, int K, int accumulate,
              int group_rows, int* status, cudaStream_t st) {
    auto k = gemm_tc_kernel<BN>;
    static bool attr_done = false;
    static int sms = 0;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return (int)cudaErrorInvalidValue;
        attr_done = true;
    }
    const long long tiles = (long long)((N + kTileW - 1) / kTileW) * ((M + BN - 1) / BN);
    dim3 grid((unsigned)(tiles < sms ? tiles : sms));
    FB_LAUNCH((k), grid, kThreads, Cfg<BN>::kSmem, st, tw, tx, out, ldo, M, N, K, accumulate, group_rows, status);
    return FB_LAUNCH_CHECK();
}

}  // namespace

// W [N, K] bf16 row-major, x [M, K] bf16 row-major (row stride ldx elements), out [M, N] f32.
// K % 8 == 0, ldx % 8 == 0, 16-byte aligned bases.  status: int[4] device buffer.
// group_rows > 0: block-diagonal form, rows [g group_rows, (g + 1) group_rows) of W contract with x columns
// [g K, (g + 1) K); group_rows % 128 == 0, K % 64 == 0, N % group_rows == 0.
FB_API int fb_gemm_tc_bf16_grouped(const void* W, const void* x, int64_t ldx, float* out, int64_t ldo, int64_t M, int64_t N,
                                   int64_t K, int64_t group_rows, int64_t accumulate, int* status, cudaStream_t st) {
    if ((K % 8) || (ldx % 8) || M < 1) return (int)cudaErrorInvalidValue;
    if (group_rows > 0 && ((group_rows % kTileW) || (K % kBK) || (N % group_rows))) return (int)cudaErrorInvalidValue;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const uint64_t xcols = group_rows > 0 ? (uint64_t)(N / group_rows) * (uint64_t)K : (uint64_t)K;
    CUtensorMap tw, tx;
    int rc = fb_make_tmap_2d(&tw, W, (uint64_t)N, (uint64_t)K, kTileW, kBK, 2);
    if (rc) return rc;
    rc = fb_make_tmap_2d_strided(&tx, x, (uint64_t)M, xcols, (uint64_t)ldx, (uint32_t)bn, kBK, 2);
    if (rc) return rc;
    const int g = (int)group_rows;
    switch (bn) {
        case 16: return launch_tc<16>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, g, status, st);
        case 32: return launch_tc<32>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, g, status, st);
        case 64: return launch_tc<64>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, g, status, st);
        case 128: return launch_tc<128>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, g, status, st);
        default: return launch_tc<256>(tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, g, status, st);
    }
}

FB_API int fb_gemm_tc_bf16(const void* W, const void* x, int64_t ldx, float* out, int64_t ldo, int64_t M, int64_t N,
                           int64_t K, int64_t accumulate, int* status, cudaStream_t st) {
    return fb_gemm_tc_bf16_grouped(W, x, ldx, out, ldo, M, N, K, 0, accumulate, status, st);
}

// ---- decode-sized row counts: split-K tcgen05 GEMV ----------------------------------------------
// out[m, n] (+)= sum_k (x_hi + x_lo)[m, k] * W[n, k] for m <= 16 rows.  Same pipeline as the GEMM above
// (TMA -> shared-memory ring -> tcgen05.mma -> TMEM), with three changes that make it a weight-streaming
// kernel: (1) the reduction dim is split over blockIdx.z so that N / 128 x splits CTAs keep every SM
// loading; (2) the activations come as a bf16 hi plane and a bf16 lo plane (x = hi + lo to ~16 bits):
// both are multiplied into the same TMEM accumulator, so the result matches the split-activation
// mma.sync GEMV; (3) split partials go to a scratch buffer and the LAST CTA of a weight tile (ticket)
// sums them in split order - deterministic, no atomics on the output.
namespace {

constexpr int kGvBN = 16;
constexpr int kGvStages = 5;     // 5 x 20 KB: two CTAs per SM
constexpr int kGvStageBytes = kTileW * kBK * 2 + 2 * kGvBN * kBK * 2;   // weights + hi + lo
constexpr size_t kGvSmem = (size_t)kGvStages * kGvStageBytes + 1024 + 256;

__global__ void __launch_bounds__(kThreads, 2)
gemv_tc_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_hi,
                      const __grid_constant__ CUtensorMap tmap_lo, float* __restrict__ out, int ldo, int M, int N, int K,
                      int accumulate, float* __restrict__ part, unsigned* __restrict__ ticket, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + kGvStages * kGvStageBytes;
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (kGvStages + s); };
    const uint32_t accum_bar = bars + 8u * (2 * kGvStages);
    const uint32_t tmem_slot = accum_bar + 8u;
    __shared__ int s_fail, s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileW;
    const int nsplit = gridDim.z, sp = blockIdx.z;
    const int nkb_all = (K + kBK - 1) / kBK;
    const int per = (nkb_all + nsplit - 1) / nsplit;
    const int kb0 = sp * per, kb1 = min(nkb_all, kb0 + per);
    const int nkb = max(kb1 - kb0, 0);

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < kGvStages; ++s) { tc::mbar_init(full(s), 1); tc::mbar_init(empty(s), 1); }
        tc::mbar_init(accum_bar, 1);
        tc::mbar_fence_init();
        tc::prefetch_tmap(&tmap_w);
        tc::prefetch_tmap(&tmap_hi);
        tc::prefetch_tmap(&tmap_lo);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, 32);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    pdl_launch();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < nkb; ++i) {
            const int s = i % kGvStages;
            if (i >= kGvStages && !tc::mbar_wait(empty(s), ((i / kGvStages) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
            const uint32_t a = base + s * kGvStageBytes, bh = a + kTileW * kBK * 2, bl = bh + kGvBN * kBK * 2;
            tc::mbar_expect_tx(full(s), kGvStageBytes);
            tc::tma_load_2d(a, &tmap_w, (kb0 + i) * kBK, n0, full(s));
            tc::tma_load_2d(bh, &tmap_hi, (kb0 + i) * kBK, 0, full(s));
            tc::tma_load_2d(bl, &tmap_lo, (kb0 + i) * kBK, 0, full(s));
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = tc::umma_idesc_bf16(kTileW, kGvBN);
        for (int i = 0; i < nkb; ++i) {
            const int s = i % kGvStages;
            if (!tc::mbar_wait(full(s), (i / kGvStages) & 1)) { atomicExch(&s_fail, 1); break; }
            tc::tc_fence_after();
            const uint32_t a = base + s * kGvStageBytes, bh = a + kTileW * kBK * 2, bl = bh + kGvBN * kBK * 2;
            const uint64_t ad = tc::umma_desc_sw128(a), hd = tc::umma_desc_sw128(bh), ld = tc::umma_desc_sw128(bl);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
                tc::umma_bf16(tmem_base, ad + 2u * k, hd + 2u * k, idesc, (i | k) ? 1u : 0u);
                tc::umma_bf16(tmem_base, ad + 2u * k, ld + 2u * k, idesc, 1u);
            }
            tc::umma_commit(empty(s));
        }
        tc::umma_commit(accum_bar);
    } else if (warp >= 2) {
        const int q = warp & 3;
        bool ok = true;
        if (nkb > 0) ok = tc::mbar_wait(accum_bar, 0, 4000000000ll);
        tc::tc_fence_after();
        if (!ok) atomicExch(&s_fail, 1);
        const bool go = __shfl_sync(0xffffffffu, (ok && s_fail == 0) ? 1 : 0, 0) != 0;
        const int n = n0 + q * 32 + lane;
        // partial tile of this split: part[tile][split][m][128]
        float* pp = part + (((size_t)blockIdx.x * nsplit + sp) * kGvBN) * kTileW + q * 32 + lane;
#pragma unroll
        for (int c = 0; c < kGvBN; c += 8) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (go && nkb > 0) tc::tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) pp[(size_t)(c + i) * kTileW] = v[i];
        }
        (void)n;
    }
    tc::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_fail) { status[0] = FB_TIMEOUT; status[1] = blockIdx.x; status[2] = blockIdx.z; status[3] = nkb; }
        __threadfence();
        s_last = (atomicAdd(ticket + blockIdx.x, 1u) == (unsigned)nsplit - 1u) ? 1 : 0;
    }
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, 32);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the last CTA of this weight tile sums the splits in order and writes the rows
    for (int i = threadIdx.x; i < M * kTileW; i += blockDim.x) {
        const int m = i / kTileW, j = i % kTileW;
        if (n0 + j >= N) continue;
        float v = 0.f;
        for (int s = 0; s < nsplit; ++s) v += __ldcg(part + (((size_t)blockIdx.x * nsplit + s) * kGvBN + m) * kTileW + j);
        float* o = out + (size_t)m * ldo + n0 + j;
        *o = accumulate ? *o + v : v;
    }
    if (threadIdx.x == 0) ticket[blockIdx.x] = 0u;
}

}  // namespace

// W [N, K] bf16; xs: split activation planes (plane 0 = bf16 hi, plane 1 = bf16 lo), rows of xs_ld elements,
// planes xs_plane elements apart; m <= 16.  part: scratch of ceil(N/128) * nsplit * 16 * 128 floats,
// ticket: ceil(N/128) zero-initialised words (left at zero).  status: int[4].
FB_API int fb_gemv_tc_bf16(const void* W, const void* xs, int64_t xs_ld, int64_t xs_plane, float* out, int64_t ldo, int64_t m,
                           int64_t N, int64_t K, int64_t accumulate, int64_t nsplit, float* part, void* ticket, int* status,
                           cudaStream_t st) {
    if ((K % 8) || (xs_ld % 8) || m < 1 || m > kGvBN || nsplit < 1) return (int)cudaErrorInvalidValue;
    CUtensorMap tw, th, tl;
    int rc = fb_make_tmap_2d(&tw, W, (uint64_t)N, (uint64_t)K, kTileW, kBK, 2);
    if (rc) return rc;
    const uint16_t* hi = (const uint16_t*)xs;
    const uint16_t* lo = hi + xs_plane;
    rc = fb_make_tmap_2d_strided(&th, hi, (uint64_t)m, (uint64_t)K, (uint64_t)xs_ld, kGvBN, kBK, 2);
    if (rc) return rc;
    rc = fb_make_tmap_2d_strided(&tl, lo, (uint64_t)m, (uint64_t)K, (uint64_t)xs_ld, kGvBN, kBK, 2);
    if (rc) return rc;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(gemv_tc_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGvSmem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid((unsigned)((N + kTileW - 1) / kTileW), 1, (unsigned)nsplit);
    FB_LAUNCH((gemv_tc_splitk_kernel), grid, kThreads, kGvSmem, st, tw, th, tl, out, (int)ldo, (int)m, (int)N, (int)K,
              (int)accumulate, part, (unsigned*)ticket, status);
    return FB_LAUNCH_CHECK();
}
