// Expert-grouped W8A16 GEMM on the 5th-generation tensor cores for prefill-sized row counts:
//
//   out[p, n] = sum_j  S[e(p)][n / 128][j] * sum_{k in 128-block j}  e4m3 W[e(p)][n, k] * x[p, k]      x: f16 rows sorted by expert
//
// GLM-5.3-Flash's routed experts keep their checkpoint format in HBM (e4m3 values, one f32 scale per 128 x 128 block).
// tcgen05.mma wants both operands in 16-bit types, so the weight tile is widened on the way: a TMA box of raw e4m3
// bytes [128 rows x 128 B] lands in a staging ring, eight expander warps turn it into f16 (exact: one cvt per two
// values) and store it with tcgen05.st into TENSOR MEMORY, from where the MMA takes its A operand (row = TMEM lane,
// two f16 per 32-bit column); the B operand is the f16 activation tile that TMA delivered into shared memory in the
// 128-byte-swizzled K-major layout.  The block scale is NOT applied to the operands: each 128-wide k-block is
// accumulated into a TMEM accumulator of its own, and eight epilogue warps drain the finished block (tcgen05.ld)
// into f32 registers with one FMA by the block's scale while the next blocks run into the other accumulators.
// Weights are the UMMA A operand (128 weight rows per CTA = the TMEM lanes), the rows of one expert the B operand
// (UMMA N = BN).  HBM traffic stays one byte per weight.
//
// What the shape of the kernel answers to (each measured on the 128-expert gate/up case, 2.1 GB of weights):
//   * 64-byte-wide raw boxes read half lines of 128 rows: 847 us.  128-byte-wide boxes: 705 us.
//   * the widened tile written to and read back from shared memory costs 4 bytes of shared-memory traffic per
//     weight byte (LSU + tensor-core shared wavefronts at 76 % of peak with DRAM at 50 %), and an 8-way bank
//     conflict pattern in its stores cost more: 615 us with ordered stores, 588 us with the tile in tensor memory.
//   * with every role but the MMAs switched off the pipeline ran at the HBM copy rate (377 us); one thread issues
//     an M128 x N<=64 x K16 MMA only about every 150 cycles whatever N is.  Stages therefore go round-robin over
//     several issuer threads with one accumulator each: 496 us with two, 444 us (0.81 of the copy rate) with four.
//
// The kernel is persistent: one CTA per SM walks (row tile, 128-row weight tile) pairs, consecutive CTAs taking the
// weight tiles of the same rows (their activations stay in L2), and all rings run across tile boundaries, so the
// weight stream never drains between tiles.  Three rings: raw e4m3 and activations in shared memory, expanded
// weights in tensor memory.  Warp roles: warp 0 weight producer, warp 1 MMA issuer, warp 2 activation producer
// (TMA, no cluster multicast), warps 3..10 expanders, warps 11..18 epilogue (two per TMEM lane quarter, half of the
// columns each), warps 19.. further MMA issuers.  Every mbarrier wait has a clock budget; on expiry the kernel
// reports FB_TIMEOUT, skips its stores and still releases its tensor memory.
//
// Replaces the mma.sync grouped kernels (moe_grouped.cu: 8 pairs per tile, about 60 TFLOP/s at 1024 rows) for row
// counts of 64 and more; counterpart of the reference's e4m3 expert GEMMs (kernels/cuda/dsv41_experts_mxf4.cu:6770,
// 7171 e4m3_gemm(_grouped)) and of its cuBLAS prefill path (crates/ferrite-kernel/src/cuda.rs:2268-2396).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "tc_common.cuh"

namespace {

constexpr int kTileW = 128;     // weight rows per CTA (UMMA M)
constexpr int kBK = 128;        // values per stage = one block-scale span = two 128-byte f16 swizzle atoms
constexpr int kAtom = 64;       // f16 values per swizzle atom
constexpr int kExpWarps = 8, kEpiWarps = 8;
constexpr int kMmaXWarp = 3 + kExpWarps + kEpiWarps;     // first of the extra MMA issuer warps

template <int BN>
struct FwCfg {
    // Ring depths follow each ring's own round trip (bytes in flight = rate x latency): HBM -> shared memory for the
    // raw bytes, L2 -> shared memory -> MMA -> commit for the activations, expander -> MMA -> commit for the f16 tile.
    static constexpr int kRaw = BN <= 64 ? 8 : 5;                    // raw e4m3 stages (16 KB)
    // Activation and expanded-weight ring depths are multiples of the issuer count: ring slot s is then always
    // consumed by issuer s % kIssuers, in order.  (With several consumers on one mbarrier, a consumer that runs a
    // whole ring ahead of another would see the parity of the slot's previous use and take it for its own.)
    static constexpr int kSB = BN <= 32 ? 8 : 4;                     // activation stages
    static constexpr int kSA = 4;                                    // expanded weight stages (64 TMEM columns each)
    static constexpr int kRawBytes = kTileW * kBK;
    static constexpr int kBAtomBytes = BN * kAtom * 2;
    static constexpr int kBBytes = 2 * kBAtomBytes;
    static constexpr int kBOff = 0;
    static constexpr int kRawOff = kBOff + kSB * kBBytes;
    static constexpr int kBarOff = kRawOff + kRaw * kRawBytes;
    static constexpr int kNumBars = 2 * kRaw + 2 * kSB + 2 * kSA + 2 * (BN <= 64 ? 4 : 2);
    // One thread issues a tcgen05.mma of this shape about every 150 cycles whatever its N (measured: 8 MMAs per stage
    // from one issuer bound the kernel at 0.6 of the HBM rate, two issuers gave 0.72), so stages go round-robin
    // over several issuer threads, each with its own accumulator.
    static constexpr int kIssuers = BN <= 64 ? 4 : 2;
    static_assert(kSA % (BN <= 64 ? 4 : 2) == 0 && kSB % (BN <= 64 ? 4 : 2) == 0, "one consumer per ring slot");
    static constexpr int kThreads = 32 * (3 + kExpWarps + kEpiWarps + kIssuers - 1);
    static constexpr int kACols = kBK / 2;                           // 32-bit columns of one expanded stage
    static constexpr int kAccCols = kIssuers * BN;                   // one accumulator per issuer
    static constexpr int kTmemCols = kAccCols + kSA * kACols <= 256 ? 256 : 512;
    static_assert(kAccCols + kSA * kACols <= 512, "tensor memory");
    static constexpr size_t kSmem = (size_t)kBarOff + 8 * kNumBars + 16 + 1024 /*align*/;
};

struct FwTile { int expert, row0, nrows, pad; };

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Instruction descriptor for kind::f16 with f16 A/B (both K-major) and f32 accumulation.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// D[tmem] (+)= A[tmem] . B[smem]^T ; issued by ONE thread.  A: 128 lanes (rows) x 8 columns (16 f16 of K).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes lane (base lane + i).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Four e4m3 bytes -> two f16x2 words, exact: the 16-bit halves of the source register are named directly, so the
// whole conversion is the two cvt instructions.
__device__ __forceinline__ void e4m3x4_f16x4(uint32_t four, uint32_t& lo, uint32_t& hi) {
    asm("{\n .reg .b16 a, b;\n mov.b32 {a, b}, %2;\n cvt.rn.f16x2.e4m3x2 %0, a;\n cvt.rn.f16x2.e4m3x2 %1, b;\n}"
        : "=r"(lo), "=r"(hi) : "r"(four));
}

template <int BN>
__global__ void __launch_bounds__(FwCfg<BN>::kThreads, 1)
fp8w_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const float* __restrict__ scales, const FwTile* __restrict__ tiles, const int* __restrict__ n_tiles,
                 float* __restrict__ out, int ldo, int m_total, int N, int K, int* __restrict__ status) {
    using C = FwCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_g = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t bars = base + C::kBarOff;
    auto raw_full = [&](int s) { return bars + 8u * s; };
    auto raw_empty = [&](int s) { return bars + 8u * (C::kRaw + s); };
    auto b_full = [&](int s) { return bars + 8u * (2 * C::kRaw + s); };
    auto b_empty = [&](int s) { return bars + 8u * (2 * C::kRaw + C::kSB + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * C::kRaw + 2 * C::kSB + s); };
    auto a_empty = [&](int s) { return bars + 8u * (2 * C::kRaw + 2 * C::kSB + C::kSA + s); };
    auto acc_full = [&](int s) { return bars + 8u * (2 * C::kRaw + 2 * C::kSB + 2 * C::kSA + s); };
    auto acc_empty = [&](int s) { return bars + 8u * (2 * C::kRaw + 2 * C::kSB + 2 * C::kSA + C::kIssuers + s); };
    const uint32_t tmem_slot = bars + 8u * C::kNumBars;
    __shared__ int s_fail;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch();
    pdl_wait();   // the tile list is written by the kernel before this one
    const int NT = N / kTileW;
    const int total = *n_tiles * NT;
    const int nkb = K / kBK;

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < C::kRaw; ++s) { tc::mbar_init(raw_full(s), 1); tc::mbar_init(raw_empty(s), kExpWarps); }
        for (int s = 0; s < C::kSB; ++s) { tc::mbar_init(b_full(s), 1); tc::mbar_init(b_empty(s), 1); }
        for (int s = 0; s < C::kSA; ++s) { tc::mbar_init(a_full(s), kExpWarps); tc::mbar_init(a_empty(s), 1); }
        for (int s = 0; s < C::kIssuers; ++s) { tc::mbar_init(acc_full(s), 1); tc::mbar_init(acc_empty(s), kEpiWarps); }
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
        // ---- weight producer: boxes of 128 rows x 128 raw bytes (whole 128-byte lines of every row), as far ahead
        //      as the ring allows ----
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const FwTile tl = tiles[t / NT];
                const int wrow = tl.expert * N + (t % NT) * kTileW;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % C::kRaw;
                    if (it >= C::kRaw && !tc::mbar_wait(raw_empty(s), ((it / C::kRaw) - 1) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                    tc::mbar_expect_tx(raw_full(s), C::kRawBytes);
                    tc::tma_load_2d(base + C::kRawOff + s * C::kRawBytes, &tmap_w, kb * kBK, wrow, raw_full(s));
                }
            }
        }
    } else if (warp == 2) {
        // ---- activation producer: two swizzle atoms per stage ----
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const FwTile tl = tiles[t / NT];
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % C::kSB;
                    if (it >= C::kSB && !tc::mbar_wait(b_empty(s), ((it / C::kSB) - 1) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                    tc::mbar_expect_tx(b_full(s), C::kBBytes);
                    const uint32_t dst = base + C::kBOff + s * C::kBBytes;
                    tc::tma_load_2d(dst, &tmap_x, kb * kBK, tl.row0, b_full(s));
                    tc::tma_load_2d(dst + C::kBAtomBytes, &tmap_x, kb * kBK + kAtom, tl.row0, b_full(s));
                }
            }
        }
    } else if (warp == 1 || warp >= kMmaXWarp) {
        // ---- MMA issuers: one 128-wide k-block (one stage) per accumulator; issuer p takes the stages with
        //      it % kIssuers == p and accumulator p ----
        const int par = warp == 1 ? 0 : warp - kMmaXWarp + 1;
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(kTileW, BN < 16 ? 16 : BN);
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int slot = it % C::kIssuers;
                    if (slot != par) continue;
                    if (it >= C::kIssuers && !tc::mbar_wait(acc_empty(slot), ((it / C::kIssuers) - 1) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                    const int sa = it % C::kSA, sb = it % C::kSB;
                    if (!tc::mbar_wait(a_full(sa), (it / C::kSA) & 1) || !tc::mbar_wait(b_full(sb), (it / C::kSB) & 1)) {
                        atomicExch(&s_fail, 1); ok = false; break;
                    }
                    tc::tc_fence_after();
                    const uint32_t d = tmem_base + (uint32_t)(slot * BN);
                    const uint32_t at = tmem_base + (uint32_t)(C::kAccCols + sa * C::kACols);
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const uint64_t bd = tc::umma_desc_sw128(base + C::kBOff + sb * C::kBBytes + a * C::kBAtomBytes);
#pragma unroll
                        for (int k = 0; k < kAtom / 16; ++k)
                            umma_f16_ts(d, at + (uint32_t)((a * 4 + k) * 8), bd + 2u * k, idesc, (a | k) ? 1u : 0u);
                    }
                    tc::umma_commit(a_empty(sa));
                    tc::umma_commit(b_empty(sb));
                    tc::umma_commit(acc_full(slot));
                }
            }
        }
    } else if (warp < 3 + kExpWarps) {
        // ---- expanders: warp w owns TMEM lanes 32 (w % 4) .. + 31 = weight rows of the tile; the two warps of a
        //      lane quarter take one 64-value half of the stage each.  A thread reads its row's four 16-byte chunks
        //      (the raw box arrives with the 128-byte swizzle: chunk c of row r sits at chunk c ^ (r & 7), so eight
        //      consecutive rows read eight different bank groups), converts, and stores 32 columns of f16 pairs ----
        const int q = warp & 3, kh = (warp - 3) >> 2;
        const int row = q * 32 + lane, sw = row & 7;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % C::kRaw, sa = it % C::kSA;
                if (!tc::mbar_wait(raw_full(s), (it / C::kRaw) & 1) ||
                    (it >= C::kSA && !tc::mbar_wait(a_empty(sa), ((it / C::kSA) - 1) & 1))) { atomicExch(&s_fail, 1); ok = false; break; }
                tc::tc_fence_after();
                const uint8_t* rawp = base_g + C::kRawOff + s * C::kRawBytes + row * 128;
                uint32_t w[32];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 p = *reinterpret_cast<const uint4*>(rawp + (((kh * 4 + j) ^ sw) << 4));
                    e4m3x4_f16x4(p.x, w[8 * j + 0], w[8 * j + 1]); e4m3x4_f16x4(p.y, w[8 * j + 2], w[8 * j + 3]);
                    e4m3x4_f16x4(p.z, w[8 * j + 4], w[8 * j + 5]); e4m3x4_f16x4(p.w, w[8 * j + 6], w[8 * j + 7]);
                }
                tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(C::kAccCols + sa * C::kACols + kh * 32), w);
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(a_full(sa)); mbar_arrive(raw_empty(s)); }
            }
        }
    } else {
        // ---- epilogue: TMEM lane quarter warp % 4, columns [half CW, (half + 1) CW) of the tile ----
        constexpr int CW = BN / 2;
        const int q = warp & 3, half = (warp - (3 + kExpWarps)) >> 2;
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const FwTile tl = tiles[t / NT];
            const int nx = t % NT;
            const float* srow = scales + ((size_t)tl.expert * NT + nx) * nkb;
            float acc[CW];
#pragma unroll
            for (int i = 0; i < CW; ++i) acc[i] = 0.f;
            for (int j = 0; j < nkb; ++j, ++it) {
                const int slot = it % C::kIssuers;
                const float sc = __ldg(srow + j);   // in flight before the wait
                bool done = tc::mbar_wait(acc_full(slot), (it / C::kIssuers) & 1);
                done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
                if (!done) { atomicExch(&s_fail, 1); ok = false; break; }
                tc::tc_fence_after();
                const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * BN + half * CW);
#pragma unroll
                for (int c = 0; c < CW; c += 16) {
                    float v[16];
                    tmem_ld16(ta + (uint32_t)c, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[c + i] = fmaf(v[i], sc, acc[c + i]);
                }
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(slot));
            }
            if (ok && s_fail == 0) {
                const int n = nx * kTileW + q * 32 + lane;
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    const int r = half * CW + i;
                    if (r < tl.nrows && tl.row0 + r < m_total) out[(size_t)(tl.row0 + r) * ldo + n] = acc[i];
                }
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

int make_tmap_u8_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                      bool swizzle128) {
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
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return (int)cudaErrorInvalidValue;
    }
    const long long most = (long long)max_tiles * (N / kTileW);
    dim3 grid((unsigned)(most < sms ? most : sms));
    FB_LAUNCH((k), grid, FwCfg<BN>::kThreads, FwCfg<BN>::kSmem, st, tw, tx, scales, tiles, n_tiles, out, ldo, m_total, N, K, status);
    return FB_LAUNCH_CHECK();
}

// dst[pos[r * topk + k]] = f16(src[r]) for every pair with pos >= 0: the rows of an expert become contiguous.
__global__ void __launch_bounds__(256)
scatter_rows_f16_kernel(const float* __restrict__ src, int ld, const int* __restrict__ pos, int topk, int K,
                        __half* __restrict__ dst) {
    PDL_PROLOGUE();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= K) return;
    const float4 a = *reinterpret_cast<const float4*>(src + (size_t)r * ld + c);
    const float4 b = *reinterpret_cast<const float4*>(src + (size_t)r * ld + c + 4);
    __half2 h[4] = {__floats2half2_rn(a.x, a.y), __floats2half2_rn(a.z, a.w), __floats2half2_rn(b.x, b.y),
                    __floats2half2_rn(b.z, b.w)};
    const uint4 v = *reinterpret_cast<const uint4*>(h);
    for (int k = 0; k < topk; ++k) {
        const int p = pos[r * topk + k];
        if (p >= 0) *reinterpret_cast<uint4*>(dst + (size_t)p * K + c) = v;
    }
}

// dst[pos[r * topk + k]] = src[r] for rows that are 16-bit already (one plane of a split activation buffer).
__global__ void __launch_bounds__(256)
scatter_rows_16_kernel(const uint16_t* __restrict__ src, int ld, const int* __restrict__ pos, int topk, int K,
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

// h [m, ldh] = [gate (I) | up (I)] of sorted row p -> act[p] = f16(wts[p] * silu(min(g, L)) * clamp(u, -L, L)).
__global__ void __launch_bounds__(256)
swiglu_rows_f16_kernel(const float* __restrict__ h, int ldh, const float* __restrict__ wts, const int* __restrict__ m_ptr,
                       int I, float limit, __half* __restrict__ act) {
    PDL_PROLOGUE();
    const int p = blockIdx.y;
    if (p >= *m_ptr) return;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= I) return;
    const float4 g = *reinterpret_cast<const float4*>(h + (size_t)p * ldh + i);
    const float4 u = *reinterpret_cast<const float4*>(h + (size_t)p * ldh + I + i);
    const float w = wts[p];
    const float ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w};
    __half o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = __float2half_rn(siluf_(fminf(ga[j], limit)) * fminf(fmaxf(ua[j], -limit), limit) * w);
    *reinterpret_cast<uint2*>(act + (size_t)p * I + i) = *reinterpret_cast<const uint2*>(o);
}

}  // namespace

// W      [E * N, K] e4m3, scales [E][N / 128][K / 128] f32; N % 128 == 0, K % 128 == 0
// X      [m_total, K] f16 rows sorted by expert
// tiles  [max_tiles] of (expert, first row, rows, 0) with n_tiles on the device (fb_mx_sort builds both)
// out    [m_total, N] f32 (row stride ldo); bn: rows per tile, one of 32 / 64 / 128
FB_API int fb_fp8w_gemm_grouped(const void* W, const float* scales, const void* X, const void* tiles, const int* n_tiles,
                                int64_t max_tiles, float* out, int64_t ldo, int64_t m_total, int64_t E, int64_t N, int64_t K,
                                int64_t bn, int* status, cudaStream_t st) {
    if ((N % kTileW) || (K % 128) || m_total < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    int rc = make_tmap_u8_rows(&tw, W, (uint64_t)(E * N), (uint64_t)K, kTileW, kBK, true);
    if (rc) return rc;
    rc = fb_make_tmap_2d(&tx, X, (uint64_t)m_total, (uint64_t)K, (uint32_t)bn, kAtom, 2);
    if (rc) return rc;
#define FW_ARGS tw, tx, scales, (const FwTile*)tiles, n_tiles, (int)max_tiles, out, (int)ldo, (int)m_total, (int)N, (int)K, status, st
    switch (bn) {
        case 32: return launch_fw<32>(FW_ARGS);
        case 64: return launch_fw<64>(FW_ARGS);
        case 128: return launch_fw<128>(FW_ARGS);
        default: return (int)cudaErrorInvalidValue;
    }
#undef FW_ARGS
}

FB_API int fb_scatter_rows_f16(const float* src, int64_t ld, const int* pos, int64_t topk, int64_t n, int64_t K, void* dst,
                               cudaStream_t st) {
    if ((K % 8) || (ld % 4)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((scatter_rows_f16_kernel), dim3((unsigned)((K / 8 + 255) / 256), (unsigned)n), 256, 0, st, src,
              (int)ld, pos, (int)topk, (int)K, (__half*)dst);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_scatter_rows_16(const void* src, int64_t ld, const int* pos, int64_t topk, int64_t n, int64_t K, void* dst,
                              cudaStream_t st) {
    if ((K % 8) || (ld % 8)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((scatter_rows_16_kernel), dim3((unsigned)((K / 8 + 255) / 256), (unsigned)n), 256, 0, st, (const uint16_t*)src,
              (int)ld, pos, (int)topk, (int)K, (uint16_t*)dst);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_swiglu_rows_f16(const float* h, int64_t ldh, const float* wts_sorted, const int* m_ptr, int64_t max_m, int64_t I,
                              float limit, void* act, cudaStream_t st) {
    if ((I % 4) || (ldh % 4)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((swiglu_rows_f16_kernel), dim3((unsigned)((I / 4 + 255) / 256), (unsigned)max_m), 256, 0, st, h, (int)ldh,
              wts_sorted, m_ptr, (int)I, limit, (__half*)act);
    return FB_LAUNCH_CHECK();
}
