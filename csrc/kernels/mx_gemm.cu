// Block-scaled grouped GEMM on the 5th-generation tensor cores (tcgen05.mma kind::mxf8f6f4.block_scale):
//
//   out[p, n] = sum_k  Wdq[e(p)][n, k] * Xdq[p, k]
//   Wdq = e2m1 value * 2^(ue8m0 scale per 32 values along k)       (MXFP4 expert weights, packed two per byte)
//   Xdq = e4m3 value * 2^(ue8m0 scale per 32 values along k)       (activation rows, sorted by expert)
//
// for the rows p of a list of (expert, first row, row count) tiles: the routed experts of the DeepSeek-V4.1-style
// model for prefill-sized and batched row counts.  The weights are the UMMA A operand ("swapAB": 128 weight rows
// per CTA = the 128 TMEM lanes), the activation rows are the B operand (UMMA N = BN = 32..256), the accumulator
// D[128 x BN] f32 lives in tensor memory, and the hardware applies both scale vectors (scale factors in tensor
// memory, written there by tcgen05.cp from shared memory) inside the MMA: nothing is dequantised in registers.
//
// Warp roles (320 threads):
//   warp 0     producer : per 128-value k-block arms the stage's mbarrier and issues three copies, none with cluster
//                         multicast: a TMA box of the packed weight bytes [128 rows x 64 B], a TMA box of the e4m3
//                         activation rows [BN x 128 B, 128-byte swizzle] and a 512-byte bulk copy of the stage's
//                         weight scale factors (pre-arranged at load time in the 32 x 16-byte shape tcgen05.cp reads);
//   warps 2..9 expand   : kind::mxf8f6f4 takes 4-bit operands only in a padded 8-bit container, so the packed
//                         nibbles are expanded to e4m3 bytes (exact: every e2m1 value is an e4m3 value) with one
//                         byte-permute per four values, written in the 128-byte-swizzled K-major layout the UMMA
//                         descriptor expects; the same warps lay the activation rows' scale bytes out for
//                         tcgen05.cp.  HBM traffic stays 0.5 byte per weight;
//   warp 1     MMA      : copies the stage's scale factors into tensor memory (tcgen05.cp 32x128b.warpx4), issues
//                         four MMAs (K = 32 each, scale-factor byte 0..3 of the same TMEM column), commits to the
//                         stage's "empty" barrier;
//   warps 2..5 epilogue : tcgen05.ld of their TMEM lane quarter, masked f32 stores.
// Every mbarrier wait has a clock budget; on expiry the kernel reports FB_TIMEOUT, skips its stores and still
// releases its tensor memory.
//
// Scale-factor layout in tensor memory (UMMA, scale_vec::1X): matrix row r = 32 g + i keeps its four scale bytes
// of a 128-value k-block in the 32-bit column g at lane i of every lane quarter; the MMA's instruction descriptor
// picks the byte (k sub-block).  In shared memory that is a 512-byte chunk per 128 rows with byte
// (i * 16 + g * 4 + s), which tcgen05.cp broadcasts to the four lane quarters.
//
// Counterpart of the reference's tcgen05 expert kernels (kernels/cuda/dsv41_experts_mxf4.cu:437 mxf4_gemm_kernel,
// :5292 swapAB gate/up, :7171 e4m3_gemm_grouped; kernels/cuda/tilelang_gen/moe_bs_up_tl.cu:24-158).
#include "tc_common.cuh"

namespace {

constexpr int kTileW = 128;     // weight rows per CTA (UMMA M)
constexpr int kBK = 128;        // values per k-block = bytes per expanded row = one swizzle atom
constexpr int kMxThreads = 320;
constexpr int kConvWarps = 8;

template <int BN>
struct MxCfg {
    static constexpr int kStages = BN == 128 ? 4 : 3;   // BN <= 64: two CTAs per SM (two sets of expander warps)
    static constexpr int kABytes = kTileW * kBK;          // expanded e4m3 weights
    static constexpr int kRawBytes = kTileW * kBK / 2;    // packed nibbles
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kSfaBytes = 512;
    static constexpr int kSfbAtoms = (BN + 127) / 128;
    static constexpr int kSfbBytes = 512 * kSfbAtoms;
    static constexpr int kStageBytes = (kABytes + kBBytes + kRawBytes + kSfaBytes + kSfbBytes + 1023) / 1024 * 1024;
    static constexpr int kAccCols = BN < 32 ? 32 : BN;
    static constexpr int kSfCols = 2 * (4 + 4 * kSfbAtoms);
    static constexpr int kTmemCols = (kAccCols + kSfCols) <= 64 ? 64 : (kAccCols + kSfCols) <= 128 ? 128
                                   : (kAccCols + kSfCols) <= 256 ? 256 : 512;
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct MxTile { int expert, row0, nrows, pad; };

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Shared-memory descriptor of a 32 x 16-byte chunk without swizzle (8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(16 >> 4) << 16;     // leading byte offset (one 16-byte unit along K: not stepped)
    d |= (uint64_t)(128 >> 4) << 32;    // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// kind::mxf8f6f4 with e4m3 A and B (both K-major), ue8m0 scales, f32 accumulation; sf: scale byte (k sub-block).
__host__ __device__ constexpr uint32_t mx_idesc(int M, int N, int sf) {
    return ((uint32_t)sf << 4) | ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24) | ((uint32_t)sf << 29);
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                        uint32_t sfb, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}

// Four e2m1 codes (16 bits, element j in nibble j) -> four e4m3 bytes (element j in byte j).  Magnitudes 0, .5, 1,
// 1.5, 2, 3, 4, 6 are the e4m3 bytes 00 30 38 3C 40 44 48 4C; the sign bit moves from nibble bit 3 to byte bit 7.
__device__ __forceinline__ uint32_t e2m1x4_to_e4m3x4(uint32_t h) {
    const uint32_t mag = __byte_perm(0x3C383000u, 0x4C484440u, h & 0x7777u);
    const uint32_t sgn = __byte_perm(0x00008000u, 0u, (h >> 3) & 0x1111u);   // byte j = 0x80 if nibble j is negative
    return mag | sgn;
}

template <int BN>
__global__ void __launch_bounds__(kMxThreads, (BN <= 64 ? 2 : 1))
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const uint8_t* __restrict__ sfa_packed, const uint8_t* __restrict__ x_sf, int ld_xsf,
               const MxTile* __restrict__ tiles, const int* __restrict__ n_tiles, float* __restrict__ out, int ldo,
               int m_total, int N, int K, int quad, int* __restrict__ status) {
    using C = MxCfg<BN>;
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
    if ((int)blockIdx.y >= *n_tiles) return;   // uniform for the CTA; nothing allocated yet
    const MxTile tl = tiles[blockIdx.y];
    const int nkb = (K + kBK - 1) / kBK;   // a last k-block past K reads zeros (TMA fill) with scale bytes the caller padded
    // stage layout: [A expanded 16 KB][B BN*128][raw 8 KB][sfa 512][sfb 512 * atoms]
    auto a_off = [&](int s) { return (uint32_t)(s * C::kStageBytes); };
    auto b_off = [&](int s) { return a_off(s) + C::kABytes; };
    auto raw_off = [&](int s) { return b_off(s) + C::kBBytes; };
    auto sfa_off = [&](int s) { return raw_off(s) + C::kRawBytes; };
    auto sfb_off = [&](int s) { return sfa_off(s) + C::kSfaBytes; };

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
            // ---- producer ----
            const size_t sfa_tile = ((size_t)tl.expert * (N / kTileW) + blockIdx.x) * nkb;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % C::kStages;
                if (kb >= C::kStages && !tc::mbar_wait(empty(s), ((kb / C::kStages) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
                tc::mbar_expect_tx(raw_full(s), C::kRawBytes + C::kBBytes + C::kSfaBytes);
                tc::tma_load_2d(base + raw_off(s), &tmap_w, kb * (kBK / 2), tl.expert * N + n0, raw_full(s));
                tc::tma_load_2d(base + b_off(s), &tmap_x, kb * kBK, tl.row0, raw_full(s));
                bulk_load(base + sfa_off(s), sfa_packed + (sfa_tile + kb) * C::kSfaBytes, C::kSfaBytes, raw_full(s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            const uint32_t sf_base = tmem_base + C::kAccCols;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % C::kStages;
                if (!tc::mbar_wait(conv_full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; break; }
                tc::tc_fence_after();
                const uint32_t sfa_t = sf_base + (uint32_t)(kb & 1) * (4 + 4 * C::kSfbAtoms);
                const uint32_t sfb_t = sfa_t + 4;
                tmem_cp_sf(sfa_t, sf_desc(base + sfa_off(s)));
#pragma unroll
                for (int a = 0; a < C::kSfbAtoms; ++a) tmem_cp_sf(sfb_t + 4 * a, sf_desc(base + sfb_off(s) + 512 * a));
                const uint64_t ad = tc::umma_desc_sw128(base + a_off(s)), bd = tc::umma_desc_sw128(base + b_off(s));
#pragma unroll
                for (int k = 0; k < 4; ++k)   // 32 bytes per K = 32 step inside the swizzle atom; scale byte k
                    umma_mx(tmem_base, ad + 2u * k, bd + 2u * k, mx_idesc(kTileW, BN, k), sfa_t, sfb_t, (kb | k) ? 1u : 0u);
                tc::umma_commit(empty(s));
            }
            tc::umma_commit(accum_bar);
        }
    } else {
        // ---- expanders (warps 2..9), then epilogue (warps 2..5) ----
        const int ct = threadIdx.x - 64;           // 0..255
        bool ok = true;
        const bool sf_row = ct < BN && ct < tl.nrows && tl.row0 + ct < m_total;
        const uint8_t* sf_src = x_sf + (size_t)(tl.row0 + (sf_row ? ct : 0)) * ld_xsf;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % C::kStages;
            // this k-block's activation scale bytes (global) go in flight before the wait: they do not depend on it
            uint32_t sv = 0x7f7f7f7fu;
            if (sf_row) sv = __ldg(reinterpret_cast<const uint32_t*>(sf_src + kb * 4));
            if (!tc::mbar_wait(raw_full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); ok = false; }
            if (ok) {
                // 512 units of 16 packed bytes per stage; consecutive threads take consecutive units (conflict-free
                // loads), each unit becomes two 16-byte chunks of e4m3 at their swizzled place in the row
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int q = ct + 256 * u;
                    const int row = q >> 2, c16 = q & 3;
                    const uint4 p = *reinterpret_cast<const uint4*>(base_g + raw_off(s) + q * 16);
                    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
                    uint32_t o[8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o[2 * j] = e2m1x4_to_e4m3x4(w[j] & 0xffffu);
                        o[2 * j + 1] = e2m1x4_to_e4m3x4(w[j] >> 16);
                    }
                    uint8_t* arow = base_g + a_off(s) + row * kBK;
                    if (!quad) {
                        const int c0 = c16 * 2;        // 16-byte chunk index inside the 128-byte row
                        *reinterpret_cast<uint4*>(arow + (((c0) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(arow + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    } else if (kb * kBK + kBK <= K) {
                        // quad-interleaved weight bytes (the decode kernels' load-time repack): word j of unit c16 is
                        // word c16 of the ORIGINAL unit j, i.e. the 8 values 32 j + 8 c16 .. + 8 of the k-block
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint2*>(arow + (((2 * j + (c16 >> 1)) ^ (row & 7)) << 4) + (c16 & 1) * 8) =
                                make_uint2(o[2 * j], o[2 * j + 1]);
                    } else {
                        // 64-value tail of a quad-interleaved row: word (block b, position q) sits at q * 2 + b;
                        // units 2 and 3 are past the row (zeros from the TMA fill) and expand to zeros in place
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int qq = 2 * c16 + (j >> 1), bb = j & 1;
                            const int chunk = c16 < 2 ? 2 * bb + (qq >> 1) : 2 * c16 + (j >> 1);
                            const int hf = c16 < 2 ? (qq & 1) : (j & 1);
                            *reinterpret_cast<uint2*>(arow + ((chunk ^ (row & 7)) << 4) + hf * 8) = make_uint2(o[2 * j], o[2 * j + 1]);
                        }
                    }
                }
                // activation rows' scale bytes of this k-block -> tcgen05.cp layout (rows past the tile: scale 1)
                if (ct < BN)
                    *reinterpret_cast<uint32_t*>(base_g + sfb_off(s) + (ct >> 7) * 512 + (ct & 31) * 16 + ((ct >> 5) & 3) * 4) = sv;
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(conv_full(s));   // also after a failed wait: the MMA warp must not starve
        }
        if (warp < 6) {
            const int q = warp & 3;   // warps 2,3,4,5 -> lane quarters 2,3,0,1
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

// 2-D uint8 tensor map without swizzle (the packed weight bytes go through the expander, not straight to the MMA).
int make_tmap_u8_plain(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
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
int launch_mx(const CUtensorMap& tw, const CUtensorMap& tx, const uint8_t* sfa, const uint8_t* xsf, int ld_xsf,
              const MxTile* tiles, const int* n_tiles, int max_tiles, float* out, int ldo, int m_total, int N, int K,
              int quad, int* status, cudaStream_t st) {
    auto k = mx_gemm_kernel<BN>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MxCfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid(N / kTileW, max_tiles);
    FB_LAUNCH((k), grid, kMxThreads, MxCfg<BN>::kSmem, st, tw, tx, sfa, xsf, ld_xsf, tiles, n_tiles, out, ldo, m_total, N, K,
              quad, status);
    return FB_LAUNCH_CHECK();
}

// Builds the tile list of a grouped GEMM from per-expert row counts: rows of expert e are [off[e], off[e] + cnt[e])
// of the sorted activation buffer; every tile covers up to bn of them.  One thread: E is a few hundred.
__global__ void mx_tiles_kernel(const int* __restrict__ counts, int E, int bn, MxTile* __restrict__ tiles, int* __restrict__ n_tiles,
                                int* __restrict__ offsets, int max_tiles) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int off = 0, t = 0;
    for (int e = 0; e < E; ++e) {
        offsets[e] = off;
        for (int r = 0; r < counts[e]; r += bn) {
            if (t < max_tiles) tiles[t] = MxTile{e, off + r, min(bn, counts[e] - r), 0};
            ++t;
        }
        off += counts[e];
    }
    offsets[E] = off;
    *n_tiles = min(t, max_tiles);
}

}  // namespace

// Wp        [E * N, K / 2] packed e2m1 (even k in the low nibble), N % 128 == 0, K % 32 == 0; quad != 0: the bytes of
//           every 64-byte group are quad-interleaved (fb_d4_fp4_repack), which needs K % 64 == 0
// sfa       [E][N / 128][ceil(K / 128)][512] ue8m0 weight scales in the tcgen05.cp chunk layout
// X8        [m_total, K] e4m3 activation rows sorted by expert;  x_sf [m_total, ld_xsf] their ue8m0 scales per 32,
//           ld_xsf >= 4 * ceil(K / 128); scale bytes of blocks past K must be valid exponents (they meet zeros)
// tiles     [max_tiles] of (expert, first row, rows, 0);  n_tiles: device int (CTAs past it exit)
// out       [m_total, N] f32 (row stride ldo);  bn: activation rows per tile, one of 32 / 64 / 128 / 256
FB_API int fb_mx_gemm_grouped(const void* Wp, const void* sfa, const void* X8, const void* x_sf, int64_t ld_xsf,
                              const void* tiles, const int* n_tiles, int64_t max_tiles, float* out, int64_t ldo,
                              int64_t m_total, int64_t E, int64_t N, int64_t K, int64_t bn, int64_t quad, int* status,
                              cudaStream_t st) {
    if ((N % kTileW) || (K % 32) || (quad && (K % 64)) || m_total < 1 || max_tiles < 1 || (ld_xsf % 4) ||
        ld_xsf < 4 * ((K + kBK - 1) / kBK))
        return (int)cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    int rc = make_tmap_u8_plain(&tw, Wp, (uint64_t)(E * N), (uint64_t)(K / 2), kTileW, kBK / 2);
    if (rc) return rc;
    rc = fb_make_tmap_2d(&tx, X8, (uint64_t)m_total, (uint64_t)K, (uint32_t)bn, kBK, 1);
    if (rc) return rc;
#define MX_ARGS tw, tx, (const uint8_t*)sfa, (const uint8_t*)x_sf, (int)ld_xsf, (const MxTile*)tiles, n_tiles, (int)max_tiles, \
                out, (int)ldo, (int)m_total, (int)N, (int)K, (int)quad, status, st
    switch (bn) {
        case 32: return launch_mx<32>(MX_ARGS);
        case 64: return launch_mx<64>(MX_ARGS);
        case 128: return launch_mx<128>(MX_ARGS);
        case 256: return launch_mx<256>(MX_ARGS);
        default: return (int)cudaErrorInvalidValue;
    }
#undef MX_ARGS
}

FB_API int fb_mx_tiles(const int* counts, int64_t E, int64_t bn, void* tiles, int* n_tiles, int* offsets, int64_t max_tiles,
                       cudaStream_t st) {
    FB_LAUNCH((mx_tiles_kernel), 1, 32, 0, st, counts, (int)E, (int)bn, (MxTile*)tiles, n_tiles, offsets, (int)max_tiles);
    return FB_LAUNCH_CHECK();
}
