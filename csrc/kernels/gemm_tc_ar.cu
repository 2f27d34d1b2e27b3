// Row-parallel prefill GEMM fused with its all-reduce: ONE kernel for
//   out[m, n] = sum_ranks ( x_rank[m, :] . W_rank[n, :] (+ out_rank[m, n]) )      m up to a few hundred rows
//
// The math is the TMA + tcgen05 pipeline of gemm_tc.cu (weights as the 128-row A operand, the
// activation tile as B, f32 accumulator in tensor memory).  The collective is a two-shot
// all-reduce over peer memory, done tile by tile inside the same launch:
//   scatter  the epilogue warps read the accumulator tile out of TMEM and store it straight
//            into slot `rank` of the tile OWNER's staging buffer (tile t belongs to rank
//            t % world), so every partial crosses NVLink once and the stores of finished tiles
//            overlap the MMAs of the tiles still being computed;
//   publish  a CTA fences at GPU scope and takes a ticket; the CTA that takes the last ticket
//            of the grid fences at system scope ONCE and stamps this launch's epoch on every
//            peer (one system fence per launch, not per tile);
//   reduce   the owner's CTA of a tile waits (bounded) for the stamps of all ranks, sums the
//            `world` partials in rank order - every rank later reads the same bits - and
//            stores the reduced tile into the gather buffer of every peer;
//   gather   second ticket + stamp among the tiles this rank owns; every CTA then waits
//            (bounded) for the stamp of its tile's owner and copies the tile to `out`.
// Per rank (world - 1) / world of the output crosses NVLink twice: the reduce-scatter +
// all-gather volume, against (world - 1) x for a one-shot push of whole tiles.  With two ranks, or
// when the whole one-shot volume is under 1 MiB, the kernel runs ONE-SHOT instead: every tile goes to
// every rank, one publish / wait round, and each CTA reduces its tile straight into `out`.
// The grid must be co-resident (checked on the host with the occupancy API): a CTA only
// waits for CTAs of OTHER ranks that are running or done, never for an unscheduled one.
// Every wait is bounded; on expiry the kernel records {TIMEOUT, phase * 16 + peer, epoch,
// tile}, skips what depends on the missing data, still releases TMEM and returns.
// With world == 1 the kernel degenerates to the plain GEMM epilogue.
//
// Replaces the reference's cuBLAS prefill GEMM followed by a separate NCCL / P2P all-reduce
// (crates/ferrite-kernel/src/cuda.rs:2268-2396; crates/ferrite-exec/src/tp.rs:729-1059).
#include "tc_common.cuh"

namespace {

constexpr int kTileW = 128;
constexpr int kBK = 64;
constexpr int kThreads = 192;
constexpr int kMaxWorld = 8;
constexpr int kFlagPad = 32;   // one 128-byte line per flag word

struct GarPtrs {
    float* scatter[kMaxWorld];   // [2][world][tiles_per_rank][BN * 128]  partial tiles, at the owner
    float* gather[kMaxWorld];    // [2][ntiles][BN * 128]                  reduced tiles, at everyone
    uint32_t* flags[kMaxWorld];  // [2][2 phases][world][kFlagPad]
};

template <int BN>
struct Cfg {
    static constexpr int kStages = BN >= 256 ? 4 : 6;
    static constexpr int kABytes = kTileW * kBK * 2;
    static constexpr int kBBytes = (BN < 16 ? 16 : BN) * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr int kTileElems = BN * kTileW;
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 + 256;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Bounded poll of a flag word that a peer writes into LOCAL memory; false on expiry.
__device__ __forceinline__ bool wait_flag(const uint32_t* f, uint32_t e, int max_spins, const int* status) {
    int spins = 0;
    const int budget = fb_spin_budget(status, max_spins);
    while (ld_relaxed_sys(f) < e) {
        if (++spins > budget) return false;
        __nanosleep(64);
    }
    (void)ld_acquire_sys(f);
    return true;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_ar_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                  float* __restrict__ out, int ldo, int M, int N, int K, int accumulate, GarPtrs t,
                  uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket, int* __restrict__ status, int rank, int world,
                  int tiles_per_rank, int max_spins, int oneshot) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + C::kStages * C::kStageBytes;
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (C::kStages + s); };
    const uint32_t accum_bar = bars + 8u * (2 * C::kStages);
    const uint32_t tmem_slot = accum_bar + 8u;
    __shared__ int s_fail;
    __shared__ uint32_t s_epoch;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileW;
    const int m0 = blockIdx.y * BN;
    const int nkb = (K + kBK - 1) / kBK;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int ntiles = gridDim.x * gridDim.y;
    const int owner = tile % world;
    const int rows = min(BN, M - m0);   // live rows of this tile

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < C::kStages; ++s) { tc::mbar_init(full(s), 1); tc::mbar_init(empty(s), 1); }
        tc::mbar_init(accum_bar, 1);
        tc::mbar_fence_init();
        tc::prefetch_tmap(&tmap_w);
        tc::prefetch_tmap(&tmap_x);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, C::kTmemCols);
    pdl_launch();
    pdl_wait();
    if (threadIdx.x == 0) s_epoch = epoch[0] + 1u;   // read before this CTA can take a ticket
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    const uint32_t e = s_epoch;
    const int par = e & 1u;

    if (warp == 0 && lane == 0) {
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % C::kStages;
            if (kb >= C::kStages && !tc::mbar_wait(empty(s), ((kb / C::kStages) - 1) & 1)) { atomicExch(&s_fail, 1); break; }
            const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
            tc::mbar_expect_tx(full(s), C::kStageBytes);
            tc::tma_load_2d(a, &tmap_w, kb * kBK, n0, full(s));
            tc::tma_load_2d(b, &tmap_x, kb * kBK, m0, full(s));
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = tc::umma_idesc_bf16(kTileW, BN < 16 ? 16 : BN);
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % C::kStages;
            if (!tc::mbar_wait(full(s), (kb / C::kStages) & 1)) { atomicExch(&s_fail, 1); break; }
            tc::tc_fence_after();
            const uint32_t a = base + s * C::kStageBytes, b = a + C::kABytes;
            const uint64_t ad = tc::umma_desc_sw128(a), bd = tc::umma_desc_sw128(b);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
                tc::umma_bf16(tmem_base, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
            tc::umma_commit(empty(s));
        }
        tc::umma_commit(accum_bar);
    } else if (warp >= 2) {
        // ---- epilogue: accumulator -> the owner's scatter slot (or `out` when there is one rank) ----
        const int q = warp & 3;
        const bool ok = tc::mbar_wait(accum_bar, 0, 4000000000ll);
        tc::tc_fence_after();
        if (!ok) atomicExch(&s_fail, 1);
        const bool go = __shfl_sync(0xffffffffu, (ok && s_fail == 0) ? 1 : 0, 0) != 0;
        if (go) {
            const int nl = q * 32 + lane;
            const int n = n0 + nl;
            // two-shot: the tile goes to its owner only; one-shot: to every rank (slot index = tile)
            const size_t slot_off = (((size_t)par * world + rank) * tiles_per_rank + (oneshot ? tile : tile / world)) * C::kTileElems + nl;
            float* dst = world > 1 && !oneshot ? t.scatter[owner] + slot_off : nullptr;
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                float v[8];
                tc::tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (c + i < rows) {
                        float a = v[i];
                        if (n < N) {
                            float* o = out + (size_t)(m0 + c + i) * ldo + n;
                            if (accumulate) a += *o;
                            if (world == 1) *o = a;
                        }
                        if (dst) dst[(size_t)(c + i) * kTileW] = a;   // 128 bytes per warp and row
                        else if (world > 1) {
                            for (int p = 0; p < world; ++p) t.scatter[p][slot_off + (size_t)(c + i) * kTileW] = a;
                        }
                    }
                }
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, C::kTmemCols);
    }
    if (world == 1) {
        if (threadIdx.x == 0 && s_fail) { status[0] = FB_TIMEOUT; status[1] = 0; status[2] = blockIdx.x; status[3] = blockIdx.y; }
        return;
    }
    // ---- publish the scatter phase: one system-scope fence per launch ----
    if (threadIdx.x == 0) {
        if (s_fail) { status[0] = FB_TIMEOUT; status[1] = 0; status[2] = (int)e; status[3] = tile; }
        __threadfence();
        if (atomicAdd(ticket, 1u) == (unsigned)ntiles - 1u) {
            __threadfence_system();
            for (int p = 0; p < world; ++p)
                st_release_sys(t.flags[p] + (((size_t)par * 2 + 0) * world + rank) * kFlagPad, e);
            ticket[0] = 0u;
            epoch[0] = e;   // every CTA read the old value before it took its ticket
        }
    }
    const bool mine = oneshot || owner == rank;
    if (mine && threadIdx.x < world) {
        const uint32_t* f = t.flags[rank] + (((size_t)par * 2 + 0) * world + threadIdx.x) * kFlagPad;
        if (!wait_flag(f, e, max_spins, status) && atomicCAS(&s_fail, 0, 1) == 0) {
            status[0] = FB_TIMEOUT; status[1] = 16 + threadIdx.x; status[2] = (int)e; status[3] = tile;
        }
    }
    __syncthreads();
    if (oneshot) {
        // ---- one-shot: every rank holds all partials of every tile; reduce in rank order straight into `out` ----
        if (s_fail == 0) {
            const float* src0 = t.scatter[rank] + ((size_t)par * world * tiles_per_rank + tile) * C::kTileElems;
            const size_t slot = (size_t)tiles_per_rank * C::kTileElems;
            for (int i = threadIdx.x; i < rows * (kTileW / 4); i += kThreads) {
                const int rr = i / (kTileW / 4), c4 = i % (kTileW / 4);
                const int n = n0 + c4 * 4;
                if (n >= N) continue;
                float4 a = ld_cg_f4(src0 + (size_t)i * 4);
                for (int s = 1; s < world; ++s) {
                    const float4 b = ld_cg_f4(src0 + s * slot + (size_t)i * 4);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                *reinterpret_cast<float4*>(out + (size_t)(m0 + rr) * ldo + n) = a;
            }
        }
        return;
    }
    if (mine && s_fail == 0) {
        // ---- reduce this tile in rank order and hand it to every rank ----
        const float* src0 = t.scatter[rank] + ((size_t)par * world * tiles_per_rank + tile / world) * C::kTileElems;
        const size_t slot = (size_t)tiles_per_rank * C::kTileElems;
        const size_t goff = ((size_t)par * ntiles + tile) * C::kTileElems;
        for (int i = threadIdx.x; i < rows * (kTileW / 4); i += kThreads) {
            float4 a = ld_cg_f4(src0 + (size_t)i * 4);
            for (int s = 1; s < world; ++s) {
                const float4 b = ld_cg_f4(src0 + s * slot + (size_t)i * 4);
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            for (int p = 0; p < world; ++p) *reinterpret_cast<float4*>(t.gather[p] + goff + (size_t)i * 4) = a;
        }
    }
    __syncthreads();
    if (mine && threadIdx.x == 0) {
        const unsigned owned = (unsigned)((ntiles - rank + world - 1) / world);
        __threadfence();
        if (atomicAdd(ticket + 1, 1u) == owned - 1u) {
            __threadfence_system();
            for (int p = 0; p < world; ++p)
                st_release_sys(t.flags[p] + (((size_t)par * 2 + 1) * world + rank) * kFlagPad, e);
            ticket[1] = 0u;
        }
    }
    // ---- gather: wait for the owner's stamp, copy the reduced tile out ----
    if (threadIdx.x == 0) {
        const uint32_t* f = t.flags[rank] + (((size_t)par * 2 + 1) * world + owner) * kFlagPad;
        if (!wait_flag(f, e, max_spins, status) && atomicCAS(&s_fail, 0, 1) == 0) {
            status[0] = FB_TIMEOUT; status[1] = 32 + owner; status[2] = (int)e; status[3] = tile;
        }
    }
    __syncthreads();
    if (s_fail == 0) {
        const float* g = t.gather[rank] + ((size_t)par * ntiles + tile) * C::kTileElems;
        for (int i = threadIdx.x; i < rows * (kTileW / 4); i += kThreads) {
            const int r = i / (kTileW / 4), c4 = i % (kTileW / 4);
            const int n = n0 + c4 * 4;
            if (n < N) *reinterpret_cast<float4*>(out + (size_t)(m0 + r) * ldo + n) = ld_cg_f4(g + (size_t)i * 4);
        }
    }
}

template <int BN>
int launch_gar(const CUtensorMap& tw, const CUtensorMap& tx, float* out, int ldo, int M, int N, int K, int accumulate,
               const GarPtrs& t, uint32_t* epoch, unsigned* ticket, int* status, int rank, int world, int64_t scatter_cap,
               int64_t gather_cap, int max_spins, int mode, cudaStream_t st) {
    auto k = gemm_tc_ar_kernel<BN>;
    static int resident = -1;
    if (resident < 0) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, sms = 0, per = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, k, kThreads, Cfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        resident = sms * per;
    }
    dim3 grid((N + kTileW - 1) / kTileW, (M + BN - 1) / BN);
    const int ntiles = (int)(grid.x * grid.y);
    // one round trip instead of two when the one-shot volume is the same (two ranks) or small, and it fits
    const int64_t tile_elems = Cfg<BN>::kTileElems;
    const bool want_one = mode == 1 || (mode == 0 && (world == 2 || (int64_t)(world - 1) * ntiles * tile_elems * 4 <= (1 << 20)));
    const bool oneshot = world > 1 && want_one && (int64_t)2 * world * ntiles * tile_elems <= scatter_cap;
    const int tpr = oneshot ? ntiles : (ntiles + world - 1) / world;
    if (world > 1) {
        if (ntiles > resident || ntiles < world) return (int)cudaErrorInvalidValue;   // co-residency; every rank owns a tile
        if ((int64_t)2 * world * tpr * tile_elems > scatter_cap) return (int)cudaErrorInvalidValue;
        if (!oneshot && (int64_t)2 * ntiles * tile_elems > gather_cap) return (int)cudaErrorInvalidValue;
    }
    FB_LAUNCH((k), grid, kThreads, Cfg<BN>::kSmem, st, tw, tx, out, ldo, M, N, K, accumulate, t, epoch, ticket, status, rank,
              world, tpr, max_spins, (int)oneshot);
    return FB_LAUNCH_CHECK();
}

}  // namespace

// Number of CTAs the fused kernel would launch for an [M, N] output (the host uses it to size buffers).
FB_API int fb_gemm_tc_ar_plan(int64_t M, int64_t N, int* bn_out, int* ntiles_out) {
    const int ct = (int)((N + kTileW - 1) / kTileW);
    int bn = 16;
    while (bn < 256 && ct * (int)((M + bn - 1) / bn) > 148) bn *= 2;
    *bn_out = bn;
    *ntiles_out = ct * (int)((M + bn - 1) / bn);
    return 0;
}

// W [N, K] bf16 row-major (this rank's K slice), x [M, K] bf16 (row stride ldx), out [M, N] f32 (row stride
// ldo, ldo % 4 == 0, 16-byte aligned).  scatter_ptrs / gather_ptrs / flag_ptrs: host arrays of `world` device
// pointers into peer-mapped buffers of scatter_cap / gather_cap floats and 4 * world * 32 words; epoch: one
// word, ticket: two words (all zero-initialised, private to this collective).  With accumulate != 0 the local
// `out` is added to this rank's partial before the reduction.  mode: 0 = choose, 1 = one-shot, 2 = two-shot.
FB_API int fb_gemm_tc_ar(const void* W, const void* x, int64_t ldx, float* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                         int64_t accumulate, const void* const* scatter_ptrs, const void* const* gather_ptrs,
                         const void* const* flag_ptrs, int64_t scatter_cap, int64_t gather_cap, void* epoch, void* ticket,
                         int* status, int64_t rank, int64_t world, int64_t max_spins, int64_t mode, cudaStream_t st) {
    if ((K % 8) || (ldx % 8) || (ldo % 4) || (N % 4) || M < 1 || world < 1 || world > kMaxWorld || ((uintptr_t)x & 15) ||
        ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    int bn, ntiles;
    fb_gemm_tc_ar_plan(M, N, &bn, &ntiles);
    if (ntiles > 148 && world > 1) return (int)cudaErrorInvalidValue;
    GarPtrs t = {};
    for (int i = 0; i < world && world > 1; ++i) {
        t.scatter[i] = (float*)scatter_ptrs[i];
        t.gather[i] = (float*)gather_ptrs[i];
        t.flags[i] = (uint32_t*)flag_ptrs[i];
    }
    CUtensorMap tw, tx;
    int rc = fb_make_tmap_2d(&tw, W, (uint64_t)N, (uint64_t)K, kTileW, kBK, 2);
    if (rc) return rc;
    rc = fb_make_tmap_2d_strided(&tx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)(bn < 16 ? 16 : bn), kBK, 2);
    if (rc) return rc;
#define GAR_ARGS tw, tx, out, (int)ldo, (int)M, (int)N, (int)K, (int)accumulate, t, (uint32_t*)epoch, (unsigned*)ticket, status, \
                 (int)rank, (int)world, scatter_cap, gather_cap, (int)max_spins, (int)mode, st
    switch (bn) {
        case 16: return launch_gar<16>(GAR_ARGS);
        case 32: return launch_gar<32>(GAR_ARGS);
        case 64: return launch_gar<64>(GAR_ARGS);
        case 128: return launch_gar<128>(GAR_ARGS);
        default: return launch_gar<256>(GAR_ARGS);
    }
#undef GAR_ARGS
}
