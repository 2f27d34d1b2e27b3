// Row-parallel GEMV fused with its all-reduce and the hyper-connection fold: ONE kernel for
//   y = sum_ranks ( x_rank . W_rank^T (+ y_rank) )         [m <= 8 rows, N outputs]
//   R'[i] = post_i * y + sum_k comb[k][i] R[k]              (optional)
//   part  = per-tile mix dots of R' with the next site's fn, and |R'|^2   (optional)
//
// A CTA owns 16 or 32 output columns.  Its warps stream the CTA's weight rows with the
// tensor-core GEMV core (mma.sync m16n8k16, software-pipelined weight loads), reduce their
// partial tiles through shared memory, and then run the collective on that 8-row tile alone:
//   push    16-byte peer stores of the tile into slot `rank` of every peer's staging buffer,
//   publish tiles go out in groups (by default one group = the grid): the CTA that completes a group
//           fences at system scope once and stamps the group's epoch on every peer,
//   wait    bounded poll of the local flag words of all ranks (peers write them into local
//           memory, so a poll never crosses NVLink); on expiry the kernel records
//           {TIMEOUT, peer, epoch, tile}, skips the reduction and still returns,
//   reduce  rank-ordered sum from the local staging, so all ranks get identical bits.
// The transfer of one tile overlaps the weight streaming of the CTAs still computing.  Tiles
// only depend on the same tile of the peers, and the host picks a tile shape whose grid is
// co-resident on a 148-SM part, so no CTA waits for a CTA that cannot be scheduled.
// Epochs and parity double-buffering follow the stand-alone all-reduce (collective.cu).
// With world == 1 the collective is skipped and the kernel is a GEMV with the fold epilogue.
//
// Replaces the reference's store-carrying GEMV epilogues + `p2p_ar_pubred_v5(_hcpost)`
// (kernels/cuda/ferrite_kernels.cu:8968-9524; crates/ferrite-exec/src/tp.rs:742-1059).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxTiles = 512;
constexpr int kMaxMix = 24;
constexpr int kFlagPad = 32;   // words per flag: pollers of different tiles never share a cache line

struct ArPtrs {
    float* staging[kMaxWorld];   // [2][world][max_elems]
    uint32_t* flags[kMaxWorld];  // [2][world][kMaxTiles][kFlagPad]: one 128-byte line per flag
};

struct HcFold {
    const float* Rin;   // [m][4][N]   (null: no fold)
    float* Rout;        // [m][4][N]
    const float* post;  // [m][4]
    const float* comb;  // [m][16]
    const float* fn;    // [mix][4 * N]  (null: no mix dots)
    float* acc;         // [m][kMaxMix + 1]
    int mix;
    float* part;        // [8][kMaxMix + 1][kMaxTiles] per-tile partial dots, summed by the consumer
    int* part_n;        // [8] number of valid tiles per row (the consumer clears it)
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
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}

template <int RT, int NW, bool FP8>
__global__ void __launch_bounds__(NW * 32, (NW >= 16 ? 2 : (RT >= 2 ? 2 : 4)))
gemv_ar_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales, const uint16_t* __restrict__ xhi,
               const uint16_t* __restrict__ xlo, int ldx, float* __restrict__ y, int ldo, int mrows, int N, int K,
               int accumulate, int store_y, ArPtrs t, uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket, int* __restrict__ status,
               int rank, int world, int max_elems, int max_spins, int group, HcFold hc, int l2_ahead) {
    pdl_launch();
    constexpr int kTileN = 16 * RT;
    constexpr int KB = FP8 ? 128 : 64;
    constexpr int XW = FP8 ? 16 : 8;
    __shared__ float red[NW][RT][32][4];
    __shared__ __align__(16) float tile[8][16 * RT];
    __shared__ __align__(16) float fn_s[kMaxMix][4][16 * RT];   // next site's mix rows, this CTA's columns
    __shared__ __align__(16) float r_s[8][4][16 * RT];          // residual tile in, folded tile out
    __shared__ int s_fail;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * kTileN;
    const int nkb = K / KB;
    const int kblocks = (K + 127) >> 7;
    float acc[RT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
    const uint8_t* wa[RT];
    const uint8_t* wb[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const size_t esz = FP8 ? 1 : 2;
        wa[r] = W + (size_t)min(n0 + r * 16 + g, N - 1) * K * esz + (size_t)tq * 32;
        wb[r] = W + (size_t)min(n0 + r * 16 + g + 8, N - 1) * K * esz + (size_t)tq * 32;
    }
    // two fragment sets alternate roles (one is loaded while the other is multiplied): no register copies per k-block
    WFrag fa[RT], fb[RT];
    auto fetch = [&](WFrag (&f)[RT], int kb) {
#pragma unroll
        for (int r = 0; r < RT; ++r) f[r] = load_wfrag(wa[r] + (size_t)kb * 128, wb[r] + (size_t)kb * 128);
        const int kp = kb + (l2_ahead - 1) * NW;   // read-ahead into L2, one lane per 128-byte line
        if (l2_ahead > 1 && kp < nkb && tq == 0) {
#pragma unroll
            for (int r = 0; r < RT; ++r) { prefetch_l2(wa[r] + (size_t)kp * 128); prefetch_l2(wb[r] + (size_t)kp * 128); }
        }
    };
    auto compute = [&](const WFrag (&f)[RT], int kb) {
        uint32_t xh[XW], xl[XW];
        load_xfrag<XW, !FP8>(xhi, xlo, ldx, g, mrows, kb * KB + tq * (KB / 4), xh, xl);
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
    const bool fold = hc.Rin != nullptr;
    if (fold && hc.fn) {   // weights: may be fetched before the previous kernel has finished
        constexpr int Q4 = kTileN / 4;
        for (int i = threadIdx.x; i < hc.mix * 4 * Q4; i += blockDim.x) {
            const int q = i / (4 * Q4), k = (i / Q4) % 4, c4 = i % Q4;
            cp_async16(&fn_s[q][k][c4 * 4], hc.fn + ((size_t)q * 4 + k) * N + n0 + c4 * 4);
        }
    }
    pdl_wait();
    if (fold) {
        constexpr int Q4 = kTileN / 4;
        for (int i = threadIdx.x; i < mrows * 4 * Q4; i += blockDim.x) {
            const int mm = i / (4 * Q4), k = (i / Q4) % 4, c4 = i % Q4;
            cp_async16(&r_s[mm][k][c4 * 4], hc.Rin + ((size_t)mm * 4 + k) * N + n0 + c4 * 4);
        }
    }
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
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    // ---- this rank's partial tile: tile[m][n_local] ----
    if (threadIdx.x < RT * 128) {
        const int idx = threadIdx.x;
        const int r = idx >> 7, l = (idx & 127) >> 2, c = idx & 3;
        const int nl = r * 16 + (l >> 2) + 8 * (c >> 1);
        const int m = 2 * (l & 3) + (c & 1);
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w][r][l][c];
        if (accumulate && m < mrows && n0 + nl < N) v += y[(size_t)m * ldo + n0 + nl];
        tile[m][nl] = v;
    }
    __syncthreads();
    const int m = threadIdx.x / kTileN, nl = threadIdx.x % kTileN;   // (row, column) owned in the epilogue
    const bool owner = threadIdx.x < 8 * kTileN;
    const bool live = owner && m < mrows && n0 + nl < N;
    float v = owner ? tile[m][nl] : 0.f;
    if (world > 1) {
        // Tiles are published in groups of `group`: a CTA pushes its tile, fences at GPU scope and takes
        // a ticket; the CTA that takes the group's last ticket fences at system scope and stamps the
        // group's flag on every peer (one system fence per group instead of one per CTA: the GPU-scope
        // release/acquire chain through the ticket makes the other CTAs' peer stores part of what the
        // publishing thread's fence orders).  Every CTA of the group then waits for the group stamps.
        const int tl = blockIdx.x;
        const int grp = tl / group;
        const int gsize = min(group, (int)gridDim.x - grp * group);
        const uint32_t e = epoch[grp] + 1u;
        const int par = e & 1u;
        constexpr int Q4 = kTileN / 4;
        for (int i = threadIdx.x; i < world * 8 * Q4; i += blockDim.x) {
            const int p = i / (8 * Q4), j = i % (8 * Q4), mm = j / Q4, c4 = j % Q4;
            if (mm < mrows && n0 + c4 * 4 < N) {
                float* dst = t.staging[p] + ((size_t)par * world + rank) * max_elems + (size_t)mm * N + n0 + c4 * 4;
                *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(&tile[mm][c4 * 4]);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(ticket + grp, 1u) == (unsigned)gsize - 1u) {
                __threadfence_system();
                for (int p = 0; p < world; ++p)
                    st_release_sys(t.flags[p] + (((size_t)par * world + rank) * kMaxTiles + grp) * kFlagPad, e);
                ticket[grp] = 0u;
                epoch[grp] = e;   // every CTA of the group read the old value before it took its ticket
            }
        }
        if (threadIdx.x < world) {
            const uint32_t* f = t.flags[rank] + (((size_t)par * world + threadIdx.x) * kMaxTiles + grp) * kFlagPad;
            int spins = 0;
        const int budget = fb_spin_budget(status, max_spins);
            // relaxed polls (cheap, no cache maintenance), one acquire load once the stamp is there
            while (ld_relaxed_sys(f) < e) {
                if (++spins > budget) {
                    if (atomicCAS(&s_fail, 0, 1) == 0) {
                        status[0] = FB_TIMEOUT; status[1] = threadIdx.x; status[2] = (int)e; status[3] = grp;
                    }
                    break;
                }
                __nanosleep(64);
            }
            (void)ld_acquire_sys(f);
        }
        __syncthreads();
        if (s_fail == 0 && live) {
            v = 0.f;
            for (int src = 0; src < world; ++src)
                v += ld_cg_f32(t.staging[rank] + ((size_t)par * world + src) * max_elems + (size_t)m * N + n0 + nl);
        }
    }
    if (store_y && live) y[(size_t)m * ldo + n0 + nl] = v;
    if (!fold) return;
    // ---- hyper-connection fold on this tile (operands were prefetched into shared memory) ----
    cp_async_wait_all();
    __syncthreads();
    if (live) {
        float rk[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) rk[k] = r_s[m][k][nl];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float o = hc.post[m * 4 + i] * v;
#pragma unroll
            for (int k = 0; k < 4; ++k) o = fmaf(hc.comb[m * 16 + k * 4 + i], rk[k], o);
            hc.Rout[((size_t)m * 4 + i) * N + n0 + nl] = o;
            r_s[m][i][nl] = o;   // the inputs of this column are already in rk
        }
    }
    if (!hc.fn) return;
    __syncthreads();
    // mix dots of R' with fn and |R'|^2 as per-tile partials; the consumer (hc_pre) sums the tiles.
    // One warp per mix row q (q == mix: the sum of squares); lanes cover the 4 x kTileN tile.
    const int tl = blockIdx.x;
    constexpr int EPL = 4 * kTileN / 32;   // tile elements per lane
    for (int q = warp; q <= hc.mix; q += NW) {
        float fv[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) fv[e] = q < hc.mix ? (&fn_s[q][0][0])[lane + 32 * e] : 0.f;
        for (int mm = 0; mm < mrows; ++mm) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float rv = (&r_s[mm][0][0])[lane + 32 * e];
                d = fmaf(q < hc.mix ? fv[e] : rv, rv, d);
            }
            d = warp_sum(d);
            if (lane == 0) hc.part[((size_t)mm * (kMaxMix + 1) + (q < hc.mix ? q : kMaxMix)) * kMaxTiles + tl] = d;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < mrows) hc.part_n[threadIdx.x] = gridDim.x;
}

}  // namespace

FB_API int fb_gemv_ar_limits(int* max_tiles, int* max_world, int* flag_words) {
    *max_tiles = kMaxTiles; *max_world = kMaxWorld; *flag_words = kFlagPad;
    return 0;
}

template <int RT, int NW, bool FP8, typename... A>
static void launch_ar(int N, cudaStream_t st, A... a) {
    FB_LAUNCH((gemv_ar_kernel<RT, NW, FP8>), (N + 16 * RT - 1) / (16 * RT), NW * 32, 0, st, a...);
}

// W [N, K] bf16 (scales == null) or e4m3 with 128x128 f32 block scales; xs: split activation planes
// (see fb_gemv_mma_bf16).  staging_ptrs / flag_ptrs: host arrays of `world` device pointers, or null
// when world == 1.  Rin == null disables the fold; fn == null keeps the fold but skips the mix dots.
// part: 8 * 25 * max_tiles floats of per-tile mix-dot partials and part_n: 8 ints (tiles per row), both
// consumed and cleared by fb_hc_pre_apply / fb_d4_hc_pre; `acc` is not written by this kernel.
FB_API int fb_gemv_ar(const void* W, const float* scales, const void* xs, int64_t xs_ld, int64_t xs_plane, float* y,
                      int64_t ldo, int64_t m, int64_t N, int64_t K, int64_t accumulate, int64_t store_y,
                      const void* const* staging_ptrs, const void* const* flag_ptrs, void* epoch, void* ticket,
                      int* status, int64_t rank, int64_t world, int64_t max_elems, int64_t max_spins, int64_t group, const float* Rin, float* Rout,
                      const float* post, const float* comb, const float* fn, float* acc, int64_t mix, float* part,
                      int* part_n, cudaStream_t st) {
    const bool fp8 = scales != nullptr;
    const int kb = fp8 ? 128 : 64;
    if (m < 1 || m > 8 || (N % 4) || (K % kb) || (xs_ld % 8) || world > kMaxWorld || mix > kMaxMix ||
        (world > 1 && m * N > max_elems) || (Rin && Rin == Rout))
        return (int)cudaErrorInvalidValue;
    ArPtrs t = {};
    for (int i = 0; i < world && world > 1; ++i) {
        t.staging[i] = (float*)staging_ptrs[i];
        t.flags[i] = (uint32_t*)flag_ptrs[i];
    }
    // One published group per launch (`group` is kept in the ABI and ignored): with several groups each group has
    // its own epoch, launches of different widths advance them unevenly, and two launches could then meet on the
    // same staging parity while a peer still reduces the earlier one.  One group = one epoch per launch.
    (void)group;
    HcFold hc{Rin, Rout, post, comb, fn, acc, (int)mix, part, part_n};
    if (Rin && fn && (!part || !part_n)) return (int)cudaErrorInvalidValue;
    if (Rin && (N % 32)) return (int)cudaErrorInvalidValue;  // the fold works on whole column tiles
    const uint16_t* base = (const uint16_t*)xs;
    const uint16_t* hi = base + (fp8 ? 2 * xs_plane : 0);
    const uint16_t* lo = hi + xs_plane;
    const int nkb = (int)(K / kb);
    const int t16 = (int)((N + 15) / 16);
    // tile shape: every CTA of the grid must be resident at once (148 SMs x CTAs per SM of the bounds)
    int shape;  // 0: <1,16> (2 per SM), 1: <1,8> (4 per SM), 2: <2,8> (2 per SM)
    if (nkb >= 64 && t16 <= 256) shape = 0;
    else if (t16 <= 512) shape = 1;
    else if ((N + 31) / 32 <= 256) shape = 2;
    else return (int)cudaErrorInvalidValue;
#define AR_ARGS (const uint8_t*)W, scales, hi, lo, (int)xs_ld, y, (int)ldo, (int)m, (int)N, (int)K, (int)accumulate, \
                (int)store_y, t, (uint32_t*)epoch, (unsigned*)ticket, status, (int)rank, (int)world, (int)max_elems, (int)max_spins, (int)kMaxTiles, hc, g_fb_l2_ahead
    if (fp8) {
        if (shape == 0) launch_ar<1, 16, true>((int)N, st, AR_ARGS);
        else if (shape == 1) launch_ar<1, 8, true>((int)N, st, AR_ARGS);
        else launch_ar<2, 8, true>((int)N, st, AR_ARGS);
    } else {
        if (shape == 0) launch_ar<1, 16, false>((int)N, st, AR_ARGS);
        else if (shape == 1) launch_ar<1, 8, false>((int)N, st, AR_ARGS);
        else launch_ar<2, 8, false>((int)N, st, AR_ARGS);
    }
#undef AR_ARGS
    return FB_LAUNCH_CHECK();
}
