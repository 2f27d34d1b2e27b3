// Row-parallel GEMV fused with its all-reduce and the hyper-connection fold: ONE kernel for
//   y = sum_ranks ( x_rank . W_rank^T (+ y_rank) )         [m <= 8 rows, N outputs]
//   R'[i] = post_i * y + sum_k comb[k][i] R[k]              (optional)
//   part  = per-tile mix dots of R' with the next site's fn, and |R'|^2   (optional)
//
// A CTA owns 16 or 32 output columns.  Its warps stream the CTA's weight rows with the
// tensor-core GEMV core (mma.sync m16n8k16, software-pipelined weight loads), reduce their
// partial tiles through shared memory, and then run the collective on that 8-row tile alone:
//   push    every value travels as an 8-byte (value, epoch) pair (two pairs per 16-byte peer store) into slot
//           `rank` of every peer's staging buffer: a pair that carries the launch's epoch IS the data, so there is
//           no fence, no flag and no grid-wide ticket between a CTA's stores and a peer's reduction
//           (measured at 4 GPUs with tile stores + one system fence + one flag per launch: 20 us per fused
//           GEMV + all-reduce against 10 us for the same GEMV on one rank),
//   wait    bounded poll of this CTA's own pairs in LOCAL staging (peers write them there, so a poll never
//           crosses NVLink); on expiry the kernel records {TIMEOUT, peer, epoch, tile}, keeps its local partial
//           and still returns,
//   reduce  rank-ordered sum, so all ranks get identical bits.
// The transfer of one tile overlaps the weight streaming of the CTAs still computing.  Tiles
// only depend on the same tile of the peers, and the host picks a tile shape whose grid is
// co-resident on a 148-SM part, so no CTA waits for a CTA that cannot be scheduled.
// Staging is double-buffered by epoch parity (a peer is at most one launch ahead: it needs this rank's pairs to
// finish a launch); the last CTA of a launch advances the epoch, nobody waits on that ticket.
// With world == 1 the collective is skipped and the kernel is a GEMV with the fold epilogue.
//
// Two more stages can ride in the same launch, so that a sublayer boundary is ONE kernel:
//   * activation source: instead of split planes the GEMV can read the f32 [gate | up] row a previous GEMV left
//     and apply SwiGLU while it builds its B fragments (the shared expert's and the dense FFN's down projection);
//   * hyper-connection front of the NEXT site: besides the mix dots every tile leaves the 10 Gram dots
//     <R'_i, R'_j> of its columns.  CTAs meet on a grid barrier (the grid is co-resident by construction); the
//     last CTA to arrive sums the tiles' partials in tile order, derives pre = sigmoid(mix * r * s0 + b) + eps
//     and the RMS of x = sum_i pre_i R'_i from the Gram matrix (|x|^2 = sum_ij pre_i pre_j G_ij), publishes
//     both, and goes on to post / comb (softmax + Sinkhorn), which only the next fold reads.  Every CTA then
//     contracts and normalises its own columns of x and writes them in f32 and split form.  This replaces a
//     one-CTA-per-row kernel (11 us, 90 launches per decode step) by about 3 us inside a kernel that is
//     running anyway.
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

struct HcPre {
    const float* scale;  // [3]   (null: no front)
    const float* base;   // [mix]
    const float* ln_w;   // [N]
    float* post;         // [m][4]   next site's coefficients (may alias HcFold::post: written after the barrier)
    float* comb;         // [m][16]
    float* x;            // [m][N] normalised layer input
    SplitBuf xs;         // ... and its split planes
    float* gram;         // [8][10][kMaxTiles] per-tile Gram partials
    float* coef;         // [8][8]: pre[4], rms factor of x
    unsigned* bar;       // [2]: arrivals of this launch, generation
    float rms_eps, hc_eps;
    int iters;
};

struct XSrc {            // where the activations come from
    const float* gu;     // null: split planes; else f32 rows [gate(I) | up(I)] with stride ld
    int ld, up_off;
    float limit;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// B fragment built from f32 [gate | up]: act = silu(min(g, L)) * clamp(u, -L, L), split into a 16-bit high and low
// part (bf16 pair for bf16 weights, f16 high part only for e4m3 weights, as the plane-reading path does).
template <int WORDS, bool FP8>
__device__ __forceinline__ void swiglu_xfrag(const XSrc& xs, int g, int mrows, int k0, uint32_t (&xh)[WORDS], uint32_t (&xl)[WORDS]) {
    if (g >= mrows) {
#pragma unroll
        for (int i = 0; i < WORDS; ++i) { xh[i] = 0u; xl[i] = 0u; }
        return;
    }
    const float4* pg = reinterpret_cast<const float4*>(xs.gu + (size_t)g * xs.ld + k0);
    const float4* pu = reinterpret_cast<const float4*>(xs.gu + (size_t)g * xs.ld + xs.up_off + k0);
#pragma unroll
    for (int i = 0; i < WORDS / 2; ++i) {
        const float4 a = pg[i], b = pu[i];
        const float ga[4] = {a.x, a.y, a.z, a.w}, ua[4] = {b.x, b.y, b.z, b.w};
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = siluf_(fminf(ga[j], xs.limit)) * fminf(fmaxf(ua[j], -xs.limit), xs.limit);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (FP8) {
                const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                xh[2 * i + j] = *reinterpret_cast<const uint32_t*>(&h);
                xl[2 * i + j] = 0u;
            } else {
                const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * j]), h1 = __float2bfloat16_rn(v[2 * j + 1]);
                const __nv_bfloat16 l0 = __float2bfloat16_rn(v[2 * j] - __bfloat162float(h0));
                const __nv_bfloat16 l1 = __float2bfloat16_rn(v[2 * j + 1] - __bfloat162float(h1));
                xh[2 * i + j] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
                xl[2 * i + j] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
            }
        }
    }
}

__device__ __forceinline__ float2 ld_relaxed_sys_f2(const float2* p) {
    float2 v;
    asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
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

constexpr int kGram = 10;   // pairs (i <= j) of the four residual streams

template <int RT, int NW, bool FP8, bool SWIGLU>
__global__ void __launch_bounds__(NW * 32, (NW >= 16 ? 2 : (RT >= 2 ? 2 : 4)))
gemv_ar_kernel(const uint8_t* __restrict__ W, const float* __restrict__ scales, const uint16_t* __restrict__ xhi,
               const uint16_t* __restrict__ xlo, int ldx, float* __restrict__ y, int ldo, int mrows, int N, int K,
               int accumulate, int store_y, ArPtrs t, uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket, int* __restrict__ status,
               int rank, int world, int max_elems, int max_spins, int group, HcFold hc, int l2_ahead, XSrc xsrc, HcPre pre) {
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
        if (SWIGLU) swiglu_xfrag<XW, FP8>(xsrc, g, mrows, kb * KB + tq * (KB / 4), xh, xl);
        else load_xfrag<XW, !FP8>(xhi, xlo, ldx, g, mrows, kb * KB + tq * (KB / 4), xh, xl);
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
    const bool front = fold && hc.fn && pre.scale != nullptr;
    // generation of the grid barrier: read before this CTA arrives, so it is the value of this launch
    const uint32_t gen0 = front ? ld_acquire_gpu(pre.bar + 1) : 0u;
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
        // Low-latency exchange: every value travels as an 8-byte (value, epoch) pair, so a pair that shows the
        // launch's epoch IS the data: no fence, no flag, no grid-wide ticket on the critical path.  A CTA pushes its
        // tile to every peer (two pairs per 16-byte store) and then polls its own tile's pairs in its own staging
        // until each peer's have arrived; CTAs of one launch never wait for each other.  Staging is double-buffered
        // by epoch parity: a peer can be at most one launch ahead (it needs this rank's pairs to finish a launch).
        const int grp = 0;
        const uint32_t e = epoch[grp] + 1u;
        const int par = e & 1u;
        const float ef = __uint_as_float(e);
        constexpr int Q2 = kTileN / 2;
        for (int i = threadIdx.x; i < world * 8 * Q2; i += blockDim.x) {
            const int p = i / (8 * Q2), j = i % (8 * Q2), mm = j / Q2, c2 = j % Q2;
            if (p != rank && mm < mrows && n0 + c2 * 2 < N) {
                float2* dst = reinterpret_cast<float2*>(t.staging[p]) + ((size_t)par * world + rank) * max_elems + (size_t)mm * N + n0 + c2 * 2;
                *reinterpret_cast<float4*>(dst) = make_float4(tile[mm][c2 * 2], ef, tile[mm][c2 * 2 + 1], ef);
            }
        }
        if (live) {
            const int budget = fb_spin_budget(status, max_spins);
            float sum = 0.f;
            for (int src = 0; src < world; ++src) {     // rank order: every rank adds in the same order
                if (src == rank) { sum += v; continue; }
                const float2* f = reinterpret_cast<const float2*>(t.staging[rank]) + ((size_t)par * world + src) * max_elems + (size_t)m * N + n0 + nl;
                float2 pr = ld_relaxed_sys_f2(f);
                int spins = 0;
                while (__float_as_uint(pr.y) != e) {
                    if (++spins > budget) {
                        if (atomicCAS(&s_fail, 0, 1) == 0) {
                            status[0] = FB_TIMEOUT; status[1] = src; status[2] = (int)e; status[3] = (int)blockIdx.x;
                        }
                        break;
                    }
                    pr = ld_relaxed_sys_f2(f);
                }
                sum += pr.x;
            }
            v = sum;
        }
        __syncthreads();
        if (s_fail != 0) v = owner ? tile[m][nl] : 0.f;   // a peer never answered: keep the local partial, the status word says so
        // the last CTA to get here advances the launch's epoch (nobody waits on this ticket)
        if (threadIdx.x == 0 && atomicAdd(ticket + grp, 1u) == gridDim.x - 1u) {
            ticket[grp] = 0u;
            epoch[grp] = e;
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
    if (!hc.fn) {
        // a fold without a next site ends a forward: leave the tile counts at zero, so that the first front of the
        // next forward (which has no producer) never sees partials of this one
        if (blockIdx.x == 0 && threadIdx.x < mrows && hc.part_n) hc.part_n[threadIdx.x] = 0;
        return;
    }
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
    if (!front && blockIdx.x == 0 && threadIdx.x < mrows) hc.part_n[threadIdx.x] = gridDim.x;
    if (!pre.gram) return;
    // ---- hyper-connection front of the next site ------------------------------------------------------------
    // Gram partials of this tile: pair p = (i, j), i <= j, one warp per (row, pair).  With them the consumer gets
    // |x|^2 of x = sum_i pre_i R'_i as sum_ij pre_i pre_j G_ij, i.e. the RMSNorm of x needs no pass over x.
    for (int w = warp; w < mrows * kGram; w += NW) {
        const int mm = w / kGram, p = w % kGram;
        int i = 0, rem = p;
        while (rem >= 4 - i) { rem -= 4 - i; ++i; }
        const int j = i + rem;
        float d = 0.f;
        for (int c = lane; c < kTileN; c += 32) d = fmaf(r_s[mm][i][c], r_s[mm][j][c], d);
        d = warp_sum(d);
        if (lane == 0) pre.gram[((size_t)mm * kGram + p) * kMaxTiles + tl] = d;
    }
    if (!front) return;   // the column-parallel front kernel (fb_hc_pre_wide) consumes the partials
    __shared__ int s_last;
    __shared__ float s_sum[8][kMaxMix + 1 + kGram];
    __shared__ float s_coef[8][8];
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(pre.bar, 1u) == gridDim.x - 1u;
    }
    __syncthreads();
    const int nt = gridDim.x;
    // Sums the tiles' partials of nq quantities per row in a fixed order: one warp per (row, quantity), every lane
    // loads its tiles (lane, lane + 32, ...) with all loads in flight before the first add, then a shuffle tree.
    // Two pairs per warp iteration keep twice as many loads in flight.  sel(q): index of the q-th quantity in
    // [0, kMaxMix] (mix dot / sum of squares) or kMaxMix + 1 + p (Gram pair p).
    auto part_src = [&](int mm, int qi) -> const float* {
        return qi <= kMaxMix ? hc.part + ((size_t)mm * (kMaxMix + 1) + qi) * kMaxTiles
                             : pre.gram + ((size_t)mm * kGram + (qi - kMaxMix - 1)) * kMaxTiles;
    };
    auto reduce_parts = [&](int row0, int nrows, int q0, int nq, auto sel) {
        const int npairs = nrows * nq;
        constexpr int TPL = kMaxTiles / 32;   // tiles per lane
        for (int pr = warp * 2; pr < npairs; pr += NW * 2) {
            float v[2][TPL];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int p = min(pr + u, npairs - 1);
                const float* src = part_src(row0 + p / nq, sel(q0 + p % nq));
#pragma unroll
                for (int j = 0; j < TPL; ++j) v[u][j] = (lane + 32 * j < nt) ? __ldcg(src + lane + 32 * j) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < TPL; ++j) a += v[u][j];
                a = warp_sum(a);
                const int p = pr + u;
                if (lane == 0 && p < npairs) s_sum[row0 + p / nq][sel(q0 + p % nq)] = a;
            }
        }
        __syncthreads();
    };
    if (s_last) {
        __threadfence();
        // phase 1: what x needs: mix dots 0..3, the sum of squares, the Gram matrix
        reduce_parts(0, mrows, 0, 5 + kGram, [&](int q) { return q < 4 ? q : (q == 4 ? kMaxMix : kMaxMix + 1 + (q - 5)); });
        if (threadIdx.x < mrows) {
            const int mm = threadIdx.x;
            const float rr = rsqrtf(s_sum[mm][kMaxMix] / (float)(4 * N) + pre.rms_eps);
            float pw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pw[i] = sigmoidf_(s_sum[mm][i] * rr * pre.scale[0] + pre.base[i]) + pre.hc_eps;
            float xss = 0.f;
            int p = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = i; j < 4; ++j, ++p) xss += (i == j ? 1.f : 2.f) * pw[i] * pw[j] * s_sum[mm][kMaxMix + 1 + p];
            const float inv = rsqrtf(fmaxf(xss, 0.f) / (float)N + pre.rms_eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) { s_coef[mm][i] = pw[i]; pre.coef[mm * 8 + i] = pw[i]; }
            s_coef[mm][4] = inv; pre.coef[mm * 8 + 4] = inv;
            s_coef[mm][5] = rr; pre.coef[mm * 8 + 5] = rr;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            pre.bar[0] = 0u;
            __threadfence();
            st_release_gpu(pre.bar + 1, gen0 + 1u);   // everyone else may go on
        }
    } else {
        if (threadIdx.x == 0) {
            int spins = 0;
            const int budget = fb_spin_budget(status, max_spins);
            while (ld_acquire_gpu(pre.bar + 1) == gen0) {
                if (++spins > budget) {
                    status[0] = FB_TIMEOUT; status[1] = -1; status[2] = (int)gen0; status[3] = tl;
                    s_fail = 1;
                    break;
                }
                __nanosleep(32);
            }
        }
        __syncthreads();
        if (s_fail) return;
        if (threadIdx.x < mrows * 8) s_coef[threadIdx.x >> 3][threadIdx.x & 7] = ld_cg_f32(pre.coef + threadIdx.x);
        __syncthreads();
    }
    if (live) {
        const float* cf = s_coef[m];
        const float xv = cf[0] * r_s[m][0][nl] + cf[1] * r_s[m][1][nl] + cf[2] * r_s[m][2][nl] + cf[3] * r_s[m][3][nl];
        const float o = xv * cf[4] * __ldg(pre.ln_w + n0 + nl);
        pre.x[(size_t)m * N + n0 + nl] = o;
        split_store(pre.xs, m, n0 + nl, o);
    }
    // phase 2 (only the next fold reads it): post and comb of the next site, row r by CTA r, side by side with the
    // other CTAs' x tiles
    if ((int)blockIdx.x >= mrows) return;
    __syncthreads();
    reduce_parts(blockIdx.x, 1, 4, hc.mix - 4, [&](int q) { return q; });
    if (warp == 0) {
        const int mm = blockIdx.x;
        const float rr = s_coef[mm][5];
        const float* a = s_sum[mm];
        if (lane < 4) pre.post[mm * 4 + lane] = 2.f * sigmoidf_(a[4 + lane] * rr * pre.scale[1] + pre.base[4 + lane]);
        // comb element (i = lane / 4, k = lane % 4): row softmax + eps, column normalise, then Sinkhorn rounds
        float c = 0.f;
        const bool on = lane < 16;
        if (on) c = a[8 + lane] * rr * pre.scale[2] + pre.base[8 + lane];
        float mx = on ? c : -INFINITY;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float e = on ? __expf(c - mx) : 0.f;
        float den = e + __shfl_xor_sync(0xffffffffu, e, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        c = on ? e / den + pre.hc_eps : 0.f;
        float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        c = __fdividef(c, cs + pre.hc_eps);
        for (int it = 1; it < pre.iters; ++it) {
            float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            c = __fdividef(c, rs + pre.hc_eps);
            cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            c = __fdividef(c, cs + pre.hc_eps);
        }
        if (on) pre.comb[mm * 16 + lane] = c;
    }
}

}  // namespace

FB_API int fb_gemv_ar_limits(int* max_tiles, int* max_world, int* flag_words) {
    *max_tiles = kMaxTiles; *max_world = kMaxWorld; *flag_words = kFlagPad;
    return 0;
}

template <int RT, int NW, bool FP8, bool SWIGLU, typename... A>
static void launch_ar(int N, cudaStream_t st, A... a) {
    FB_LAUNCH((gemv_ar_kernel<RT, NW, FP8, SWIGLU>), (N + 16 * RT - 1) / (16 * RT), NW * 32, 0, st, a...);
}

// Optional stages of fb_gemv_ar (all pointers null / zero: off).
struct FbGemvArExt {
    // activation source: f32 rows [gate | up] (stride gu_ld, up at column gu_up_off) instead of split planes
    const float* gu; int64_t gu_ld, gu_up_off; float limit;
    // hyper-connection front of the next site (needs the fold with fn): see HcPre
    const float* pre_scale; const float* pre_base; const float* pre_ln_w;
    float* pre_post; float* pre_comb; float* pre_x;
    void* xs_base; int64_t xs_ld, xs_plane, xs_mask;
    float* gram; float* coef; void* bar;
    float rms_eps, hc_eps; int64_t iters;
};

// W [N, K] bf16 (scales == null) or e4m3 with 128x128 f32 block scales; xs: split activation planes
// (see fb_gemv_mma_bf16).  staging_ptrs / flag_ptrs: host arrays of `world` device pointers, or null
// when world == 1.  Rin == null disables the fold; fn == null keeps the fold but skips the mix dots.
// part: 8 * 25 * max_tiles floats of per-tile mix-dot partials and part_n: 8 ints (tiles per row), both
// consumed and cleared by fb_hc_pre_apply / fb_d4_hc_pre; `acc` is not written by this kernel.
// ext (may be null): the SwiGLU activation source and the next site's hyper-connection front.
FB_API int fb_gemv_ar(const void* W, const float* scales, const void* xs, int64_t xs_ld, int64_t xs_plane, float* y,
                      int64_t ldo, int64_t m, int64_t N, int64_t K, int64_t accumulate, int64_t store_y,
                      const void* const* staging_ptrs, const void* const* flag_ptrs, void* epoch, void* ticket,
                      int* status, int64_t rank, int64_t world, int64_t max_elems, int64_t max_spins, int64_t group, const float* Rin, float* Rout,
                      const float* post, const float* comb, const float* fn, float* acc, int64_t mix, float* part,
                      int* part_n, const FbGemvArExt* ext, cudaStream_t st) {
    const bool fp8 = scales != nullptr;
    const int kb = fp8 ? 128 : 64;
    const bool swiglu = ext && ext->gu;
    if (m < 1 || m > 8 || (N % 4) || (K % kb) || (!swiglu && (xs_ld % 8)) || world > kMaxWorld || mix > kMaxMix ||
        (world > 1 && m * N > max_elems) || (Rin && Rin == Rout))
        return (int)cudaErrorInvalidValue;
    if (swiglu && ((ext->gu_ld % 4) || (ext->gu_up_off % 4) || ((uintptr_t)ext->gu % 16))) return (int)cudaErrorInvalidValue;
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
    XSrc xsrc{};
    if (swiglu) xsrc = XSrc{ext->gu, (int)ext->gu_ld, (int)ext->gu_up_off, ext->limit};
    HcPre pre{};
    if (ext && ext->gram && !ext->pre_scale) {   // Gram partials only
        if (!Rin || !fn) return (int)cudaErrorInvalidValue;
        pre.gram = ext->gram;
    }
    if (ext && ext->pre_scale) {
        if (N < 512 /* one CTA per row finishes post / comb */ || !Rin || !fn || mix < 8 || !ext->pre_base || !ext->pre_ln_w || !ext->pre_post || !ext->pre_comb || !ext->pre_x ||
            !ext->gram || !ext->coef || !ext->bar)
            return (int)cudaErrorInvalidValue;
        pre = HcPre{ext->pre_scale, ext->pre_base, ext->pre_ln_w, ext->pre_post, ext->pre_comb, ext->pre_x,
                    SplitBuf{(uint16_t*)ext->xs_base, (int)ext->xs_ld, (int)ext->xs_plane, (int)ext->xs_mask},
                    ext->gram, ext->coef, (unsigned*)ext->bar, ext->rms_eps, ext->hc_eps, (int)ext->iters};
    }
    const uint16_t* base = (const uint16_t*)xs;
    const uint16_t* hi = base ? base + (fp8 ? 2 * xs_plane : 0) : nullptr;
    const uint16_t* lo = hi ? hi + xs_plane : nullptr;
    const int nkb = (int)(K / kb);
    const int t16 = (int)((N + 15) / 16);
    // tile shape: every CTA of the grid must be resident at once (148 SMs x CTAs per SM of the bounds)
    int shape;  // 0: <1,16> (2 per SM), 1: <1,8> (4 per SM), 2: <2,8> (2 per SM)
    if (nkb >= 64 && t16 <= 256) shape = 0;
    else if (t16 <= 512) shape = 1;
    else if ((N + 31) / 32 <= 256) shape = 2;
    else return (int)cudaErrorInvalidValue;
#define AR_ARGS (const uint8_t*)W, scales, hi, lo, (int)xs_ld, y, (int)ldo, (int)m, (int)N, (int)K, (int)accumulate, \
                (int)store_y, t, (uint32_t*)epoch, (unsigned*)ticket, status, (int)rank, (int)world, (int)max_elems, (int)max_spins, (int)kMaxTiles, hc, g_fb_l2_ahead, xsrc, pre
#define AR_SHAPES(F8, SW)                                                       \
    do {                                                                        \
        if (shape == 0) launch_ar<1, 16, F8, SW>((int)N, st, AR_ARGS);          \
        else if (shape == 1) launch_ar<1, 8, F8, SW>((int)N, st, AR_ARGS);      \
        else launch_ar<2, 8, F8, SW>((int)N, st, AR_ARGS);                      \
    } while (0)
    if (fp8) { if (swiglu) AR_SHAPES(true, true); else AR_SHAPES(true, false); }
    else { if (swiglu) AR_SHAPES(false, true); else AR_SHAPES(false, false); }
#undef AR_SHAPES
#undef AR_ARGS
    return FB_LAUNCH_CHECK();
}
