// Sparse MLA attention over the latent cache on the tensor cores (decode / verify rows).
//
// With the key/value up-projection absorbed into q and o, all heads of a row share ONE key/value
// sequence - the 512-wide latents of the selected tokens - so a row's attention is two small GEMMs:
//   S[heads x tokens] = Q[heads x 512] . L[tokens x 512]^T      P = softmax(S)      O[heads x 512] += P . L
// One CTA = (split of the selected-token list, row).  It keeps Q (bf16 hi + lo, pre-scaled) in shared
// memory, streams 64-token latent tiles (bf16, gathered through the page table; tokens of foreign DCP
// shards are masked), runs both GEMMs with mma.sync m16n8k16 (ldmatrix operands; .trans for the P.L
// product), keeps the online-softmax state in registers and writes the same un-normalised
// (o, m, l) partials as the SIMT kernel, so the split-K merge and the cross-rank DCP merge are shared.
// Warp w owns heads 16*(w&3).. in both GEMMs; in S it takes tokens 32*(w>>2).., in O columns
// 256*(w>>2)...
// The SIMT form of this op was bound by shared-memory bandwidth (215 us per layer at 1k context,
// 64 heads); this form replaces the reference's sparse_attn_v2 / _split kernels
// (kernels/cuda/ferrite_kernels.cu:2159,2296,7648-7792).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

struct PageViewT {
    const int* table;  // [slots][max_pages]
    int max_pages;
    int page_size;
};

constexpr int DL = 512;
constexpr int TT = 64;          // tokens per tile
constexpr int QS = DL + 8;      // padded row (bf16 elements): 16-byte rows of ldmatrix hit different banks
constexpr int PS = TT + 8;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__global__ void __launch_bounds__(256, 1)
dsa_attn_partial_tc_kernel(const float* __restrict__ qabs, const __nv_bfloat16* __restrict__ lat_cache,
                           const int* __restrict__ idx, int ld_idx, const int* __restrict__ cnt,
                           float* __restrict__ o_part, float* __restrict__ ml_part, const RowMeta* __restrict__ meta,
                           PageViewT pv, int hl, int nsplit, int shard, int nshard, float scale) {
    PDL_PROLOGUE();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* Qh = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [64][QS]
    __nv_bfloat16* Ql = Qh + 64 * QS;                                         // [64][QS]
    __nv_bfloat16* Lt = Ql + 64 * QS;                                         // [TT][QS]
    __nv_bfloat16* Ps = Lt + TT * QS;                                         // [64][PS]
    float* rmax = reinterpret_cast<float*>(Ps + 64 * PS);                    // [2][64]
    float* lsum = rmax + 128;                                                 // [2][64]
    long long* toff = reinterpret_cast<long long*>(lsum + 128);              // [TT] element offsets, -1 = masked

    const int r = blockIdx.y, sp = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mt = warp & 3, half = warp >> 2;
    const RowMeta m = meta[r];
    const int n_tok = cnt[r];
    const int per = ((n_tok + nsplit - 1) / nsplit + TT - 1) / TT * TT;
    const int lo = sp * per, hi = min(n_tok, lo + per);

    // Q -> bf16 hi / lo, pre-scaled; heads >= hl are zero rows
    for (int i = tid; i < 64 * (DL / 2); i += 256) {
        const int h = i / (DL / 2), d = (i % (DL / 2)) * 2;
        float a = 0.f, b = 0.f;
        if (h < hl) {
            const float2 v = *reinterpret_cast<const float2*>(qabs + ((size_t)r * hl + h) * DL + d);
            a = v.x * scale;
            b = v.y * scale;
        }
        const __nv_bfloat16 ah = __float2bfloat16_rn(a), bh = __float2bfloat16_rn(b);
        *reinterpret_cast<__nv_bfloat162*>(Qh + h * QS + d) = __nv_bfloat162(ah, bh);
        *reinterpret_cast<__nv_bfloat162*>(Ql + h * QS + d) =
            __nv_bfloat162(__float2bfloat16_rn(a - __bfloat162float(ah)), __float2bfloat16_rn(b - __bfloat162float(bh)));
    }
    float mrun[2] = {-INFINITY, -INFINITY};   // rows g and g + 8 of this warp's head tile
    float lrun[2] = {0.f, 0.f};               // partial over this warp's token half and this lane's columns
    float O[32][4];
#pragma unroll
    for (int j = 0; j < 32; ++j) { O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f; }

    for (int t0 = lo; t0 < hi; t0 += TT) {
        __syncthreads();   // previous tile fully consumed (and Q staged, first time)
        if (tid < TT) {
            int t = (t0 + tid < hi) ? idx[(size_t)r * ld_idx + t0 + tid] : -1;
            if (t >= 0 && nshard > 1 && ((t / pv.page_size) % nshard) != shard) t = -1;   // DCP ownership
            long long off = -1;
            if (t >= 0) {
                const int pg = pv.table[(size_t)m.slot * pv.max_pages + t / pv.page_size];
                off = ((long long)pg * pv.page_size + (t % pv.page_size)) * DL;
            }
            toff[tid] = off;
        }
        __syncthreads();
        for (int i = tid; i < TT * (DL / 8); i += 256) {   // 16-byte pieces
            const int t = i / (DL / 8), d = (i % (DL / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (toff[t] >= 0) v = *reinterpret_cast<const uint4*>(lat_cache + toff[t] + d);
            *reinterpret_cast<uint4*>(Lt + t * QS + d) = v;
        }
        __syncthreads();
        // ---- S = Q . L^T for heads 16*mt.., tokens 32*half.. ----
        float S[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { S[j][0] = S[j][1] = S[j][2] = S[j][3] = 0.f; }
#pragma unroll 4
        for (int ks = 0; ks < DL / 16; ++ks) {
            uint32_t ah[4], al[4], b01[4], b23[4];
            const int arow = mt * 16 + (lane & 15), acol = ks * 16 + (lane >> 4) * 8;
            ldsm_x4(ah, Qh + arow * QS + acol);
            ldsm_x4(al, Ql + arow * QS + acol);
            // B: two token groups of 8 per ldmatrix.x4: lanes 0-7 rows of group 0 (k lo), 8-15 (k hi), 16-31 group 1
            const int brow = half * 32 + (lane >> 4) * 8 + (lane & 7), bcol = ks * 16 + ((lane >> 3) & 1) * 8;
            ldsm_x4(b01, Lt + brow * QS + bcol);
            ldsm_x4(b23, Lt + (brow + 16) * QS + bcol);
            mma_bf16_16816(S[0], ah[0], ah[1], ah[2], ah[3], b01[0], b01[1]);
            mma_bf16_16816(S[1], ah[0], ah[1], ah[2], ah[3], b01[2], b01[3]);
            mma_bf16_16816(S[2], ah[0], ah[1], ah[2], ah[3], b23[0], b23[1]);
            mma_bf16_16816(S[3], ah[0], ah[1], ah[2], ah[3], b23[2], b23[3]);
            mma_bf16_16816(S[0], al[0], al[1], al[2], al[3], b01[0], b01[1]);
            mma_bf16_16816(S[1], al[0], al[1], al[2], al[3], b01[2], b01[3]);
            mma_bf16_16816(S[2], al[0], al[1], al[2], al[3], b23[0], b23[1]);
            mma_bf16_16816(S[3], al[0], al[1], al[2], al[3], b23[2], b23[3]);
        }
        // mask, per-row max over this warp's 32 tokens
        float pm[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int tk = half * 32 + j * 8 + 2 * t4 + (c & 1);
                if (toff[tk] < 0) S[j][c] = -INFINITY;
                pm[c >> 1] = fmaxf(pm[c >> 1], S[j][c]);
            }
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            pm[q] = fmaxf(pm[q], __shfl_xor_sync(0xffffffffu, pm[q], 1));
            pm[q] = fmaxf(pm[q], __shfl_xor_sync(0xffffffffu, pm[q], 2));
        }
        if (t4 == 0) {
            rmax[half * 64 + mt * 16 + g] = pm[0];
            rmax[half * 64 + mt * 16 + g + 8] = pm[1];
        }
        __syncthreads();
        float alpha[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int row = mt * 16 + g + 8 * q;
            const float mnew = fmaxf(mrun[q], fmaxf(rmax[row], rmax[64 + row]));
            alpha[q] = (mnew == -INFINITY) ? 1.f : __expf(mrun[q] - mnew);
            mrun[q] = mnew;
            lrun[q] *= alpha[q];
        }
        // P = exp(S - m) -> bf16 tile in shared memory, partial row sums in registers
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float p[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float mm = mrun[c >> 1];
                p[c] = (S[j][c] == -INFINITY || mm == -INFINITY) ? 0.f : __expf(S[j][c] - mm);
                lrun[c >> 1] += p[c];
            }
            const int col = half * 32 + j * 8 + 2 * t4;
            *reinterpret_cast<__nv_bfloat162*>(Ps + (mt * 16 + g) * PS + col) = __floats2bfloat162_rn(p[0], p[1]);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (mt * 16 + g + 8) * PS + col) = __floats2bfloat162_rn(p[2], p[3]);
        }
        __syncthreads();
        // ---- O = alpha * O + P . L for heads 16*mt.., columns 256*half.. ----
#pragma unroll
        for (int j = 0; j < 32; ++j) { O[j][0] *= alpha[0]; O[j][1] *= alpha[0]; O[j][2] *= alpha[1]; O[j][3] *= alpha[1]; }
#pragma unroll
        for (int kt = 0; kt < TT / 16; ++kt) {
            uint32_t a[4];
            ldsm_x4(a, Ps + (mt * 16 + (lane & 15)) * PS + kt * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int jp = 0; jp < 16; ++jp) {   // two 8-column tiles per ldmatrix
                uint32_t b[4];
                const int trow = kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int col = half * 256 + jp * 16 + (lane >> 4) * 8;
                ldsm_x4_trans(b, Lt + trow * QS + col);
                mma_bf16_16816(O[2 * jp], a[0], a[1], a[2], a[3], b[0], b[1]);
                mma_bf16_16816(O[2 * jp + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
            }
        }
    }
    // ---- partials: o [n][nsplit][hl][DL] un-normalised, ml [n][nsplit][hl][2] ----
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        lrun[q] += __shfl_xor_sync(0xffffffffu, lrun[q], 1);
        lrun[q] += __shfl_xor_sync(0xffffffffu, lrun[q], 2);
    }
    __syncthreads();
    if (t4 == 0) {
        lsum[half * 64 + mt * 16 + g] = lrun[0];
        lsum[half * 64 + mt * 16 + g + 8] = lrun[1];
    }
    float* op = o_part + ((size_t)r * nsplit + sp) * hl * DL;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int h = mt * 16 + g + 8 * q;
        if (h < hl) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int col = half * 256 + j * 8 + 2 * t4;
                *reinterpret_cast<float2*>(op + (size_t)h * DL + col) = make_float2(O[j][2 * q], O[j][2 * q + 1]);
            }
        }
    }
    __syncthreads();
    if (half == 0 && t4 == 0) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int h = mt * 16 + g + 8 * q;
            if (h < hl) {
                float* ml = ml_part + (((size_t)r * nsplit + sp) * hl + h) * 2;
                ml[0] = mrun[q];
                ml[1] = lsum[h] + lsum[64 + h];
            }
        }
    }
}

constexpr size_t kSmemBytes = (size_t)(64 * QS * 2 + TT * QS + 64 * PS) * 2 + 256 * 4 + TT * 8;

}  // namespace

// Same contract as fb_dsa_attn_partial for a bf16 latent cache with DL == 512 and hl <= 64.
FB_API int fb_dsa_attn_partial_tc(const float* qabs, const void* lat_cache, const int* idx, int64_t ld_idx,
                                  const int* cnt, float* o_part, float* ml_part, const void* meta,
                                  const int* page_table, int64_t max_pages, int64_t page_size, int64_t n, int64_t hl,
                                  int64_t latent_dim, int64_t nsplit, int64_t shard, int64_t nshard, float scale,
                                  cudaStream_t st) {
    if (latent_dim != DL || hl < 1 || hl > 64) return (int)cudaErrorInvalidValue;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(dsa_attn_partial_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    PageViewT pv{page_table, (int)max_pages, (int)page_size};
    FB_LAUNCH((dsa_attn_partial_tc_kernel), dim3((unsigned)nsplit, (unsigned)n), 256, kSmemBytes, st, qabs,
              (const __nv_bfloat16*)lat_cache, idx, (int)ld_idx, cnt, o_part, ml_part, (const RowMeta*)meta, pv, (int)hl,
              (int)nsplit, (int)shard, (int)nshard, scale);
    return FB_LAUNCH_CHECK();
}
