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

// Where a row's keys and its query come from.  A source gives the number of keys of row r, the address of key i
// (null = masked) and one adjacent pair of the pre-scaled query.
struct GlmSrc {   // selected tokens of the paged latent cache (GLM DSA)
    const float* qabs; const __nv_bfloat16* lat_cache; const int* idx; int ld_idx; const int* cnt;
    PageViewT pv; int hl, shard, nshard; float scale;
    __device__ int n_keys(int r, const RowMeta&) const { return cnt[r]; }
    __device__ const __nv_bfloat16* key(int r, const RowMeta& m, int i) const {
        const int t = idx[(size_t)r * ld_idx + i];
        if (t < 0) return nullptr;
        if (nshard > 1 && ((t / pv.page_size) % nshard) != shard) return nullptr;   // DCP ownership
        const int pg = pv.table[(size_t)m.slot * pv.max_pages + t / pv.page_size];
        if (pg < 0) return nullptr;                                                  // page not held on this rank
        return lat_cache + ((long long)pg * pv.page_size + (t % pv.page_size)) * DL;
    }
    __device__ float2 q_pair(int r, const RowMeta&, int h, int d) const {
        const float2 v = *reinterpret_cast<const float2*>(qabs + ((size_t)r * hl + h) * DL + d);
        return make_float2(v.x * scale, v.y * scale);
    }
};
struct D4Src {    // DSV41: the row's window positions of the KV ring, then the selected compressed rows; q is rotated here
    const float* q; int ldq; const __nv_bfloat16* ring; int cap, window; const __nv_bfloat16* comp; int ccap;
    const int* idx; int ldi, ktop; const float* freqs; int rd, pos_off, win_mode; float scale;
    __device__ int wpos(const RowMeta& m) const { return win_mode ? m.ctx0 - 1 : m.pos; }
    __device__ int n_win(const RowMeta& m) const { return max(min(wpos(m) + 1, window), 0); }
    __device__ int n_keys(int, const RowMeta& m) const { return n_win(m) + ktop; }
    __device__ const __nv_bfloat16* key(int r, const RowMeta& m, int i) const {
        const int nw = n_win(m);
        if (i < nw) return ring + ((size_t)m.slot * cap + ((wpos(m) - nw + 1 + i) % cap)) * DL;
        const int c = idx[(size_t)r * ldi + (i - nw)];
        return (c >= 0 && c < ccap) ? comp + ((size_t)m.slot * ccap + c) * DL : nullptr;
    }
    __device__ float2 q_pair(int r, const RowMeta& m, int h, int d) const {
        const float2 v = *reinterpret_cast<const float2*>(q + (size_t)r * ldq + (size_t)h * DL + d);
        float a = v.x, b = v.y;
        if (d >= DL - rd) {
            float sn, cs;
            sincosf((float)(m.pos + pos_off) * freqs[(d - (DL - rd)) >> 1], &sn, &cs);
            a = v.x * cs - v.y * sn;
            b = v.x * sn + v.y * cs;
        }
        return make_float2(a * scale, b * scale);
    }
};

template <class Src>
__global__ void __launch_bounds__(256, 1)
attn_partial_tc_kernel(Src src, float* __restrict__ o_part, float* __restrict__ ml_part, const RowMeta* __restrict__ meta,
                       int hl, int nsplit) {
    PDL_PROLOGUE();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* Qh = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [64][QS]
    __nv_bfloat16* Ql = Qh + 64 * QS;                                         // [64][QS]
    __nv_bfloat16* Lt = Ql + 64 * QS;                                         // [TT][QS]
    __nv_bfloat16* Ps = Lt + TT * QS;                                         // [64][PS]
    float* rmax = reinterpret_cast<float*>(Ps + 64 * PS);                    // [2][64]
    float* lsum = rmax + 128;                                                 // [2][64]
    const __nv_bfloat16** tptr = reinterpret_cast<const __nv_bfloat16**>(lsum + 128);   // [TT] key rows, null = masked

    const int r = blockIdx.y, sp = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mt = warp & 3, half = warp >> 2;
    const RowMeta m = meta[r];
    const int n_tok = src.n_keys(r, m);
    const int per = ((n_tok + nsplit - 1) / nsplit + TT - 1) / TT * TT;
    const int lo = sp * per, hi = min(n_tok, lo + per);

    // Q -> bf16 hi / lo, pre-scaled; heads >= hl are zero rows
    for (int i = tid; i < 64 * (DL / 2); i += 256) {
        const int h = i / (DL / 2), d = (i % (DL / 2)) * 2;
        float a = 0.f, b = 0.f;
        if (h < hl) {
            const float2 v = src.q_pair(r, m, h, d);
            a = v.x;
            b = v.y;
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
        if (tid < TT) tptr[tid] = (t0 + tid < hi) ? src.key(r, m, t0 + tid) : nullptr;
        __syncthreads();
        for (int i = tid; i < TT * (DL / 8); i += 256) {   // 16-byte pieces
            const int t = i / (DL / 8), d = (i % (DL / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tptr[t]) v = *reinterpret_cast<const uint4*>(tptr[t] + d);
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
                if (!tptr[tk]) S[j][c] = -INFINITY;
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
        cudaError_t e = cudaFuncSetAttribute(attn_partial_tc_kernel<GlmSrc>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    PageViewT pv{page_table, (int)max_pages, (int)page_size};
    GlmSrc src{qabs, (const __nv_bfloat16*)lat_cache, idx, (int)ld_idx, cnt, pv, (int)hl, (int)shard, (int)nshard, scale};
    FB_LAUNCH((attn_partial_tc_kernel<GlmSrc>), dim3((unsigned)nsplit, (unsigned)n), 256, kSmemBytes, st, src, o_part, ml_part,
              (const RowMeta*)meta, (int)hl, (int)nsplit);
    return FB_LAUNCH_CHECK();
}

namespace {

// DSV41 merge of the tensor-core partials (o [n][nsplit][hl][DL], ml [n][nsplit][hl][2]): max-shifted sum, the sink
// logit joins the denominator, the output gets the inverse rotation.  grid (heads, rows), 128 threads.
__global__ void __launch_bounds__(128)
d4_attn_merge_tc_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, const float* __restrict__ sink,
                        const float* __restrict__ freqs, int rd, const RowMeta* __restrict__ meta, int pos_off, int hl,
                        int nsplit, float* __restrict__ out, int ldo, SplitBuf osp) {
    PDL_PROLOGUE();
    const int h = blockIdx.x, r = blockIdx.y;
    auto ml = [&](int s) { return ml_part + (((size_t)r * nsplit + s) * hl + h) * 2; };
    float M = -1e30f;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml(s)[0]);
    float den = __expf(sink[h] - M);
    for (int s = 0; s < nsplit; ++s) den += ml(s)[1] * __expf(ml(s)[0] - M);
    const float inv = 1.f / den;
    const float pos = (float)(meta[r].pos + pos_off);
    for (int e = 2 * threadIdx.x; e < DL; e += 2 * blockDim.x) {
        float a = 0.f, b = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float w = __expf(ml(s)[0] - M);
            if (w != 0.f) {   // an empty split holds no data
                const float2 o = *reinterpret_cast<const float2*>(o_part + (((size_t)r * nsplit + s) * hl + h) * DL + e);
                a = fmaf(o.x, w, a);
                b = fmaf(o.y, w, b);
            }
        }
        a *= inv; b *= inv;
        float x0 = a, x1 = b;
        if (e >= DL - rd) {
            float sn, cs;
            sincosf(pos * freqs[(e - (DL - rd)) >> 1], &sn, &cs);
            x0 = a * cs + b * sn;    // inverse rotation
            x1 = -a * sn + b * cs;
        }
        float* o = out + (size_t)r * ldo + (size_t)h * DL + e;
        o[0] = x0;
        o[1] = x1;
        split_store(osp, r, h * DL + e, x0);
        split_store(osp, r, h * DL + e + 1, x1);
    }
}

}  // namespace

// DSV41 sparse attention with a sink on the tensor cores: head_dim 512, up to 64 heads, keys = the row's window
// positions of the ring + the selected compressed rows (no extra rows).  o_part: n * nsplit * heads * 512 floats,
// ml_part: n * nsplit * heads * 2 floats; q is un-rotated, out gets the inverse rotation.
FB_API int fb_d4_sparse_attn_tc(const float* q, int64_t ldq, const void* ring, int64_t cap, int64_t window, const void* comp,
                                int64_t ccap, const int* idx, int64_t ldi, int64_t ktop, const float* sink, const float* freqs,
                                int64_t rd, const void* meta, int64_t pos_off, int64_t win_mode, float scale, int64_t heads,
                                float* out, int64_t ldo, int64_t n, int64_t nsplit, float* o_part, float* ml_part,
                                void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if (heads < 1 || heads > 64 || nsplit < 1 || (rd % 2) || rd > DL || (ldq % 2)) return (int)cudaErrorInvalidValue;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_partial_tc_kernel<D4Src>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    if (!idx) ktop = 0;
    D4Src src{q, (int)ldq, (const __nv_bfloat16*)ring, (int)cap, (int)window, (const __nv_bfloat16*)comp, (int)ccap, idx,
              (int)ldi, (int)ktop, freqs, (int)rd, (int)pos_off, (int)win_mode, scale};
    FB_LAUNCH((attn_partial_tc_kernel<D4Src>), dim3((unsigned)nsplit, (unsigned)n), 256, kSmemBytes, st, src, o_part, ml_part,
              (const RowMeta*)meta, (int)heads, (int)nsplit);
    int rc = FB_LAUNCH_CHECK();
    if (rc) return rc;
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    FB_LAUNCH((d4_attn_merge_tc_kernel), dim3((unsigned)heads, (unsigned)n), 128, 0, st, o_part, ml_part, sink, freqs, (int)rd,
              (const RowMeta*)meta, (int)pos_off, (int)heads, (int)nsplit, out, (int)ldo, osp);
    return FB_LAUNCH_CHECK();
}
