// DSA (DeepSeek sparse attention) for GLM-5.3-Flash: paged latent KV cache, k-pool
// indexer, top-k selection and sparse MLA attention in its weight-absorbed latent form.
//
// Reference math: crates/ferrite-exec/src/lib.rs:717-1040 and
// crates/ferrite-kernel/src/cpu.rs:375-524.  The reference caches per-head K and V
// (64 x 512 values per token); here only the normalised 512-wide latent is cached and
// kv_b is absorbed into the query (q_abs[h] = Wk_h^T q_h) and the output
// (o_h = Wv_h ctx_h), which is the same function and 64x less cache traffic.
// Replaces dsa_cache_append*, quant_kv, kpool_compress*, pool_expand*, indexer_topk*,
// layernorm_affine, sparse_attn_v2*, sparse_attn_*_split, sparse_attn_merge
// (kernels/cuda/ferrite_kernels.cu:1557-2296,6465-7871).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

struct PageView {
    const int* table;  // [slots][max_pages]
    int max_pages;
    int page_size;
};

__device__ __forceinline__ size_t tok_index(const PageView& pv, int slot, int pos) {
    const int pg = pv.table[(size_t)slot * pv.max_pages + pos / pv.page_size];
    return (size_t)pg * pv.page_size + (pos % pv.page_size);
}

template <typename T> __device__ __forceinline__ void st_kv(T* p, float v);
template <> __device__ __forceinline__ void st_kv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_kv<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// proj row = [qa_raw (QL) | latent_raw (DL) | ki_raw (ID) | wi_raw (IH) | kg (ID)]
template <typename KVT>
__global__ void __launch_bounds__(512)
dsa_prep_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ qa_ln,
                const float* __restrict__ kv_ln, const float* __restrict__ kn_w,
                const float* __restrict__ kn_b, float* __restrict__ qa_out, float* __restrict__ wi_out,
                KVT* __restrict__ lat_cache, float* __restrict__ kidx_cache, float* __restrict__ kgate_cache,
                const RowMeta* __restrict__ meta, PageView pv, const int* __restrict__ lat_table, int QL, int DL, int ID,
                int IH, float eps, SplitBuf osp) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const RowMeta m = meta[r];
    const float* p = proj + (size_t)r * ld;
    const size_t ti = tok_index(pv, m.slot, m.pos);
    // the latent cache may have a page table of its own (decode context parallel: a rank stores only the latent
    // pages it owns, compactly; entries of the other ranks' pages are negative and the row's latent is not stored)
    long long tl = (long long)ti;
    if (lat_table) {
        const int pg = lat_table[(size_t)m.slot * pv.max_pages + m.pos / pv.page_size];
        tl = pg < 0 ? -1 : (long long)pg * pv.page_size + (m.pos % pv.page_size);
    }
    // q_a RMSNorm
    float ss = 0.f;
    for (int j = threadIdx.x; j < QL; j += blockDim.x) ss += p[j] * p[j];
    ss = block_sum(ss, red);
    float inv = rsqrtf(ss / QL + eps);
    for (int j = threadIdx.x; j < QL; j += blockDim.x) {
        const float o = p[j] * inv * qa_ln[j];
        qa_out[(size_t)r * QL + j] = o;
        split_store(osp, r, j, o);
    }
    // latent RMSNorm -> cache
    const float* pl = p + QL;
    ss = 0.f;
    for (int j = threadIdx.x; j < DL; j += blockDim.x) ss += pl[j] * pl[j];
    ss = block_sum(ss, red);
    inv = rsqrtf(ss / DL + eps);
    if (tl >= 0)
        for (int j = threadIdx.x; j < DL; j += blockDim.x) st_kv(lat_cache + tl * DL + j, pl[j] * inv * kv_ln[j]);
    // indexer key LayerNorm (mean/var) -> cache; gate -> cache; head weights scaled
    const float* pk = pl + DL;
    float s1 = 0.f;
    for (int j = threadIdx.x; j < ID; j += blockDim.x) s1 += pk[j];
    s1 = block_sum(s1, red);
    const float mean = s1 / ID;
    float s2 = 0.f;
    for (int j = threadIdx.x; j < ID; j += blockDim.x) { float d = pk[j] - mean; s2 += d * d; }
    s2 = block_sum(s2, red);
    inv = rsqrtf(s2 / ID + eps);
    const float* pw = pk + ID;
    const float* pg = pw + IH;
    for (int j = threadIdx.x; j < ID; j += blockDim.x) {
        kidx_cache[ti * ID + j] = (pk[j] - mean) * inv * kn_w[j] + kn_b[j];
        kgate_cache[ti * ID + j] = pg[j];
    }
    const float wscale = rsqrtf((float)IH);
    for (int j = threadIdx.x; j < IH; j += blockDim.x) wi_out[(size_t)r * IH + j] = pw[j] * wscale;
}

// Recompute the pooled key of the pool that holds this row's token from the tokens that
// exist (t < total).  Rows of one pool write identical values.
__global__ void dsa_pool_kernel(const float* __restrict__ kidx_cache, const float* __restrict__ kgate_cache,
                                const float* __restrict__ ape, float* __restrict__ pool_cache,
                                const RowMeta* __restrict__ meta, PageView pv, int ID, int kpool) {
    PDL_PROLOGUE();
    const RowMeta m = meta[blockIdx.x];
    const int p = m.pos / kpool;
    const int ppp = pv.page_size / kpool;  // pools per page
    const int pg = pv.table[(size_t)m.slot * pv.max_pages + p / ppp];
    float* dst = pool_cache + ((size_t)pg * ppp + (p % ppp)) * ID;
    for (int d = threadIdx.x; d < ID; d += blockDim.x) {
        float mx = -INFINITY;
        for (int j = 0; j < kpool; ++j) {
            const int t = p * kpool + j;
            if (t < m.total) mx = fmaxf(mx, kgate_cache[tok_index(pv, m.slot, t) * ID + d] + ape[j * ID + d]);
        }
        float den = 0.f, num = 0.f;
        for (int j = 0; j < kpool; ++j) {
            const int t = p * kpool + j;
            if (t < m.total) {
                const size_t ti = tok_index(pv, m.slot, t);
                const float w = __expf(kgate_cache[ti * ID + d] + ape[j * ID + d] - mx);
                den += w;
                num += w * kidx_cache[ti * ID + d];
            }
        }
        dst[d] = num / den;
    }
}

// scores[r][p] = ID^-0.5 * sum_h wi[r][h] * relu(qi[r][h] . pool_key[p]).  A CTA of 128 threads owns kScPools pools;
// thread (pool, head group) covers IH / kScGroups heads of one pool, the groups' partial sums meet in shared memory
// (a decode step scores a few hundred pools: one thread per pool would leave a 4096-FMA chain on 2 % of the GPU).
constexpr int kScPools = 16, kScGroups = 8;
template <int ID>
__global__ void __launch_bounds__(kScPools * kScGroups)
dsa_score_kernel(const float* __restrict__ qi, int ld_qi, const float* __restrict__ wi,
                 const float* __restrict__ pool_cache, float* __restrict__ scores, int ld_sc,
                 const RowMeta* __restrict__ meta, PageView pv, int IH, int kpool) {
    PDL_PROLOGUE();
    extern __shared__ float sq[];  // [IH][ID] then [IH]
    float* sw = sq + IH * ID;
    __shared__ float part[kScGroups][kScPools];
    const int r = blockIdx.y;
    const RowMeta m = meta[r];
    const int npools = (m.total + kpool - 1) / kpool;
    const int nvis = min(npools, m.ctx0 / kpool + m.off + 1);
    if ((int)(blockIdx.x * kScPools) >= nvis) return;
    for (int i = threadIdx.x; i < IH * ID; i += blockDim.x) sq[i] = qi[(size_t)r * ld_qi + i];
    for (int i = threadIdx.x; i < IH; i += blockDim.x) sw[i] = wi[(size_t)r * IH + i];
    __syncthreads();
    const int pl = threadIdx.x % kScPools, hg = threadIdx.x / kScPools;
    const int p = blockIdx.x * kScPools + pl;
    float s = 0.f;
    if (p < nvis) {
        const int ppp = pv.page_size / kpool;
        const int pg = pv.table[(size_t)m.slot * pv.max_pages + p / ppp];
        const float4* src = reinterpret_cast<const float4*>(pool_cache + ((size_t)pg * ppp + (p % ppp)) * ID);
        float4 pk[ID / 4];
#pragma unroll
        for (int i = 0; i < ID / 4; ++i) pk[i] = src[i];
        const int hper = (IH + kScGroups - 1) / kScGroups;
        for (int h = hg * hper; h < min(IH, (hg + 1) * hper); ++h) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + h * ID);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < ID / 4; ++i) {
                const float4 q = q4[i];
                d += q.x * pk[i].x + q.y * pk[i].y + q.z * pk[i].z + q.w * pk[i].w;
            }
            s += sw[h] * fmaxf(d, 0.f);
        }
    }
    part[hg][pl] = s;
    __syncthreads();
    if (hg == 0 && p < nvis) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < kScGroups; ++g) t += part[g][pl];   // fixed order: every rank gets the same bits
        scores[(size_t)r * ld_sc + p] = t * rsqrtf((float)ID);
    }
}

__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Exclusive block scan of a packed pair (lo 16 bits, hi 16 bits); blockDim.x == 1024.
__device__ __forceinline__ uint32_t block_scan_excl(uint32_t v, uint32_t* wsum, uint32_t* total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) wsum[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        uint32_t w = wsum[lane];
        uint32_t winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        wsum[lane] = winc - w;
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return inc - v + wsum[wid];
}

// Per row: choose the top `select_k` visible pools (ties to the lower index), expand them to
// token ids that are complete pools before the causal frontier, then append the frontier
// tail.  Only valid ids are written, in ascending order; cnt[r] is their number.
__global__ void __launch_bounds__(1024)
dsa_select_kernel(const float* __restrict__ scores, int ld_sc, int* __restrict__ idx, int ld_idx,
                  int* __restrict__ cnt, const RowMeta* __restrict__ meta, int kpool, int select_max) {
    PDL_PROLOGUE();
    __shared__ uint32_t hist[256];
    __shared__ uint32_t wsum[32];
    __shared__ uint32_t s_total, s_prefix, s_need, s_below;
    const int r = blockIdx.x;
    const RowMeta m = meta[r];
    const int npools = (m.total + kpool - 1) / kpool;
    const int nvis = min(npools, m.ctx0 / kpool + m.off + 1);
    const int select_k = min(select_max, npools);
    const float* sc = scores + (size_t)r * ld_sc;
    const int vc = m.pos + 1;
    const int tail = vc % kpool;
    const int start = vc - tail;
    const int frontier = start / kpool;  // pools below it are complete and visible

    if (threadIdx.x == 0) s_below = 0;
    __syncthreads();
    uint32_t thr_key = 0;  // select keys > thr_key, plus `need_eq` lowest-index keys == thr_key
    uint32_t need_eq = 0;
    const bool all = nvis <= select_k;
    if (!all) {
        uint32_t prefix = 0, need = (uint32_t)select_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int p = threadIdx.x; p < nvis; p += blockDim.x) {
                const uint32_t k = order_key(sc[p]);
                if ((k & himask) == prefix) atomicAdd(&hist[(k >> shift) & 0xffu], 1u);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                uint32_t acc = 0;
                int b = 255;
                for (; b > 0; --b) {
                    if (acc + hist[b] >= need) break;
                    acc += hist[b];
                }
                s_prefix = prefix | ((uint32_t)b << shift);
                s_need = need - acc;
            }
            __syncthreads();
            prefix = s_prefix;
            need = s_need;
            __syncthreads();
        }
        thr_key = prefix;
        need_eq = need;
    }
    // ordered compaction
    uint32_t run_sel = 0, run_eq = 0;
    for (int base = 0; base < nvis; base += blockDim.x) {
        const int p = base + threadIdx.x;
        uint32_t gt = 0, eq = 0;
        if (p < nvis) {
            if (all) gt = 1;
            else {
                const uint32_t k = order_key(sc[p]);
                gt = k > thr_key;
                eq = k == thr_key;
            }
        }
        const uint32_t ex = block_scan_excl(gt | (eq << 16), wsum, &s_total);
        const uint32_t gt_before = ex & 0xffffu, eq_before = ex >> 16;
        const uint32_t eq_rank = run_eq + eq_before;
        const bool sel = gt || (eq && eq_rank < need_eq);
        const uint32_t sel_before = run_sel + gt_before + (min(eq_rank, need_eq) - min(run_eq, need_eq));
        if (sel && p < frontier) {
            atomicAdd(&s_below, 1u);
            int* o = idx + (size_t)r * ld_idx + (size_t)sel_before * kpool;
            for (int j = 0; j < kpool; ++j) o[j] = p * kpool + j;
        }
        const uint32_t tot = s_total;
        const uint32_t chunk_gt = tot & 0xffffu, chunk_eq = tot >> 16;
        run_sel += chunk_gt + (min(run_eq + chunk_eq, need_eq) - min(run_eq, need_eq));
        run_eq += chunk_eq;
        __syncthreads();
    }
    // Pools are visited in index order, so the selected pools below the frontier come first
    // and their output slots are dense; pools at or past the frontier emit nothing.
    if (threadIdx.x == 0) {
        const int nsel = (int)s_below;
        int* o = idx + (size_t)r * ld_idx + (size_t)nsel * kpool;
        for (int j = 0; j < tail; ++j) o[j] = start + j;
        cnt[r] = nsel * kpool + tail;
    }
}

// ---- sparse attention over the latent cache (weight-absorbed MLA) ------------------------
constexpr int kTT = 16;  // tokens per tile

template <int HLMAX, int DL, typename KVT>
__global__ void __launch_bounds__(256)
dsa_attn_partial_kernel(const float* __restrict__ qabs, const KVT* __restrict__ lat_cache,
                        const int* __restrict__ idx, int ld_idx, const int* __restrict__ cnt,
                        float* __restrict__ o_part, float* __restrict__ ml_part,
                        const RowMeta* __restrict__ meta, PageView pv, int hl, int nsplit,
                        int shard, int nshard, float scale) {
    PDL_PROLOGUE();
    constexpr int QS = DL + 4;                 // padded row stride (floats)
    constexpr int HPT = (HLMAX + 15) / 16;     // heads per thread in the score phase
    constexpr int CPT = (DL >= 256) ? DL / 256 : 1;
    constexpr int ACT = DL / CPT;              // threads that own output columns
    extern __shared__ float sm[];
    float* q_s = sm;                            // [HLMAX][QS]
    float* l_s = q_s + HLMAX * QS;              // [kTT][QS]
    float* p_s = l_s + kTT * QS;                // [kTT][HLMAX]
    float* a_s = p_s + kTT * HLMAX;             // [HLMAX] rescale factors
    __shared__ int tok_s[kTT];
    __shared__ size_t off_s[kTT];

    const int r = blockIdx.y, sp = blockIdx.x;
    const RowMeta m = meta[r];
    const int n_tok = cnt[r];
    const int per = ((n_tok + nsplit - 1) / nsplit + kTT - 1) / kTT * kTT;
    const int lo = sp * per, hi = min(n_tok, lo + per);
    const int tid = threadIdx.x;

    {
        const float4* q4 = reinterpret_cast<const float4*>(qabs + (size_t)r * hl * DL);
#pragma unroll 8
        for (int i = tid; i < hl * DL / 4; i += 256) {
            const int h = (i * 4) / DL, d = (i * 4) % DL;
            *reinterpret_cast<float4*>(q_s + h * QS + d) = __ldg(q4 + i);
        }
    }
    const int t_l = tid % kTT, hg = tid / kTT;  // score phase: token lane, head group
    float mrun[HPT], lrun[HPT];
#pragma unroll
    for (int i = 0; i < HPT; ++i) { mrun[i] = -INFINITY; lrun[i] = 0.f; }
    float acc[HLMAX][CPT];
#pragma unroll
    for (int h = 0; h < HLMAX; ++h)
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[h][c] = 0.f;

    for (int t0 = lo; t0 < hi; t0 += kTT) {
        __syncthreads();
        if (tid < kTT) {
            int t = (t0 + tid < hi) ? idx[(size_t)r * ld_idx + t0 + tid] : -1;
            if (t >= 0 && nshard > 1 && ((t / pv.page_size) % nshard) != shard) t = -1;  // DCP ownership
            if (t >= 0 && pv.table[(size_t)m.slot * pv.max_pages + t / pv.page_size] < 0) t = -1;   // page not held here
            tok_s[tid] = t;
            off_s[tid] = t >= 0 ? tok_index(pv, m.slot, t) * DL : 0;
        }
        __syncthreads();
        {
            constexpr int EPV = 16 / (int)sizeof(KVT);  // elements per 16-byte load
            for (int i = tid; i < kTT * DL / EPV; i += 256) {
                const int t = i / (DL / EPV), d = (i % (DL / EPV)) * EPV;
                float* dst = l_s + t * QS + d;
                if (tok_s[t] >= 0) {
                    const uint4 v = *reinterpret_cast<const uint4*>(lat_cache + off_s[t] + d);
                    if (sizeof(KVT) == 4) {
                        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(&v);
                    } else {
                        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
                        for (int e = 0; e < 4; ++e) { dst[2 * e] = bf16lo(w[e]); dst[2 * e + 1] = bf16hi(w[e]); }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) dst[e] = 0.f;
                }
            }
        }
        __syncthreads();
        // scores
        const bool tvalid = tok_s[t_l] >= 0;
#pragma unroll
        for (int i = 0; i < HPT; ++i) {
            const int h = hg + 16 * i;
            float s = -INFINITY;
            if (h < hl) {
                float d = 0.f;
                const float4* q4 = reinterpret_cast<const float4*>(q_s + h * QS);
                const float4* l4 = reinterpret_cast<const float4*>(l_s + t_l * QS);
#pragma unroll 8
                for (int k = 0; k < DL / 4; ++k) {
                    const float4 a = q4[k], b = l4[k];
                    d += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
                }
                s = tvalid ? d * scale : -INFINITY;
            }
            float mx = s;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mnew = fmaxf(mrun[i], mx);
            const float p = (s == -INFINITY) ? 0.f : __expf(s - mnew);
            float ps = p;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            const float alpha = (mnew == -INFINITY) ? 1.f : __expf(mrun[i] - mnew);
            lrun[i] = lrun[i] * alpha + ps;
            mrun[i] = mnew;
            if (h < hl) {
                p_s[t_l * HLMAX + h] = p;
                if (t_l == 0) a_s[h] = alpha;
            }
        }
        __syncthreads();
        // accumulate
        if (tid < ACT) {
#pragma unroll
            for (int h = 0; h < HLMAX; ++h) {
                if (h < hl) {
                    const float al = a_s[h];
#pragma unroll
                    for (int c = 0; c < CPT; ++c) acc[h][c] *= al;
                }
            }
            for (int t = 0; t < kTT; ++t) {
                float lv[CPT];
#pragma unroll
                for (int c = 0; c < CPT; ++c) lv[c] = l_s[t * QS + tid * CPT + c];
#pragma unroll
                for (int h = 0; h < HLMAX; ++h) {
                    if (h < hl) {
                        const float p = p_s[t * HLMAX + h];
#pragma unroll
                        for (int c = 0; c < CPT; ++c) acc[h][c] = fmaf(p, lv[c], acc[h][c]);
                    }
                }
            }
        }
    }
    // write partials: o_part [n][nsplit][hl][DL] (unnormalised), ml_part [n][nsplit][hl][2]
    float* op = o_part + ((size_t)r * nsplit + sp) * hl * DL;
    if (tid < ACT) {
#pragma unroll
        for (int h = 0; h < HLMAX; ++h)
            if (h < hl)
#pragma unroll
                for (int c = 0; c < CPT; ++c) op[(size_t)h * DL + tid * CPT + c] = acc[h][c];
    }
    if (t_l == 0) {
#pragma unroll
        for (int i = 0; i < HPT; ++i) {
            const int h = hg + 16 * i;
            if (h < hl) {
                float* ml = ml_part + (((size_t)r * nsplit + sp) * hl + h) * 2;
                ml[0] = mrun[i];
                ml[1] = lrun[i];
            }
        }
    }
}

// ctx[r][h][:] = sum_s o_s e^{m_s - M} / (sum_s l_s e^{m_s - M} + eps_f32); optional lse out.
__global__ void dsa_attn_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                      float* __restrict__ ctx, float* __restrict__ lse_out, int hl, int DL,
                                      int nsplit, int normalise, SplitBuf osp) {
    PDL_PROLOGUE();
    __shared__ float w_s[64];     // per-split weight e^{m_s - M} (0 for an empty split); nsplit <= 64
    __shared__ float s_inv;
    const int r = blockIdx.y, h = blockIdx.x;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int s = threadIdx.x; s < nsplit; s += 32) M = fmaxf(M, ml_part[(((size_t)r * nsplit + s) * hl + h) * 2]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = threadIdx.x; s < nsplit; s += 32) {
            const float* ml = ml_part + (((size_t)r * nsplit + s) * hl + h) * 2;
            const float w = (ml[0] != -INFINITY) ? __expf(ml[0] - M) : 0.f;
            w_s[s] = w;
            L += ml[1] * w;
        }
        L = warp_sum(L);
        if (threadIdx.x == 0) {
            s_inv = normalise ? 1.f / (L + 1.1920929e-07f) : 1.f;
            if (lse_out) {
                lse_out[((size_t)r * hl + h) * 2] = M;
                lse_out[((size_t)r * hl + h) * 2 + 1] = L;
            }
        }
    }
    __syncthreads();
    const float inv = s_inv;
    for (int d = threadIdx.x; d < DL; d += blockDim.x) {
        float o = 0.f;
        // 16 splits at a time with every load in flight before the first add (an empty split's partial is never
        // read: it may hold anything)
        for (int s0 = 0; s0 < nsplit; s0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int sp = s0 + j;
                v[j] = (sp < nsplit && w_s[sp] != 0.f) ? o_part[(((size_t)r * nsplit + sp) * hl + h) * DL + d] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) o = fmaf(v[j], s0 + j < nsplit ? w_s[s0 + j] : 0.f, o);
        }
        ctx[((size_t)r * hl + h) * DL + d] = o * inv;
        split_store(osp, r, h * DL + d, o * inv);
    }
}

}  // namespace

static PageView make_pv(const int* table, int64_t max_pages, int64_t page_size) {
    PageView pv;
    pv.table = table; pv.max_pages = (int)max_pages; pv.page_size = (int)page_size;
    return pv;
}

FB_API int fb_dsa_prep(const float* proj, int64_t ld, const float* qa_ln, const float* kv_ln,
                       const float* kn_w, const float* kn_b, float* qa_out, float* wi_out, void* lat_cache,
                       float* kidx_cache, float* kgate_cache, const void* meta, const int* page_table,
                       const int* lat_table, int64_t max_pages, int64_t page_size, int64_t n, int64_t QL, int64_t DL,
                       int64_t ID, int64_t IH, float eps, int64_t kv_f32, void* s_base, int64_t s_ld, int64_t s_plane,
                       int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    PageView pv = make_pv(page_table, max_pages, page_size);
    if (kv_f32)
        FB_LAUNCH((dsa_prep_kernel<float>), n, 512, 0, st, proj, (int)ld, qa_ln, kv_ln, kn_w, kn_b, qa_out, wi_out,
            (float*)lat_cache, kidx_cache, kgate_cache, (const RowMeta*)meta, pv, lat_table, (int)QL, (int)DL, (int)ID, (int)IH, eps, osp);
    else
        FB_LAUNCH((dsa_prep_kernel<__nv_bfloat16>), n, 512, 0, st, proj, (int)ld, qa_ln, kv_ln, kn_w, kn_b, qa_out, wi_out,
            (__nv_bfloat16*)lat_cache, kidx_cache, kgate_cache, (const RowMeta*)meta, pv, lat_table, (int)QL, (int)DL, (int)ID, (int)IH, eps, osp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_dsa_pool(const float* kidx_cache, const float* kgate_cache, const float* ape, float* pool_cache,
                       const void* meta, const int* page_table, int64_t max_pages, int64_t page_size,
                       int64_t n, int64_t ID, int64_t kpool, cudaStream_t st) {
    PageView pv = make_pv(page_table, max_pages, page_size);
    FB_LAUNCH((dsa_pool_kernel), n, 128, 0, st, kidx_cache, kgate_cache, ape, pool_cache, (const RowMeta*)meta, pv, (int)ID, (int)kpool);
    return FB_LAUNCH_CHECK();
}

// scores [n, ld_sc] scratch; max_pools bounds the grid (>= pools of the longest row).
FB_API int fb_dsa_scores(const float* qi, int64_t ld_qi, const float* wi, const float* pool_cache,
                         float* scores, int64_t ld_sc, const void* meta, const int* page_table,
                         int64_t max_pages, int64_t page_size, int64_t n, int64_t IH, int64_t ID,
                         int64_t kpool, int64_t max_pools, cudaStream_t st) {
    PageView pv = make_pv(page_table, max_pages, page_size);
    dim3 grid((unsigned)((max_pools + kScPools - 1) / kScPools), (unsigned)n);
    size_t sm = (size_t)(IH * ID + IH) * sizeof(float);
#define SC_ARGS qi, (int)ld_qi, wi, pool_cache, scores, (int)ld_sc, (const RowMeta*)meta, pv, (int)IH, (int)kpool
    if (ID == 128) FB_LAUNCH((dsa_score_kernel<128>), grid, 128, sm, st, SC_ARGS);
    else if (ID == 32) FB_LAUNCH((dsa_score_kernel<32>), grid, 128, sm, st, SC_ARGS);
    else if (ID == 16) FB_LAUNCH((dsa_score_kernel<16>), grid, 128, sm, st, SC_ARGS);
    else return (int)cudaErrorInvalidValue;
#undef SC_ARGS
    return FB_LAUNCH_CHECK();
}

FB_API int fb_dsa_select(const float* scores, int64_t ld_sc, int* idx, int64_t ld_idx, int* cnt,
                         const void* meta, int64_t n, int64_t kpool, int64_t select_max, cudaStream_t st) {
    FB_LAUNCH((dsa_select_kernel), n, 1024, 0, st, scores, (int)ld_sc, idx, (int)ld_idx, cnt, (const RowMeta*)meta,
                                          (int)kpool, (int)select_max);
    return FB_LAUNCH_CHECK();
}

template <int HLMAX, int DL, typename KVT>
static int launch_attn(const float* qabs, const void* lat, const int* idx, int64_t ld_idx, const int* cnt,
                       float* o_part, float* ml_part, const void* meta, PageView pv, int64_t n, int64_t hl,
                       int64_t nsplit, int64_t shard, int64_t nshard, float scale, cudaStream_t st) {
    constexpr int QS = DL + 4;
    size_t sm = (size_t)(HLMAX * QS + kTT * QS + kTT * HLMAX + HLMAX) * sizeof(float);
    auto k = dsa_attn_partial_kernel<HLMAX, DL, KVT>;
    if (sm > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return (int)e;
    }
    FB_LAUNCH((k), dim3((unsigned)nsplit, (unsigned)n), 256, sm, st, qabs, (const KVT*)lat, idx, (int)ld_idx, cnt, o_part,
        ml_part, (const RowMeta*)meta, pv, (int)hl, (int)nsplit, (int)shard, (int)nshard, scale);
    return FB_LAUNCH_CHECK();
}

// qabs [n, hl, DL]; o_part [n, nsplit, hl, DL]; ml_part [n, nsplit, hl, 2].  With nshard > 1
// only tokens on pages p with p % nshard == shard take part (decode context parallel).
FB_API int fb_dsa_attn_partial(const float* qabs, const void* lat_cache, const int* idx, int64_t ld_idx,
                               const int* cnt, float* o_part, float* ml_part, const void* meta,
                               const int* page_table, int64_t max_pages, int64_t page_size, int64_t n,
                               int64_t hl, int64_t DL, int64_t nsplit, int64_t shard, int64_t nshard,
                               float scale, int64_t kv_f32, cudaStream_t st) {
    PageView pv = make_pv(page_table, max_pages, page_size);
#define AT(HM, D) \
    return kv_f32 ? launch_attn<HM, D, float>(qabs, lat_cache, idx, ld_idx, cnt, o_part, ml_part, meta, pv, n, hl, nsplit, shard, nshard, scale, st) \
                  : launch_attn<HM, D, __nv_bfloat16>(qabs, lat_cache, idx, ld_idx, cnt, o_part, ml_part, meta, pv, n, hl, nsplit, shard, nshard, scale, st)
    if (DL == 512) {
        if (hl <= 16) { AT(16, 512); }
        if (hl <= 64) { AT(64, 512); }
    } else if (DL == 64) {
        if (hl <= 4) { AT(4, 64); }
        if (hl <= 16) { AT(16, 64); }
    }
#undef AT
    return (int)cudaErrorInvalidValue;
}

FB_API int fb_dsa_attn_merge(const float* o_part, const float* ml_part, float* ctx, float* lse_out, int64_t n,
                             int64_t hl, int64_t DL, int64_t nsplit, int64_t normalise, void* s_base, int64_t s_ld,
                             int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    if (nsplit > 64) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((dsa_attn_merge_kernel), dim3((unsigned)hl, (unsigned)n), 128, 0, st, o_part, ml_part, ctx, lse_out, (int)hl,
                                                                           (int)DL, (int)nsplit, (int)normalise, osp);
    return FB_LAUNCH_CHECK();
}
