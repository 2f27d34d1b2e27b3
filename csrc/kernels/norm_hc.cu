// Row metadata, embedding, RMSNorm family and the manifold-hyper-connection (MHC) chain.
//
// MHC per site (reference crates/ferrite-exec/src/mhc.rs:58-213):
//   r = rsqrt(mean(R_flat^2) + rms_eps);  mixes = (fn . R_flat) * r              (24 values)
//   pre_i = sigmoid(mix_i*s0 + b_i) + eps;  post_i = 2 sigmoid(mix_{4+i}*s1 + b_{4+i})
//   comb = Sinkhorn_20(softmax_rows(mix_{8..}*s2 + b_{8..}) + eps)
//   x = sum_i pre_i R_i  -> rmsnorm -> sublayer -> y;   R'_i = post_i*y + sum_k comb[k][i] R_k
// Here a site is two launches: hc_post_mix (the previous site's hc_post fused with this
// site's split-K mix dots, accumulated with atomics) and hc_pre_apply (coefficients by one
// warp, contraction and the following RMSNorm fused).  Replaces hc_pre_fuse/hc_pre/hc_post/hc_pre_mix_split/hc_pre_rest345/hc_contract
// (kernels/cuda/ferrite_kernels.cu:2370-2679,8001-8451).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

// Every position a forward pass touches derives from the RowMeta written here, so this is the one place
// that enforces the context limit on the device: a group that would run past `max_pos` is moved back so
// that its last row sits on position max_pos - 1 (it overwrites the tail of its OWN sequence, never a
// page-table entry or cache row of another one) and the status word reports FB_BAD_ARG with the slot and
// the offending length.  The host stops a sequence before this point; the clamp is the backstop.
__global__ void prep_rows_kernel(const int* __restrict__ row_slot, const int* __restrict__ row_off,
                                 const int* __restrict__ row_gsize, const int* __restrict__ seq_len,
                                 RowMeta* __restrict__ meta, int n, int max_pos, int* __restrict__ status) {
    PDL_PROLOGUE();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    RowMeta m;
    m.slot = row_slot[r];
    m.off = row_off[r];
    m.gsize = row_gsize[r];
    m.ctx0 = seq_len[m.slot];
    if (m.ctx0 < 0 || m.ctx0 + m.gsize > max_pos) {
        if (status && m.off == 0) { status[0] = FB_BAD_ARG; status[1] = m.slot; status[2] = m.ctx0; status[3] = m.gsize; }
        m.ctx0 = max(0, min(m.ctx0, max_pos - m.gsize));
    }
    m.pos = m.ctx0 + m.off;
    m.total = m.ctx0 + m.gsize;
    m.first = (m.off == 0);
    m.pad = 0;
    meta[r] = m;
}

// seq_len[slot] += (accept ? accept[slot] : gsize) for the first row of each group.
__global__ void advance_rows_kernel(const RowMeta* __restrict__ meta, const int* __restrict__ accept,
                                    int* __restrict__ seq_len, int n) {
    PDL_PROLOGUE();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    RowMeta m = meta[r];
    if (!m.first) return;
    seq_len[m.slot] = m.ctx0 + (accept ? accept[m.slot] : m.gsize);
}

__global__ void embed_expand_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ emb,
                                    float* __restrict__ out, int H, int mult, int vocab) {
    PDL_PROLOGUE();
    const int r = blockIdx.x;
    int id = ids[r];
    id = min(max(id, 0), vocab - 1);
    const __nv_bfloat16* e = emb + (size_t)id * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = __bfloat162float(e[j]);
        for (int c = 0; c < mult; ++c) out[((size_t)r * mult + c) * H + j] = v;
    }
}

// out = rmsnorm(a (+ b)) * w; optionally stores the sum.
__global__ void rmsnorm_kernel(const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ sum_out, const float* __restrict__ w,
                               float* __restrict__ out, int d, int lda, int ldo, float eps, SplitBuf osp) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* red = sh;
    float* buf = sh + 32;
    const int r = blockIdx.x;
    float ss = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = a[(size_t)r * lda + j];
        if (b) v += b[(size_t)r * lda + j];
        buf[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / d + eps);
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = buf[j];
        if (sum_out) sum_out[(size_t)r * lda + j] = v;
        const float o = v * inv * w[j];
        out[(size_t)r * ldo + j] = o;
        split_store(osp, r, j, o);
    }
}

// cat(rmsnorm(embed[id], enorm), rmsnorm(h_prev, hnorm)) -> out [n, 2H]
__global__ void mtp_prep_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ emb,
                                const float* __restrict__ h_prev, const float* __restrict__ enorm,
                                const float* __restrict__ hnorm, float* __restrict__ out, int H,
                                int vocab, float eps, SplitBuf osp) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* red = sh;
    float* buf = sh + 32;
    const int r = blockIdx.x, half = blockIdx.y;
    float ss = 0.f;
    int id = min(max(ids[r], 0), vocab - 1);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = half == 0 ? __bfloat162float(emb[(size_t)id * H + j]) : h_prev[(size_t)r * H + j];
        buf[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / H + eps);
    const float* w = half == 0 ? enorm : hnorm;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float o = buf[j] * inv * w[j];
        out[(size_t)r * 2 * H + (size_t)half * H + j] = o;
        split_store(osp, r, half * H + j, o);
    }
}

constexpr int kMaxMix = 24;
constexpr int kMixGroups = 4;   // the mix rows are split over blockIdx.z
constexpr int kPmThreads = 128; // one float4 column of R per thread -> 512 columns per CTA

// Fused hc_post of one site and hc_mix of the next (n == 4 residual copies):
//   if y:  Rout[r][i][j] = post[r][i]*y[r][j] + sum_k comb[r][k][i] Rin[r][k][j]
//   if fn: acc[r][m] += sum_{i,j} fn[m][i*H + j] * R'[r][i][j];  acc[r][24] += sum R'^2
// grid = (ceil(H/512), n, kMixGroups); every z recomputes R' for its columns (cheap), z == 0
// writes it and owns the sum of squares.  With a mix (several z) Rout must not alias Rin:
// the other z blocks still read Rin.
template <int G>
__global__ void __launch_bounds__(kPmThreads)
hc_post_mix_kernel(const float* Rin, float* Rout, const float* __restrict__ y, const float* __restrict__ post,
                   const float* __restrict__ comb, const float* __restrict__ fn, float* __restrict__ acc,
                   int H, int mix) {
    PDL_PROLOGUE();
    constexpr int PER = (kMaxMix + G - 1) / G;     // mix rows per z block: 6 with four groups, 24 with one
    __shared__ float red[kPmThreads / 32][PER + 1];
    const int r = blockIdx.y, z = blockIdx.z;
    const int j = (blockIdx.x * kPmThreads + threadIdx.x) * 4;
    const bool act = j < H;
    const float* row = Rin + (size_t)r * 4 * H;
    float* orow = Rout + (size_t)r * 4 * H;
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = act ? *reinterpret_cast<const float4*>(row + (size_t)k * H + j) : make_float4(0, 0, 0, 0);
    if (y) {
        const float4 yy = act ? *reinterpret_cast<const float4*>(y + (size_t)r * H + j) : make_float4(0, 0, 0, 0);
        float p[4], c[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = post[r * 4 + i];
#pragma unroll
        for (int i = 0; i < 16; ++i) c[i] = comb[r * 16 + i];
        float4 o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[i].x = p[i] * yy.x; o[i].y = p[i] * yy.y; o[i].z = p[i] * yy.z; o[i].w = p[i] * yy.w;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float ck = c[k * 4 + i];
                o[i].x += ck * v[k].x; o[i].y += ck * v[k].y; o[i].z += ck * v[k].z; o[i].w += ck * v[k].w;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = o[i];
            if (act && z == 0) *reinterpret_cast<float4*>(orow + (size_t)i * H + j) = o[i];
        }
    }
    if (!fn) return;
    const int per = (mix + G - 1) / G;  // <= PER
    const int m0 = z * per;
    float part[PER + 1];
#pragma unroll
    for (int q = 0; q < PER + 1; ++q) part[q] = 0.f;
    if (act) {
#pragma unroll
        for (int q = 0; q < PER; ++q) {
            const int m = m0 + q;
            if (q < per && m < mix) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 f = __ldg(reinterpret_cast<const float4*>(fn + (size_t)m * 4 * H + (size_t)i * H + j));
                    part[q] += v[i].x * f.x + v[i].y * f.y + v[i].z * f.z + v[i].w * f.w;
                }
            }
        }
        if (z == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) part[PER] += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int q = 0; q < PER + 1; ++q) {
        const float s = warp_sum(part[q]);
        if (lane == 0) red[wid][q] = s;
    }
    __syncthreads();
    if (threadIdx.x < PER + 1) {
        const int q = threadIdx.x;
        float s = 0.f;
        for (int w = 0; w < kPmThreads / 32; ++w) s += red[w][q];
        float* a = acc + (size_t)r * (kMaxMix + 1);
        if (q == PER) { if (z == 0) atomicAdd(a + kMaxMix, s); }
        else if (q < per && m0 + q < mix) atomicAdd(a + m0 + q, s);
    }
}

// One block per row: C contraction warps (a thread owns up to two float4 columns, loaded before the first
// barrier) plus one coefficient warp.  After the per-tile partial dots are summed, every contraction thread
// derives the four `pre` weights itself (four sigmoids of the accumulated dots) and contracts right away,
// while the coefficient warp runs the serial part - `post`, the row softmax and the Sinkhorn iterations of
// `comb` - side by side.  The contraction warps meet on a named barrier of their own; a second named
// barrier lets the coefficient warp clear the accumulator only after everyone has read it.
__global__ void __launch_bounds__(1024)
hc_pre_apply_kernel(const float* __restrict__ R, float* __restrict__ acc, const float* __restrict__ scale,
                    const float* __restrict__ base, const float* __restrict__ ln_w,
                    float* __restrict__ x_out, float* __restrict__ xn_out, float* __restrict__ post_out,
                    float* __restrict__ comb_out, int H, int n, float rms_eps, float hc_eps, int iters,
                    SplitBuf osp, const float* __restrict__ part, int* __restrict__ part_n, int part_ld) {
    PDL_PROLOGUE();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int nct = blockDim.x - 32;
    const bool coef_warp = (int)threadIdx.x >= nct;
    const float* row = R + (size_t)r * n * H;
    float4 v[2][4], lw[2];
    bool act[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int j = (threadIdx.x + c * nct) * 4;
        act[c] = !coef_warp && j < H;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            v[c][k] = act[c] ? *reinterpret_cast<const float4*>(row + (size_t)k * H + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        lw[c] = act[c] ? *reinterpret_cast<const float4*>(ln_w + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (part_n) {
        // per-tile partial mix dots left by a fused GEMV epilogue: one warp per dot sums the tiles
        const int nt = part_n[r];
        if (nt > 0) {
            const int lane = threadIdx.x & 31;
            for (int o = threadIdx.x >> 5; o <= kMaxMix; o += blockDim.x >> 5) {
                const float* pp = part + ((size_t)r * (kMaxMix + 1) + o) * part_ld;
                float sum = 0.f;
                for (int i = lane; i < nt; i += 32) sum += pp[i];
                sum = warp_sum(sum);
                if (lane == 0) acc[(size_t)r * (kMaxMix + 1) + o] += sum;
            }
            __syncthreads();
            if (threadIdx.x == 0) part_n[r] = 0;
        }
    }
    float* a = acc + (size_t)r * (kMaxMix + 1);
    const float rr = rsqrtf(a[kMaxMix] / (float)(n * H) + rms_eps);
    if (coef_warp) {
        const int lane = threadIdx.x & 31;
        if (lane < n) post_out[(size_t)r * n + lane] = 2.f * sigmoidf_(a[n + lane] * rr * scale[1] + base[n + lane]);
        // comb element (i = lane / n, k = lane % n); n == 4 so rows are 4-lane groups
        float c = 0.f;
        const bool on = lane < n * n;
        if (on) c = a[2 * n + lane] * rr * scale[2] + base[2 * n + lane];
        float mx = on ? c : -INFINITY;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float e = on ? __expf(c - mx) : 0.f;
        float den = e + __shfl_xor_sync(0xffffffffu, e, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        c = on ? e / den + hc_eps : 0.f;
        float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        c = __fdividef(c, cs + hc_eps);
        for (int it = 1; it < iters; ++it) {
            float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            c = __fdividef(c, rs + hc_eps);
            cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            c = __fdividef(c, cs + hc_eps);
        }
        if (on) comb_out[(size_t)r * n * n + lane] = c;
        asm volatile("bar.sync 2, %0;" ::"r"((int)blockDim.x) : "memory");   // everyone has read the accumulator
        if (lane <= kMaxMix) a[lane] = 0.f;
        return;
    }
    const float s0 = scale[0];
    const float p0 = sigmoidf_(a[0] * rr * s0 + base[0]) + hc_eps, p1 = sigmoidf_(a[1] * rr * s0 + base[1]) + hc_eps;
    const float p2 = sigmoidf_(a[2] * rr * s0 + base[2]) + hc_eps, p3 = sigmoidf_(a[3] * rr * s0 + base[3]) + hc_eps;
    asm volatile("bar.arrive 2, %0;" ::"r"((int)blockDim.x) : "memory");
    float4 x[2];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        x[c].x = p0 * v[c][0].x + p1 * v[c][1].x + p2 * v[c][2].x + p3 * v[c][3].x;
        x[c].y = p0 * v[c][0].y + p1 * v[c][1].y + p2 * v[c][2].y + p3 * v[c][3].y;
        x[c].z = p0 * v[c][0].z + p1 * v[c][1].z + p2 * v[c][2].z + p3 * v[c][3].z;
        x[c].w = p0 * v[c][0].w + p1 * v[c][1].w + p2 * v[c][2].w + p3 * v[c][3].w;
        if (act[c]) ss += x[c].x * x[c].x + x[c].y * x[c].y + x[c].z * x[c].z + x[c].w * x[c].w;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    asm volatile("bar.sync 1, %0;" ::"r"(nct) : "memory");
    float tot = 0.f;
    for (int w = 0; w < (nct >> 5); ++w) tot += red[w];
    const float inv = rsqrtf(tot / H + rms_eps);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        if (!act[c]) continue;
        const int j = (threadIdx.x + c * nct) * 4;
        if (x_out) *reinterpret_cast<float4*>(x_out + (size_t)r * H + j) = x[c];
        float4 o;
        o.x = x[c].x * inv * lw[c].x; o.y = x[c].y * inv * lw[c].y; o.z = x[c].z * inv * lw[c].z; o.w = x[c].w * inv * lw[c].w;
        *reinterpret_cast<float4*>(xn_out + (size_t)r * H + j) = o;
        split_store(osp, r, j, o.x); split_store(osp, r, j + 1, o.y);
        split_store(osp, r, j + 2, o.z); split_store(osp, r, j + 3, o.w);
    }
}

// Column-parallel hyper-connection front for decode rows, fed by the per-tile partials the fused GEMV + fold kernel
// leaves (24 mix dots, the sum of squares and the 10 Gram dots <R_i, R_j> per tile):
//   CTA (c, r), c < nx : columns [512 c, 512 c + 512) of row r.  15 warps sum one quantity each over the tiles
//                         (all loads in flight, fixed order), every thread derives pre_i = sigmoid(mix_i r s0 + b_i)
//                         + eps and the RMS factor of x from the Gram matrix (|x|^2 = sum_ij pre_i pre_j G_ij), and
//                         writes its column of x = rmsnorm(sum_i pre_i R_i) * w in f32 and split form;
//   CTA (nx, r)         : post and comb of row r (softmax + Sinkhorn), which only the next fold reads, side by side
//                         with the x CTAs.
// No CTA waits for another one, and the serial part (Sinkhorn) is off the path to x.
// e4m3-per-32 round trip with a power-of-two scale (the DSV41 activation quantiser, csrc/kernels/dsv41.cu)
__device__ __forceinline__ float wide_e4m3_rt(float v, float amax) {
    const float t = fmaxf(amax, 1e-4f) * (1.f / 448.f);
    const uint32_t b = __float_as_uint(t);
    const int e = (int)((b >> 23) & 0xff) + ((b & 0x7fffffu) ? 1 : 0);
    const float s = __uint_as_float((uint32_t)min(max(e, 0), 254) << 23);
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v / s, __NV_SATFINITE, __NV_E4M3);
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h)) * s;
}

constexpr int kWideCols = 512;
constexpr int kGramPairs = 10;

__device__ __forceinline__ float tile_sum(const float* __restrict__ src, int nt, int lane) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (lane + 32 * j < nt) ? __ldcg(src + lane + 32 * j) : 0.f;
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) a += v[j];
    return warp_sum(a);
}

__global__ void __launch_bounds__(kWideCols)
hc_pre_wide_kernel(const float* __restrict__ R, const float* __restrict__ part, const float* __restrict__ gram,
                   const int* __restrict__ part_n, int part_ld, const float* __restrict__ scale,
                   const float* __restrict__ base, const float* __restrict__ ln_w, float* __restrict__ xn_out,
                   float* __restrict__ post_out, float* __restrict__ comb_out, int H, int mix, float rms_eps,
                   float hc_eps, int iters, SplitBuf osp, const float* __restrict__ pre_in, float* __restrict__ pre_out,
                   float* __restrict__ xq_out, SplitBuf qsp) {
    // pre_in / pre_out: the offset form of the hyper-connections (the contraction uses the PREVIOUS site's `pre`, given
    // in pre_in; this site's `pre` is only stored for the next one).  xq_out / qsp: also the e4m3-per-32 round trip of
    // the normed row (a warp's 32 columns are one quantisation block).
    PDL_PROLOGUE();
    __shared__ float s_sum[kMaxMix + 1 + kGramPairs];
    const int r = blockIdx.y, nx = gridDim.x - 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nt = min(part_n[r], 512);
    const float* prow = part + (size_t)r * (kMaxMix + 1) * part_ld;
    const float* grow = gram + (size_t)r * kGramPairs * part_ld;
    if ((int)blockIdx.x == nx) {
        // ---- coefficient CTA: all 24 mix dots + the sum of squares, then post / comb ----
        // 16 warps, 25 sums: a warp issues the loads of both of its sums before it reduces either (one L2 round trip)
        for (int q = warp; q <= mix; q += 2 * (kWideCols / 32)) {
            const int q2 = q + kWideCols / 32;
            const int qi = q < mix ? q : kMaxMix, qi2 = q2 < mix ? q2 : kMaxMix;
            const float* s1 = prow + (size_t)qi * part_ld;
            const float* s2 = prow + (size_t)qi2 * part_ld;
            const int nt2 = q2 <= mix ? nt : 0;
            float v1[16], v2[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v1[j] = (lane + 32 * j < nt) ? __ldcg(s1 + lane + 32 * j) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) v2[j] = (lane + 32 * j < nt2) ? __ldcg(s2 + lane + 32 * j) : 0.f;
            float a1 = 0.f, a2 = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) { a1 += v1[j]; a2 += v2[j]; }
            a1 = warp_sum(a1);
            a2 = warp_sum(a2);
            if (lane == 0) {
                s_sum[qi] = a1;
                if (q2 <= mix) s_sum[qi2] = a2;
            }
        }
        __syncthreads();
        if (warp != 0) return;
        const float rr = rsqrtf(s_sum[kMaxMix] / (float)(4 * H) + rms_eps);
        if (lane < 4) post_out[(size_t)r * 4 + lane] = 2.f * sigmoidf_(s_sum[4 + lane] * rr * scale[1] + base[4 + lane]);
        if (pre_out && lane < 4) pre_out[(size_t)r * 4 + lane] = sigmoidf_(s_sum[lane] * rr * scale[0] + base[lane]) + hc_eps;
        float c = 0.f;
        const bool on = lane < 16;
        if (on) c = s_sum[8 + lane] * rr * scale[2] + base[8 + lane];
        float mx = on ? c : -INFINITY;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float e = on ? __expf(c - mx) : 0.f;
        float den = e + __shfl_xor_sync(0xffffffffu, e, 1);
        den += __shfl_xor_sync(0xffffffffu, den, 2);
        c = on ? e / den + hc_eps : 0.f;
        float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        c = __fdividef(c, cs + hc_eps);
        for (int it = 1; it < iters; ++it) {
            float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            c = __fdividef(c, rs + hc_eps);
            cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            c = __fdividef(c, cs + hc_eps);
        }
        if (on) comb_out[(size_t)r * 16 + lane] = c;
        return;
    }
    // ---- x CTA ----
    const int j = blockIdx.x * kWideCols + threadIdx.x;
    const bool act = j < H;
    float rv[4] = {0.f, 0.f, 0.f, 0.f};
    float lw = 0.f;
    if (act) {
#pragma unroll
        for (int k = 0; k < 4; ++k) rv[k] = R[((size_t)r * 4 + k) * H + j];
        lw = __ldg(ln_w + j);
    }
    if (warp < 5 + kGramPairs) {   // mix dots 0..3, the sum of squares, the Gram pairs
        const float* src = warp < 4 ? prow + (size_t)warp * part_ld
                                    : (warp == 4 ? prow + (size_t)kMaxMix * part_ld : grow + (size_t)(warp - 5) * part_ld);
        const float v = tile_sum(src, nt, lane);
        if (lane == 0) s_sum[warp < 4 ? warp : (warp == 4 ? kMaxMix : kMaxMix + 1 + (warp - 5))] = v;
    }
    __syncthreads();
    const float rr = rsqrtf(s_sum[kMaxMix] / (float)(4 * H) + rms_eps);
    float pw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pw[i] = pre_in ? pre_in[(size_t)r * 4 + i] : sigmoidf_(s_sum[i] * rr * scale[0] + base[i]) + hc_eps;
    float xss = 0.f;
    int p = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = i; k < 4; ++k, ++p) xss += (i == k ? 1.f : 2.f) * pw[i] * pw[k] * s_sum[kMaxMix + 1 + p];
    const float inv = rsqrtf(fmaxf(xss, 0.f) / (float)H + rms_eps);
    const float o = act ? (pw[0] * rv[0] + pw[1] * rv[1] + pw[2] * rv[2] + pw[3] * rv[3]) * inv * lw : 0.f;
    if (act) {
        xn_out[(size_t)r * H + j] = o;
        split_store(osp, r, j, o);
    }
    if (xq_out || qsp.base) {
        const float q = wide_e4m3_rt(o, warp_max(fabsf(o)));      // whole warps: H is a multiple of 32
        if (act) {
            if (xq_out) xq_out[(size_t)r * H + j] = q;
            split_store(qsp, r, j, q);
        }
    }
}

// h_final = mean_i R_i ; xn = rmsnorm(h_final) * w
__global__ void hc_head_kernel(const float* __restrict__ R, const float* __restrict__ w,
                               float* __restrict__ h_final, float* __restrict__ xn, int H, int n, float eps,
                               SplitBuf osp) {
    PDL_PROLOGUE();
    extern __shared__ float sh[];
    float* red = sh;
    float* buf = sh + 32;
    const int r = blockIdx.x;
    const float* row = R + (size_t)r * n * H;
    float ss = 0.f;
    const float invn = 1.f / n;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = 0.f;
        for (int i = 0; i < n; ++i) v += row[(size_t)i * H + j];
        v *= invn;
        buf[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        h_final[(size_t)r * H + j] = buf[j];
        const float o = buf[j] * inv * w[j];
        xn[(size_t)r * H + j] = o;
        split_store(osp, r, j, o);
    }
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o, size_t n) {
    PDL_PROLOGUE();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) o[i] = a[i] + b[i];
}

}  // namespace

// max_pos: positions are kept below it (<= 0: no limit); status: 4 ints or null (see the kernel).
FB_API int fb_prep_rows(const int* row_slot, const int* row_off, const int* row_gsize, const int* seq_len,
                        void* meta, int64_t n, int64_t max_pos, int* status, cudaStream_t st) {
    const int lim = max_pos > 0 && max_pos < 0x7fffffff ? (int)max_pos : 0x7fffffff;
    FB_LAUNCH((prep_rows_kernel), (n + 127) / 128, 128, 0, st, row_slot, row_off, row_gsize, seq_len, (RowMeta*)meta, (int)n,
              lim, status);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_advance_rows(const void* meta, const int* accept, int* seq_len, int64_t n, cudaStream_t st) {
    FB_LAUNCH((advance_rows_kernel), (n + 127) / 128, 128, 0, st, (const RowMeta*)meta, accept, seq_len, (int)n);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_embed_expand(const int* ids, const void* emb, float* out, int64_t n, int64_t H, int64_t mult,
                           int64_t vocab, cudaStream_t st) {
    FB_LAUNCH((embed_expand_kernel), n, 256, 0, st, ids, (const __nv_bfloat16*)emb, out, (int)H, (int)mult, (int)vocab);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_rmsnorm(const float* a, const float* b, float* sum_out, const float* w, float* out, int64_t n,
                      int64_t d, int64_t lda, int64_t ldo, float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    size_t sm = (32 + d) * sizeof(float);
    if (sm > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    FB_LAUNCH((rmsnorm_kernel), n, 512, sm, st, a, b, sum_out, w, out, (int)d, (int)lda, (int)ldo, eps, osp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_mtp_prep(const int* ids, const void* emb, const float* h_prev, const float* enorm,
                       const float* hnorm, float* out, int64_t n, int64_t H, int64_t vocab, float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask,
                       cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    size_t sm = (32 + H) * sizeof(float);
    FB_LAUNCH((mtp_prep_kernel), dim3(n, 2), 512, sm, st, ids, (const __nv_bfloat16*)emb, h_prev, enorm, hnorm, out,
                                                  (int)H, (int)vocab, eps, osp);
    return FB_LAUNCH_CHECK();
}

// acc is [n, 25] f32 and must be zero on entry; fb_hc_pre_apply clears it again.
// y == nullptr skips the post update, fn == nullptr skips the mix.
FB_API int fb_hc_post_mix(const float* Rin, float* Rout, const float* y, const float* post, const float* comb,
                          const float* fn, float* acc, int64_t n, int64_t H, int64_t mix, cudaStream_t st) {
    if (mix > kMaxMix || (H % 4) || (y && fn && Rin == Rout)) return (int)cudaErrorInvalidValue;
    // few rows: the mix rows go over four z blocks (each re-reads the row: latency matters, traffic does not);
    // prefill-sized row counts: one block per (columns, row) does all of them and the row is read once
    const bool wide = fn && n < 64;
    dim3 grid((unsigned)((H / 4 + kPmThreads - 1) / kPmThreads), (unsigned)n, wide ? kMixGroups : 1);
    if (wide) FB_LAUNCH((hc_post_mix_kernel<kMixGroups>), grid, kPmThreads, 0, st, Rin, Rout, y, post, comb, fn, acc, (int)H, (int)mix);
    else FB_LAUNCH((hc_post_mix_kernel<1>), grid, kPmThreads, 0, st, Rin, Rout, y, post, comb, fn, acc, (int)H, (int)mix);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_hc_mix(const float* R, const float* fn, float* acc, int64_t n, int64_t D, int64_t mix,
                     cudaStream_t st) {
    return fb_hc_post_mix(R, nullptr, nullptr, nullptr, nullptr, fn, acc, n, D / 4, mix, st);
}

FB_API int fb_hc_pre_apply(const float* R, float* acc, const float* scale, const float* base,
                           const float* ln_w, float* x_out, float* xn_out, float* post_out, float* comb_out,
                           int64_t n, int64_t H, int64_t mult, float rms_eps, float hc_eps, int64_t iters, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask,
                           const float* part, int* part_n, int64_t part_ld, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    if (mult != 4 || (H % 4) || (part_n && n > 64)) return (int)cudaErrorInvalidValue;
    const int nct = (int)(((H / 4 + 1) / 2 + 31) / 32 * 32);   // two float4 columns per contraction thread
    if (nct + 32 > 1024) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((hc_pre_apply_kernel), n, nct + 32, 0, st, R, acc, scale, base, ln_w, x_out, xn_out, post_out, comb_out,
                                               (int)H, (int)mult, rms_eps, hc_eps, (int)iters, osp, part, part_n, (int)part_ld);
    return FB_LAUNCH_CHECK();
}

// Decode-row front from the partials of fb_gemv_ar (part: [n][25][part_ld], gram: [n][10][part_ld], part_n[r] tiles;
// none of them is modified).  n <= 8 rows, mult == 4, at most 512 tiles.
FB_API int fb_hc_pre_wide(const float* R, const float* part, const float* gram, const int* part_n, int64_t part_ld,
                          const float* scale, const float* base, const float* ln_w, float* xn_out, float* post_out,
                          float* comb_out, int64_t n, int64_t H, int64_t mix, float rms_eps, float hc_eps, int64_t iters,
                          void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    if (n < 1 || n > 8 || mix > kMaxMix || mix < 24 || !part || !gram || !part_n) return (int)cudaErrorInvalidValue;
    const unsigned nx = (unsigned)((H + kWideCols - 1) / kWideCols);
    FB_LAUNCH((hc_pre_wide_kernel), dim3(nx + 1, (unsigned)n), kWideCols, 0, st, R, part, gram, part_n, (int)part_ld, scale,
              base, ln_w, xn_out, post_out, comb_out, (int)H, (int)mix, rms_eps, hc_eps, (int)iters, osp,
              (const float*)nullptr, (float*)nullptr, (float*)nullptr, SplitBuf{nullptr, 0, 0, 0});
    return FB_LAUNCH_CHECK();
}

// The same front for the offset form (DSV41): x = rmsnorm(sum_i pre_in[r][i] R_i) * ln_w with the PREVIOUS site's
// coefficients, this site's (pre, post, comb) stored for later; optionally the e4m3-per-32 round trip of x as well
// (xq_out f32 and / or its split planes).  H % 32 == 0.
FB_API int fb_hc_pre_wide_offset(const float* R, const float* part, const float* gram, const int* part_n, int64_t part_ld,
                                 const float* scale, const float* base, const float* ln_w, const float* pre_in,
                                 float* pre_out, float* xn_out, float* post_out, float* comb_out, int64_t n, int64_t H,
                                 int64_t mix, float rms_eps, float hc_eps, int64_t iters, void* s_base, int64_t s_ld,
                                 int64_t s_plane, int64_t s_mask, float* xq_out, void* q_base, int64_t q_ld, int64_t q_plane,
                                 int64_t q_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    SplitBuf qsp{(uint16_t*)q_base, (int)q_ld, (int)q_plane, (int)q_mask};
    if (n < 1 || n > 8 || mix > kMaxMix || mix < 24 || !part || !gram || !part_n || !pre_in || !pre_out || (H % 32))
        return (int)cudaErrorInvalidValue;
    const unsigned nx = (unsigned)((H + kWideCols - 1) / kWideCols);
    FB_LAUNCH((hc_pre_wide_kernel), dim3(nx + 1, (unsigned)n), kWideCols, 0, st, R, part, gram, part_n, (int)part_ld, scale,
              base, ln_w, xn_out, post_out, comb_out, (int)H, (int)mix, rms_eps, hc_eps, (int)iters, osp, pre_in, pre_out,
              xq_out, qsp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_hc_post(float* R, const float* y, const float* post, const float* comb, int64_t n, int64_t H,
                      cudaStream_t st) {
    return fb_hc_post_mix(R, R, y, post, comb, nullptr, nullptr, n, H, 0, st);
}

FB_API int fb_hc_head(const float* R, const float* w, float* h_final, float* xn, int64_t n, int64_t H,
                      int64_t mult, float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    size_t sm = (32 + H) * sizeof(float);
    FB_LAUNCH((hc_head_kernel), n, 512, sm, st, R, w, h_final, xn, (int)H, (int)mult, eps, osp);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_add(const float* a, const float* b, float* o, int64_t n, cudaStream_t st) {
    FB_LAUNCH((add_kernel), (n + 255) / 256, 256, 0, st, a, b, o, (size_t)n);
    return FB_LAUNCH_CHECK();
}
