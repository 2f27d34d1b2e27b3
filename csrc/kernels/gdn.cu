// GatedDeltaNet (KDA) linear attention: fused decode / verify / serial-prefill kernel.
//
// One CTA per (head, sequence group) walks the group's rows in order with the head's
// [dk, dv] f32 state held in registers (4*dk threads, dk/4 state rows each).  Per row it
// does everything between the input projections and o_proj:
//   causal depthwise conv (k=4, rolling tail) -> SiLU -> split q,k,v -> L2-norm q,k ->
//   q *= dk^-0.5 -> beta = sigmoid(b) -> decay = exp(lb * sigmoid(exp(A_log)(fb + dt_bias)))
//   S *= decay (rows); u = S^T k; S += beta k (v - u)^T; o = S^T q
//   -> gated RMSNorm with sigmoid(gb) and o_norm.
// For decode-sized groups (<= 8 rows) the kernel can also apply the second halves of the low-rank decay / gate
// projections itself (fb = f_b . f_a_out, gb = g_b . g_a_out: 2 * dk rows of 128 weights per head), which removes
// the GEMV launch that would otherwise sit between the input projection and this kernel.
// State and conv tails live in `nbuf` rotating buffers per sequence slot: with snapshots on
// (MTP verify) the state after row i goes to buffer (cur+1+i) % nbuf, so accepting k rows is
// just cur += k (see fb_mtp_commit) -- no state copy, where the reference restores from
// per-token snapshots with a commit kernel (kernels/cuda/ferrite_kernels.cu:10415,10580).
// Math: crates/ferrite-kernel/src/cpu.rs:207-351, crates/ferrite-exec/src/lib.rs:531-713.
// Replaces gdn_step_v2/v2p, gdn_chunk_batched, gdn_chunk_fused, gdn_prep, conv1d*,
// conv_prep_fused, gated_rmsnorm (ferrite_kernels.cu:345-1042,2743-2850,10123-10415).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

template <int DK>
__global__ void __launch_bounds__(4 * DK)
gdn_fused_kernel(const float* __restrict__ proj, int ld_proj, const float* __restrict__ fb,
                 const float* __restrict__ gb, int ld_fg, const float* __restrict__ conv_w,
                 const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                 const float* __restrict__ o_norm_w, float* __restrict__ state,
                 float* __restrict__ conv_state, const int* __restrict__ cur,
                 const RowMeta* __restrict__ meta, const int* __restrict__ group_first,
                 float* __restrict__ out, int ld_out, int H, int b_off, int nbuf, int snapshots, float lb, float eps,
                 SplitBuf osp, const __nv_bfloat16* __restrict__ fgw, int fa_off, int lr) {
    PDL_PROLOGUE();
    constexpr int RPT = DK / 4;  // state rows per thread
    constexpr int kFgRows = 8;   // rows per group the in-kernel low-rank projection covers
    constexpr int kLrMax = 128;
    __shared__ float qs[DK], ks[DK], vs[DK], dec[DK];
    __shared__ float part[4][DK];
    __shared__ float red[32];
    __shared__ float s_beta;
    __shared__ float fg_s[kFgRows][2][DK];       // [row][f | g][channel]
    __shared__ float fin_s[kFgRows][2 * kLrMax];  // f_a | g_a outputs of the group's rows

    const int h = blockIdx.x;
    const int row0 = group_first[blockIdx.y];
    const RowMeta m0 = meta[row0];
    const int slot = m0.slot, gsize = m0.gsize;
    const int P = H * DK;
    const int tid = threadIdx.x;
    const int c = tid % DK, rg = tid / DK;
    const int cbuf = (nbuf > 1) ? cur[slot] % nbuf : 0;

    const size_t head_elems = (size_t)DK * DK;
    const size_t st_slot = (size_t)nbuf * H * head_elems;
    float* st_base = state + (size_t)slot * st_slot;
    const size_t cv_buf = (size_t)3 * P * 3;
    float* cv_base = conv_state + (size_t)slot * nbuf * cv_buf;

    float s[RPT];
    {
        const float* src = st_base + ((size_t)cbuf * H + h) * head_elems;
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) s[ii] = src[(size_t)(rg * RPT + ii) * DK + c];
    }
    // conv ownership: tid < 3*DK owns channel (part = tid / DK in {q,k,v}, elem = tid % DK)
    const bool conv_owner = tid < 3 * DK;
    const int ch = conv_owner ? (tid / DK) * P + h * DK + (tid % DK) : 0;
    float hist[3] = {0.f, 0.f, 0.f}, cw[4] = {0.f, 0.f, 0.f, 0.f};
    if (conv_owner) {
        const float* t = cv_base + (size_t)cbuf * cv_buf + (size_t)ch * 3;
        hist[0] = t[0]; hist[1] = t[1]; hist[2] = t[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) cw[i] = conv_w[(size_t)ch * 4 + i];
    }
    const float a_exp = __expf(a_log[h]);
    const float qscale = rsqrtf((float)DK);
    const bool own_fg = fgw != nullptr;   // host guarantees gsize <= kFgRows and lr <= kLrMax then
    if (own_fg) {
        // two adjacent lanes share an output channel, each takes half of the low-rank dimension
        const int o = tid >> 1, half = tid & 1;          // o in [0, 2 DK): f channels then g channels
        const int isg = o / DK, e = o % DK;
        const int kh = lr / 2;
        const __nv_bfloat16* wrow = fgw + ((size_t)isg * P + (size_t)h * DK + e) * lr + half * kh;
        // this thread's weights (constant: may be read before the previous kernel's output) go in flight first,
        // then the rows' f_a | g_a outputs are staged
        constexpr int KV = kLrMax / 16;   // 16-byte weight loads per thread
        uint4 wv[KV];
#pragma unroll
        for (int j = 0; j < KV; ++j) wv[j] = (8 * j < kh) ? ldg_nc_v4(wrow + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid; i < gsize * 2 * lr; i += blockDim.x) {
            const int rr = i / (2 * lr), k = i % (2 * lr);
            fin_s[rr][k] = proj[(size_t)(row0 + rr) * ld_proj + fa_off + k];
        }
        __syncthreads();
        float acc[kFgRows];
#pragma unroll
        for (int rr = 0; rr < kFgRows; ++rr) acc[rr] = 0.f;
#pragma unroll
        for (int kj = 0; kj < KV; ++kj) {
            const int k = 8 * kj;
            if (k >= kh) break;
            const uint4 w4 = wv[kj];
            const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
            float wf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { wf[2 * j] = bf16lo(ww[j]); wf[2 * j + 1] = bf16hi(ww[j]); }
#pragma unroll
            for (int rr = 0; rr < kFgRows; ++rr) {
                if (rr < gsize) {
                    const float* xin = &fin_s[rr][isg * lr + half * kh + k];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[rr] = fmaf(wf[j], xin[j], acc[rr]);
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < kFgRows; ++rr) {
            const float tot = acc[rr] + __shfl_xor_sync(0xffffffffu, acc[rr], 1);
            if (half == 0 && rr < gsize) fg_s[rr][isg][e] = tot;
        }
        __syncthreads();
    }

    for (int i = 0; i < gsize; ++i) {
        const int r = row0 + i;
        const float* prow = proj + (size_t)r * ld_proj;
        float val = 0.f;
        if (conv_owner) {
            const float xin = prow[ch];
            val = cw[0] * hist[0] + cw[1] * hist[1] + cw[2] * hist[2] + cw[3] * xin;
            hist[0] = hist[1]; hist[1] = hist[2]; hist[2] = xin;
            val = siluf_(val);
        } else {
            const int e = tid - 3 * DK;
            const float g = (own_fg ? fg_s[i][0][e] : fb[(size_t)r * ld_fg + h * DK + e]) + dt_bias[h * DK + e];
            dec[e] = __expf(lb * sigmoidf_(a_exp * g));
            if (e == 0) s_beta = sigmoidf_(prow[b_off + h]);
        }
        // L2 norms of q (threads [0,DK)) and k (threads [DK,2DK)): warp partials -> red
        float sq = (tid < 2 * DK) ? val * val : 0.f;
        sq = warp_sum(sq);
        __syncthreads();  // previous iteration's readers of qs/ks/vs/part are done
        if ((tid & 31) == 0) red[tid >> 5] = sq;
        __syncthreads();
        if (conv_owner) {
            const int prt = tid / DK;
            if (prt < 2) {
                float tot = 0.f;
                constexpr int WPP = DK / 32;  // warps per part
#pragma unroll
                for (int w = 0; w < WPP; ++w) tot += red[prt * WPP + w];
                const float nrm = sqrtf(tot);
                const float inv = nrm > 0.f ? 1.f / nrm : 0.f;
                if (prt == 0) qs[c] = val * inv * qscale; else ks[c] = val * inv;
            } else {
                vs[c] = val;
            }
        }
        __syncthreads();
        const float beta = s_beta;
        float up = 0.f;
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) {
            const int row = rg * RPT + ii;
            s[ii] *= dec[row];
            up = fmaf(ks[row], s[ii], up);
        }
        part[rg][c] = up;
        __syncthreads();
        const float u = part[0][c] + part[1][c] + part[2][c] + part[3][c];
        const float delta = beta * (vs[c] - u);
        float op = 0.f;
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) {
            const int row = rg * RPT + ii;
            s[ii] = fmaf(ks[row], delta, s[ii]);
            op = fmaf(qs[row], s[ii], op);
        }
        __syncthreads();  // everyone has read part[] (u) before it is reused for o
        part[rg][c] = op;
        __syncthreads();
        float o = 0.f, o2 = 0.f;
        if (rg == 0) {
            o = part[0][c] + part[1][c] + part[2][c] + part[3][c];
            o2 = o * o;
        }
        const float tot = block_sum(o2, red);
        if (rg == 0) {
            const float inv = rsqrtf(tot / DK + eps);
            const float gate = sigmoidf_(own_fg ? fg_s[i][1][c] : gb[(size_t)r * ld_fg + h * DK + c]);
            const float ov = o * inv * o_norm_w[c] * gate;
            out[(size_t)r * ld_out + h * DK + c] = ov;
            split_store(osp, r, h * DK + c, ov);
        }
        const bool last = (i == gsize - 1);
        if ((snapshots && nbuf > 1) || last) {
            const int wb = (snapshots && nbuf > 1) ? (cbuf + 1 + i) % nbuf : cbuf;
            float* dst = st_base + ((size_t)wb * H + h) * head_elems;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) dst[(size_t)(rg * RPT + ii) * DK + c] = s[ii];
            if (conv_owner) {
                float* t = cv_base + (size_t)wb * cv_buf + (size_t)ch * 3;
                t[0] = hist[0]; t[1] = hist[1]; t[2] = hist[2];
            }
        }
    }
}

}  // namespace

// proj [n, ld_proj] holds q|k|v (3P) per row and b (H heads) at column b_off; fb/gb [n, ld_fg] hold the
// decay and output-gate pre-activations (P each).  state [slots][nbuf][H][dk][dk],
// conv_state [slots][nbuf][3P][3].  group_first[g] = first row of group g; rows of a group
// are contiguous and ordered.  snapshots=1 requires gsize < nbuf.
// fg_w (may be null): bf16 [2 * H * dk, lr] = f_b rows then g_b rows.  When given, fb / gb are not read: the kernel
// applies f_b / g_b itself to the f_a | g_a outputs at columns [fa_off, fa_off + 2 lr) of proj; every group must
// then have at most 8 rows (max_gsize) and lr <= 128, lr % 16 == 0.
FB_API int fb_gdn_fused(const float* proj, int64_t ld_proj, const float* fb, const float* gb, int64_t ld_fg,
                        const float* conv_w, const float* a_log, const float* dt_bias,
                        const float* o_norm_w, float* state, float* conv_state, const int* cur,
                        const void* meta, const int* group_first, int64_t n_groups, float* out,
                        int64_t ld_out, int64_t H, int64_t dk, int64_t b_off, int64_t nbuf, int64_t snapshots, float lb,
                        float eps, void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask,
                        const void* fg_w, int64_t fa_off, int64_t lr, int64_t max_gsize, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    if (fg_w && (max_gsize > 8 || lr > 128 || (lr % 16) || lr < 16)) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)H, (unsigned)n_groups);
#define GDN_ARGS proj, (int)ld_proj, fb, gb, (int)ld_fg, conv_w, a_log, dt_bias, o_norm_w, state, conv_state, cur, \
        (const RowMeta*)meta, group_first, out, (int)ld_out, (int)H, (int)b_off, (int)nbuf, (int)snapshots, lb, eps, osp, \
        (const __nv_bfloat16*)fg_w, (int)fa_off, (int)lr
    if (dk == 128) FB_LAUNCH((gdn_fused_kernel<128>), grid, 512, 0, st, GDN_ARGS);
    else if (dk == 64) FB_LAUNCH((gdn_fused_kernel<64>), grid, 256, 0, st, GDN_ARGS);
    else if (dk == 32) FB_LAUNCH((gdn_fused_kernel<32>), grid, 128, 0, st, GDN_ARGS);
    else return (int)cudaErrorInvalidValue;
#undef GDN_ARGS
    return FB_LAUNCH_CHECK();
}

// ---- WY-chunked scan for prefill-sized groups ------------------------------------------------------
// The recurrence above costs a dozen block-wide barriers per token; over a prompt that serial chain is the whole
// cost (2.4 us per token and layer).  Here a CTA (one head of one sequence, state [dk x dv] resident in shared
// memory) advances C = 32 tokens at a time with matrix products (crates/ferrite-kernel/src/wyf.rs:38-147 is the
// reference's statement of the same algebra for its older decay form):
//   L[t]   = sum_{r <= t} g[r]                 per-channel log decay, cumulative inside the chunk (all <= 0)
//   K+ = k * e^{L - Lref},  K- = k * e^{Lref - L},  Q+ = q * e^{L - Lref}      Lref = L[15]: every exponent stays
//                                                                             inside +-80, no overflow for g >= -5
//   Kb = k * e^{L},  Qb = q * e^{L}            the decayed rows that meet the chunk's incoming state S0
//   B  = Kb S0            C = K+ K-^T (strictly lower)        M = Q+ K-^T (lower)
//   W  = (I + diag(beta) C)^-1 diag(beta) (V - B)             forward substitution down the 32 rows, one thread per
//                                                             value channel with its column of W in registers
//   O  = Qb S0 + M W      S_C = diag(e^{L[C-1]}) S0 + diag(e^{L[C-1] - Lref}) K-^T W
// All products are f32 FMAs on register tiles: the state is f32 and the oracle is the step recurrence, so no
// precision is given away to the tensor cores here.  Shared memory bandwidth, not the FMA pipe, bounds a naive
// tiling (one LDS per two FMAs): the tiles below are 4 x 4 (B, O) and 8 x 4 (state) outputs per thread with the
// broadcast operand read four reduction steps at a time (LDS.128), which leaves the FMAs as the longer side.
// B / O run on half of the CTA while the other half builds C and M.
namespace {

constexpr int kWyC = 32;      // tokens per chunk
constexpr int kWyRef = 15;    // reference row of the decay exponents

__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
    return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}
__device__ __forceinline__ float f4c(const float4& a, int i) { return i == 0 ? a.x : i == 1 ? a.y : i == 2 ? a.z : a.w; }

template <int DK>
__global__ void __launch_bounds__(512, 1)
gdn_chunk_kernel(const float* __restrict__ proj, int ld_proj, const float* __restrict__ fb, const float* __restrict__ gb,
                 int ld_fg, const float* __restrict__ conv_w, const float* __restrict__ a_log,
                 const float* __restrict__ dt_bias, const float* __restrict__ o_norm_w, float* __restrict__ state,
                 float* __restrict__ conv_state, const int* __restrict__ cur, const RowMeta* __restrict__ meta,
                 const int* __restrict__ group_first, float* __restrict__ out, int ld_out, int H, int b_off, int nbuf,
                 float lb, float eps, SplitBuf osp) {
    PDL_PROLOGUE();
    constexpr int C = kWyC;
    constexpr int LDK = DK + 4;                      // padded row of K-: float4 reads by 8 lanes hit 32 distinct banks
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                                   // [DK][DK]   state, row = key channel, column = value channel
    float* Qp = S + DK * DK;                         // [C][DK]    Q+
    float* Kp = Qp + C * DK;                         // [C][DK]    K+
    float* Qb = Kp + C * DK;                         // [C][DK]
    float* Kb = Qb + C * DK;                         // [C][DK]
    float* Vb = Kb + C * DK;                         // [C][DK]    v, then beta (v - b)
    float* Bm = Vb + C * DK;                         // [C][DK]    cumulative log decay L, later W
    float* Lb = Bm;
    float* Km = Bm + C * DK;                         // [C][LDK]   K-
    float* Cm = Km + C * LDK;                        // [C][C]     A = diag(beta) C
    float* Mm = Cm + C * C;                          // [C][C]
    float* beta = Mm + C * C;                        // [C]
    float* nq = beta + C;                            // [C]
    float* nk = nq + C;                              // [C]
    float* eref = nk + C;                            // [DK]  e^{Lref}
    float* elast = eref + DK;                        // [DK]  e^{L[C-1] - Lref}

    const int h = blockIdx.x;
    const int row0g = group_first[blockIdx.y];
    const RowMeta m0 = meta[row0g];
    const int slot = m0.slot, gsize = m0.gsize;
    const int P = H * DK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cbuf = (nbuf > 1) ? cur[slot] % nbuf : 0;
    const size_t head_elems = (size_t)DK * DK;
    float* st = state + ((size_t)slot * nbuf + cbuf) * H * head_elems + (size_t)h * head_elems;
    const size_t cv_buf = (size_t)3 * P * 3;
    float* cv = conv_state + ((size_t)slot * nbuf + cbuf) * cv_buf;

    for (int i = tid; i < DK * DK; i += blockDim.x) S[i] = st[i];
    const bool conv_owner = tid < 3 * DK;
    const int ch = conv_owner ? (tid / DK) * P + h * DK + (tid % DK) : 0;
    float hist[3] = {0.f, 0.f, 0.f}, cw[4] = {0.f, 0.f, 0.f, 0.f};
    if (conv_owner) {
        hist[0] = cv[(size_t)ch * 3]; hist[1] = cv[(size_t)ch * 3 + 1]; hist[2] = cv[(size_t)ch * 3 + 2];
#pragma unroll
        for (int i = 0; i < 4; ++i) cw[i] = conv_w[(size_t)ch * 4 + i];
    }
    const float a_exp = __expf(a_log[h]);
    const float qscale = rsqrtf((float)DK);
    // register-tile mappings: (4 rows x 4 columns) of a [C x DK] product, (8 rows x 4 columns) of the state
    constexpr int Q4 = DK / 4;                       // float4 columns per row
    constexpr int NB = (C / 4) * Q4;                 // threads of the B / O tiles (DK = 128: 256)
    const bool rt_on = tid < NB;
    const int rt_t = (tid / Q4) * 4, rt_c = (tid % Q4) * 4;
    constexpr int SG = DK / 8;
    const bool st_on = tid < SG * Q4;
    const int st_i = (tid / Q4) * 8, st_c = (tid % Q4) * 4;

    for (int c0 = 0; c0 < gsize; c0 += C) {
        const int nc = min(C, gsize - c0);
        const int row0 = row0g + c0;
        const int tref = min(kWyRef, nc - 1);
        // ---- A: conv + SiLU, decay prefix sums, beta ----
        // a thread's 32 global loads go in flight together (the serial part is arithmetic on registers)
        if (conv_owner) {
            float xin[C];
#pragma unroll
            for (int t = 0; t < C; ++t) xin[t] = t < nc ? proj[(size_t)(row0 + t) * ld_proj + ch] : 0.f;
            float* dstb = (tid / DK == 0) ? Qp : (tid / DK == 1 ? Kp : Vb);
            const int e = tid % DK;
#pragma unroll
            for (int t = 0; t < C; ++t) {
                float val = 0.f;
                if (t < nc) {
                    val = cw[0] * hist[0] + cw[1] * hist[1] + cw[2] * hist[2] + cw[3] * xin[t];
                    hist[0] = hist[1]; hist[1] = hist[2]; hist[2] = xin[t];
                    val = siluf_(val);
                }
                dstb[t * DK + e] = val;
            }
        } else if (tid < 4 * DK) {
            const int e = tid - 3 * DK;
            float fv[C];
#pragma unroll
            for (int t = 0; t < C; ++t) fv[t] = t < nc ? fb[(size_t)(row0 + t) * ld_fg + h * DK + e] : 0.f;
            float L = 0.f;
            const float db = dt_bias[h * DK + e];
#pragma unroll
            for (int t = 0; t < C; ++t) {
                if (t < nc) L += lb * sigmoidf_(a_exp * (fv[t] + db));
                Lb[t * DK + e] = L;
            }
        }
        if (tid < C) beta[tid] = tid < nc ? sigmoidf_(proj[(size_t)(row0 + tid) * ld_proj + b_off + h]) : 0.f;
        __syncthreads();
        // L2 norms of the q and k rows: warp per (row, q | k)
        for (int w = warp; w < 2 * C; w += (int)(blockDim.x >> 5)) {
            const float* src = (w < C ? Qp : Kp) + (w % C) * DK;
            float ss = 0.f;
            for (int e = lane; e < DK; e += 32) ss += src[e] * src[e];
            ss = warp_sum(ss);
            if (lane == 0) {
                const float nrm = sqrtf(ss);
                (w < C ? nq : nk)[w % C] = nrm > 0.f ? 1.f / nrm : 0.f;
            }
        }
        if (tid < DK) {
            const float lr = Lb[tref * DK + tid];
            eref[tid] = expf(lr);
            elast[tid] = expf(Lb[(nc - 1) * DK + tid] - lr);
        }
        __syncthreads();
        for (int i = tid; i < C * DK; i += blockDim.x) {
            const int t = i / DK, e = i % DK;
            const float d = Lb[i] - Lb[tref * DK + e];
            const float ep = expf(d), em = expf(-d);
            const float ea = ep * eref[e];
            const float kk = Kp[i] * nk[t];
            const float qq = Qp[i] * nq[t] * qscale;
            Qp[i] = qq * ep;
            Kp[i] = kk * ep;
            Qb[i] = qq * ea;
            Kb[i] = kk * ea;
            Km[t * LDK + e] = kk * em;
        }
        __syncthreads();
        // ---- B: b = Kb S0, o1 = Qb S0 on the first NB threads; C and M on the others ----
        float o1[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) o1[r][j] = 0.f;
        if (rt_on) {
            float bt[4][4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j) bt[r][j] = 0.f;
#pragma unroll 1
            for (int i4 = 0; i4 < DK; i4 += 4) {
                float4 kx[4], qx[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    kx[r] = *reinterpret_cast<const float4*>(Kb + (rt_t + r) * DK + i4);
                    qx[r] = *reinterpret_cast<const float4*>(Qb + (rt_t + r) * DK + i4);
                }
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const float4 s4 = *reinterpret_cast<const float4*>(S + (i4 + ii) * DK + rt_c);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float kv = f4c(kx[r], ii), qv = f4c(qx[r], ii);
                        bt[r][0] = fmaf(kv, s4.x, bt[r][0]); bt[r][1] = fmaf(kv, s4.y, bt[r][1]);
                        bt[r][2] = fmaf(kv, s4.z, bt[r][2]); bt[r][3] = fmaf(kv, s4.w, bt[r][3]);
                        o1[r][0] = fmaf(qv, s4.x, o1[r][0]); o1[r][1] = fmaf(qv, s4.y, o1[r][1]);
                        o1[r][2] = fmaf(qv, s4.z, o1[r][2]); o1[r][3] = fmaf(qv, s4.w, o1[r][3]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                // Vb <- beta (v - b)
                float4 v4 = *reinterpret_cast<float4*>(Vb + (rt_t + r) * DK + rt_c);
                const float bb = beta[rt_t + r];
                v4.x = bb * (v4.x - bt[r][0]); v4.y = bb * (v4.y - bt[r][1]);
                v4.z = bb * (v4.z - bt[r][2]); v4.w = bb * (v4.w - bt[r][3]);
                *reinterpret_cast<float4*>(Vb + (rt_t + r) * DK + rt_c) = v4;
            }
        } else {
            // C[t][s] = K+_t . K-_s (s < t),  M[t][s] = Q+_t . K-_s (s <= t); A = beta C.  A thread owns rows
            // (ta, ta + 16) x columns (sb, sb + 16); the (ta, sb + 16) corner is above the diagonal.
            for (int blk = tid - NB; blk < (C / 2) * (C / 2); blk += (int)blockDim.x - NB) {
                const int ta = blk / (C / 2), sb = blk % (C / 2);
                float cc0 = 0.f, cc1 = 0.f, cc2 = 0.f, mm0 = 0.f, mm1 = 0.f, mm2 = 0.f;
#pragma unroll 2
                for (int i4 = 0; i4 < DK; i4 += 4) {
                    const float4 k0 = *reinterpret_cast<const float4*>(Kp + ta * DK + i4);
                    const float4 k1 = *reinterpret_cast<const float4*>(Kp + (ta + C / 2) * DK + i4);
                    const float4 q0 = *reinterpret_cast<const float4*>(Qp + ta * DK + i4);
                    const float4 q1 = *reinterpret_cast<const float4*>(Qp + (ta + C / 2) * DK + i4);
                    const float4 n0 = *reinterpret_cast<const float4*>(Km + sb * LDK + i4);
                    const float4 n1 = *reinterpret_cast<const float4*>(Km + (sb + C / 2) * LDK + i4);
                    cc0 += dot4(k0, n0); mm0 += dot4(q0, n0);
                    cc1 += dot4(k1, n0); mm1 += dot4(q1, n0);
                    cc2 += dot4(k1, n1); mm2 += dot4(q1, n1);
                }
                const int tb = ta + C / 2, sc = sb + C / 2;
                Cm[ta * C + sb] = sb < ta ? beta[ta] * cc0 : 0.f;
                Mm[ta * C + sb] = sb <= ta ? mm0 : 0.f;
                Cm[ta * C + sc] = 0.f;
                Mm[ta * C + sc] = 0.f;
                Cm[tb * C + sb] = beta[tb] * cc1;
                Mm[tb * C + sb] = mm1;
                Cm[tb * C + sc] = sb < ta ? beta[tb] * cc2 : 0.f;
                Mm[tb * C + sc] = sb <= ta ? mm2 : 0.f;
            }
        }
        __syncthreads();
        // ---- C: (I + A) W = U by forward substitution; thread c keeps column c of W in registers ----
        if (tid < DK) {
            float w[C];
#pragma unroll
            for (int t = 0; t < C; ++t) {
                float a0 = Vb[t * DK + tid], a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < t; s4 += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(Cm + t * C + s4);   // same address in every lane
                    a0 = fmaf(-a.x, w[s4], a0);
                    if (s4 + 1 < t) a1 = fmaf(-a.y, w[s4 + 1], a1);
                    if (s4 + 2 < t) a2 = fmaf(-a.z, w[s4 + 2], a2);
                    if (s4 + 3 < t) a3 = fmaf(-a.w, w[s4 + 3], a3);
                }
                w[t] = (a0 + a1) + (a2 + a3);
                Bm[t * DK + tid] = w[t];
            }
        }
        __syncthreads();
        // ---- E: O = o1 + M W, gated RMSNorm, store ----
        if (rt_on) {
#pragma unroll 1
            for (int s4 = 0; s4 < C; s4 += 4) {
                float4 mx[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) mx[r] = *reinterpret_cast<const float4*>(Mm + (rt_t + r) * C + s4);
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const float4 w4 = *reinterpret_cast<const float4*>(Bm + (s4 + ii) * DK + rt_c);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float mv = f4c(mx[r], ii);
                        o1[r][0] = fmaf(mv, w4.x, o1[r][0]); o1[r][1] = fmaf(mv, w4.y, o1[r][1]);
                        o1[r][2] = fmaf(mv, w4.z, o1[r][2]); o1[r][3] = fmaf(mv, w4.w, o1[r][3]);
                    }
                }
            }
            // one row's DK columns are spread over Q4 consecutive threads (a whole warp for DK = 128)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float ss = o1[r][0] * o1[r][0] + o1[r][1] * o1[r][1] + o1[r][2] * o1[r][2] + o1[r][3] * o1[r][3];
#pragma unroll
                for (int off = Q4 / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                const int t = rt_t + r;
                if (t < nc) {
                    const float inv = rsqrtf(ss / DK + eps);
                    const int row = row0 + t;
                    const float4 g4 = *reinterpret_cast<const float4*>(gb + (size_t)row * ld_fg + h * DK + rt_c);
                    const float4 n4 = *reinterpret_cast<const float4*>(o_norm_w + rt_c);
                    float4 ov;
                    ov.x = o1[r][0] * inv * n4.x * sigmoidf_(g4.x);
                    ov.y = o1[r][1] * inv * n4.y * sigmoidf_(g4.y);
                    ov.z = o1[r][2] * inv * n4.z * sigmoidf_(g4.z);
                    ov.w = o1[r][3] * inv * n4.w * sigmoidf_(g4.w);
                    *reinterpret_cast<float4*>(out + (size_t)row * ld_out + h * DK + rt_c) = ov;
                    split_store(osp, row, h * DK + rt_c, ov.x);
                    split_store(osp, row, h * DK + rt_c + 1, ov.y);
                    split_store(osp, row, h * DK + rt_c + 2, ov.z);
                    split_store(osp, row, h * DK + rt_c + 3, ov.w);
                }
            }
        }
        // ---- F: S = diag(e^{L[C-1]}) S0 + diag(elast) K-^T W ----
        if (st_on) {
            float acc[8][4];
#pragma unroll
            for (int r = 0; r < 8; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; acc[r][2] = 0.f; acc[r][3] = 0.f; }
#pragma unroll 2
            for (int s2 = 0; s2 < C; ++s2) {
                const float4 w4 = *reinterpret_cast<const float4*>(Bm + s2 * DK + st_c);
                const float4 ka = *reinterpret_cast<const float4*>(Km + s2 * LDK + st_i);
                const float4 kb = *reinterpret_cast<const float4*>(Km + s2 * LDK + st_i + 4);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float km = r < 4 ? f4c(ka, r) : f4c(kb, r - 4);
                    acc[r][0] = fmaf(km, w4.x, acc[r][0]); acc[r][1] = fmaf(km, w4.y, acc[r][1]);
                    acc[r][2] = fmaf(km, w4.z, acc[r][2]); acc[r][3] = fmaf(km, w4.w, acc[r][3]);
                }
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float el = elast[st_i + r], et = el * eref[st_i + r];
                float4 s4 = *reinterpret_cast<const float4*>(S + (st_i + r) * DK + st_c);
                s4.x = fmaf(s4.x, et, acc[r][0] * el); s4.y = fmaf(s4.y, et, acc[r][1] * el);
                s4.z = fmaf(s4.z, et, acc[r][2] * el); s4.w = fmaf(s4.w, et, acc[r][3] * el);
                *reinterpret_cast<float4*>(S + (st_i + r) * DK + st_c) = s4;
            }
        }
        __syncthreads();
    }
    for (int i = tid; i < DK * DK; i += blockDim.x) st[i] = S[i];
    if (conv_owner) { cv[(size_t)ch * 3] = hist[0]; cv[(size_t)ch * 3 + 1] = hist[1]; cv[(size_t)ch * 3 + 2] = hist[2]; }
}

template <int DK>
constexpr size_t wy_smem() {
    return sizeof(float) * ((size_t)DK * DK + 6 * kWyC * DK + (size_t)kWyC * (DK + 4) + 2 * kWyC * kWyC + 3 * kWyC + 2 * DK);
}

}  // namespace

// Same contract as fb_gdn_fused without snapshots: rows of a group are contiguous and ordered, the group's state
// and conv tail are read from and written to buffer cur % nbuf.  For prefill-sized groups (any size; 32 tokens per
// chunk).  dk: 64 or 128.
FB_API int fb_gdn_chunk(const float* proj, int64_t ld_proj, const float* fb, const float* gb, int64_t ld_fg,
                        const float* conv_w, const float* a_log, const float* dt_bias, const float* o_norm_w, float* state,
                        float* conv_state, const int* cur, const void* meta, const int* group_first, int64_t n_groups,
                        float* out, int64_t ld_out, int64_t H, int64_t dk, int64_t b_off, int64_t nbuf, float lb, float eps,
                        void* s_base, int64_t s_ld, int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    dim3 grid((unsigned)H, (unsigned)n_groups);
#define WY_ARGS proj, (int)ld_proj, fb, gb, (int)ld_fg, conv_w, a_log, dt_bias, o_norm_w, state, conv_state, cur, \
        (const RowMeta*)meta, group_first, out, (int)ld_out, (int)H, (int)b_off, (int)nbuf, lb, eps, osp
    if (dk == 128) {
        static bool done = false;
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wy_smem<128>());
            if (e != cudaSuccess) return (int)e;
            done = true;
        }
        FB_LAUNCH((gdn_chunk_kernel<128>), grid, 512, wy_smem<128>(), st, WY_ARGS);
    } else if (dk == 64) {
        static bool done = false;
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wy_smem<64>());
            if (e != cudaSuccess) return (int)e;
            done = true;
        }
        FB_LAUNCH((gdn_chunk_kernel<64>), grid, 512, wy_smem<64>(), st, WY_ARGS);
    } else {
        return (int)cudaErrorInvalidValue;
    }
#undef WY_ARGS
    return FB_LAUNCH_CHECK();
}
