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
//   S' = diag(e^{Lref}) S0
//   B  = K+ S'            C = K+ K-^T (strictly lower)        M = Q+ K-^T (lower)
//   W  = (I + diag(beta) C)^-1 diag(beta) (V - B)             inverse of a unit lower-triangular 32 x 32 matrix as
//                                                             (I - A)(I + A^2)(I + A^4)(I + A^8)(I + A^16), A nilpotent
//   O  = Q+ S' + M W      S_C = diag(e^{L[C-1] - Lref}) (S' + K-^T W)
// All products are f32 FMAs on register tiles (2 x 4 or 8 x 4 outputs per thread, operands from shared memory): the
// state is f32 and the oracle is the step recurrence, so no precision is given away to the tensor cores here.
// About 4600 FMAs per thread and chunk against 32 x 12 barriers of the serial form.
namespace {

constexpr int kWyC = 32;      // tokens per chunk
constexpr int kWyRef = 15;    // reference row of the decay exponents

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
    constexpr int LDT = C + 1;                       // padded row of the small matrices
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                                   // [DK][DK]   state, row = key channel, column = value channel
    float* Qp = S + DK * DK;                         // [C][DK]
    float* Kp = Qp + C * DK;                         // [C][DK]
    float* Vb = Kp + C * DK;                         // [C][DK]    v, then beta (v - b)
    float* Bm = Vb + C * DK;                         // [C][DK]    b, then w
    float* Lb = Bm + C * DK;                         // [C][DK]    cumulative log decay
    float* KmT = Lb + C * DK;                        // [DK][LDT]  K- transposed
    float* Cm = KmT + DK * LDT;                      // [C][LDT]   A = beta C, then its powers
    float* Mm = Cm + C * LDT;                        // [C][LDT]
    float* Tm = Mm + C * LDT;                        // [C][LDT]   running product -> (I + A)^-1
    float* Xm = Tm + C * LDT;                        // [C][LDT]   scratch
    float* beta = Xm + C * LDT;                      // [C]
    float* nq = beta + C;                            // [C]
    float* nk = nq + C;                              // [C]
    float* eref = nk + C;                            // [DK]
    float* elast = eref + DK;                        // [DK]

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
    // register-tile mappings: (2 rows x 4 columns) of a [C x DK] product, (8 rows x 4 columns) of the state
    constexpr int Q4 = DK / 4;                       // float4 columns per row
    const bool rt_on = tid < (C / 2) * Q4;           // DK = 128: all 512 threads
    const int rt_t = (tid / Q4) * 2, rt_c = (tid % Q4) * 4;
    constexpr int SG = DK / 8;
    const bool st_on = tid < SG * Q4;
    const int st_i = (tid / Q4) * 8, st_c = (tid % Q4) * 4;

    for (int c0 = 0; c0 < gsize; c0 += C) {
        const int nc = min(C, gsize - c0);
        const int row0 = row0g + c0;
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
            const float lr = Lb[min(kWyRef, nc - 1) * DK + tid];
            eref[tid] = expf(lr);
            elast[tid] = expf(Lb[(nc - 1) * DK + tid] - lr);
        }
        __syncthreads();
        for (int i = tid; i < C * DK; i += blockDim.x) {
            const int t = i / DK, e = i % DK;
            const float d = Lb[i] - Lb[min(kWyRef, nc - 1) * DK + e];
            const float ep = expf(d), em = expf(-d);
            const float kk = Kp[i] * nk[t];
            Qp[i] = Qp[i] * nq[t] * qscale * ep;
            Kp[i] = kk * ep;
            KmT[e * LDT + t] = kk * em;
        }
        for (int i = tid; i < DK * DK; i += blockDim.x) S[i] *= eref[i / DK];
        __syncthreads();
        // ---- B: b = K+ S', o1 = Q+ S' (register tiles), C and M ----
        float o1[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        if (rt_on) {
            float bt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
            for (int i = 0; i < DK; ++i) {
                const float4 s4 = *reinterpret_cast<const float4*>(S + i * DK + rt_c);
                const float k0 = Kp[rt_t * DK + i], k1 = Kp[(rt_t + 1) * DK + i];
                const float q0 = Qp[rt_t * DK + i], q1 = Qp[(rt_t + 1) * DK + i];
                bt[0][0] = fmaf(k0, s4.x, bt[0][0]); bt[0][1] = fmaf(k0, s4.y, bt[0][1]);
                bt[0][2] = fmaf(k0, s4.z, bt[0][2]); bt[0][3] = fmaf(k0, s4.w, bt[0][3]);
                bt[1][0] = fmaf(k1, s4.x, bt[1][0]); bt[1][1] = fmaf(k1, s4.y, bt[1][1]);
                bt[1][2] = fmaf(k1, s4.z, bt[1][2]); bt[1][3] = fmaf(k1, s4.w, bt[1][3]);
                o1[0][0] = fmaf(q0, s4.x, o1[0][0]); o1[0][1] = fmaf(q0, s4.y, o1[0][1]);
                o1[0][2] = fmaf(q0, s4.z, o1[0][2]); o1[0][3] = fmaf(q0, s4.w, o1[0][3]);
                o1[1][0] = fmaf(q1, s4.x, o1[1][0]); o1[1][1] = fmaf(q1, s4.y, o1[1][1]);
                o1[1][2] = fmaf(q1, s4.z, o1[1][2]); o1[1][3] = fmaf(q1, s4.w, o1[1][3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                // Vb <- beta (v - b)
                float4 v4 = *reinterpret_cast<float4*>(Vb + (rt_t + r) * DK + rt_c);
                const float bb = beta[rt_t + r];
                v4.x = bb * (v4.x - bt[r][0]); v4.y = bb * (v4.y - bt[r][1]);
                v4.z = bb * (v4.z - bt[r][2]); v4.w = bb * (v4.w - bt[r][3]);
                *reinterpret_cast<float4*>(Vb + (rt_t + r) * DK + rt_c) = v4;
            }
        }
        // C[t][s] = K+_t . K-_s (s < t),  M[t][s] = Q+_t . K-_s (s <= t); A = beta C
        for (int o = tid; o < C * C; o += blockDim.x) {
            const int t = o / C, s2 = o % C;
            float cc = 0.f, mm = 0.f;
            if (s2 <= t) {
#pragma unroll 4
                for (int i = 0; i < DK; ++i) {
                    const float km = KmT[i * LDT + s2];
                    cc = fmaf(Kp[t * DK + i], km, cc);
                    mm = fmaf(Qp[t * DK + i], km, mm);
                }
            }
            const float a = (s2 < t) ? beta[t] * cc : 0.f;
            Cm[t * LDT + s2] = a;
            Mm[t * LDT + s2] = (s2 <= t) ? mm : 0.f;
            Tm[t * LDT + s2] = (s2 == t ? 1.f : 0.f) - a;      // I - A
        }
        __syncthreads();
        // ---- C: (I + A)^-1 = (I - A)(I + A^2)(I + A^4)(I + A^8)(I + A^16) ----
        for (int pw = 0; pw < 4; ++pw) {
            for (int o = tid; o < C * C; o += blockDim.x) {     // X = A A
                const int t = o / C, s2 = o % C;
                float a = 0.f;
#pragma unroll 8
                for (int j = 0; j < C; ++j) a = fmaf(Cm[t * LDT + j], Cm[j * LDT + s2], a);
                Xm[t * LDT + s2] = a;
            }
            __syncthreads();
            for (int o = tid; o < C * C; o += blockDim.x) Cm[(o / C) * LDT + o % C] = Xm[(o / C) * LDT + o % C];
            __syncthreads();
            for (int o = tid; o < C * C; o += blockDim.x) {     // X = T (I + A)
                const int t = o / C, s2 = o % C;
                float a = Tm[t * LDT + s2];
#pragma unroll 8
                for (int j = 0; j < C; ++j) a = fmaf(Tm[t * LDT + j], Cm[j * LDT + s2], a);
                Xm[t * LDT + s2] = a;
            }
            __syncthreads();
            for (int o = tid; o < C * C; o += blockDim.x) Tm[(o / C) * LDT + o % C] = Xm[(o / C) * LDT + o % C];
            __syncthreads();
        }
        // ---- D: W = T U (U in Vb) -> Bm ----
        if (rt_on) {
            float wt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
            for (int s2 = 0; s2 < C; ++s2) {
                const float4 u4 = *reinterpret_cast<const float4*>(Vb + s2 * DK + rt_c);
                const float t0 = Tm[rt_t * LDT + s2], t1 = Tm[(rt_t + 1) * LDT + s2];
                wt[0][0] = fmaf(t0, u4.x, wt[0][0]); wt[0][1] = fmaf(t0, u4.y, wt[0][1]);
                wt[0][2] = fmaf(t0, u4.z, wt[0][2]); wt[0][3] = fmaf(t0, u4.w, wt[0][3]);
                wt[1][0] = fmaf(t1, u4.x, wt[1][0]); wt[1][1] = fmaf(t1, u4.y, wt[1][1]);
                wt[1][2] = fmaf(t1, u4.z, wt[1][2]); wt[1][3] = fmaf(t1, u4.w, wt[1][3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
                *reinterpret_cast<float4*>(Bm + (rt_t + r) * DK + rt_c) = make_float4(wt[r][0], wt[r][1], wt[r][2], wt[r][3]);
        }
        __syncthreads();
        // ---- E: O = o1 + M W, gated RMSNorm, store ----
        if (rt_on) {
#pragma unroll 4
            for (int s2 = 0; s2 < C; ++s2) {
                const float4 w4 = *reinterpret_cast<const float4*>(Bm + s2 * DK + rt_c);
                const float m0 = Mm[rt_t * LDT + s2], m1 = Mm[(rt_t + 1) * LDT + s2];
                o1[0][0] = fmaf(m0, w4.x, o1[0][0]); o1[0][1] = fmaf(m0, w4.y, o1[0][1]);
                o1[0][2] = fmaf(m0, w4.z, o1[0][2]); o1[0][3] = fmaf(m0, w4.w, o1[0][3]);
                o1[1][0] = fmaf(m1, w4.x, o1[1][0]); o1[1][1] = fmaf(m1, w4.y, o1[1][1]);
                o1[1][2] = fmaf(m1, w4.z, o1[1][2]); o1[1][3] = fmaf(m1, w4.w, o1[1][3]);
            }
        }
        // one row's DK columns are spread over Q4 consecutive threads (a whole warp for DK = 128)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float ss = rt_on ? o1[r][0] * o1[r][0] + o1[r][1] * o1[r][1] + o1[r][2] * o1[r][2] + o1[r][3] * o1[r][3] : 0.f;
#pragma unroll
            for (int off = Q4 / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            const int t = rt_t + r;
            if (rt_on && t < nc) {
                const float inv = rsqrtf(ss / DK + eps);
                const int row = row0 + t;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int cidx = rt_c + j;
                    const float gate = sigmoidf_(gb[(size_t)row * ld_fg + h * DK + cidx]);
                    const float ov = o1[r][j] * inv * o_norm_w[cidx] * gate;
                    out[(size_t)row * ld_out + h * DK + cidx] = ov;
                    split_store(osp, row, h * DK + cidx, ov);
                }
            }
        }
        // ---- F: S = diag(elast) (S' + K-^T W) ----
        if (st_on) {
            float acc[8][4];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float4 s4 = *reinterpret_cast<const float4*>(S + (st_i + r) * DK + st_c);
                acc[r][0] = s4.x; acc[r][1] = s4.y; acc[r][2] = s4.z; acc[r][3] = s4.w;
            }
#pragma unroll 2
            for (int s2 = 0; s2 < C; ++s2) {
                const float4 w4 = *reinterpret_cast<const float4*>(Bm + s2 * DK + st_c);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float km = KmT[(st_i + r) * LDT + s2];
                    acc[r][0] = fmaf(km, w4.x, acc[r][0]); acc[r][1] = fmaf(km, w4.y, acc[r][1]);
                    acc[r][2] = fmaf(km, w4.z, acc[r][2]); acc[r][3] = fmaf(km, w4.w, acc[r][3]);
                }
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float el = elast[st_i + r];
                *reinterpret_cast<float4*>(S + (st_i + r) * DK + st_c) =
                    make_float4(acc[r][0] * el, acc[r][1] * el, acc[r][2] * el, acc[r][3] * el);
            }
        }
        __syncthreads();
    }
    for (int i = tid; i < DK * DK; i += blockDim.x) st[i] = S[i];
    if (conv_owner) { cv[(size_t)ch * 3] = hist[0]; cv[(size_t)ch * 3 + 1] = hist[1]; cv[(size_t)ch * 3 + 2] = hist[2]; }
}

template <int DK>
constexpr size_t wy_smem() {
    return sizeof(float) * ((size_t)DK * DK + 5 * kWyC * DK + (size_t)DK * (kWyC + 1) + 4 * kWyC * (kWyC + 1) + 3 * kWyC + 2 * DK);
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
