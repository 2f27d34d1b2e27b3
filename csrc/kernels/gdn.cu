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
