// Decode context parallel (DCP) merge of sparse-attention partials, inside the attention epilogue.
//
// Every rank of the DCP group ran fb_dsa_attn_partial over the GLOBAL top-k index list but only
// over the pages it owns (page % n_dcp == d), leaving split-K partials (o, m, l) per row and head.
// This kernel finishes the attention in ONE launch per layer:
//   1. merge the rank's own split-K partials (max-shifted, un-normalised),
//   2. push (o[DL], m, l) of every (row, head) into slot `rank` of every peer's staging buffer
//      with 16-byte peer stores over NVLink,
//   3. publish: CTAs fence at GPU scope and take a ticket; the CTA that takes the last ticket
//      fences at system scope once and stamps the epoch on every peer,
//   4. wait (bounded) for all ranks' stamps on the local flag words,
//   5. merge across ranks in rank order:  M = max m_r,  ctx = sum o_r e^{m_r - M} / sum l_r e^{m_r - M}.
// The grid (heads x rows CTAs of 128 threads) must be co-resident; the host checks that.
// On a timeout the kernel writes {TIMEOUT, peer, epoch, -3} to the status word, leaves the
// rank-local result in ctx and returns.
// GPU counterpart of the reference's CPU-only DCP (crates/ferrite-kernel/src/dcp.rs:49-174;
// crates/ferrite-exec/src/distributed.rs:473-).
#include "common.cuh"
#include "mma_gemv.cuh"

namespace {

constexpr int kMaxWorld = 8;

struct DcpTables {
    float* staging[kMaxWorld];   // [2][world][max_rows * heads * (DL + 4)]
    uint32_t* flags[kMaxWorld];  // [2][world] padded to 32 words each
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

// grid (heads, rows), 128 threads; DL % 4 == 0, DL <= 512.
__global__ void __launch_bounds__(128)
dsa_merge_dcp_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, float* __restrict__ ctx,
                     int hl, int DL, int nsplit, DcpTables t, uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket,
                     int* __restrict__ status, int rank, int world, int slot_elems, int max_spins, SplitBuf osp) {
    PDL_PROLOGUE();
    __shared__ int s_fail;
    __shared__ float s_ml[kMaxWorld][2];
    const int r = blockIdx.y, h = blockIdx.x;
    const int rec = DL + 4;                                   // record: o[DL], m, l, pad, pad
    const size_t rec_off = ((size_t)r * hl + h) * rec;
    const uint32_t e = epoch[0] + 1u;
    const int par = e & 1u;
    if (threadIdx.x == 0) s_fail = 0;
    // 1. local split-K merge (un-normalised)
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml_part[(((size_t)r * nsplit + s) * hl + h) * 2]);
    float L = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float* ml = ml_part + (((size_t)r * nsplit + s) * hl + h) * 2;
        if (ml[0] != -INFINITY) L += ml[1] * __expf(ml[0] - M);
    }
    float4 mine = make_float4(0.f, 0.f, 0.f, 0.f);
    const int d4 = threadIdx.x * 4;
    if (d4 < DL) {
        for (int s = 0; s < nsplit; ++s) {
            const float ms = ml_part[(((size_t)r * nsplit + s) * hl + h) * 2];
            if (ms != -INFINITY) {
                const float w = __expf(ms - M);
                const float4 o = *reinterpret_cast<const float4*>(o_part + (((size_t)r * nsplit + s) * hl + h) * DL + d4);
                mine.x += o.x * w; mine.y += o.y * w; mine.z += o.z * w; mine.w += o.w * w;
            }
        }
    }
    // 2. push the record to every rank (own slot included)
    for (int p = 0; p < world; ++p) {
        float* dst = t.staging[p] + ((size_t)par * world + rank) * slot_elems + rec_off;
        if (d4 < DL) *reinterpret_cast<float4*>(dst + d4) = mine;
        if (threadIdx.x == 0) *reinterpret_cast<float4*>(dst + DL) = make_float4(M, L, 0.f, 0.f);
    }
    __syncthreads();
    // 3. one publish per launch
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned total = gridDim.x * gridDim.y;
        if (atomicAdd(ticket, 1u) == total - 1u) {
            __threadfence_system();
            for (int p = 0; p < world; ++p) st_release_sys(t.flags[p] + (par * world + rank) * 32, e);
            *ticket = 0u;
            epoch[0] = e;   // every CTA read the old value before it took its ticket
        }
    }
    // 4. bounded wait for every rank's stamp
    if (threadIdx.x < world) {
        const uint32_t* f = t.flags[rank] + (par * world + threadIdx.x) * 32;
        int spins = 0;
        const int budget = fb_spin_budget(status, max_spins);
        while (ld_relaxed_sys(f) < e) {
            if (++spins > budget) {
                if (atomicCAS(&s_fail, 0, 1) == 0) {
                    status[0] = FB_TIMEOUT; status[1] = threadIdx.x; status[2] = (int)e; status[3] = -3;
                }
                break;
            }
            __nanosleep(64);
        }
        (void)ld_acquire_sys(f);
    }
    __syncthreads();
    const bool ok = s_fail == 0;
    // 5. cross-rank merge in rank order
    float Mg = M, Lg = L;
    float4 acc = mine;
    if (ok) {
        if (threadIdx.x < world) {
            const float4 ml = ld_cg_f4(t.staging[rank] + ((size_t)par * world + threadIdx.x) * slot_elems + rec_off + DL);
            s_ml[threadIdx.x][0] = ml.x;
            s_ml[threadIdx.x][1] = ml.y;
        }
        __syncthreads();
        Mg = -INFINITY;
        for (int s = 0; s < world; ++s) Mg = fmaxf(Mg, s_ml[s][0]);
        Lg = 0.f;
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < world; ++s) {
            if (s_ml[s][0] == -INFINITY) continue;
            const float w = __expf(s_ml[s][0] - Mg);
            Lg += s_ml[s][1] * w;
            if (d4 < DL) {
                const float4 o = ld_cg_f4(t.staging[rank] + ((size_t)par * world + s) * slot_elems + rec_off + d4);
                acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
            }
        }
    }
    const float inv = 1.f / (Lg + 1.1920929e-07f);
    if (d4 < DL) {
        float* c = ctx + ((size_t)r * hl + h) * DL + d4;
        c[0] = acc.x * inv; c[1] = acc.y * inv; c[2] = acc.z * inv; c[3] = acc.w * inv;
        split_store(osp, r, h * DL + d4, acc.x * inv);
        split_store(osp, r, h * DL + d4 + 1, acc.y * inv);
        split_store(osp, r, h * DL + d4 + 2, acc.z * inv);
        split_store(osp, r, h * DL + d4 + 3, acc.w * inv);
    }
}

}  // namespace

// o_part [n, nsplit, hl, DL], ml_part [n, nsplit, hl, 2] from fb_dsa_attn_partial (run with this rank's
// shard); ctx [n, hl, DL] gets the attention output over ALL ranks' pages.  slot_elems: floats per
// (parity, rank) staging slot, >= n * hl * (DL + 4).
FB_API int fb_dsa_attn_merge_dcp(const float* o_part, const float* ml_part, float* ctx, int64_t n, int64_t hl,
                                 int64_t DL, int64_t nsplit, const void* const* staging_ptrs,
                                 const void* const* flag_ptrs, void* epoch, void* ticket, int* status, int64_t rank,
                                 int64_t world, int64_t slot_elems, int64_t max_spins, void* s_base, int64_t s_ld,
                                 int64_t s_plane, int64_t s_mask, cudaStream_t st) {
    if ((DL % 4) || DL > 512 || world > kMaxWorld || n * hl * (DL + 4) > slot_elems || n * hl > 148 * 8)
        return (int)cudaErrorInvalidValue;   // all CTAs must be resident at once
    DcpTables t = {};
    for (int i = 0; i < world; ++i) {
        t.staging[i] = (float*)staging_ptrs[i];
        t.flags[i] = (uint32_t*)flag_ptrs[i];
    }
    SplitBuf osp{(uint16_t*)s_base, (int)s_ld, (int)s_plane, (int)s_mask};
    FB_LAUNCH((dsa_merge_dcp_kernel), dim3((unsigned)hl, (unsigned)n), 128, 0, st, o_part, ml_part, ctx, (int)hl, (int)DL,
              (int)nsplit, t, (uint32_t*)epoch, (unsigned*)ticket, status, (int)rank, (int)world, (int)slot_elems,
              (int)max_spins, osp);
    return FB_LAUNCH_CHECK();
}
