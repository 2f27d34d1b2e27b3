// Expert-parallel MoE: all-to-all dispatch and combine over NVLink peer memory.
//
// Every rank owns E / world whole experts and `n_loc` token rows of its own.  One MoE layer is
//   route (local)  ->  fb_ep_dispatch  ->  expert gate/up + down over the gathered rows (local experts
//   only: the grouped tensor-core kernels skip slots whose expert lives elsewhere)  ->  fb_ep_combine.
//
// fb_ep_dispatch   each CTA handles one local row: its routing (expert ids, weights: a few bytes) goes into this
//                  rank's row block of every rank's gather buffers, its split activation planes ONLY to the ranks
//                  that own one of its top-k experts (16-byte peer stores): NVLink carries a row once per distinct
//                  owner, not once per rank.  The grid publishes one epoch stamp per peer (GPU-scope fence + ticket,
//                  a single system-scope fence) and waits, bounded, until all ranks' rows have arrived.  A row block
//                  entry whose ids name no local expert keeps stale planes; the expert kernels never read them.
// fb_ep_combine    each CTA pushes one gathered row's partial output (the sum over this rank's experts,
//                  already scaled by the routing weights) back to the rank that owns the token, into
//                  slot `rank` of its staging; publish, bounded wait; the first n_loc CTAs then sum the
//                  owners' slots in rank order (+ an optional local addend, e.g. the shared expert).
// Gather buffers need no double buffering: the combine's wait is a barrier after every rank's expert
// compute, the next dispatch's wait is a barrier after every rank's combine.
// The reference has no all-to-all (its EP mode zero-fills remote slots and all-reduces,
// kernels/cuda/ferrite_kernels.cu:4021; crates/ferrite-exec/src/lib.rs:1083-1166).
#include "common.cuh"

namespace {

constexpr int kMaxWorld = 8;

struct EpPtrs {
    uint16_t* xs[kMaxWorld];     // [planes][world * n_max][H] split activation planes
    int* ids[kMaxWorld];         // [world * n_max][topk]
    float* wts[kMaxWorld];       // [world * n_max][topk]
    float* ybuf[kMaxWorld];      // [world][n_max][H] combine staging
    uint32_t* flags[kMaxWorld];  // [2 phases][world] padded to 32 words
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

// Grid-wide publish + bounded wait shared by both phases.  Returns false after a timeout.
__device__ __forceinline__ bool publish_and_wait(const EpPtrs& t, int phase, uint32_t e, unsigned* ticket, int rank,
                                                 int world, int max_spins, int* status, int* s_fail) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1u) {
            __threadfence_system();
            for (int p = 0; p < world; ++p) st_release_sys(t.flags[p] + (phase * world + rank) * 32, e);
            *ticket = 0u;
        }
    }
    if (threadIdx.x < world) {
        const uint32_t* f = t.flags[rank] + (phase * world + threadIdx.x) * 32;
        int spins = 0;
        const int budget = fb_spin_budget(status, max_spins);
        while (ld_relaxed_sys(f) < e) {
            if (++spins > budget) {
                if (atomicCAS(s_fail, 0, 1) == 0) {
                    status[0] = FB_TIMEOUT; status[1] = threadIdx.x; status[2] = (int)e; status[3] = -10 - phase;
                }
                break;
            }
            __nanosleep(64);
        }
        (void)ld_acquire_sys(f);
    }
    __syncthreads();
    return *s_fail == 0;
}

// grid = n_loc CTAs (>= 1), 256 threads.  xs_local: [planes][n_loc_ld rows][H] planes of the local rows.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint16_t* __restrict__ xs_local, int local_plane, const int* __restrict__ ids,
                   const float* __restrict__ wts, int n_loc, int n_max, int H, int topk, int planes, int e_per_rank,
                   EpPtrs t, uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket, int* __restrict__ status,
                   int rank, int world, int max_spins) {
    PDL_PROLOGUE();
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    const int r = blockIdx.x;
    const uint32_t e = epoch[0] + 1u;
    const size_t gather_plane = (size_t)world * n_max * H;
    const int grow = rank * n_max + r;   // this row's place in every rank's gather buffers
    unsigned owners = 0xffffffffu;          // bit p: rank p owns one of this row's experts
    if (e_per_rank > 0 && r < n_loc) {
        owners = 0u;
        for (int k = 0; k < topk; ++k) {
            const int e = ids[(size_t)r * topk + k];
            if (e >= 0) owners |= 1u << min(e / e_per_rank, 31);
        }
    }
    for (int p = 0; p < world; ++p) {
        if (r < n_loc && ((owners >> p) & 1u)) {
            for (int pl = 0; pl < planes; ++pl) {
                const uint4* src = reinterpret_cast<const uint4*>(xs_local + (size_t)pl * local_plane + (size_t)r * H);
                uint4* dst = reinterpret_cast<uint4*>(t.xs[p] + (size_t)pl * gather_plane + (size_t)grow * H);
                for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
            }
        }
        if (threadIdx.x < topk) {
            t.ids[p][(size_t)grow * topk + threadIdx.x] = r < n_loc ? ids[(size_t)r * topk + threadIdx.x] : -1;
            t.wts[p][(size_t)grow * topk + threadIdx.x] = r < n_loc ? wts[(size_t)r * topk + threadIdx.x] : 0.f;
        }
    }
    publish_and_wait(t, 0, e, ticket, rank, world, max_spins, status, &s_fail);
    if (blockIdx.x == 0 && threadIdx.x == 0) epoch[0] = e;   // dispatch and combine of one layer share the epoch
}

// grid = world * n_max CTAs, 256 threads.  y_all [world * n_max][H]: this rank's experts' weighted sum per
// gathered row.  y_out [n_loc][H] = sum over ranks (+ addend).
__global__ void __launch_bounds__(256)
ep_combine_kernel(const float* __restrict__ y_all, const float* __restrict__ addend, float* __restrict__ y_out,
                  int n_loc, int n_max, int H, EpPtrs t, const uint32_t* __restrict__ epoch, unsigned* __restrict__ ticket,
                  int* __restrict__ status, int rank, int world, int max_spins) {
    PDL_PROLOGUE();
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    const int g = blockIdx.x;
    const int src = g / n_max, r = g % n_max;   // the token's home rank and its row there
    const uint32_t e = epoch[0];                 // the stamp its dispatch used
    {
        const float4* s4 = reinterpret_cast<const float4*>(y_all + (size_t)g * H);
        float4* d4 = reinterpret_cast<float4*>(t.ybuf[src] + ((size_t)rank * n_max + r) * H);
        for (int i = threadIdx.x; i < H / 4; i += blockDim.x) d4[i] = s4[i];
    }
    const bool ok = publish_and_wait(t, 1, e, ticket, rank, world, max_spins, status, &s_fail);
    if (g >= n_loc) return;
    // this CTA reduces local row g over the owners
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
        float4 acc = addend ? *reinterpret_cast<const float4*>(addend + (size_t)g * H + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (ok) {
            for (int o = 0; o < world; ++o) {
                const float4 v = ld_cg_f4(t.ybuf[rank] + ((size_t)o * n_max + g) * H + i * 4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        *reinterpret_cast<float4*>(y_out + (size_t)g * H + i * 4) = acc;
    }
}

}  // namespace

// ptrs: host array of 5 * world device pointers: [xs..., ids..., wts..., ybuf..., flags...] (index = rank).
static void fill_ptrs(EpPtrs& t, const void* const* ptrs, int world) {
    for (int i = 0; i < world; ++i) {
        t.xs[i] = (uint16_t*)ptrs[0 * world + i];
        t.ids[i] = (int*)ptrs[1 * world + i];
        t.wts[i] = (float*)ptrs[2 * world + i];
        t.ybuf[i] = (float*)ptrs[3 * world + i];
        t.flags[i] = (uint32_t*)ptrs[4 * world + i];
    }
}

// e_per_rank > 0: experts [p * e_per_rank, (p + 1) * e_per_rank) live on rank p and a row's planes go to its owners
// only; 0: every row goes to every rank.
FB_API int fb_ep_dispatch(const void* xs_local, int64_t local_plane, const int* ids, const float* wts, int64_t n_loc,
                          int64_t n_max, int64_t H, int64_t topk, int64_t planes, int64_t e_per_rank, const void* const* ptrs, void* epoch,
                          void* ticket, int* status, int64_t rank, int64_t world, int64_t max_spins, cudaStream_t st) {
    if ((H % 8) || world > kMaxWorld || n_loc > n_max || topk > 32 || n_max > 148) return (int)cudaErrorInvalidValue;
    EpPtrs t = {};
    fill_ptrs(t, ptrs, (int)world);
    FB_LAUNCH((ep_dispatch_kernel), n_max, 256, 0, st, (const uint16_t*)xs_local, (int)local_plane, ids, wts, (int)n_loc,
              (int)n_max, (int)H, (int)topk, (int)planes, (int)e_per_rank, t, (uint32_t*)epoch, (unsigned*)ticket, status,
              (int)rank, (int)world, (int)max_spins);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_ep_combine(const float* y_all, const float* addend, float* y_out, int64_t n_loc, int64_t n_max, int64_t H,
                         const void* const* ptrs, const void* epoch, void* ticket, int* status, int64_t rank, int64_t world,
                         int64_t max_spins, cudaStream_t st) {
    if ((H % 4) || world > kMaxWorld || n_loc > n_max || world * n_max > 148 * 4) return (int)cudaErrorInvalidValue;
    EpPtrs t = {};
    fill_ptrs(t, ptrs, (int)world);
    FB_LAUNCH((ep_combine_kernel), world * n_max, 256, 0, st, y_all, addend, y_out, (int)n_loc, (int)n_max, (int)H, t,
              (const uint32_t*)epoch, (unsigned*)ticket, status, (int)rank, (int)world, (int)max_spins);
    return FB_LAUNCH_CHECK();
}
