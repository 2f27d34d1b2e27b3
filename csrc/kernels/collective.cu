// One-shot all-reduce over NVLink peer memory, with bounded waits and a status word.
//
// Every rank owns a symmetric region: staging[2 parity][world][max_elems] (value, epoch) pairs and
// flags[2][world][kMaxChunks] u32, mapped into every peer through CUDA IPC.  One launch does
// the whole collective for payloads of a few rows of the hidden size (16-48 KB):
//   1. push: each CTA owns a 4096-element chunk and stores its part of the local vector into slot `rank` of
//      EVERY peer's staging as 8-byte (value, epoch) pairs, two per 16-byte peer store over NVLink.  A pair that
//      carries the launch's epoch IS the data: no fence and no flag follow the stores (with tile stores + a
//      system-scope fence + a flag per chunk the 3 x 4096 case took 18 us on 4 GPUs);
//   2. wait: each thread polls its OWN four pairs of every peer's slot in local staging (a poll never crosses
//      NVLink) -- at most `max_spins` polls, after which the kernel records {TIMEOUT, peer, epoch, chunk} in the
//      status buffer and leaves the vector unreduced instead of spinning, trapping or parking;
//   3. reduce: slots are summed in rank order, so every rank gets bit-identical sums.
// Epochs advance only inside this kernel, chunk by chunk, so warm-up, capture and replay
// keep all ranks in lockstep; staging is double-buffered by epoch parity, which is enough
// because a rank publishes epoch e+1 only after it finished reducing epoch e.
// This is the counterpart of the reference's AR v5 (kernels/cuda/ferrite_kernels.cu:8968-9524),
// whose waiter parks forever or traps on timeout (:9180-9229).
#include "common.cuh"
#include <string.h>

int g_fb_pdl = 0;  // measured neutral on the decode chain (kernel time, not launch gaps, dominates); opt-in

namespace {

constexpr int kMaxChunks = 64;
constexpr int kChunk = 4096;  // elements per CTA (1024 threads x float4)
constexpr int kMaxWorld = 8;

struct ArTables {
    float* staging[kMaxWorld];
    uint32_t* flags[kMaxWorld];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One chunk of the all-reduce: push `v`, wait, and return the rank-ordered sum of the four chunk elements owned by
// this thread.  Low-latency exchange: every value travels as an 8-byte (value, epoch) pair (two pairs per 16-byte
// peer store); a pair that carries the launch's epoch IS the data, so no fence and no flag stand between the peer
// stores and the peers' reduction, and a thread polls only its own pairs in LOCAL staging.  Staging is double-buffered
// by epoch parity (a peer can be at most one launch ahead: it needs this rank's pairs to finish one).  `ok` is false
// after a timeout (v is then returned unchanged).
__device__ __forceinline__ float2 ld_relaxed_sys_f2(const float2* p) {
    float2 v;
    asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ar_chunk(const ArTables& t, uint32_t* epoch, int* status, int rank, int world,
                                           int max_elems, int max_spins, int chunk, float4 v, bool valid, bool* ok) {
    __shared__ int s_fail;
    const uint32_t e = epoch[chunk] + 1u;
    const int par = e & 1u;
    const float ef = __uint_as_float(e);
    const size_t off = (size_t)chunk * kChunk + threadIdx.x * 4;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    float4 acc = v;
    if (valid) {
        for (int p = 0; p < world; ++p) {
            if (p == rank) continue;
            float2* dst = reinterpret_cast<float2*>(t.staging[p]) + ((size_t)par * world + rank) * max_elems + off;
            reinterpret_cast<float4*>(dst)[0] = make_float4(v.x, ef, v.y, ef);
            reinterpret_cast<float4*>(dst)[1] = make_float4(v.z, ef, v.w, ef);
        }
        const int budget = fb_spin_budget(status, max_spins);
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
        const float mine[4] = {v.x, v.y, v.z, v.w};
        bool failed = false;
        for (int src = 0; src < world && !failed; ++src) {      // rank order: identical bits on every rank
            if (src == rank) {
#pragma unroll
                for (int j = 0; j < 4; ++j) s4[j] += mine[j];
                continue;
            }
            const float2* f = reinterpret_cast<const float2*>(t.staging[rank]) + ((size_t)par * world + src) * max_elems + off;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 pr = ld_relaxed_sys_f2(f + j);
                int spins = 0;
                while (__float_as_uint(pr.y) != e) {
                    if (++spins > budget) {
                        if (atomicCAS(&s_fail, 0, 1) == 0) {
                            status[0] = FB_TIMEOUT; status[1] = src; status[2] = (int)e; status[3] = chunk;
                        }
                        failed = true;
                        break;
                    }
                    pr = ld_relaxed_sys_f2(f + j);
                }
                s4[j] += pr.x;
            }
        }
        acc = make_float4(s4[0], s4[1], s4[2], s4[3]);
    }
    __syncthreads();
    const bool good = (s_fail == 0);
    *ok = good;
    if (threadIdx.x == 0) epoch[chunk] = e;  // stay in step with the peers even after a timeout
    return good ? acc : v;
}

__global__ void __launch_bounds__(1024)
ar_oneshot_kernel(ArTables t, uint32_t* epoch, int* status, float* y, int n_elems, int rank, int world,
                  int max_elems, int max_spins) {
    PDL_PROLOGUE();
    const int chunk = blockIdx.x;
    const int i = chunk * kChunk + threadIdx.x * 4;
    const bool valid = i < n_elems;
    float4 v = valid ? *reinterpret_cast<const float4*>(y + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok;
    const float4 r = ar_chunk(t, epoch, status, rank, world, max_elems, max_spins, chunk, v, valid, &ok);
    if (ok && valid) *reinterpret_cast<float4*>(y + i) = r;
}

// Cross-rank argmax for a vocab-sliced head.  Each rank has the 64 per-slice partial keys of its
// vocab slice for n rows (fb_argmax's first pass; a key orders by value, then by LOWER global index).
// One CTA: thread r reduces row r's partials, stores the key into slot `rank` of every peer's
// staging, the CTA publishes one epoch stamp per peer, waits (bounded) for all ranks' stamps and
// takes the maximum key over the ranks - every rank ends with the same token id.  Replaces the
// reference's argmax_xchg_v5 (kernels/cuda/dsv41_kernels.cu:11329,11393).
struct XchgTables {
    unsigned long long* staging[kMaxWorld];  // [2][world][kXchgRows]
    uint32_t* flags[kMaxWorld];              // [2][world]
};
constexpr int kXchgRows = 64;

__global__ void __launch_bounds__(64)
argmax_xchg_kernel(const unsigned long long* __restrict__ part, XchgTables t, uint32_t* epoch, int* status,
                   int* __restrict__ ids, float* __restrict__ vals, int id_stride, int n, int rank, int world,
                   int max_spins) {
    PDL_PROLOGUE();
    __shared__ int s_fail;
    const int r = threadIdx.x;
    const uint32_t e = epoch[0] + 1u;
    const int par = e & 1u;
    if (r == 0) s_fail = 0;
    unsigned long long best = 0ull;
    if (r < n) {
        for (int i = 0; i < 64; ++i) {
            const unsigned long long k = part[(size_t)r * 64 + i];
            best = k > best ? k : best;
        }
        for (int p = 0; p < world; ++p) t.staging[p][((size_t)par * world + rank) * kXchgRows + r] = best;
    }
    __syncthreads();
    if (r == 0) {
        __threadfence_system();
        for (int p = 0; p < world; ++p) st_release_sys(t.flags[p] + par * world + rank, e);
    }
    if (r < world) {
        const uint32_t* f = t.flags[rank] + par * world + r;
        int spins = 0;
        const int budget = fb_spin_budget(status, max_spins);
        while (ld_acquire_sys(f) < e) {
            if (++spins > budget) {
                if (atomicCAS(&s_fail, 0, 1) == 0) { status[0] = FB_TIMEOUT; status[1] = r; status[2] = (int)e; status[3] = -2; }
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    if (r < n && s_fail == 0) {
        for (int src = 0; src < world; ++src) {
            unsigned long long k;
            const unsigned long long* p = t.staging[rank] + ((size_t)par * world + src) * kXchgRows + r;
            asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(k) : "l"(p));
            best = k > best ? k : best;
        }
    }
    if (r < n) {
        ids[(size_t)r * id_stride] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        if (vals) {
            uint32_t u = (uint32_t)(best >> 32);
            u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
            vals[r] = __uint_as_float(u);
        }
    }
    __syncthreads();
    if (r == 0) epoch[0] = e;
}

// A wait that nothing satisfies: used by the failure-detection test to check that a bounded
// wait gives up with a status word and leaves the context usable.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, int max_spins, int* status) {
    PDL_PROLOGUE();
    int spins = 0;
    const int budget = fb_spin_budget(status, max_spins);
    while (ld_acquire_sys(flag) < want) {
        if (++spins > budget) {
            status[0] = FB_TIMEOUT; status[1] = -1; status[2] = (int)want; status[3] = spins;
            return;
        }
        __nanosleep(64);
    }
    status[0] = FB_OK;
}

}  // namespace

// ---- symmetric memory plumbing (cudaMalloc + CUDA IPC) ----------------------------------------
FB_API int fb_symm_alloc(int64_t bytes, void** out) {
    cudaError_t e = cudaMalloc(out, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(*out, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();   // zeroed before any peer can learn the address
    return (int)e;
}
FB_API int fb_symm_free(void* p) { return (int)cudaFree(p); }
FB_API int fb_ipc_get_handle(void* p, void* handle64) {
    return (int)cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), p);
}
FB_API int fb_ipc_open(const void* handle64, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
FB_API int fb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
FB_API int fb_memcpy_d2h(void* dst, const void* src, int64_t bytes) {
    return (int)cudaMemcpy(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost);
}
// 1 = launch every kernel with programmatic dependent launch allowed, 0 = plain (default).
FB_API int fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; return 0; }

FB_API int fb_ar_limits(int* max_chunks, int* chunk_elems) {
    *max_chunks = kMaxChunks; *chunk_elems = kChunk;
    return 0;
}

// staging_ptrs / flag_ptrs: host arrays of `world` device pointers (index = rank; the own
// entry is the local allocation).  y [n_elems] f32 is reduced in place; n_elems % 4 == 0 and
// n_elems <= min(max_elems, 64 * 4096).
FB_API int fb_ar_oneshot(const void* const* staging_ptrs, const void* const* flag_ptrs, void* epoch, int* status,
                         float* y, int64_t n_elems, int64_t rank, int64_t world, int64_t max_elems,
                         int64_t max_spins, cudaStream_t st) {
    if (world > kMaxWorld || n_elems > max_elems || (n_elems % 4) || n_elems > (int64_t)kMaxChunks * kChunk)
        return (int)cudaErrorInvalidValue;
    ArTables t;
    for (int i = 0; i < world; ++i) { t.staging[i] = (float*)staging_ptrs[i]; t.flags[i] = (uint32_t*)flag_ptrs[i]; }
    const int chunks = (int)((n_elems + kChunk - 1) / kChunk);
    FB_LAUNCH((ar_oneshot_kernel), chunks, 1024, 0, st, t, (uint32_t*)epoch, status, y, (int)n_elems, (int)rank, (int)world,
                                               (int)max_elems, (int)max_spins);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_wait_flag(const void* flag, int64_t want, int64_t max_spins, int* status, cudaStream_t st) {
    FB_LAUNCH((wait_flag_kernel), 1, 1, 0, st, (const uint32_t*)flag, (uint32_t)want, (int)max_spins, status);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_argmax_xchg_limits(int* max_rows) { *max_rows = kXchgRows; return 0; }

// part: this rank's first-pass argmax keys [n][64] (global indices: run fb_argmax_partial with the
// slice's vocab offset).  staging_ptrs / flag_ptrs: `world` device pointers each.
FB_API int fb_argmax_xchg(const void* part, const void* const* staging_ptrs, const void* const* flag_ptrs, void* epoch,
                          int* status, int* ids, float* vals, int64_t id_stride, int64_t n, int64_t rank, int64_t world,
                          int64_t max_spins, cudaStream_t st) {
    if (n < 1 || n > kXchgRows || world > kMaxWorld) return (int)cudaErrorInvalidValue;
    XchgTables t;
    for (int i = 0; i < world; ++i) {
        t.staging[i] = (unsigned long long*)staging_ptrs[i];
        t.flags[i] = (uint32_t*)flag_ptrs[i];
    }
    FB_LAUNCH((argmax_xchg_kernel), 1, 64, 0, st, (const unsigned long long*)part, t, (uint32_t*)epoch, status, ids, vals,
              (int)id_stride, (int)n, (int)rank, (int)world, (int)max_spins);
    return FB_LAUNCH_CHECK();
}
