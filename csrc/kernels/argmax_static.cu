// fb_argmax_static: the two-pass greedy argmax of sample.cu with its partials in a fixed
// array of this library instead of a buffer the caller allocates.  See argmax_static.h for
// who needs that and for the rules (row limit, first call outside capture, shared array).
//
// This file allocates nothing: no cudaMalloc/cudaFree, no stream or event creation, no
// tensor library.  The host work is one cudaGetDevice per call, one cudaGetSymbolAddress
// per device for the life of the process, and two kernel launches.
#include "argmax_static.h"

#include <mutex>

#include "common.cuh"

constexpr int kSlices = 64;  // partials per row, same split as fb_argmax
constexpr int kMaxDevices = 64;

// The scratch: one u64 key per (row, slice).  64 rows x 64 slices x 8 bytes = 32 KiB per
// device.  The name below is a host-side handle for the symbol, NOT a device address: the
// kernels get the address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned long long g_partials[FB_ARGMAX_STATIC_MAX_ROWS * kSlices];

namespace {

std::mutex g_mu;
unsigned long long* g_dev_ptr[kMaxDevices] = {};  // per device, filled on that device's first call

// Ordered key: larger value wins, on ties the smaller index wins; 0 is below every real key.
__device__ __forceinline__ unsigned long long key_of(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, k, o);
        k = t > k ? t : k;
    }
    return k;
}

// grid (kSlices, n): block (s, r) scans columns [s*per, (s+1)*per) of row r and writes
// part[r*kSlices + s].  Every (r, s) with r < n is written, also for an empty slice (key 0).
__global__ void __launch_bounds__(256)
static_partial_kernel(const float* __restrict__ logits, int ld, unsigned long long* __restrict__ part, int V) {
    __shared__ unsigned long long wb[8];
    const int r = blockIdx.y;
    const int per = (V + kSlices - 1) / kSlices;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    unsigned long long best = 0ull;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = logits[(size_t)r * ld + i];
        if (v == v) {  // a NaN never wins
            const unsigned long long k = key_of(v, i);
            best = k > best ? k : best;
        }
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0) wb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = wb[w] > best ? wb[w] : best;
        part[(size_t)r * kSlices + blockIdx.x] = best;
    }
}

// grid n, one warp per row: reduces the row's kSlices partials.
__global__ void static_final_kernel(const unsigned long long* __restrict__ part, int* __restrict__ ids,
                                    float* __restrict__ vals, int id_stride, int vocab_offset) {
    const int r = blockIdx.x;
    unsigned long long best = part[(size_t)r * kSlices + threadIdx.x];
    const unsigned long long t = part[(size_t)r * kSlices + threadIdx.x + 32];
    best = warp_max_u64(t > best ? t : best);
    if (threadIdx.x == 0) {
        const int idx = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        ids[(size_t)r * id_stride] = idx + vocab_offset;
        if (vals) {
            uint32_t u = (uint32_t)(best >> 32);
            u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
            vals[r] = __uint_as_float(u);
        }
    }
}

// Device address of g_partials on the current device.  Set-up happens here, once per device.
int scratch_for_current_device(unsigned long long** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return FB_ARGMAX_STATIC_E_SYMBOL;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_partials);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();  // do not leave the error for an unrelated later check
            return FB_ARGMAX_STATIC_E_SYMBOL;
        }
        if (!p) return FB_ARGMAX_STATIC_E_SYMBOL;
        g_dev_ptr[dev] = (unsigned long long*)p;
    }
    *out = g_dev_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int fb_argmax_static(const float* logits, int64_t ld, int* ids, float* vals, int64_t n, int64_t V,
                                int64_t id_stride, int64_t vocab_offset, cudaStream_t st) {
    if (n < 1 || n > FB_ARGMAX_STATIC_MAX_ROWS) return FB_ARGMAX_STATIC_E_ROWS;
    if (!logits || !ids || V < 1 || ld < V || V > 0x7fffffffll || ld > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    unsigned long long* part = nullptr;
    const int rc = scratch_for_current_device(&part);
    if (rc) return rc;
    static_partial_kernel<<<dim3(kSlices, (unsigned)n), 256, 0, st>>>(logits, (int)ld, part, (int)V);
    static_final_kernel<<<(unsigned)n, 32, 0, st>>>(part, ids, vals, (int)id_stride, (int)vocab_offset);
    return (int)cudaGetLastError();
}

extern "C" const char* fb_argmax_static_strerror(int rc) {
    if (rc == 0) return "ok";
    if (rc == FB_ARGMAX_STATIC_E_ROWS)
        return "fb_argmax_static: row count outside 1..64 (FB_ARGMAX_STATIC_MAX_ROWS); the fixed scratch array holds "
               "64 rows of partials - split the batch or use fb_argmax with a caller-owned buffer";
    if (rc == FB_ARGMAX_STATIC_E_SYMBOL)
        return "fb_argmax_static: could not obtain the device address of the scratch array on the current device";
    return cudaGetErrorString((cudaError_t)rc);
}
