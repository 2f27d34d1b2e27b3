// Shared device helpers for the sm_100a kernel library.
//
// Conventions of the C ABI exported by this library:
//   * every entry point is `extern "C" int fb_<name>(..., cudaStream_t stream)` and returns
//     the cudaError_t of its launch (0 = success); nothing synchronises the stream;
//   * activations are f32, weights bf16 or fp8-e4m3 (128x128 block scales), ids are int32;
//   * a kernel that waits on another agent (peer GPU, flag, mbarrier) counts its polls and,
//     when the limit runs out, writes a status word and returns -- it never traps or parks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#define FB_API extern "C" __attribute__((visibility("default")))

// Status words written by kernels with bounded waits (host reads them after the step).
enum FbStatus : int {
    FB_OK = 0,
    FB_TIMEOUT = 1,     // a bounded wait ran out; payload words say who/what
    FB_BAD_CANARY = 2,  // a guard word next to a signal pad was overwritten
    FB_BAD_ARG = 3,     // an index failed its bounds check; the access was skipped
};

#define FB_LAUNCH_CHECK() ((int)cudaGetLastError())

// ---- programmatic dependent launch (PDL) ---------------------------------------------------
// Every kernel is launched with programmatic stream serialization allowed and starts with
// PDL_PROLOGUE(): it lets the NEXT kernel in the stream be scheduled right away and then
// waits until the PREVIOUS kernel has completed and flushed its memory.  Launch latency and
// the ramp-up of a kernel therefore overlap the tail of its predecessor; because every
// kernel waits before it touches any buffer, completion is transitive along the stream.
// Only data that no kernel of the step writes (weights) may be read before pdl_wait().
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define PDL_PROLOGUE() do { pdl_launch(); pdl_wait(); } while (0)

extern int g_fb_pdl;  // 1 = launch with the PDL attribute, 0 = plain launches (default)

template <typename... KArgs, typename... Args>
inline cudaError_t fb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_fb_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define FB_LAUNCH(kernel, grid, block, smem, st, ...) \
    (void)fb_launch(kernel, dim3(grid), dim3(block), (size_t)(smem), st, __VA_ARGS__)

// Wait budget of a collective kernel: once a wait of this collective has run out (status word = FB_TIMEOUT),
// later launches do not wait again, so one missing peer costs one budget and not one per queued launch.
// The host clears the status word when it reads the failure.
__device__ __forceinline__ int fb_spin_budget(const int* status, int max_spins) {
    return (*reinterpret_cast<const volatile int*>(status) == FB_TIMEOUT) ? 0 : max_spins;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `red` is a shared array of >= 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + __expf(-x)); }

// bf16 pair packed in a 32-bit word -> two floats (exact: bf16 is the top half of f32).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Four e4m3 bytes packed in a 32-bit word -> four floats.
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t w, float* o) {
    __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
    __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
    float2 fa = __half22float2(*reinterpret_cast<__half2*>(&a));
    float2 fb = __half22float2(*reinterpret_cast<__half2*>(&b));
    o[0] = fa.x; o[1] = fa.y; o[2] = fb.x; o[3] = fb.y;
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 r;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// Per-forward row metadata, filled on the device by fb_prep_rows so that a replayed CUDA
// graph advances without host writes.
struct RowMeta {
    int slot;   // sequence slot (state / page-table row)
    int pos;    // absolute position of this row's token
    int ctx0;   // position of the first row of this row's group (tokens already cached)
    int total;  // ctx0 + rows in the group
    int first;  // 1 if this row is the first row of its group
    int off;    // row index inside its group
    int gsize;  // rows in the group
    int pad;
};
