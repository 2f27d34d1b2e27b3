// Lean device runtime behind the C ABI: prioritised streams with fork/join events, stream capture and
// graph instantiate/launch, pinned host staging, async copies (host, device, 2-D, peer).  The engines
// normally ride on PyTorch's streams and graphs; this is the runtime for hosts without a tensor
// library and for side-stream scheduling inside a captured step (main stream forks to a side stream,
// both record kernels, the main stream joins).  Counterpart of the reference's DevRuntime
// (crates/ferrite-kernel/src/devrt.rs:540-1617: streams/events :823-945, peer :1036-1060, copies
// :1160-1351, capture/graph :1510-1587).  Nothing here changes a device-wide setting.
#include "common.cuh"

namespace {
constexpr int kMaxSide = 4;
struct FbRuntime {
    int device;
    cudaStream_t main;
    cudaStream_t side[kMaxSide];
    cudaEvent_t fork_ev, join_ev[kMaxSide];
    int n_side;
};
}  // namespace

FB_API int fb_rt_create(int64_t device, int64_t n_side, void** out) {
    if (n_side < 0 || n_side > kMaxSide) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaSetDevice((int)device);
    if (e != cudaSuccess) return (int)e;
    FbRuntime* rt = new FbRuntime();
    rt->device = (int)device;
    rt->n_side = (int)n_side;
    int lo = 0, hi = 0;   // numerically lower = higher priority
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    e = cudaStreamCreateWithPriority(&rt->main, cudaStreamNonBlocking, hi);
    for (int i = 0; i < rt->n_side && e == cudaSuccess; ++i) {
        e = cudaStreamCreateWithPriority(&rt->side[i], cudaStreamNonBlocking, lo);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&rt->join_ev[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&rt->fork_ev, cudaEventDisableTiming);
    if (e != cudaSuccess) { delete rt; return (int)e; }
    *out = rt;
    return 0;
}

FB_API int fb_rt_destroy(void* h) {
    FbRuntime* rt = (FbRuntime*)h;
    if (!rt) return 0;
    cudaStreamDestroy(rt->main);
    for (int i = 0; i < rt->n_side; ++i) { cudaStreamDestroy(rt->side[i]); cudaEventDestroy(rt->join_ev[i]); }
    cudaEventDestroy(rt->fork_ev);
    delete rt;
    return 0;
}

FB_API void* fb_rt_stream(void* h, int64_t which) {   // -1 = main, 0.. = side streams
    FbRuntime* rt = (FbRuntime*)h;
    if (which < 0) return rt->main;
    return which < rt->n_side ? rt->side[which] : nullptr;
}

// Side stream `which` waits for everything recorded on the main stream so far.
FB_API int fb_rt_fork(void* h, int64_t which) {
    FbRuntime* rt = (FbRuntime*)h;
    if (which < 0 || which >= rt->n_side) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaEventRecord(rt->fork_ev, rt->main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->side[which], rt->fork_ev, 0);
    return (int)e;
}

// The main stream waits for everything recorded on side stream `which` so far.
FB_API int fb_rt_join(void* h, int64_t which) {
    FbRuntime* rt = (FbRuntime*)h;
    if (which < 0 || which >= rt->n_side) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaEventRecord(rt->join_ev[which], rt->side[which]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->main, rt->join_ev[which], 0);
    return (int)e;
}

FB_API int fb_rt_sync(void* h) { return (int)cudaStreamSynchronize(((FbRuntime*)h)->main); }

// ---- capture / graphs (thread-local capture mode: other threads of the process are unaffected) ----
FB_API int fb_rt_capture_begin(void* h) {
    return (int)cudaStreamBeginCapture(((FbRuntime*)h)->main, cudaStreamCaptureModeThreadLocal);
}
FB_API int fb_rt_capture_end(void* h, void** graph_exec) {
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(((FbRuntime*)h)->main, &g);
    if (e != cudaSuccess) return (int)e;
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiateWithFlags(&ex, g, cudaGraphInstantiateFlagUseNodePriority);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return (int)e;
    *graph_exec = ex;
    return 0;
}
FB_API int fb_rt_graph_launch(void* h, void* graph_exec) {
    return (int)cudaGraphLaunch((cudaGraphExec_t)graph_exec, ((FbRuntime*)h)->main);
}
FB_API int fb_rt_graph_free(void* graph_exec) { return (int)cudaGraphExecDestroy((cudaGraphExec_t)graph_exec); }

// ---- memory ------------------------------------------------------------------------------------
FB_API int fb_rt_pinned_alloc(int64_t bytes, void** out) { return (int)cudaHostAlloc(out, (size_t)bytes, cudaHostAllocDefault); }
FB_API int fb_rt_pinned_free(void* p) { return (int)cudaFreeHost(p); }
FB_API int fb_rt_copy(void* h, void* dst, const void* src, int64_t bytes, int64_t which) {
    FbRuntime* rt = (FbRuntime*)h;
    cudaStream_t st = which < 0 ? rt->main : rt->side[which];
    return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, st);
}
FB_API int fb_rt_copy_2d(void* h, void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                         int64_t which) {
    FbRuntime* rt = (FbRuntime*)h;
    cudaStream_t st = which < 0 ? rt->main : rt->side[which];
    return (int)cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width, (size_t)height, cudaMemcpyDefault, st);
}
FB_API int fb_rt_copy_peer(void* h, void* dst, int64_t dst_dev, const void* src, int64_t src_dev, int64_t bytes) {
    return (int)cudaMemcpyPeerAsync(dst, (int)dst_dev, src, (int)src_dev, (size_t)bytes, ((FbRuntime*)h)->main);
}
