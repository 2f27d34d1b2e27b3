// Greedy argmax that allocates nothing.  This entry point has no counterpart in the reference.
//
// fb_argmax needs a caller-supplied partials buffer, which in practice a tensor library
// allocates.  Some callers cannot allocate at the point where they sample: a thread that
// drives the device from a signal-safe or real-time loop, a C host that links this library
// without any tensor library, or code that runs while another thread holds the allocator's
// lock.  For them the partials live in a fixed array inside the library image.
//
// Limits and rules
//   * n (rows) <= FB_ARGMAX_STATIC_MAX_ROWS; a larger n is refused with
//     FB_ARGMAX_STATIC_E_ROWS and nothing is launched.
//   * The first call on each device looks up the array's device address (no allocation, but
//     it is a host-side runtime query): make that first call outside any stream capture.
//   * All calls on one device share the one array.  Two calls whose kernels can overlap
//     (different streams, or different host threads on different streams) race on it; keep
//     calls on one stream or order them with events.
//   * Every partial slot that the final pass reads is written by the first pass of the same
//     call, so the array needs no clearing between calls and stale contents are harmless.
//   * A NaN never wins a comparison.  A row that holds nothing but NaNs therefore has no
//     winner: its id comes back as vocab_offset - 1 (one below the first valid id of the
//     slice, i.e. -1 for vocab_offset = 0) and its value as a NaN.  A
//     caller that samples from unchecked logits should treat an id below vocab_offset as
//     "no token" rather than index with it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FB_ARGMAX_STATIC_MAX_ROWS 64
#define FB_ARGMAX_STATIC_E_ROWS (-2)    // n outside 1..FB_ARGMAX_STATIC_MAX_ROWS
#define FB_ARGMAX_STATIC_E_SYMBOL (-3)  // the device address of the array could not be obtained

#if defined(__GNUC__)
#define FB_ARGMAX_STATIC_EXPORT __attribute__((visibility("default")))
#else
#define FB_ARGMAX_STATIC_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

// logits [n, ld] f32 (V <= ld used columns); ids[r * id_stride] = first index of the row maximum
// (+ vocab_offset); vals (may be null) [n] = the maximum.  Returns 0, a cudaError_t value, or
// one of the negative codes above.
FB_ARGMAX_STATIC_EXPORT int fb_argmax_static(const float* logits, int64_t ld, int* ids, float* vals, int64_t n, int64_t V, int64_t id_stride,
                     int64_t vocab_offset, cudaStream_t st);

// Text for a return code of fb_argmax_static (static storage, never null).
FB_ARGMAX_STATIC_EXPORT const char* fb_argmax_static_strerror(int rc);

#ifdef __cplusplus
}
#endif
