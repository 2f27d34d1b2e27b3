// Greedy sampling (first maximum wins) and the device-side MTP accept/commit.
//
// argmax is two launches (per-slice partials, then a per-row final) and can take a vocab
// offset so that a vocab-sliced head publishes global ids.  fb_mtp_accept is the whole
// "accept -> commit" phase of a speculative step as ONE small kernel: it walks the shared
// accept chain (reference crates/ferrite-types/src/spec_step.rs:91-112), publishes the
// emitted tokens, advances sequence lengths and the GatedDeltaNet snapshot cursor (commit
// without copying state; the reference restores state with mtp_commit_kernel,
// kernels/cuda/ferrite_kernels.cu:10580,11455), and stages the next step's MTP inputs.
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long amax_key(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

constexpr int kSlices = 64;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int ld, unsigned long long* __restrict__ part, int V,
                      int key_offset) {
    PDL_PROLOGUE();
    __shared__ unsigned long long wb[8];
    const int r = blockIdx.y;
    const int per = (V + kSlices - 1) / kSlices;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    unsigned long long best = 0ull;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = logits[(size_t)r * ld + i];
        if (v == v) {  // NaN never wins
            const unsigned long long k = amax_key(v, i + key_offset);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) wb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = wb[w] > best ? wb[w] : best;
        part[(size_t)r * kSlices + blockIdx.x] = best;
    }
}

// Counter-based noise: one 32-bit hash per (seed, row key, global vocab index), the same on every
// rank of a vocab-sliced head and on every replay of a captured step (the row key is the position).
__device__ __forceinline__ uint32_t mix32(uint32_t h) {
    h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}
__device__ __forceinline__ float gumbel_noise(uint32_t seed, uint32_t key, uint32_t idx) {
    const uint32_t h = mix32(mix32(seed ^ (key * 0x9e3779b1u)) ^ (idx * 0x85ebca77u));
    const float u = ((float)(h >> 8) + 0.5f) * (1.f / 16777216.f);   // (0, 1)
    return -logf(-logf(u));
}

// First pass of temperature sampling by the Gumbel-max trick: argmax_i (logit_i / T + G_i) is a draw
// from softmax(logits / T) (reference sampler: softmax(l / T) / Exp(1), ref_inference/model.py:1285-1292).
__global__ void __launch_bounds__(256)
gumbel_partial_kernel(const float* __restrict__ logits, int ld, unsigned long long* __restrict__ part, int V,
                      int key_offset, float inv_t, uint32_t seed, const RowMeta* __restrict__ meta) {
    PDL_PROLOGUE();
    __shared__ unsigned long long wb[8];
    const int r = blockIdx.y;
    const uint32_t key = meta ? (uint32_t)meta[r].pos : (uint32_t)r;
    const int per = (V + kSlices - 1) / kSlices;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    unsigned long long best = 0ull;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = logits[(size_t)r * ld + i] * inv_t + gumbel_noise(seed, key, (uint32_t)(i + key_offset));
        if (v == v) {
            const unsigned long long k = amax_key(v, i + key_offset);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) wb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = wb[w] > best ? wb[w] : best;
        part[(size_t)r * kSlices + blockIdx.x] = best;
    }
}

__global__ void argmax_final_kernel(const unsigned long long* __restrict__ part, int* __restrict__ ids,
                                    float* __restrict__ vals, int id_stride, int vocab_offset) {
    PDL_PROLOGUE();
    const int r = blockIdx.x;
    unsigned long long best = part[(size_t)r * kSlices + threadIdx.x];
    if (threadIdx.x + 32 < kSlices) {
        unsigned long long t = part[(size_t)r * kSlices + threadIdx.x + 32];
        best = t > best ? t : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
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

// One block per sequence group g (rows g*nv .. g*nv+nv-1 of the verify block).
//   block_ids [G][nv]  : [t_last, d1..d_nd]      (in)  -> block_ids[g][0] = next t_last (out)
//   judges    [G*nv]   : verify argmax per row   (in)
//   out_tokens[G][nv+1]: [k, emitted tokens...]  (out)
//   h_final   [G*nv][H]: contracted residual per verify row (in)
//   mtp_ids [G][2], mtp_h [G][2][H]: the next draft pass's two (token, hidden) pairs (in/out)
//   main_len/mtp_len/cur [slots]: device-resident sequence bookkeeping
__global__ void __launch_bounds__(256)
mtp_accept_kernel(int* __restrict__ block_ids, const int* __restrict__ judges, int* __restrict__ out_tokens,
                  const float* __restrict__ h_final, int* __restrict__ mtp_ids, float* __restrict__ mtp_h,
                  const int* __restrict__ group_slot, int* __restrict__ main_len, int* __restrict__ mtp_len,
                  int* __restrict__ cur, int nv, int H, int nbuf) {
    PDL_PROLOGUE();
    __shared__ int s_k;
    const int g = blockIdx.x;
    int* blk = block_ids + (size_t)g * nv;
    const int* jd = judges + (size_t)g * nv;
    if (threadIdx.x == 0) {
        int matched = 0;
        while (matched < nv - 1 && blk[1 + matched] == jd[matched]) ++matched;
        const int k = matched + 1;  // anchor row is in the block: emitted = accepted drafts + bonus
        s_k = k;
        int* o = out_tokens + (size_t)g * (nv + 1);
        o[0] = k;
        for (int i = 0; i < nv; ++i) o[1 + i] = i < k ? jd[i] : -1;
    }
    __syncthreads();
    const int k = s_k;
    float* h0 = mtp_h + (size_t)g * 2 * H;
    float* h1 = h0 + H;
    const float* hf = h_final + (size_t)g * nv * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float a = (k == 1) ? h1[j] : hf[(size_t)(k - 2) * H + j];
        const float b = hf[(size_t)(k - 1) * H + j];
        h0[j] = a;
        h1[j] = b;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int slot = group_slot[g];
        mtp_ids[g * 2 + 0] = blk[k - 1];
        mtp_ids[g * 2 + 1] = jd[k - 1];
        blk[0] = jd[k - 1];
        const int new_len = main_len[slot] + k;
        main_len[slot] = new_len;
        mtp_len[slot] = new_len - 2;
        if (nbuf > 1) cur[slot] = (cur[slot] + k) % nbuf;
    }
}

__global__ void copy_i32_kernel(const int* __restrict__ src, int* __restrict__ dst, int n, int src_stride,
                                int dst_stride) {
    PDL_PROLOGUE();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[(size_t)i * dst_stride] = src[(size_t)i * src_stride];
}

}  // namespace

// part: scratch of n*64 u64.  ids[r*id_stride] = argmax (+ vocab_offset); vals (optional) = max.
FB_API int fb_argmax(const float* logits, int64_t ld, void* part, int* ids, float* vals, int64_t n, int64_t V,
                     int64_t id_stride, int64_t vocab_offset, cudaStream_t st) {
    FB_LAUNCH((argmax_partial_kernel), dim3(kSlices, (unsigned)n), 256, 0, st, logits, (int)ld, (unsigned long long*)part, (int)V, 0);
    FB_LAUNCH((argmax_final_kernel), n, 32, 0, st, (const unsigned long long*)part, ids, vals, (int)id_stride, (int)vocab_offset);
    return FB_LAUNCH_CHECK();
}

// First pass only: part[r][64] keys over this rank's vocab slice with GLOBAL indices (i + vocab_offset),
// to be merged across ranks by fb_argmax_xchg.
FB_API int fb_argmax_partial(const float* logits, int64_t ld, void* part, int64_t n, int64_t V, int64_t vocab_offset,
                             cudaStream_t st) {
    FB_LAUNCH((argmax_partial_kernel), dim3(kSlices, (unsigned)n), 256, 0, st, logits, (int)ld, (unsigned long long*)part, (int)V,
              (int)vocab_offset);
    return FB_LAUNCH_CHECK();
}

// Temperature sampling (Gumbel-max).  With `final` != 0 the ids are written here; with 0 only the
// partial keys are produced (global indices), to be merged across ranks by fb_argmax_xchg.
// meta (optional): row metadata, the row's position keys the noise; otherwise the row index does.
FB_API int fb_sample_gumbel(const float* logits, int64_t ld, void* part, int* ids, int64_t n, int64_t V,
                            int64_t id_stride, int64_t vocab_offset, float temperature, int64_t seed, const void* meta,
                            int64_t final, cudaStream_t st) {
    if (!(temperature > 0.f)) return (int)cudaErrorInvalidValue;
    FB_LAUNCH((gumbel_partial_kernel), dim3(kSlices, (unsigned)n), 256, 0, st, logits, (int)ld, (unsigned long long*)part, (int)V,
              (int)vocab_offset, 1.f / fmaxf(temperature, 1e-5f), (uint32_t)seed, (const RowMeta*)meta);
    if (final)
        FB_LAUNCH((argmax_final_kernel), n, 32, 0, st, (const unsigned long long*)part, ids, (float*)nullptr, (int)id_stride, 0);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_mtp_accept(int* block_ids, const int* judges, int* out_tokens, const float* h_final, int* mtp_ids,
                         float* mtp_h, const int* group_slot, int* main_len, int* mtp_len, int* cur,
                         int64_t n_groups, int64_t nv, int64_t H, int64_t nbuf, cudaStream_t st) {
    FB_LAUNCH((mtp_accept_kernel), n_groups, 256, 0, st, block_ids, judges, out_tokens, h_final, mtp_ids, mtp_h, group_slot,
                                                main_len, mtp_len, cur, (int)nv, (int)H, (int)nbuf);
    return FB_LAUNCH_CHECK();
}

FB_API int fb_copy_i32(const int* src, int* dst, int64_t n, int64_t src_stride, int64_t dst_stride, cudaStream_t st) {
    FB_LAUNCH((copy_i32_kernel), (n + 127) / 128, 128, 0, st, src, dst, (int)n, (int)src_stride, (int)dst_stride);
    return FB_LAUNCH_CHECK();
}
