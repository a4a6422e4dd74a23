// Packed-FP8 dot product for sm_100a:  *out = sum_i decode(a[i]) * decode(b[i]).
//
// Replaces the reference kernel feather/routines/dot.py:144-192, which adds one
// partial sum per 1024-word block into the result with a float atomic (so its
// last bits change from run to run).  Here a persistent grid streams both
// operands with 128-bit loads, every CTA writes ONE partial sum to the
// workspace, and the CTA that finishes last (a ticket counter in the
// workspace) adds the partials in index order: a single launch, and the same
// bits every run.
#pragma once
#include "gemv_common.cuh"  // ldg_stream, warp_sum, decode_word_h2, fma_h2

namespace feather {

constexpr int kDotThreads = 256;
constexpr int kDotMaxCtas = 2048;  // partial slots in the workspace
constexpr int kDotWorkspaceBytes = 16 + 4 * kDotMaxCtas;

// Four code pairs: both words decoded to FP16 pairs, multiplied with the
// mixed-precision FMA (FP16 operands, FP32 accumulate; the product of two FP16
// values is exact in FP32).
template <int MODE>
__device__ __forceinline__ void dot_words(uint32_t wa, uint32_t wb, float (&acc)[4]) {
    uint32_t alo, ahi, blo, bhi;
    decode_word_h2<MODE>(wa, alo, ahi);
    decode_word_h2<MODE>(wb, blo, bhi);
    fma_h2(alo, blo, acc[0], acc[1]);
    fma_h2(ahi, bhi, acc[2], acc[3]);
}

// a, b: n_words words.  VEC: both pointers are 16-byte aligned, so whole
// uint4 chunks are streamed and only the last n_words % 4 words use word loads.
template <int MODE, bool VEC, int UNROLL>
__global__ void __launch_bounds__(kDotThreads)
dot_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, float* __restrict__ out,
           unsigned int* __restrict__ ticket, float* __restrict__ partial, long long n_words) {
    __shared__ float warp_part[kDotThreads / 32];
    __shared__ bool is_last;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const long long tid = (long long)blockIdx.x * kDotThreads + threadIdx.x;
    const long long n_threads = (long long)gridDim.x * kDotThreads;

    long long done_words = 0;
    if (VEC) {
        // Grid-stride over 16-byte chunks; a thread keeps UNROLL chunks of each
        // operand in flight.  Chunks past the end are replaced by zero words
        // (code 0 decodes to +0.0), so there is no remainder loop.
        const long long n_chunks = n_words >> 2;
        const uint4* a4 = reinterpret_cast<const uint4*>(a);
        const uint4* b4 = reinterpret_cast<const uint4*>(b);
        for (long long c = tid; c < n_chunks; c += UNROLL * n_threads) {
            uint4 xa[UNROLL], xb[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const long long cu = c + u * n_threads;
                if (cu < n_chunks) {
                    xa[u] = ldg_stream(a4 + cu);
                    xb[u] = ldg_stream(b4 + cu);
                } else {
                    xa[u] = make_uint4(0, 0, 0, 0);
                    xb[u] = make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                dot_words<MODE>(xa[u].x, xb[u].x, acc);
                dot_words<MODE>(xa[u].y, xb[u].y, acc);
                dot_words<MODE>(xa[u].z, xb[u].z, acc);
                dot_words<MODE>(xa[u].w, xb[u].w, acc);
            }
        }
        done_words = n_chunks << 2;
    }
    for (long long w = done_words + tid; w < n_words; w += n_threads)
        dot_words<MODE>(__ldg(a + w), __ldg(b + w), acc);

    // CTA partial: lanes -> warp (shuffles) -> CTA (fixed order over warps)
    const float s = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_part[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kDotThreads / 32; ++w) t += warp_part[w];
        partial[blockIdx.x] = t;
        __threadfence();  // the partial is visible before the ticket is taken
        const unsigned int n = atomicAdd(ticket, 1u);
        is_last = (n == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;

    // Last CTA: add the partials in index order (thread-strided, then the same
    // fixed tree as above), and hand the ticket counter back as zero.
    __threadfence();
    float t = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += kDotThreads)
        t += __ldcg(partial + i);
    t = warp_sum(t);
    if (lane == 0) warp_part[warp] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < kDotThreads / 32; ++w) r += warp_part[w];
        *out = r;
        *ticket = 0u;
    }
}

}  // namespace feather
