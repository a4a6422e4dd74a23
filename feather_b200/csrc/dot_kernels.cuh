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
#include "gemv_ring.cuh"    // mbarrier and bulk-copy helpers

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

// dot_ring_kernel: the same sum for long operands, streamed through shared
// memory.  The load-to-register kernel above can keep only as many bytes in
// flight as its registers hold; B200 wants well over 64 KB per SM.  Here one
// producer warp keeps a ring of stages full with cp.async.bulk (a stage holds
// the same number of 16-byte chunks of EACH operand), so ~190 KB per SM
// are in flight whatever the consumers do; kDotWarps consumer warps read the
// stage with conflict-free 128-bit shared loads.  One CTA per SM; CTA b owns
// the contiguous chunks [n*b/G, n*(b+1)/G).  The reduction (lanes, warps,
// CTA partial, ticket, last CTA adds in index order) is the one above, so the
// result has the same bits on every run.  Needs 16-byte aligned operands; the
// last n_words % 4 words are added by one thread.  Waits are bounded like the
// GEMV ring's.
constexpr int kDotWarps = 16;
constexpr int kDotRingThreads = (kDotWarps + 1) * 32;
constexpr int dot_ring_smem_bytes(int stages, int stage_chunks) {
    return stages * 2 * stage_chunks * 16 + 2 * stages * 8 + 16 + 4 * kDotWarps;
}

// kDotStages stages of kDotStageChunks 16-byte chunks per operand.
template <int MODE, int kDotStages, int kDotStageChunks>
__global__ void __launch_bounds__(kDotRingThreads, 1)
dot_ring_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, float* __restrict__ out,
                unsigned int* __restrict__ ticket, float* __restrict__ partial, long long n_words,
                unsigned int* __restrict__ status, int pre_bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(128) unsigned char dsm[];
    const uint32_t ring_s = smem_u32(dsm);
    unsigned char* bar_mem = dsm + kDotStages * 2 * kDotStageChunks * 16;
    const uint32_t bars = smem_u32(bar_mem);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kDotStages + s); };
    bool* is_last = reinterpret_cast<bool*>(bar_mem + 2 * kDotStages * 8);
    float* warp_part = reinterpret_cast<float*>(bar_mem + 2 * kDotStages * 8 + 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long n_chunks = n_words >> 2;
    const long long c_begin = n_chunks * blockIdx.x / gridDim.x;
    const long long c_end = n_chunks * (blockIdx.x + 1) / gridDim.x;
    const int n_stage = (int)((c_end - c_begin + kDotStageChunks - 1) / kDotStageChunks);
    const uint4* a4 = reinterpret_cast<const uint4*>(a);
    const uint4* b4 = reinterpret_cast<const uint4*>(b);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kDotStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kDotWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDotWarps && pre_bytes > 0 && lane < 2) {
        // ahead of the stream-order wait: ask L2 for the start of both ranges
        // (safe whatever the kernel before this one still writes: L2 is where
        // writes to this GPU's memory land too)
        long long bytes = (c_end - c_begin) * 16;
        if (bytes > pre_bytes / 2) bytes = (pre_bytes / 2) & ~15;
        if (bytes > 0) bulk_prefetch_l2((lane ? b4 : a4) + c_begin, (uint32_t)bytes);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp == kDotWarps) {
        // ------------------------------------------------------- producer --
        // lanes 0..3 each issue one bulk copy per stage: A low half, A high
        // half, B low half, B high half
        int s = 0;
        uint32_t round = 0;
        bool alive = true;
        for (int st = 0; st < n_stage && alive; ++st) {
            if (round > 0 && !mbar_wait(empty_bar(s), (round & 1u) ^ 1u, status)) {
                alive = false;
                break;
            }
            const long long c0 = c_begin + (long long)st * kDotStageChunks;
            const int chunks = (int)min((long long)kDotStageChunks, c_end - c0);
            const int lo = min(chunks, kDotStageChunks / 2), hi = chunks - lo;
            if (lane == 0) mbar_arrive_expect_tx(full_bar(s), 2u * (uint32_t)chunks * 16u);
            __syncwarp();
            if (lane < 4) {
                const int op = lane >> 1, half = lane & 1;
                const int n = half ? hi : lo;
                if (n > 0)
                    bulk_load(ring_s + ((s * 2 + op) * kDotStageChunks + half * (kDotStageChunks / 2)) * 16,
                              (op ? b4 : a4) + c0 + half * (kDotStageChunks / 2), (uint32_t)n * 16u,
                              full_bar(s));
            }
            if (++s == kDotStages) { s = 0; ++round; }
        }
        if (!alive) {
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 1000000ull) {}
        }
    } else {
        // ------------------------------------------------------ consumers --
        int s = 0;
        uint32_t phase = 0;
        const uint4* ring4 = reinterpret_cast<const uint4*>(dsm);
        for (int st = 0; st < n_stage; ++st) {
            if (!mbar_wait(full_bar(s), phase, status)) break;
            const long long c0 = c_begin + (long long)st * kDotStageChunks;
            const int chunks = (int)min((long long)kDotStageChunks, c_end - c0);
            const uint4* sa = ring4 + (s * 2) * kDotStageChunks;
            const uint4* sb = sa + kDotStageChunks;
#pragma unroll
            for (int k = 0; k < kDotStageChunks / (kDotWarps * 32); ++k) {
                const int i = (k * kDotWarps + warp) * 32 + lane;
                if (i < chunks) {
                    const uint4 xa = sa[i], xb = sb[i];
                    dot_words<MODE>(xa.x, xb.x, acc);
                    dot_words<MODE>(xa.y, xb.y, acc);
                    dot_words<MODE>(xa.z, xb.z, acc);
                    dot_words<MODE>(xa.w, xb.w, acc);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
            if (++s == kDotStages) { s = 0; phase ^= 1u; }
        }
        if (blockIdx.x == 0 && threadIdx.x == 0)
            for (long long w = n_chunks << 2; w < n_words; ++w) dot_words<MODE>(__ldg(a + w), __ldg(b + w), acc);
        const float sum = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (lane == 0) warp_part[warp] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kDotWarps; ++w) t += warp_part[w];
        partial[blockIdx.x] = t;
        __threadfence();  // the partial is visible before the ticket is taken
        *is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!*is_last) return;
    // last CTA: the partials in index order over the consumer threads, then the
    // same fixed tree (warp_part was read before the barrier above, so it is free)
    __threadfence();
    float t = 0.f;
    if (warp < kDotWarps)
        for (int i = threadIdx.x; i < (int)gridDim.x; i += kDotWarps * 32) t += __ldcg(partial + i);
    t = warp_sum(t);
    if (lane == 0 && warp < kDotWarps) warp_part[warp] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < kDotWarps; ++w) r += warp_part[w];
        *out = r;
        *ticket = 0u;
    }
}

}  // namespace feather
