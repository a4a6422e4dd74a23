// Packed-FP8 GEMV against several vectors in one pass over the matrix (sm_100a):
//
//   out[b, r] = sum_j decode(m[r, j]) * decode(v[b, j]),   b < B <= NB
//
// The reference multiplies one vector per launch (feather/routines/gemv.py:8-61,
// :91-133), so B right-hand sides stream the matrix B times; here every 16-byte
// chunk of a row is loaded and decoded once and multiplied with all B vectors.
// Same structure as gemv_rows_kernel: a warp owns two rows, lanes stream 128-bit
// chunks with non-allocating loads, the vectors sit in shared memory as FP16
// pairs (NB tiles of kRowsTileCodes / NB codes), products are exact
// (fma.rn.f32.f16), each (row, vector) sum is accumulated in the same order as
// the single-vector kernel, so out[b] has the bits of a single GEMV with v[b]
// wherever that GEMV takes gemv_rows_kernel.
#pragma once
#include "gemv_kernels.cuh"

namespace feather {

// 16 codes of a row as eight FP16 pairs, in decode_word_h2's pairing.
template <int MODE>
__device__ __forceinline__ void decode_chunk_h2(const uint4 mw, uint32_t (&h)[8]) {
    decode_word_h2<MODE>(mw.x, h[0], h[1]);
    decode_word_h2<MODE>(mw.y, h[2], h[3]);
    decode_word_h2<MODE>(mw.z, h[4], h[5]);
    decode_word_h2<MODE>(mw.w, h[6], h[7]);
}

// The FMA sequence of fma_chunk on an already decoded chunk.
__device__ __forceinline__ void fma_decoded(const uint32_t (&h)[8], const uint4 va, const uint4 vb,
                                            float (&acc)[4]) {
    fma_h2(h[0], va.x, acc[0], acc[1]);
    fma_h2(h[1], va.y, acc[2], acc[3]);
    fma_h2(h[2], va.z, acc[0], acc[1]);
    fma_h2(h[3], va.w, acc[2], acc[3]);
    fma_h2(h[4], vb.x, acc[0], acc[1]);
    fma_h2(h[5], vb.y, acc[2], acc[3]);
    fma_h2(h[6], vb.z, acc[0], acc[1]);
    fma_h2(h[7], vb.w, acc[2], acc[3]);
}

// Shared memory: nb vector regions of FP16 values, each the row length rounded up to
// 512 codes but no more than the tile of kRowsTileCodes / nb codes.
constexpr int gemv_multi_smem_bytes(int n_codes, int nb) {
    const int padded = (n_codes + 511) / 512 * 512;
    const int tile = kRowsTileCodes / nb;
    return nb * (padded < tile ? padded : tile) * 2;
}

// Grid: one CTA per group of 16 rows.  v: B vectors of n16 * 4 words each, one
// after the other; out: B rows of M floats.  Vectors B..NB-1 do not exist: their
// tiles are zero and nothing is stored for them.
template <int MODE, int NB, bool EARLY>
__global__ void __launch_bounds__(kRowsThreads)
gemv_multi_kernel(const uint4* __restrict__ m, const uint32_t* __restrict__ v,
                  float* __restrict__ out, int M, int n16, int B) {
    extern __shared__ __align__(16) unsigned char rows_smem[];
    constexpr int RW = 2, U = 2;
    constexpr int kWarps = kRowsThreads / 32;
    constexpr int kTileChunks = kRowsTileCodes / 16 / NB;  // chunks of one vector resident at a time
    // uint4 per vector region (FP16: 32 B per chunk), no more than the rows need
    const int kTileVec = min(kTileChunks, (n16 + 31) / 32 * 32) * 2;
    uint4* vec = reinterpret_cast<uint4*>(rows_smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = ((int)blockIdx.x * kWarps + warp) * RW;
    const bool active = row0 < M;                           // warp-uniform
    const uint4* rows[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) rows[r] = m + (size_t)min(row0 + r, M - 1) * n16;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4 buf[U][RW];
    auto issue = [&](int c0) {  // chunks c0 + u*32 + lane of this warp's rows
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + u * 32 + lane;
#pragma unroll
            for (int r = 0; r < RW; ++r)
                buf[u][r] = (active && c < n16) ? ldg_stream(rows[r] + c) : make_uint4(0, 0, 0, 0);
        }
    };
    if (EARLY) issue(0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!EARLY) issue(0);

    float acc[RW][NB][4];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b][0] = acc[r][b][1] = acc[r][b][2] = acc[r][b][3] = 0.f;

    for (int t0 = 0; t0 < n16; t0 += kTileChunks) {
        const int tile_chunks = min(kTileChunks, n16 - t0);
        if (t0 > 0) __syncthreads();
        {   // stage the tile of every vector (gemv_rows_kernel's layout, one region per vector)
            const int w_valid = tile_chunks * 4, w_fill = ((tile_chunks + 31) / 32) * 128;
            for (int b = 0; b < NB; ++b) {
                uint2* vec2 = reinterpret_cast<uint2*>(vec + (size_t)b * kTileVec);
                const uint32_t* vb = v + (size_t)b * n16 * 4 + (size_t)t0 * 4;
                for (int wl = threadIdx.x; wl < w_fill; wl += kRowsThreads) {
                    uint32_t lo, hi;
                    decode_word_h2<MODE>((b < B && wl < w_valid) ? __ldg(vb + wl) : 0u, lo, hi);
                    const int chunk = wl >> 2, k = wl & 3;
                    vec2[(((chunk >> 5) * 2 + (k >> 1)) * 32 + (chunk & 31)) * 2 + (k & 1)] = make_uint2(lo, hi);
                }
            }
        }
        __syncthreads();
        const int c_end = t0 + tile_chunks;
        for (int c0 = t0; c0 < c_end; c0 += U * 32) {
            uint4 cur[U][RW];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < RW; ++r) cur[u][r] = buf[u][r];
            issue(c0 + U * 32);  // next batch (zeros past the end of the rows)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int cl = c0 - t0 + u * 32;
                if (cl < tile_chunks) {  // warp-uniform; lanes past N hold zero codes
                    uint32_t h[RW][8];
#pragma unroll
                    for (int r = 0; r < RW; ++r) decode_chunk_h2<MODE>(cur[u][r], h[r]);
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        const uint4 va = vec[(size_t)b * kTileVec + ((cl >> 5) * 2) * 32 + lane];
                        const uint4 vb = vec[(size_t)b * kTileVec + ((cl >> 5) * 2 + 1) * 32 + lane];
#pragma unroll
                        for (int r = 0; r < RW; ++r) fma_decoded(h[r], va, vb, acc[r][b]);
                    }
                }
            }
        }
    }
    if (!active) return;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        float sums[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r)
            sums[r] = (acc[r][b][0] + acc[r][b][1]) + (acc[r][b][2] + acc[r][b][3]);
        warp_reduce_rows<RW>(sums, lane);
        if (b < B && (lane & (32 / RW - 1)) == 0) {
            const int row = row0 + lane / (32 / RW);
            if (row < M) out[(size_t)b * M + row] = sums[0];
        }
    }
}

}  // namespace feather
