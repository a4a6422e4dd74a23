// Packed-FP8 GEMV against up to eight vectors in one pass over a LARGE matrix
// (sm_100a), the products on the tensor cores:
//
//   out[b, r] = sum_j decode(m[r, j]) * decode(v[b, j]),   b < B <= 8
//
// With several right-hand sides the work is a skinny matrix product, and the
// FP32 FMA pipe (gemv_multi_kernel) becomes the limit long before HBM does.
// Here the codes are still decoded in registers to FP16 pairs -- the decode is
// the reference kernels' own (feather/routines/gemv.py:31-34, :83-88), which for
// E4M3 is NOT the hardware's e4m3 (exponent-0 codes are m * 2^-17, 0x7F is 480),
// so the FP8 tensor-core formats cannot be fed the raw bytes -- and the decoded
// pairs go straight from registers into mma.sync.m16n8k16 (FP16 x FP16, FP32
// accumulate): 16 rows x 16 codes x 8 vectors per instruction.  Products are
// exact; the accumulation is the tensor core's (not IEEE round-to-nearest after
// every addition), so each warp spreads its steps over eight accumulator sets
// and adds them in FP32 at the end, which keeps the result within the tolerance
// the single-vector kernels are held to.
//
// Mapping.  A CTA owns 64 rows: warp w works on rows 16 * (w & 3) .. + 15 and on
// every other 64-code unit of them (w >> 2 picks even or odd units).  In a unit,
// lane (g, t) = (lane >> 2, lane & 3) loads the 16-byte chunk t of rows g and
// g + 8; word s of those chunks, decoded, is exactly the A fragment of the s-th
// mma (k slots 2t, 2t+1 and 2t+8, 2t+9 are the word's two FP16 pairs), and the
// B fragment is the same word of vector g, read from shared memory where the
// vectors' tiles sit decoded in the same pairing.  Any one-to-one assignment of
// codes to k slots is valid as long as A and B agree, so nothing is shuffled.
#pragma once
#include "gemv_kernels.cuh"

namespace feather {

constexpr int kMmaThreads = 256;
constexpr int kMmaCtaRows = 64;
constexpr int kMmaVectors = 8;
constexpr int kMmaTileCodes = 4096;                       // codes of each vector resident at a time
constexpr int kMmaVecStride = kMmaTileCodes * 2 + 16;     // bytes; the 16 spread the vectors over the banks
constexpr int kMmaSmemBytes = kMmaVectors * kMmaVecStride;
constexpr int kMmaUnroll = 4;                             // 64-code units in flight per warp

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Grid: one CTA per 64 rows.  v: B vectors of n16 * 4 words, one after the
// other; out: B rows of M floats.  Shared memory: kMmaSmemBytes.
template <int MODE, bool EARLY>
__global__ void __launch_bounds__(kMmaThreads, 2)
gemv_mma_kernel(const uint4* __restrict__ m, const uint32_t* __restrict__ v,
                float* __restrict__ out, int M, int n16, int B) {
    extern __shared__ __align__(16) unsigned char mma_smem[];
    __shared__ float part[4][16][kMmaVectors];            // the odd-unit warps' sums
    constexpr int U = kMmaUnroll;
    constexpr int kTileChunks = kMmaTileCodes / 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp & 3, split = warp >> 2;
    const int row_a = (int)blockIdx.x * kMmaCtaRows + group * 16 + g;
    const uint4* ra = m + (size_t)min(row_a, M - 1) * n16;      // rows past M: duplicates, never stored
    const uint4* rb = m + (size_t)min(row_a + 8, M - 1) * n16;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // unit k of this warp = global 64-code unit 2k + split = chunks 4 * (2k + split) .. + 3
    uint4 buf_a[U], buf_b[U];
    auto issue = [&](int slot, int k) {
        const int c = 4 * (2 * k + split) + t;
        const bool on = c < n16;
        buf_a[slot] = on ? ldg_stream(ra + c) : make_uint4(0, 0, 0, 0);
        buf_b[slot] = on ? ldg_stream(rb + c) : make_uint4(0, 0, 0, 0);
    };
    if (EARLY) {
#pragma unroll
        for (int u = 0; u < U; ++u) issue(u, u);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!EARLY) {
#pragma unroll
        for (int u = 0; u < U; ++u) issue(u, u);
    }

    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    // A batch is U = 4 units of this warp = 32 consecutive chunks of the row for
    // the two splits together, so the tile (256 chunks) is a whole number of
    // batches and a batch never straddles tiles.  Chunks past the row end are
    // zero codes against zero vector values.
    static_assert(U == 4 && kTileChunks % 32 == 0, "batches of 32 chunks must tile the vector tile");
    const unsigned char* vec_g = mma_smem + (size_t)g * kMmaVecStride;
    for (int t0 = 0; t0 < n16; t0 += kTileChunks) {
        const int tile_chunks = min(kTileChunks, n16 - t0);
        const int fill_chunks = (tile_chunks + 31) / 32 * 32;   // whole batches
        if (t0 > 0) __syncthreads();
        {   // stage the tile of all eight vectors as FP16 pairs, word after word;
            // vectors B..7 and the chunks past the row end are zero
            // (a thread takes the same word of all eight vectors: eight loads in flight)
            const int w_valid = tile_chunks * 4, w_fill = fill_chunks * 4;
            const uint32_t* src = v + (size_t)t0 * 4;
            for (int wl = threadIdx.x; wl < w_fill; wl += kMmaThreads) {
                uint32_t w[kMmaVectors];
#pragma unroll
                for (int b = 0; b < kMmaVectors; ++b)
                    w[b] = (b < B && wl < w_valid) ? __ldg(src + (size_t)b * n16 * 4 + wl) : 0u;
#pragma unroll
                for (int b = 0; b < kMmaVectors; ++b) {
                    uint32_t lo, hi;
                    decode_word_h2<MODE>(w[b], lo, hi);
                    reinterpret_cast<uint2*>(mma_smem + (size_t)b * kMmaVecStride)[wl] = make_uint2(lo, hi);
                }
            }
        }
        __syncthreads();
        const int k_end = t0 / 8 + fill_chunks / 8;           // this warp's units: k in [t0/8, k_end)
        for (int k = t0 / 8; k < k_end; k += U) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint4 xa = buf_a[u], xb = buf_b[u];
                issue(u, k + u + U);                          // refill the slot one batch ahead
                const int cl = 4 * (2 * (k + u) + split) + t - t0;   // chunk inside the tile
                const uint4 q0 = *reinterpret_cast<const uint4*>(vec_g + (size_t)cl * 32);
                const uint4 q1 = *reinterpret_cast<const uint4*>(vec_g + (size_t)cl * 32 + 16);
                uint32_t al, ah, bl, bh;
                decode_word_h2<MODE>(xa.x, al, ah);
                decode_word_h2<MODE>(xb.x, bl, bh);
                mma_16x8x16(acc[(u & 1) * 4 + 0], al, bl, ah, bh, q0.x, q0.y);
                decode_word_h2<MODE>(xa.y, al, ah);
                decode_word_h2<MODE>(xb.y, bl, bh);
                mma_16x8x16(acc[(u & 1) * 4 + 1], al, bl, ah, bh, q0.z, q0.w);
                decode_word_h2<MODE>(xa.z, al, ah);
                decode_word_h2<MODE>(xb.z, bl, bh);
                mma_16x8x16(acc[(u & 1) * 4 + 2], al, bl, ah, bh, q1.x, q1.y);
                decode_word_h2<MODE>(xa.w, al, ah);
                decode_word_h2<MODE>(xb.w, bl, bh);
                mma_16x8x16(acc[(u & 1) * 4 + 3], al, bl, ah, bh, q1.z, q1.w);
            }
        }
    }
    // accumulator sets in fixed order, then the two halves of the row
    float d[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        d[i] = ((acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i])) +
               ((acc[4][i] + acc[5][i]) + (acc[6][i] + acc[7][i]));
    if (split == 1) {
        part[group][g][2 * t] = d[0];
        part[group][g][2 * t + 1] = d[1];
        part[group][g + 8][2 * t] = d[2];
        part[group][g + 8][2 * t + 1] = d[3];
    }
    __syncthreads();
    if (split == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row_a + (i >> 1) * 8, b = 2 * t + (i & 1);
            if (row < M && b < B)
                out[(size_t)b * M + row] = d[i] + part[group][g + (i >> 1) * 8][b];
        }
    }
}

}  // namespace feather
