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
// Mapping.  A CTA works on up to 8 groups of 16 rows at a time, two warps per
// group: warp w takes group w >> 1 and every other 128-code unit of its rows
// (w & 1 picks even or odd units).  For the mma, lane (g, t) = (lane >> 2,
// lane & 3) supplies rows g and g + 8: word s of their 16-byte chunk t (and of
// chunk 4 + t for the second half of the unit), decoded, is exactly the A
// fragment of one mma (k slots 2t, 2t+1 and 2t+8, 2t+9 are the word's two FP16
// pairs), and the B fragment is the same word of vector g, read from shared
// memory where the vectors' tiles sit decoded in the same pairing.  Any
// one-to-one assignment of codes to k slots is valid as long as A and B agree,
// so nothing is shuffled.
//
// Streaming.  A warp copies a unit with four cp.async instructions (16 bytes per
// lane, L2 only; eight lanes cover the 128 bytes of one row, so every request is
// a whole line) into a slot of its own ring, kMmaDepth units ahead, and its lanes
// read their fragments back from the slot (rows XOR-swizzled by parity so the
// quarter-warps do not collide on banks): no registers are held by loads in
// flight and the only synchronisation is cp.async.wait_group + __syncwarp -- a
// CTA (one per SM, sixteen warps) keeps up to 128 KiB of the matrix in flight.
// The grid is persistent; groups per CTA are chosen so that the waves are full.
#pragma once
#include "gemv_kernels.cuh"
#include "gemv_ring.cuh"  // mbarrier helpers with bounded waits

namespace feather {

constexpr int kMmaWarps = 16;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaMaxGroups = kMmaWarps / 2;              // 16-row groups a CTA works on at a time
constexpr int kMmaVectors = 8;
constexpr int kMmaTileCodes = 1024;                       // codes of each vector in a tile (three tiles resident)
constexpr int kMmaTileBuffers = 3;
constexpr int kMmaVecStride = kMmaTileCodes * 2 + 16;     // bytes; the 16 spread the vectors over the banks
constexpr int kMmaTileBytes = 8 * kMmaVecStride;          // one tile of all eight vectors
constexpr int kMmaDepth = 5;                              // units a warp keeps in flight
constexpr int kMmaSlotBytes = 16 * 128;                   // a unit of a warp: 128 bytes of each of its 16 rows
constexpr int kMmaRingOffset = kMmaTileBuffers * kMmaTileBytes;
constexpr int kMmaSmemBytes = kMmaRingOffset + kMmaWarps * kMmaDepth * kMmaSlotBytes;

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared, not through L1; n_src = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* src, int n_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_dst), "l"(src), "r"(n_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Grid: any size up to the number of passes; pass p covers row groups
// [p * gpc, (p + 1) * gpc), CTAs take passes blockIdx.x, blockIdx.x + gridDim.x, ...
// v: B vectors of n16 * 4 words, one after the other; out: B rows of M floats.
template <int MODE, bool EARLY>
__global__ void __launch_bounds__(kMmaThreads, 1)
gemv_mma_kernel(const uint4* __restrict__ m, const uint32_t* __restrict__ v,
                float* __restrict__ out, int M, int n16, int B, int gpc,
                unsigned int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char mma_smem[];
    __shared__ float part[2][kMmaMaxGroups][16][kMmaVectors]; // the odd-unit warps' sums, by pass parity
    __shared__ __align__(8) unsigned long long tile_bar[kMmaTileBuffers];  // "tile staged" per buffer
    constexpr int D = kMmaDepth;
    constexpr int kTileChunks = kMmaTileCodes / 16;
    static_assert(kTileChunks % 16 == 0, "a tile is a whole number of unit pairs");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp >> 1, split = warp & 1;
    const bool working = group < gpc;                         // warp-uniform
    const int n_groups = (M + 15) / 16;
    const int n_pass = (n_groups + gpc - 1) / gpc;
    // the warp's ring: [slot][row 0..15][128 bytes, chunk c of row r at c ^ 4 * (r & 1)]
    unsigned char* ring_ptr = mma_smem + kMmaRingOffset + warp * (D * kMmaSlotBytes);
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_ptr);
    // copy role: this lane moves chunk lane & 7 of rows (lane >> 3) + 0, 4, 8, 12
    const int cp_row = lane >> 3, cp_chunk = lane & 7;
    const uint32_t cp_dst = cp_row * 128 + ((cp_chunk ^ ((cp_row & 1) << 2)) << 4);   // + 512 per 4 rows
    // fragment role: chunks t (first half of the unit) and 4 + t (second half) of rows
    // g and g + 8, which have the same parity and so the same swizzle
    const int frag_off0 = g * 128 + (((0 + t) ^ ((g & 1) << 2)) << 4);
    const int frag_off1 = g * 128 + (((4 + t) ^ ((g & 1) << 2)) << 4);

    // Vector tiles: three buffers, a sequence of tiles that runs on across passes.
    // Every thread owns one word of four vectors' tile: it loads those words of
    // tile s + 2 before the CTA computes tile s and decodes them into buffer
    // (s + 1) % 3 one step later, then arrives on that buffer's mbarrier; a warp
    // starts tile s once all 512 threads have arrived for it.  Nobody waits at a
    // CTA-wide barrier: the arrivals a warp needs happened a whole compute step
    // earlier.  Vectors B..7 and chunks past the row end are zero.
    static_assert(kMmaTileCodes / 4 * 2 == kMmaThreads, "a word of four vectors' tile per thread");
    const int st_word = threadIdx.x & (kMmaTileCodes / 4 - 1);    // staging role: this word ...
    const int st_vec = (threadIdx.x / (kMmaTileCodes / 4)) * 4;   // ... of these four vectors
    uint32_t w[4];
    int fetch_t0 = 0;                                             // first chunk of the next tile to fetch
    auto fetch_tile = [&]() {
        const bool on = st_word < min(kTileChunks, n16 - fetch_t0) * 4;
#pragma unroll
        for (int b = 0; b < 4; ++b)
            w[b] = (on && st_vec + b < B) ? __ldg(v + ((size_t)(st_vec + b) * n16 + fetch_t0) * 4 + st_word) : 0u;
        fetch_t0 += kTileChunks;
        if (fetch_t0 >= n16) fetch_t0 = 0;                        // on to the next pass: same vectors
    };
    auto store_tile = [&](int buffer) {   // what fetch_tile loaded last; every thread arrives
        unsigned char* tile_smem = mma_smem + buffer * kMmaTileBytes;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t lo, hi;
            decode_word_h2<MODE>(w[b], lo, hi);
            reinterpret_cast<uint2*>(tile_smem + (size_t)(st_vec + b) * kMmaVecStride)[st_word] = make_uint2(lo, hi);
        }
        mbar_arrive(smem_u32(&tile_bar[buffer]));
    };
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < kMmaTileBuffers; ++i) mbar_init(smem_u32(&tile_bar[i]), kMmaThreads);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    bool waited = false;
    int buf = 0;                                              // buffer of the tile being computed
    uint32_t phases = 0;                                      // bit i: parity to wait for on buffer i
    for (int pass = blockIdx.x, n_done = 0; pass < n_pass; pass += gridDim.x, ++n_done) {
        const int row0 = (pass * gpc + group) * 16;
        const int row_a = row0 + g;
        const uint4* cp_src = m + (size_t)min(row0 + cp_row, M - 1) * n16;
        // unit k of this warp = chunks 8 * (2k + split) .. + 7 of its rows; one commit
        // group per unit.  Rows past M and chunks past the row end are zero-filled.
        auto issue = [&](int k) {
            if (working) {
                const int c = 8 * (2 * k + split) + cp_chunk;
                const uint32_t slot = ring + (k % D) * kMmaSlotBytes + cp_dst;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool on = c < n16 && row0 + cp_row + 4 * i < M;
                    cp_async_16(slot + i * 512, on ? cp_src + (size_t)i * 4 * n16 + c : m, on ? 16 : 0);
                }
            }
            cp_async_commit();
        };
        if (EARLY || waited) {
#pragma unroll
            for (int k = 0; k < D; ++k) issue(k);
        }
        if (!waited) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
            if (!EARLY) {
#pragma unroll
                for (int k = 0; k < D; ++k) issue(k);
            }
            fetch_tile();                // the vectors may come from the kernel before: after the wait
            store_tile(0);
            fetch_tile();
        }

        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

        for (int t0 = 0; t0 < n16; t0 += kTileChunks) {
            const int tile_chunks = min(kTileChunks, n16 - t0);
            const int fill_chunks = (tile_chunks + 15) / 16 * 16;   // whole units for both warps of a group
            // this tile is staged (by everybody, one compute step ago)
            mbar_wait(smem_u32(&tile_bar[buf]), (phases >> buf) & 1u, status);
            phases ^= 1u << buf;
            const unsigned char* vec_g = mma_smem + buf * kMmaTileBytes + (size_t)g * kMmaVecStride;
            buf = buf == kMmaTileBuffers - 1 ? 0 : buf + 1;
            store_tile(buf);             // the next tile; its buffer was last read two tiles ago
            fetch_tile();                // the tile after it, in flight while this one is computed
            if (!working) continue;
            // this warp's units inside the tile: k in [t0 / 16, t0 / 16 + fill_chunks / 16)
            const int k_end = t0 / 16 + fill_chunks / 16;
            for (int k = t0 / 16; k < k_end; ++k) {
                cp_async_wait<D - 1>();                             // this lane's part of unit k has landed
                __syncwarp();                                       // ... and everybody else's
                const unsigned char* slot = ring_ptr + (k % D) * kMmaSlotBytes;
                uint4 xa[2], xb[2];
                xa[0] = *reinterpret_cast<const uint4*>(slot + frag_off0);
                xb[0] = *reinterpret_cast<const uint4*>(slot + frag_off0 + 8 * 128);
                xa[1] = *reinterpret_cast<const uint4*>(slot + frag_off1);
                xb[1] = *reinterpret_cast<const uint4*>(slot + frag_off1 + 8 * 128);
                __syncwarp();                                       // the slot is read: refill it
                issue(k + D);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int cl = 8 * (2 * k + split) + 4 * u + t - t0;   // chunk inside the tile
                    const uint4 q0 = *reinterpret_cast<const uint4*>(vec_g + (size_t)cl * 32);
                    const uint4 q1 = *reinterpret_cast<const uint4*>(vec_g + (size_t)cl * 32 + 16);
                    float (*a)[4] = acc + 4 * u;
                    uint32_t al, ah, bl, bh;
                    decode_word_h2<MODE>(xa[u].x, al, ah);
                    decode_word_h2<MODE>(xb[u].x, bl, bh);
                    mma_16x8x16(a[0], al, bl, ah, bh, q0.x, q0.y);
                    decode_word_h2<MODE>(xa[u].y, al, ah);
                    decode_word_h2<MODE>(xb[u].y, bl, bh);
                    mma_16x8x16(a[1], al, bl, ah, bh, q0.z, q0.w);
                    decode_word_h2<MODE>(xa[u].z, al, ah);
                    decode_word_h2<MODE>(xb[u].z, bl, bh);
                    mma_16x8x16(a[2], al, bl, ah, bh, q1.x, q1.y);
                    decode_word_h2<MODE>(xa[u].w, al, ah);
                    decode_word_h2<MODE>(xb[u].w, bl, bh);
                    mma_16x8x16(a[3], al, bl, ah, bh, q1.z, q1.w);
                }
            }
        }
        cp_async_wait<0>();   // only zero-fill copies past the row end are left; the ring is free again

        // accumulator sets in fixed order, then the two halves of the row
        float d[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            d[i] = ((acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i])) +
                   ((acc[4][i] + acc[5][i]) + (acc[6][i] + acc[7][i]));
        float (*pp)[16][kMmaVectors] = part[n_done & 1];
        if (working && split == 1) {
            pp[group][g][2 * t] = d[0];
            pp[group][g][2 * t + 1] = d[1];
            pp[group][g + 8][2 * t] = d[2];
            pp[group][g + 8][2 * t + 1] = d[3];
        }
        __syncthreads();
        if (working && split == 0 && pass * gpc + group < n_groups) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = row_a + (i >> 1) * 8, b = 2 * t + (i & 1);
                if (row < M && b < B)
                    out[(size_t)b * M + row] = d[i] + pp[group][g + (i >> 1) * 8][b];
            }
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace feather
