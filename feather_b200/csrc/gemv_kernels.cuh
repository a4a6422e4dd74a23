// Packed-FP8 GEMV kernels for sm_100a, small and mid-size matrices.
//
//   out[r] = sum_j decode(m[r, j]) * decode(v[j])      (FP32 products, FP32 sums)
//
// replaces the reference kernels feather/routines/gemv.py:8-61 (E5M2) and
// gemv.py:91-133 (E4M3).  Large matrices take gemv_ring_kernel (gemv_ring.cuh).
//
// gemv_rows_kernel (N % 16 == 0, 16-byte aligned rows)
//   * each WARP owns RW rows for all columns, so a row's sum never leaves the
//     warp: one shuffle butterfly per warp, no CTA-wide reduction;
//   * lanes stream 16-byte (128-bit) chunks with non-allocating loads, RW * U
//     of them in flight per lane;
//   * the vector is decoded once per CTA to FP16 pairs in shared memory (the
//     decoded values of both formats are FP16 numbers), conflict-free layout;
//   * codes are decoded in registers and multiplied with fma.rn.f32.f16 (FP16
//     operands, FP32 accumulator; the product is exact in FP32);
//   * launched with programmatic stream serialisation; with the static-matrix
//     promise the first matrix loads are issued before the stream-order wait.
//
//   * out_code >= 0: the FP32 sums are not stored; the CTA encodes its rows'
//     sums to FP8 codes of that format (the packer's rounding) and stores
//     packed words, four rows per word, row r in byte r % 4 of word r / 4 --
//     the packed vector the next GEMV of a chain consumes.
//
// gemv_general_kernel: any N % 4 == 0, 4-byte aligned; one warp per row, word
//   loads.  Used for ragged shapes.
#pragma once
#include <type_traits>
#include "gemv_common.cuh"

namespace feather {

// Shared memory of gemv_rows_kernel: the FP16 vector tile.
constexpr int kRowsTileCodes = 32768;                 // codes of the vector resident at a time
constexpr int kRowsThreads = 256;                     // 8 warps
constexpr int gemv_rows_smem_bytes(int n_codes) {
    return (n_codes < kRowsTileCodes ? ((n_codes + 511) / 512) * 512 : kRowsTileCodes) * 2;
}

// Grid: when the whole vector fits one tile (N <= kRowsTileCodes) any grid up to
// the number of row groups works and each CTA walks groups blockIdx.x,
// blockIdx.x + gridDim.x, ... with the vector staged once; otherwise the grid
// must equal the number of row groups (one group per CTA, tiles inside).
//
// ALLREDUCE: the column-sharded GEMV of a tensor-parallel layer.  Every rank
// holds a column slice of all M rows and the matching slice of the vector; its
// row sums are partial and the result is the sum over the ranks.  Each CTA
// exchanges ITS rows with the same CTA of every peer, through peer-mapped
// inboxes: a row sum travels as an 8-byte (value, call number) pair, two per
// 16-byte store, so the receiver polls the data itself -- no fence, no separate
// flag, one NVLink crossing.  The CTA then adds the ranks' sums in rank order
// and writes `ar.result`: the same bits on every rank, no collective launch.
// The call counter lives in device memory (flag word kArEpochWord), so a
// captured CUDA graph can be replayed.  `out` is ignored.  The grid must be one
// CTA per row group and fit the GPU at once (CTAs wait for their peers).
struct NoAllReduce {};
template <int MODE, int RW, int U, bool EARLY, bool ALLREDUCE = false>
__global__ void __launch_bounds__(kRowsThreads)
gemv_rows_kernel(const uint4* __restrict__ m, const uint32_t* __restrict__ v,
                 float* __restrict__ out, int M, int n16, int out_code,
                 const __grid_constant__ std::conditional_t<ALLREDUCE, AllReduceArgs, NoAllReduce> ar,
                 unsigned int* __restrict__ status, int pre) {
    extern __shared__ __align__(16) unsigned char rows_smem[];
    uint4* vec = reinterpret_cast<uint4*>(rows_smem);
    constexpr int kWarps = kRowsThreads / 32;
    constexpr int kTileChunks = kRowsTileCodes / 16;
    constexpr int kGroupRows = kWarps * RW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_groups = (M + kGroupRows - 1) / kGroupRows;
    int group = blockIdx.x;
    int row0 = (group * kWarps + warp) * RW;
    bool active = row0 < M;                           // warp-uniform
    const uint4* rows[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) rows[r] = m + (size_t)min(row0 + r, M - 1) * n16;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // first batch of matrix chunks; with the static-matrix promise they are
    // requested before the stream-order wait
    uint4 buf[U][RW];
    auto issue = [&](const uint4* const (&rp)[RW], bool on, int c0) {  // chunks c0 + u*32 + lane
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + u * 32 + lane;
#pragma unroll
            for (int r = 0; r < RW; ++r)
                buf[u][r] = (on && c < n16 && bounds_ok(rp[r] + c >= m && rp[r] + c < m + (size_t)M * n16))
                                ? ldg_stream(rp[r] + c) : make_uint4(0, 0, 0, 0);
        }
    };
    if (EARLY) issue(rows, active, 0);
    else if (pre && active && (lane & 7) == 0) {
        // without the promise: ask L2 for the lines of the first batch (one
        // request per 128-byte line).  A prefetch moves data from HBM into L2,
        // where every write to this GPU's memory lands too, so it cannot make
        // the loads after the wait see stale bytes.
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = u * 32 + lane;
#pragma unroll
            for (int r = 0; r < RW; ++r)
                if (c < n16) asm volatile("prefetch.global.L2 [%0];" ::"l"(rows[r] + c));
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!EARLY) issue(rows, active, 0);
    __shared__ float ar_part[kGroupRows];  // a CTA's row sums, for the all-reduce / packed output
    unsigned int epoch = 0;
    if constexpr (ALLREDUCE) {
        // this call's number: one more than the calls completed on this rank
        epoch = __ldcg(ar.flags[ar.rank] + kArEpochWord) + 1u;
        if (epoch == 0u) epoch = 2u;  // 0 is the tag of an untouched inbox; keep the parity
    }

    float acc[RW][4];
#pragma unroll
    for (int r = 0; r < RW; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    auto finish_rows = [&]() {  // butterfly over the warp, the row's lane writes
        if (active) {
            float sums[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) sums[r] = (acc[r][0] + acc[r][1]) + (acc[r][2] + acc[r][3]);
            warp_reduce_rows<RW>(sums, lane);
            if ((lane & (32 / RW - 1)) == 0) {
                const int row = row0 + lane / (32 / RW);
                if (ALLREDUCE || out_code >= 0) ar_part[warp * RW + lane / (32 / RW)] = row < M ? sums[0] : 0.f;
                else if (row < M && bounds_ok(row >= 0)) out[row] = sums[0];
            }
        } else if (ALLREDUCE || out_code >= 0) {
            if (lane < RW) ar_part[warp * RW + lane] = 0.f;
        }
        if (!ALLREDUCE && out_code >= 0) {  // CTA-uniform
            // rows past M encode as code 0, like the packer's zero-padded tail
            __syncthreads();
            const int cta_row0 = group * kGroupRows;
            if (threadIdx.x < kGroupRows / 4 && cta_row0 + 4 * (int)threadIdx.x < M) {
                uint32_t word = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float x = ar_part[4 * threadIdx.x + i];
                    const bool live = cta_row0 + 4 * (int)threadIdx.x + i < M;
                    const uint32_t c = out_code == kE5M2 ? encode_f32<kE5M2>(x) : encode_f32<kE4M3>(x);
                    word |= (live ? c : 0u) << (8 * i);
                }
                if (bounds_ok(cta_row0 / 4 + (int)threadIdx.x < (M + 3) / 4))
                    reinterpret_cast<uint32_t*>(out)[cta_row0 / 4 + threadIdx.x] = word;
            }
            __syncthreads();  // ar_part is free for the next row group
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    };
    // stage `tile_chunks` chunks of the vector from chunk t0 as FP16 pairs:
    // (group g, half k, lane l) is the uint4 at (g*2 + k)*32 + l and holds
    // codes 16*(32g+l) + 8k .. +7; the last group is padded with zero codes
    auto stage = [&](int t0, int tile_chunks) {
        uint2* vec2 = reinterpret_cast<uint2*>(vec);
        const int w_valid = tile_chunks * 4, w_fill = ((tile_chunks + 31) / 32) * 128;
        for (int wl = threadIdx.x; wl < w_fill; wl += kRowsThreads) {
            uint32_t lo, hi;
            decode_word_h2<MODE>(wl < w_valid && bounds_ok(t0 * 4 + wl < n16 * 4) ? __ldg(v + t0 * 4 + wl) : 0u,
                                 lo, hi);
            const int chunk = wl >> 2, k = wl & 3;
            vec2[(((chunk >> 5) * 2 + (k >> 1)) * 32 + (chunk & 31)) * 2 + (k & 1)] = make_uint2(lo, hi);
        }
    };
    // one batch: U groups of 32 chunks starting at tile-local chunk `cl0`
    auto compute = [&](const uint4 (&cur)[U][RW], int cl0, int tile_chunks) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int cl = cl0 + u * 32;
            if (cl < tile_chunks) {  // warp-uniform; lanes past N hold zero codes
                const uint4 va = vec[((cl >> 5) * 2) * 32 + lane];
                const uint4 vb = vec[((cl >> 5) * 2 + 1) * 32 + lane];
#pragma unroll
                for (int r = 0; r < RW; ++r) fma_chunk<MODE>(cur[u][r], va, vb, acc[r]);
            }
        }
    };

    if (n16 <= kTileChunks) {
        // the whole vector is resident: walk this CTA's row groups, always one
        // batch of loads ahead (across the group boundary too)
        stage(0, n16);
        __syncthreads();
        while (group < n_groups) {
            const int next = group + (int)gridDim.x;
            const int next_row0 = (next * kWarps + warp) * RW;
            const bool next_active = next < n_groups && next_row0 < M;
            const uint4* next_rows[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) next_rows[r] = m + (size_t)min(next_row0 + r, M - 1) * n16;
            for (int c0 = 0; c0 < n16; c0 += U * 32) {
                uint4 cur[U][RW];
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int r = 0; r < RW; ++r) cur[u][r] = buf[u][r];
                if (c0 + U * 32 < n16) issue(rows, active, c0 + U * 32);
                else issue(next_rows, next_active, 0);
                compute(cur, c0, n16);
            }
            finish_rows();
            group = next;
            row0 = next_row0;
            active = next_active;
#pragma unroll
            for (int r = 0; r < RW; ++r) rows[r] = next_rows[r];
        }
    } else {
    // long rows: one row group per CTA, the vector in tiles
    for (int t0 = 0; t0 < n16; t0 += kTileChunks) {
        const int tile_chunks = min(kTileChunks, n16 - t0);
        if (t0 > 0) __syncthreads();
        stage(t0, tile_chunks);
        __syncthreads();
        const int c_end = t0 + tile_chunks;
        for (int c0 = t0; c0 < c_end; c0 += U * 32) {
            uint4 cur[U][RW];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < RW; ++r) cur[u][r] = buf[u][r];
            issue(rows, active, c0 + U * 32);  // next batch (zeros past the end of the rows)
            compute(cur, c0 - t0, tile_chunks);
        }
    }
    finish_rows();
    }
    if constexpr (ALLREDUCE) {
        // ---- exchange this CTA's rows with the peers' same CTA and add ----
        constexpr int kPieces = kGroupRows / 2;            // 16-byte pieces: two (sum, tag) pairs
        __shared__ float ar_recv[kMaxArRanks][kGroupRows];
        const int cta_row0 = (int)blockIdx.x * kGroupRows;
        const size_t slot = 2 * (((size_t)M + 15) / 16 * 16);  // floats per rank slot
        const size_t half0 = (size_t)(epoch & 1u) * ar.half;   // this call's half of an inbox
        __syncthreads();                                    // ar_part is complete
        for (int t = threadIdx.x; t < ar.world * kPieces; t += kRowsThreads) {
            const int q = t / kPieces, j = t - q * kPieces;
            const float s0 = ar_part[2 * j], s1 = ar_part[2 * j + 1];
            if (q == ar.rank) {
                ar_recv[q][2 * j] = s0;
                ar_recv[q][2 * j + 1] = s1;
                continue;
            }
            // my sums into rank q's inbox, slot `rank` ...
            st_volatile_v4(ar.inbox[q] + half0 + (size_t)ar.rank * slot + 2 * (size_t)(cta_row0 + 2 * j),
                           make_uint4(__float_as_uint(s0), epoch, __float_as_uint(s1), epoch));
        }
        for (int t = threadIdx.x; t < ar.world * kPieces; t += kRowsThreads) {
            const int q = t / kPieces, j = t - q * kPieces;
            if (q == ar.rank) continue;
            // ... and rank q's sums out of my inbox, slot q, once both tags say "this call"
            const float* src = ar.inbox[ar.rank] + half0 + (size_t)q * slot + 2 * (size_t)(cta_row0 + 2 * j);
            uint4 x = ld_volatile_v4(src);
            if (x.y != epoch || x.w != epoch) {
                const unsigned long long t0 = global_timer_ns();
                do {
                    x = ld_volatile_v4(src);
                    if (global_timer_ns() - t0 > kWaitLimitNs) {
                        atomicOr(status, 2u);  // rank q's sums did not arrive in time
                        break;
                    }
                } while (x.y != epoch || x.w != epoch);
            }
            ar_recv[q][2 * j] = __uint_as_float(x.x);
            ar_recv[q][2 * j + 1] = __uint_as_float(x.z);
        }
        __syncthreads();
        if (threadIdx.x < kGroupRows && cta_row0 + (int)threadIdx.x < M) {
            float t = ar_recv[0][threadIdx.x];  // rank 0's sum, then the others in rank order
            for (int q = 1; q < ar.world; ++q) t += ar_recv[q][threadIdx.x];
            ar.result[cta_row0 + threadIdx.x] = t;
        }
        // the CTA that finishes last records the call as completed
        if (threadIdx.x == 0) {
            unsigned int* my_flags = ar.flags[ar.rank];
            if (atomicAdd(my_flags + kArTicketWord, 1u) == gridDim.x - 1) {
                my_flags[kArTicketWord] = 0u;
                my_flags[kArEpochWord] = epoch;
            }
        }
    }
}

// One warp per row, 4-byte loads: every N % 4 == 0, any 4-byte alignment.
template <int MODE>
__global__ void __launch_bounds__(256)
gemv_general_kernel(const uint32_t* __restrict__ m, const uint32_t* __restrict__ v,
                    float* __restrict__ out, int M, int n_words) {
    const int lane = threadIdx.x & 31;
    const long long warp_global = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp_global; row < M; row += n_warps) {
        const uint32_t* mr = m + (size_t)row * n_words;
        float2 a0 = make_float2(0.f, 0.f), a1 = a0;
        for (int w = lane; w < n_words; w += 32) {
            if (!bounds_ok(row >= 0 && row < M && w < n_words)) break;
            float2 mlo, mhi, vlo, vhi;
            decode_word<MODE>(__ldg(mr + w), mlo, mhi);
            decode_word<MODE>(__ldg(v + w), vlo, vhi);
            a0 = __ffma2_rn(mlo, vlo, a0);
            a1 = __ffma2_rn(mhi, vhi, a1);
        }
        const float s = warp_sum((a0.x + a0.y) + (a1.x + a1.y));
        if (lane == 0) out[row] = s;
    }
}

}  // namespace feather
