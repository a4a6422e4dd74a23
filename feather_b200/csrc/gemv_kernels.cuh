// Packed-FP8 GEMV kernels for sm_100a.
//
//   out[r] = sum_j decode(m[r, j]) * decode(v[j])      (FP32 products, FP32 sums)
//
// replaces the reference kernels feather/routines/gemv.py:8-61 (E5M2) and
// gemv.py:91-133 (E4M3).  The work is HBM-bound integer/byte streaming: one
// byte of matrix per multiply-add, no reuse, so there are no tensor cores here.
//
// gemv_stream_kernel (fast path, N % 16 == 0, 16-byte aligned rows)
//   * persistent grid: a multiple of the SM count; each CTA owns a contiguous
//     block of rows and walks it in groups of R rows;
//   * the vector is decoded to FP32 ONCE per CTA per column tile into shared
//     memory, laid out so that every lane's float4 reads are conflict-free;
//   * all warps of a CTA split the columns of the same R rows, each lane
//     streams 16-byte (128-bit) chunks with non-allocating loads, R of them
//     per step plus the next step's R prefetched, so the matrix bytes in
//     flight do not depend on the reduction at the end of a row group;
//   * codes are decoded in registers (prmt / shifts / masks, fp8_codec.cuh),
//     multiplied with packed FP32 FMAs (fma.rn.f32x2), reduced with warp
//     shuffles and one shared-memory step across the warps.
//   Products of two decoded values are exact in FP32, so only the summation
//   order differs from the reference (whose order is unspecified as well).
//
// gemv_general_kernel: any N % 4 == 0, 4-byte aligned; one warp per row, word
//   loads.  Used for ragged shapes and tiny matrices.
#pragma once
#include "fp8_codec.cuh"

namespace feather {

// Shared memory of gemv_stream_kernel: the FP32 vector tile, then two
// buffers of WARPS x R partial sums.
constexpr int gemv_stream_smem_bytes(int tile_codes, int warps, int rows) {
    return tile_codes * 4 + 2 * warps * rows * 4;
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
    return x;
}

// Position of one step of a warp's walk: column tile, row group inside the
// CTA's row block, column step inside the tile.
struct Cursor {
    int tile, task, step;
};
template <int V>
struct IntTag {
    static constexpr int value = V;
};

// TILE_CODES: codes of the vector resident (as FP32) at a time; a multiple of 512.
template <int MODE, int WARPS, int R, int MIN_CTAS, int TILE_CODES>
__global__ void __launch_bounds__(WARPS * 32, MIN_CTAS)
gemv_stream_kernel(const uint4* __restrict__ m, const uint32_t* __restrict__ v,
                   float* __restrict__ out, int M, int n16) {
    constexpr int kTileCodes = TILE_CODES;
    constexpr int kTileChunks = kTileCodes / 16;   // 16-byte chunks per tile
    constexpr int kTileGroups = kTileChunks / 32;  // warp-wide groups per tile
    constexpr int kVecSmemBytes = kTileCodes * 4;
    static_assert(TILE_CODES % 512 == 0, "tile must hold whole warp-wide groups");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4* vec = reinterpret_cast<float4*>(smem_raw);  // kTileCodes floats
    float* red = reinterpret_cast<float*>(smem_raw + kVecSmemBytes);  // [2][WARPS][R]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // contiguous row block of this CTA
    const int row_begin = (int)(((long long)M * blockIdx.x) / gridDim.x);
    const int row_end = (int)(((long long)M * (blockIdx.x + 1)) / gridDim.x);
    const int n_tasks = (row_end - row_begin + R - 1) / R;
    if (n_tasks == 0) return;
    const int n_tiles = (n16 + kTileChunks - 1) / kTileChunks;
    // column steps per (tile, task): the widest tile decides; narrower tiles
    // mask the excess.  Every warp executes the same number of steps.
    const int tile_groups = min(kTileGroups, (n16 + 31) / 32);
    const int steps = (tile_groups + WARPS - 1) / WARPS;

    auto advance = [&](Cursor& c) {
        if (++c.step == steps) {
            c.step = 0;
            if (++c.task == n_tasks) { c.task = 0; ++c.tile; }
        }
    };
    auto issue = [&](const Cursor& c, uint4 (&buf)[R]) {
        const int q_local = (warp + c.step * WARPS) * 32 + lane;
        const int q = c.tile * kTileChunks + q_local;
        const bool ok = (c.tile < n_tiles) && (q_local < kTileChunks) && (q < n16);
        const int row0 = row_begin + c.task * R;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = min(row0 + r, row_end - 1);
            buf[r] = ok ? ldg_stream(m + (size_t)row * n16 + q) : make_uint4(0, 0, 0, 0);
        }
    };

    Cursor pre = {0, 0, 0}, cur = {0, 0, 0};
    uint4 buf[2][R];
    issue(pre, buf[0]);  // matrix bytes are on their way before the vector is staged
    advance(pre);

    float2 acc[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = make_float2(0.f, 0.f);

    int red_buf = 0;
    // One step of the walk; PAR selects which half of `buf` is consumed (the
    // other half receives the prefetch), so register indices stay static.
    auto step_fn = [&](auto par_tag) {
        constexpr int PAR = decltype(par_tag)::value;
        if (cur.task == 0 && cur.step == 0) {
            // stage this column tile of the vector: decode to FP32, permuted so
            // that (group g, quarter k, lane l) is one float4 at (g*4 + k)*32 + l
            // and holds the values in decode_word's pair order.
            __syncthreads();  // everyone is done reading the previous tile
            const int w_begin = cur.tile * (kTileCodes / 4);
            const int w_end = min(n16 * 4, w_begin + kTileCodes / 4);
            const int w_fill = w_begin + min(steps * WARPS * 128, kTileCodes / 4);
            for (int w = w_begin + threadIdx.x; w < w_fill; w += WARPS * 32) {
                float2 lo = make_float2(0.f, 0.f), hi = lo;  // beyond N: zeros
                if (w < w_end) decode_word<MODE>(__ldg(v + w), lo, hi);
                const int wl = w - w_begin, chunk = wl >> 2, k = wl & 3;
                vec[((chunk >> 5) * 4 + k) * 32 + (chunk & 31)] = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
            __syncthreads();
        }
        // prefetch the next step, then consume the current one
        issue(pre, buf[PAR ^ 1]);
        advance(pre);

        const int g = warp + cur.step * WARPS;
        if (g < kTileGroups) {
            const float4* vs = vec + (g * 4) * 32 + lane;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 vv = vs[k * 32];
                const float2 v_lo = make_float2(vv.x, vv.y), v_hi = make_float2(vv.z, vv.w);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint4 mw = buf[PAR][r];
                    const uint32_t word = k == 0 ? mw.x : k == 1 ? mw.y : k == 2 ? mw.z : mw.w;
                    float2 lo, hi;
                    decode_word<MODE>(word, lo, hi);
                    acc[r][0] = __ffma2_rn(lo, v_lo, acc[r][0]);
                    acc[r][1] = __ffma2_rn(hi, v_hi, acc[r][1]);
                }
            }
        }

        if (cur.step == steps - 1) {
            // end of a row group: reduce R sums over the CTA
            float s[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                s[r] = warp_sum((acc[r][0].x + acc[r][0].y) + (acc[r][1].x + acc[r][1].y));
                acc[r][0] = acc[r][1] = make_float2(0.f, 0.f);
            }
            float* rb = red + red_buf * (WARPS * R);
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) rb[warp * R + r] = s[r];
            }
            __syncthreads();
            if (threadIdx.x < R) {
                const int row = row_begin + cur.task * R + threadIdx.x;
                if (row < row_end) {
                    float t = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) t += rb[w * R + threadIdx.x];
                    if (cur.tile == 0) out[row] = t;
                    else out[row] += t;  // same thread owns the row in every tile
                }
            }
            red_buf ^= 1;
        }
        advance(cur);
    };
    while (true) {
        step_fn(IntTag<0>{});
        if (cur.tile >= n_tiles) break;
        step_fn(IntTag<1>{});
        if (cur.tile >= n_tiles) break;
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
