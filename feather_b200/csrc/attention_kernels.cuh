// Single-head, non-causal attention on packed E5M2 Q, K, V (sm_100a):
//
//   out = softmax(Q K^T / sqrt(d)) V,   Q, K, V: seq_len x d codes, out: seq_len x d FP32
//
// replaces _flash_attention_fp8_e5m2_acc_fp32_kernel (feather/routines/attention.py:14-108)
// and follows it step by step: key tiles of 64, scores accumulated in FP32 and divided by
// sqrt(d) (:83), online softmax with a running maximum and sum (:85-90), probabilities
// rounded to FP16 before they multiply V (:97-101), one division by the sum at the end
// (:103-106).  The division by sqrt(d) and the exponentials use the fast hardware forms
// (div.full, ex2.approx), as the compiled reference kernel does.  Like the reference, keys
// past seq_len in the last tile are read as zero
// codes and their scores (zero) are NOT masked: each takes part in the softmax.
//
// Mapping.  A CTA owns 16 query rows.  With one warp per CTA the warp walks all key tiles
// and the softmax state never leaves it.  Short sequences give too few such warps to fill
// the GPU, so a CTA may be 2, 4 or 8 warps that take every 2nd / 4th / 8th key tile of the SAME
// rows, each with its own running maximum, sum and output, merged at the end through
// shared memory (out = sum_w O_w e^(m_w - m) / sum_w l_w e^(m_w - m)): the same result up
// to the rounding of the FP16 probabilities against a per-warp instead of a global maximum.  Codes become FP16 by a byte permute
// (an E5M2 code is the high byte of an FP16 number) in registers:
//   * S = Q K^T with mma.sync.m16n8k16: lane (g, t) holds word t of each 16-code chunk of
//     query rows g and g + 8 as its A fragments and loads word t of the same chunk of key
//     8n + g as the B fragment -- any assignment of codes to k slots is valid as long as
//     both operands use it, so fragments are whole words and nothing is shuffled;
//   * the softmax runs on the accumulator fragments (row maxima and sums by two shuffles);
//   * O += P V: the S fragments, rounded to FP16, are already the A fragments.  A B
//     fragment pairs two KEYS for one output column, and V is contiguous along columns, so
//     a lane loads the same word (four columns) of two key rows and interleaves them with
//     two byte permutes: the four results are its B fragments for four column tiles.  Which
//     output column sits where in a tile is free as well: tile nn, position n holds column
//     4 (n + 8 (nn / 4)) + nn % 4, so that a lane's results are runs of four floats.
// No shared memory and no CTA barrier: warps are independent, K and V come through L1/L2.
#pragma once
#include "gemv_common.cuh"

namespace feather {

constexpr int kAttnThreads = 256;    // at most: 1, 2, 4 or 8 warps per CTA
constexpr int kAttnTile = 64;        // keys per step (the reference's tile, attention.py:9)

__device__ __forceinline__ void attn_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// D = 4 * words per row: 16, 32, 64, 128 (CS = 1), 256 (CS = 2) or 512 (CS = 4).
// Grid: one CTA per 16 queries.
//   CS = 1: blockDim.x / 32 warps split the key tiles.  Dynamic shared memory: nothing for
//           one warp, else warps * (16 * D + 32) floats.
//   CS > 1: the model dimension is too wide for one warp's registers, so the CTA is CS
//           warps that each own D / CS = 128 columns: a warp multiplies its slice of Q
//           with its slice of K (a partial S), the partials are added through shared
//           memory in warp order (every warp then holds the same S and runs the same
//           softmax), and each warp accumulates its own columns of O.  Dynamic shared
//           memory: CS * 1024 floats.
template <int D, int CS>
__global__ void __launch_bounds__(kAttnThreads)
attention_e5m2_kernel(const uint32_t* __restrict__ q, const uint32_t* __restrict__ k,
                      const uint32_t* __restrict__ v, float* __restrict__ out, int seq_len) {
    extern __shared__ __align__(16) float attn_merge[];
    constexpr int DS = D / CS;                  // columns this warp contracts over and outputs
    constexpr int KS = DS / 16;                 // k-steps of S = Q K^T (16 codes each)
    constexpr int WPR = D / 4;                  // words per row
    constexpr int NG = (DS / 4 + 7) / 8;        // groups of four 8-column tiles of O (32 columns)
    constexpr int NT = 4 * NG;                  // column tiles held (D = 16: half of them are padding)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n_split = CS > 1 ? 1 : (int)blockDim.x >> 5;   // warps that split the key tiles
    const int key_warp = CS > 1 ? 0 : warp;
    const int woff = CS > 1 ? warp * (DS / 4) : 0;            // first word of this warp's column slice
    const int row_a = (int)blockIdx.x * 16 + g, row_b = row_a + 8;

    // Q fragments, kept for the whole loop; rows past seq_len are zero codes (:36)
    uint32_t qa[KS][2], qb[KS][2];
#pragma unroll
    for (int s = 0; s < KS; ++s) {
        const uint32_t wa = row_a < seq_len ? __ldg(q + (size_t)row_a * WPR + woff + 4 * s + t) : 0u;
        const uint32_t wb = row_b < seq_len ? __ldg(q + (size_t)row_b * WPR + woff + 4 * s + t) : 0u;
        decode_word_h2<kE5M2>(wa, qa[s][0], qa[s][1]);
        decode_word_h2<kE5M2>(wb, qb[s][0], qb[s][1]);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const float sqrt_d = sqrtf((float)D);

    for (int key0 = key_warp * kAttnTile; key0 < seq_len; key0 += n_split * kAttnTile) {
        // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys ----
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
            const int key = key0 + 8 * n + g;
            const uint32_t* kr = k + (size_t)min(key, seq_len - 1) * WPR + woff + t;
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                uint32_t b0, b1;
                decode_word_h2<kE5M2>(key < seq_len ? __ldg(kr + 4 * s) : 0u, b0, b1);
                attn_mma(sc[n], qa[s][0], qb[s][0], qa[s][1], qb[s][1], b0, b1);
            }
        }
        if (CS > 1) {
            // ---- add the warps' partial scores: [warp][fragment value][lane], warps in order ----
            __syncthreads();                    // the previous tile's partials have been read
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) attn_merge[(warp * 32 + n * 4 + i) * 32 + lane] = sc[n][i];
            __syncthreads();
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float sum = attn_merge[(n * 4 + i) * 32 + lane];
                    for (int w = 1; w < CS; ++w) sum += attn_merge[(w * 32 + n * 4 + i) * 32 + lane];
                    sc[n][i] = sum;
                }
        }
        // ---- online softmax on the fragments: rows g (values 0, 1) and g + 8 (values 2, 3) ----
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[n][i] = __fdividef(sc[n][i], sqrt_d);
            mx_a = fmaxf(mx_a, fmaxf(sc[n][0], sc[n][1]));
            mx_b = fmaxf(mx_b, fmaxf(sc[n][2], sc[n][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float alpha_a = __expf(m_a - mn_a), alpha_b = __expf(m_b - mn_b);
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t p[8][2];                       // probabilities as FP16 pairs: [n][row a | row b]
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float e0 = __expf(sc[n][0] - mn_a), e1 = __expf(sc[n][1] - mn_a);
            const float e2 = __expf(sc[n][2] - mn_b), e3 = __expf(sc[n][3] - mn_b);
            sum_a += e0 + e1;
            sum_b += e2 + e3;
            p[n][0] = pack_h2(e0, e1);
            p[n][1] = pack_h2(e2, e3);
        }
        sum_a += __shfl_xor_sync(0xFFFFFFFFu, sum_a, 1);
        sum_a += __shfl_xor_sync(0xFFFFFFFFu, sum_a, 2);
        sum_b += __shfl_xor_sync(0xFFFFFFFFu, sum_b, 1);
        sum_b += __shfl_xor_sync(0xFFFFFFFFu, sum_b, 2);
        l_a = l_a * alpha_a + sum_a;
        l_b = l_b * alpha_b + sum_b;
        m_a = mn_a;
        m_b = mn_b;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= alpha_a;
            o[n][1] *= alpha_a;
            o[n][2] *= alpha_b;
            o[n][3] *= alpha_b;
        }
        // ---- O += P V: k-step j covers keys 16 j .. 16 j + 15 = S tiles 2j and 2j + 1 ----
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // this lane's k slots: keys 16 j + 2t, + 1 (first B register) and + 8, + 9 (second)
            const int kk = key0 + 16 * j + 2 * t;
#pragma unroll
            for (int c = 0; c < NG; ++c) {
                const int w = g + 8 * c;            // the word whose four columns this lane feeds
                uint32_t x[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = kk + (i & 1) + 8 * (i >> 1);
                    x[i] = (w < DS / 4 && key < seq_len) ? __ldg(v + (size_t)key * WPR + woff + w) : 0u;
                }
                // bytes (col0: key a, key b, col1: key a, key b), then the E5M2 byte -> FP16 spread
                uint32_t b0[4], b1[4];
                decode_word_h2<kE5M2>(prmt(x[0], x[1], 0x5140u), b0[0], b0[1]);
                decode_word_h2<kE5M2>(prmt(x[0], x[1], 0x7362u), b0[2], b0[3]);
                decode_word_h2<kE5M2>(prmt(x[2], x[3], 0x5140u), b1[0], b1[1]);
                decode_word_h2<kE5M2>(prmt(x[2], x[3], 0x7362u), b1[2], b1[3]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    attn_mma(o[4 * c + i], p[2 * j][0], p[2 * j][1], p[2 * j + 1][0], p[2 * j + 1][1],
                             b0[i], b1[i]);
            }
        }
    }
    if (CS == 1 && n_split > 1) {
        // ---- merge the warps' partial results: [warp][row][col] sums, then [warp][row] m and l ----
        float* so = attn_merge + (size_t)warp * (16 * D + 32);
#pragma unroll
        for (int c = 0; c < NG; ++c) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = 32 * c + 4 * (2 * t + e);
                if (col < D) {
                    *reinterpret_cast<float4*>(so + g * D + col) =
                        make_float4(o[4 * c][e], o[4 * c + 1][e], o[4 * c + 2][e], o[4 * c + 3][e]);
                    *reinterpret_cast<float4*>(so + (g + 8) * D + col) =
                        make_float4(o[4 * c][2 + e], o[4 * c + 1][2 + e], o[4 * c + 2][2 + e], o[4 * c + 3][2 + e]);
                }
            }
        }
        if (t == 0) {
            so[16 * D + g] = m_a;
            so[16 * D + g + 8] = m_b;
            so[16 * D + 16 + g] = l_a;
            so[16 * D + 16 + g + 8] = l_b;
        }
        __syncthreads();
        const int rows_here = min(16, seq_len - (int)blockIdx.x * 16);
        for (int idx = threadIdx.x; idx < rows_here * D; idx += blockDim.x) {
            const int row = idx / D, col = idx - row * D;
            float m = -INFINITY;
            for (int w = 0; w < n_split; ++w) m = fmaxf(m, attn_merge[(size_t)w * (16 * D + 32) + 16 * D + row]);
            float l = 0.f, acc = 0.f;
            for (int w = 0; w < n_split; ++w) {       // warps in order: a fixed summation order
                const float* sw = attn_merge + (size_t)w * (16 * D + 32);
                const float scale = expf(sw[16 * D + row] - m);   // a warp without tiles: e^(-inf) = 0
                l += sw[16 * D + 16 + row] * scale;
                acc += sw[row * D + col] * scale;
            }
            out[((size_t)blockIdx.x * 16 + row) * D + col] = __fdiv_rn(acc, l);
        }
        return;
    }
    // ---- out = O / l (:103-106).  Fragment (tile 4c + i, value e / 2 + e): row g or g + 8,
    // column 32 c + 4 (2t + e) + i: four consecutive floats over i ----
#pragma unroll
    for (int c = 0; c < NG; ++c) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = 32 * c + 4 * (2 * t + e);
            if (col < DS) {
                if (row_a < seq_len)
                    *reinterpret_cast<float4*>(out + (size_t)row_a * D + 4 * woff + col) = make_float4(
                        __fdiv_rn(o[4 * c][e], l_a), __fdiv_rn(o[4 * c + 1][e], l_a),
                        __fdiv_rn(o[4 * c + 2][e], l_a), __fdiv_rn(o[4 * c + 3][e], l_a));
                if (row_b < seq_len)
                    *reinterpret_cast<float4*>(out + (size_t)row_b * D + 4 * woff + col) = make_float4(
                        __fdiv_rn(o[4 * c][2 + e], l_b), __fdiv_rn(o[4 * c + 1][2 + e], l_b),
                        __fdiv_rn(o[4 * c + 2][2 + e], l_b), __fdiv_rn(o[4 * c + 3][2 + e], l_b));
            }
        }
    }
}

}  // namespace feather
