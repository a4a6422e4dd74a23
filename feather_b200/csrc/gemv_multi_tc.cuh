// E5M2 matrix times up to 16 E5M2 vectors in one pass over the matrix, on the fifth-generation
// tensor cores (sm_100a):
//
//   out[b][r] = sum_j decode(m[r][j]) * decode(v[b][j]),   b < batch <= 16
//
// No counterpart in the reference (its GEMV takes one vector); the arithmetic is the
// reference GEMV's (feather/routines/gemv.py:8-61): exact products of the decoded codes,
// FP32 accumulation.  An E5M2 code is what the tensor core calls e5m2, so nothing is decoded:
// tcgen05.mma kind::f8f6f4 reads the packed bytes of the matrix (A, 128 rows x 32 codes per
// instruction) and of the vectors (B, 16 columns) from shared memory and accumulates
// 128 x 16 FP32 sums in tensor memory.  E4M3 cannot take this road: the reference decodes
// exponent-0 codes and 0x7F / 0xFF differently from the hardware's e4m3.
//
// With several right-hand sides the work is still bound by the matrix bytes from HBM.  A CTA
// per SM owns a contiguous range of rows and walks it in blocks of at most 128 rows; per
// block it streams the rows in steps of 512 codes.  A stage of the shared-memory ring holds
// one step as four pieces of 128 codes: the block's rows x 128 bytes of the matrix and the
// 16 x 128 bytes of the vectors each (tensor-map copies, 128-byte swizzle, rows past the end
// of the matrix or of the batch arrive as zeros), so the vectors need no resident copy (they
// come from L2 again for every row block: 2 KB beside 16 KB of matrix).  Warp 0 issues the
// copies, warp 1 the products (16 per stage, then a tcgen05.commit that frees the stage),
// warps 2-5 read a finished block's sums from tensor memory and store them.
//
// The tensor core's FP32 accumulation does not round like an FMA chain: one accumulator over
// 16384 codes came out 1.0e-5 off the float64 result (normalised), growing linearly with the
// row length.  So the products of a block go round-robin into EIGHT accumulators that the
// storing warps add in FP32 at the end (1.3e-6 at 16384 codes; the single-vector kernels:
// 1.3e-7); two such sets alternate between blocks.
//
// Every wait is bounded; a CTA that gave up still frees its tensor memory.
#pragma once
#include "attention_tc.cuh"   // descriptors, tensor-map copies, tensor-memory loads

namespace feather {

constexpr int kMtcThreads = 6 * 32;
constexpr int kMtcRows = 128;                 // rows per block = lanes of tensor memory
constexpr int kMtcVectors = 16;               // columns of the product
constexpr int kMtcBox = 128;                  // codes (bytes) of a row per tensor-map copy: the swizzle width
// Measured on B200 at 16384 x 16384 with 8 vectors: one copy (128 B of every row) per stage and
// 11 stages 51.0 us, two and 5 stages 46.1 us, four and 3 stages 45.3 us -- the more of a row a
// stage takes, the more of an open DRAM page it uses; blocks of 64 rows with 8 x 2 or 4 x 4
// (copies x stages) 51.6 / 49.1 us.
constexpr int kMtcBoxes = 4;                  // copies per stage: consecutive pieces of the same rows
constexpr int kMtcStep = kMtcBox * kMtcBoxes; // codes (bytes) of a row per stage
constexpr int kMtcStages = 3;
constexpr int kMtcSlotRows = kMtcRows;        // rows a block may have: a copy's place in the stage
constexpr int kMtcChains = 8;                 // accumulators per row block, summed in FP32 at the end
constexpr int kMtcCols = 2 * kMtcChains * kMtcVectors;   // tensor-memory columns: two sets of them alternate
constexpr int kMtcStageBytes = kMtcSlotRows * kMtcStep + kMtcVectors * kMtcStep;   // 16 KB + 2 KB per box
constexpr int kMtcBar = kMtcStages * kMtcStageBytes;          // full[], empty[], acc_full[2], acc_empty[2], base
constexpr int kMtcSmemBytes = kMtcBar + 8 * (2 * kMtcStages + 4) + 16;
constexpr uint32_t kMtcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kMtcVectors / 8) << 17) | ((kMtcRows / 16) << 24);

// Grid: any number of CTAs up to the SM count; CTA c owns rows [c, c + 1) * rows_cta, walked
// in n_blk blocks of blk_rows rows each (blk_rows <= 128 is also the row count of map_m's
// boxes).  map_m: the M x N byte matrix, boxes of 128 bytes x blk_rows rows; map_v: the
// batch x N byte vectors, boxes of 128 bytes x 16 rows; both swizzled over 128 bytes.
// N is a multiple of 512.  192 threads, kMtcSmemBytes of dynamic shared memory.
__global__ void __launch_bounds__(kMtcThreads, 1)
gemv_multi_tc_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_v,
                     float* __restrict__ out, int M, int N, int batch, int rows_cta, int blk_rows, int n_blk,
                     unsigned int* status) {
    extern __shared__ __align__(1024) unsigned char mtc_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = smem_u32(mtc_smem);
    const uint32_t bars = sbase + kMtcBar;
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (kMtcStages + s); };
    auto acc_full = [&](int a) { return bars + 8u * (2 * kMtcStages + a); };
    auto acc_empty = [&](int a) { return bars + 8u * (2 * kMtcStages + 2 + a); };
    const uint32_t tmem_slot = bars + 8u * (2 * kMtcStages + 4);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (sbase & 1023u) {                      // the swizzled tiles want 1 KiB alignment (every CTA alike)
        if (tid == 0) atomicOr(status, 2u);
        return;
    }
    const int row_begin = (int)blockIdx.x * rows_cta;
    const int row_end = min(M, row_begin + rows_cta);
    const int my_blk = row_begin < M ? min(n_blk, (row_end - row_begin + blk_rows - 1) / blk_rows) : 0;
    const int n_step = N / kMtcStep;

    if (tid == 0) {
        for (int s = 0; s < kMtcStages; ++s) {
            mbar_init(full(s), 1);            // the producer's arrive + the copied bytes
            mbar_init(empty(s), 1);           // the tensor core's commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);        // the tensor core's commit
            mbar_init(acc_empty(a), 4);       // the four reading warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tmem_slot), "r"((uint32_t)kMtcCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(mtc_smem + kMtcBar + 8 * (2 * kMtcStages + 4));

    if (warp == 0) {
        // ---- producer: one lane fills the ring, stage after stage, block after block ----
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the matrix and the vectors may be the previous kernel's
            bool ok = true;
            int it = 0;
            for (int b = 0; b < my_blk && ok; ++b) {
                const int r0 = row_begin + b * blk_rows;
                for (int k = 0; k < n_step && ok; ++k, ++it) {
                    const int s = it % kMtcStages;
                    if (it >= kMtcStages) ok = mbar_wait(empty(s), (uint32_t)((it / kMtcStages - 1) & 1), status);
                    mbar_arrive_expect_tx(full(s), (uint32_t)(blk_rows * kMtcStep + kMtcVectors * kMtcStep));
#pragma unroll
                    for (int x = 0; x < kMtcBoxes; ++x) {
                        tma_load_2d(sbase + s * kMtcStageBytes + x * (kMtcSlotRows * kMtcBox), &map_m,
                                    k * kMtcStep + x * kMtcBox, r0, full(s));
                        tma_load_2d(sbase + s * kMtcStageBytes + kMtcSlotRows * kMtcStep + x * (kMtcVectors * kMtcBox), &map_v,
                                    k * kMtcStep + x * kMtcBox, 0, full(s));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- one lane issues the products: 16 x (128 x 16 x 32 codes) per stage ----
        if (lane == 0) {
            bool ok = true;
            int it = 0;
            for (int b = 0; b < my_blk && ok; ++b) {
                const int a = b & 1;
                if (b >= 2) ok = mbar_wait(acc_empty(a), (uint32_t)((b / 2 - 1) & 1), status);   // its readers are done
                tc_fence_after();
                for (int k = 0; k < n_step && ok; ++k, ++it) {
                    const int s = it % kMtcStages;
                    ok = mbar_wait(full(s), (uint32_t)((it / kMtcStages) & 1), status);
                    tc_fence_after();
                    const uint32_t at = sbase + s * kMtcStageBytes;
#pragma unroll
                    for (int j = 0; j < kMtcStep / 32; ++j) {
                        const int x = j / (kMtcBox / 32), jj = j % (kMtcBox / 32);
                        tc_mma<true>(tmem + kMtcVectors * (kMtcChains * a + j % kMtcChains),
                                     tc_desc_swizzled(at + x * (kMtcSlotRows * kMtcBox) + jj * 32, 1024, 2),
                                     tc_desc_swizzled(at + kMtcSlotRows * kMtcStep + x * (kMtcVectors * kMtcBox) + jj * 32, 1024, 2),
                                     kMtcIdesc, k != 0 || j >= kMtcChains);
                    }
                    tc_commit(empty(s));      // the stage is free once these products have read it
                }
                tc_commit(acc_full(a));       // ... and the block's sums are complete
            }
        }
    } else {
        // ---- four warps store the sums: warp w reads lanes 32 (w % 4) .. of tensor memory ----
        const int q = warp & 3;
        bool ok = true;
        bool waited = false;
        for (int b = 0; b < my_blk; ++b) {
            const int a = b & 1;
            ok = mbar_wait(acc_full(a), (uint32_t)((b / 2) & 1), status) && ok;
            tc_fence_after();
            float acc[16];
            tmem_ld<16>(tmem + kMtcVectors * kMtcChains * a + ((uint32_t)(q * 32) << 16), acc);
#pragma unroll
            for (int c = 1; c < kMtcChains; ++c) {      // the chains' sums, in order
                float more[16];
                tmem_ld<16>(tmem + kMtcVectors * (kMtcChains * a + c) + ((uint32_t)(q * 32) << 16), more);
#pragma unroll
                for (int v = 0; v < 16; ++v) acc[v] += more[v];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(a));
            if (!waited) {                    // nothing is written before the kernel in front has completed
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
            const int r_in_blk = q * 32 + lane;
            const int row = row_begin + b * blk_rows + r_in_blk;
            if (ok && r_in_blk < blk_rows && row < row_end) {
#pragma unroll
                for (int v = 0; v < kMtcVectors; ++v)
                    if (v < batch) out[(size_t)v * M + row] = acc[v];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kMtcCols) : "memory");
    }
}

}  // namespace feather
