// Single-head, non-causal attention on packed E5M2 Q, K, V for the fifth-generation
// tensor cores (sm_100a): tcgen05.mma with both operands in shared memory and the
// accumulators in tensor memory.
//
//   out = softmax(Q K^T / sqrt(d)) V,   Q, K, V: seq_len x d codes, out: seq_len x d FP32
//
// replaces _flash_attention_fp8_e5m2_acc_fp32_kernel (feather/routines/attention.py:14-108)
// with the same tile-by-tile arithmetic as the register-fed kernel beside it: key tiles of
// 64 (:9), scores accumulated in FP32 and divided by sqrt(d) (:83), online softmax with a
// running maximum and sum (:85-90), probabilities rounded to FP16 before they multiply V
// (:97-101), one division by the sum at the end (:103-106); keys past seq_len in the last
// tile are zero codes whose (zero) scores take part in the softmax, as in the reference.
//
// Mapping.  A CTA of 128 threads owns 128 query rows: thread t owns row t, which is lane
// t of tensor memory, so the softmax needs no shuffles.  The key tiles of one query block
// are split over the 1, 2, 4 or 8 CTAs of a thread-block cluster (contiguous ranges), each
// with its own running maximum, sum and output; at the end every CTA leaves its partial
// result in its own shared memory and the cluster merges them through distributed shared
// memory (out = sum_c O_c e^(m_c - m) / sum_c l_c e^(m_c - m), CTAs in rank order), each
// CTA writing 128 / cluster rows.  No global scratch, no atomics, deterministic.
//
// Per key tile:
//   1. K codes (raw bytes: the tensor core reads E5M2 itself, kind::f8f6f4) and V codes of
//      the NEXT tile are fetched with cp.async into the other half of a double buffer;
//   2. one thread issues S = Q K^T (128 x 64, d / 32 instructions) into tensor-memory
//      columns 0..63 and commits to an mbarrier;
//   3. meanwhile all threads spread this tile's V codes to FP16 (an E5M2 code is the high
//      byte of an FP16 number) in the layout the second product reads;
//   4. each thread reads its row of S (tcgen05.ld 32x32b), runs the online softmax and
//      stores the FP16 probabilities as the A operand of the second product;
//   5. one thread issues P V (128 x d, 4 instructions, kind::f16) into columns 64..64+d-1;
//   6. each thread reads its row of P V and folds it into its FP32 output registers
//      (o = o * alpha + pv).
//
// Shared-memory operand layouts (no swizzle; 16-byte units; LBO / SBO of the matrix
// descriptor):
//   * Q, K (K-major, 1 byte per element) and P (K-major, FP16): [16-byte unit along the
//     contraction][row][16 B]: rows are 16 B apart (an 8-row core matrix is 128 contiguous
//     bytes, SBO = 128) and the units along the contraction are rows * 16 B apart (LBO);
//   * V (MN-major FP16: the model dimension runs fastest, as V is stored): a core matrix
//     is 8 keys x 8 columns (128 B, key rows 16 B apart); column groups follow 144 B apart
//     (SBO; the odd 16 B keep the conversion's stores free of bank conflicts) and key
//     groups (d / 8) * 144 B apart (LBO).
//
// Every wait is bounded (mbar_wait raises the status word and gives up after the limit);
// a CTA that gave up still walks every CTA and cluster barrier and frees its tensor
// memory.  Shared memory per CTA is sized so that the CTAs resident on one SM never ask
// for more than its 512 tensor-memory columns.
#pragma once
#include "gemv_mma.cuh"    // cp.async wrappers
#include "gemv_ring.cuh"   // mbarrier wrappers, bounded waits

namespace feather {

constexpr int kAtcRows = 128;      // queries per CTA = lanes of tensor memory
constexpr int kAtcThreads = 128;
constexpr int kAtcTile = 64;       // keys per step (the reference's tile, attention.py:9)

template <int D>
struct AtcLayout {
    static constexpr int kQ = 0;                               // [D/16][128][16 B]
    static constexpr int kQBytes = kAtcRows * D;
    static constexpr int kK = kQ + kQBytes;                    // 2 x [D/16][64][16 B]
    static constexpr int kKBytes = kAtcTile * D;
    static constexpr int kVraw = kK + 2 * kKBytes;             // 2 x [64][D] codes
    static constexpr int kV = kVraw + 2 * kKBytes;             // FP16, see above
    static constexpr int kVSbo = 144;
    static constexpr int kVLbo = (D / 8) * kVSbo;
    static constexpr int kVBytes = (kAtcTile / 8) * kVLbo;
    static constexpr int kP = kV + kVBytes;                    // [8][128][16 B] FP16
    static constexpr int kPBytes = kAtcRows * kAtcTile * 2;
    static constexpr int kBar = kP + kPBytes;                  // two mbarriers, tensor-memory base
    static constexpr int kTileBytes = kBar + 32;
    // the merge reuses the operand space: O as [128][D + 4] floats (the odd 16 B keep a
    // thread-per-row's 16-byte stores free of bank conflicts), then m[128], l[128]
    static constexpr int kMergeStride = D + 4;
    static constexpr int kMergeM = kAtcRows * kMergeStride * 4;
    static constexpr int kMergeBytes = kMergeM + 2 * kAtcRows * 4;
    static constexpr int kWeightBytes = 9 * kAtcRows * 4;      // the merging CTA's own weights, behind it
    static_assert(kMergeBytes + kWeightBytes <= kBar, "the merge buffers must not reach the barriers");
    static constexpr int kCols = D > 64 ? 256 : 128;           // tensor-memory columns: 64 (S) + D (P V)
    // at most 512 / kCols CTAs of this kernel per SM: ask for more than 1 / (that + 1) of 227 KiB
    static constexpr int kMinBytes = (227 * 1024) / (512 / kCols + 1) + 1024;
    static constexpr int kBytes = kTileBytes > kMinBytes ? kTileBytes : kMinBytes;
};

// ---- tcgen05 / cp.async / cluster wrappers ----
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Matrix descriptor, no swizzle: start address, leading and stride byte offsets in 16-byte
// units, descriptor version 1 (bits 46-47).
__device__ __forceinline__ uint64_t tc_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           (1ull << 46);
}
// Instruction descriptors: FP32 accumulator (bits 4-5 = 1), operand formats (bits 7-9 and
// 10-12: E5M2 = 1 for kind::f8f6f4, FP16 = 0 for kind::f16), B MN-major (bit 16), N / 8 (bits
// 17-22), M / 16 (bits 24-28).
constexpr uint32_t kAtcIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((kAtcTile / 8) << 17) | ((kAtcRows / 16) << 24);
template <int D>
constexpr uint32_t kAtcIdescPV = (1u << 4) | (1u << 16) | ((uint32_t)(D / 8) << 17) | ((kAtcRows / 16) << 24);

template <bool F8>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    if (F8)
        asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                     "  tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
                     ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
    else
        asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                     "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
                     ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// This thread's lane of tensor memory, 32 consecutive columns from taddr.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t x[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]),
          "=r"(x[8]), "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15]),
          "=r"(x[16]), "=r"(x[17]), "=r"(x[18]), "=r"(x[19]), "=r"(x[20]), "=r"(x[21]), "=r"(x[22]), "=r"(x[23]),
          "=r"(x[24]), "=r"(x[25]), "=r"(x[26]), "=r"(x[27]), "=r"(x[28]), "=r"(x[29]), "=r"(x[30]), "=r"(x[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(x[i]);
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The cluster-wide address of CTA `rank`'s copy of this CTA's shared address `addr`, and a
// float load through such an address.
__device__ __forceinline__ uint32_t map_cluster(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
    float4 x;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "r"(addr) : "memory");
    return x;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float x;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x) : "r"(addr) : "memory");
    return x;
}

#ifdef FEATHER_ATC_STAMPS
// Diagnostic build only: the SM's cycle counter at points of CTA (0, 0)'s thread 0.
__device__ unsigned long long g_atc_stamps[256];
#define ATC_STAMP(i) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (i) < 256) g_atc_stamps[i] = (unsigned long long)clock64(); } while (0)
#else
#define ATC_STAMP(i) do { } while (0)
#endif

// D = codes per row: 32, 64 or 128.  Grid (splits, query blocks), cluster (splits, 1, 1),
// 128 threads, AtcLayout<D>::kBytes of dynamic shared memory.  q, k, v 16-byte aligned.
template <int D>
__global__ void __launch_bounds__(kAtcThreads)
attention_tc_kernel(const uint32_t* __restrict__ q, const uint32_t* __restrict__ k,
                    const uint32_t* __restrict__ v, float* __restrict__ out, int seq_len,
                    unsigned int* status) {
    extern __shared__ __align__(128) unsigned char atc_smem[];
    using L = AtcLayout<D>;
    constexpr int KU = D / 16;                    // 16-byte units per row of codes
    const int tid = threadIdx.x, warp = tid >> 5;
    const int n_split = (int)gridDim.x, split = (int)blockIdx.x;
    const int row0 = (int)blockIdx.y * kAtcRows;
    const uint32_t sbase = smem_u32(atc_smem);
    const uint32_t bar_s = sbase + L::kBar, bar_o = bar_s + 8;
    ATC_STAMP(0);

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sbase + L::kBar + 16), "r"((uint32_t)L::kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(atc_smem + L::kBar + 16);
    const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes

    // this CTA's key tiles: a contiguous range
    const int tiles = (seq_len + kAtcTile - 1) / kAtcTile;
    const int per = (tiles + n_split - 1) / n_split;
    const int t_begin = min(split * per, tiles);
    const int n = min(tiles, t_begin + per) - t_begin;

    auto load_kv = [&](int tile, int buf) {
        const int key0 = tile * kAtcTile;
#pragma unroll
        for (int c = tid; c < kAtcTile * KU; c += kAtcThreads) {
            // K: unit c = (row c % 64, 16-byte unit c / 64) lands at c * 16
            const int key = key0 + (c & (kAtcTile - 1));
            const char* src = reinterpret_cast<const char*>(k) + (size_t)min(key, seq_len - 1) * D + (c >> 6) * 16;
            cp_async_16(sbase + L::kK + buf * L::kKBytes + c * 16, src, key < seq_len ? 16 : 0);
        }
#pragma unroll
        for (int c = tid; c < kAtcTile * KU; c += kAtcThreads) {
            // V: rows as they are
            const int key = key0 + c / KU;
            const char* src = reinterpret_cast<const char*>(v) + (size_t)min(key, seq_len - 1) * D + (c % KU) * 16;
            cp_async_16(sbase + L::kVraw + buf * L::kKBytes + c * 16, src, key < seq_len ? 16 : 0);
        }
    };
    if (n > 0) {
#pragma unroll
        for (int c = tid; c < kAtcRows * KU; c += kAtcThreads) {
            const int row = row0 + (c & (kAtcRows - 1));
            const char* src = reinterpret_cast<const char*>(q) + (size_t)min(row, seq_len - 1) * D + (c >> 7) * 16;
            cp_async_16(sbase + L::kQ + c * 16, src, row < seq_len ? 16 : 0);
        }
        load_kv(t_begin, 0);
    }
    cp_async_commit();

    ATC_STAMP(1);
    float o[D];
#pragma unroll
    for (int c = 0; c < D; ++c) o[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    const float sqrt_d = sqrtf((float)D);
    uint32_t phase = 0;
    bool ok = true;

    for (int i = 0; i < n; ++i) {
        const int buf = i & 1;
        if (i + 1 < n) load_kv(t_begin + i + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();                 // all but the newest group: Q and tile i are here
        fence_proxy_async_smem();           // ... and visible to the tensor core's reads
        tc_fence_before();
        if (__syncthreads_or(!ok)) break;
        ATC_STAMP(8 + 6 * i);
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < D / 32; ++j)  // 32 codes (two 16-byte units) per instruction
                tc_mma<true>(tmem,
                             tc_desc(sbase + L::kQ + j * 2 * (kAtcRows * 16), kAtcRows * 16, 128),
                             tc_desc(sbase + L::kK + buf * L::kKBytes + j * 2 * (kAtcTile * 16), kAtcTile * 16, 128),
                             kAtcIdescQK, j > 0);
            tc_commit(bar_s);
        }
        __syncwarp();
        // ---- V codes -> FP16 (8 codes -> one 16-byte unit), the previous P V has completed ----
#pragma unroll
        for (int u = tid; u < kAtcTile * (D / 8); u += kAtcThreads) {
            const int ng = u % (D / 8), key = u / (D / 8);
            const uint2 w = *reinterpret_cast<const uint2*>(atc_smem + L::kVraw + buf * L::kKBytes + key * D + ng * 8);
            uint4 h;
            decode_word_h2<kE5M2>(w.x, h.x, h.y);
            decode_word_h2<kE5M2>(w.y, h.z, h.w);
            *reinterpret_cast<uint4*>(atc_smem + L::kV + (key >> 3) * L::kVLbo + ng * L::kVSbo + (key & 7) * 16) = h;
        }
        // ---- this row's scores and the online softmax ----
        ATC_STAMP(9 + 6 * i);
        ok = mbar_wait(bar_s, phase, status) && ok;
        tc_fence_after();
        ATC_STAMP(10 + 6 * i);
        float s[kAtcTile];
        {
            float a[32], b[32];
            tmem_ld32(tmem_row, a);
            tmem_ld32(tmem_row + 32, b);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                s[j] = a[j];
                s[32 + j] = b[j];
            }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < kAtcTile; ++j) {
            s[j] = __fdividef(s[j], sqrt_d);
            mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);   // four chains instead of one of 64
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float mn = fmaxf(m, mx);
        const float alpha = __expf(m - mn);
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < kAtcTile / 8; ++u) {
            uint32_t p[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float e0 = __expf(s[8 * u + 2 * x] - mn), e1 = __expf(s[8 * u + 2 * x + 1] - mn);
                sum4[x] += e0 + e1;
                const __half2 h = __floats2half2_rn(e0, e1);
                p[x] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(atc_smem + L::kP + u * (kAtcRows * 16) + tid * 16) = make_uint4(p[0], p[1], p[2], p[3]);
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m = mn;
        fence_proxy_async_smem();
        tc_fence_before();
        ATC_STAMP(11 + 6 * i);
        if (__syncthreads_or(!ok)) break;
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < kAtcTile / 16; ++j)   // 16 keys (two key groups) per instruction
                tc_mma<false>(tmem + kAtcTile,
                              tc_desc(sbase + L::kP + j * 2 * (kAtcRows * 16), kAtcRows * 16, 128),
                              tc_desc(sbase + L::kV + j * 2 * L::kVLbo, L::kVLbo, L::kVSbo),
                              kAtcIdescPV<D>, j > 0);
            tc_commit(bar_o);
        }
        __syncwarp();
        ATC_STAMP(12 + 6 * i);
        ok = mbar_wait(bar_o, phase, status) && ok;
        tc_fence_after();
        ATC_STAMP(13 + 6 * i);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            float pv[32];
            tmem_ld32(tmem_row + kAtcTile + 32 * c, pv);
#pragma unroll
            for (int x = 0; x < 32; ++x) o[32 * c + x] = fmaf(o[32 * c + x], alpha, pv[x]);
        }
        phase ^= 1;
    }
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();                          // operands and tensor memory are no longer read

    ATC_STAMP(2);
    // ---- partial result to shared memory, merge over the cluster ----
    float* mo = reinterpret_cast<float*>(atc_smem);
#pragma unroll
    for (int c = 0; c < D; c += 4)
        *reinterpret_cast<float4*>(mo + tid * L::kMergeStride + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
    mo[L::kMergeM / 4 + tid] = m;
    mo[L::kMergeM / 4 + kAtcRows + tid] = l;
    ATC_STAMP(3);
    cluster_sync();
    ATC_STAMP(4);
    // Every CTA merges 128 / n_split rows.  First the rows' weights: thread r of the slice
    // reads the n_split maxima and sums of its row (all loads in flight at once), and
    // leaves e^(m_c - m) per CTA and the total sum in this CTA's own shared memory, past
    // the part its peers read.
    const int rows_per = kAtcRows / n_split;
    uint32_t peer[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) peer[c] = map_cluster(sbase, (uint32_t)min(c, n_split - 1));
    float* weight = reinterpret_cast<float*>(atc_smem + L::kMergeBytes);   // [8][128], then the sums [128]
    if (tid < rows_per) {
        const int r = split * rows_per + tid;
        float mc[8], lc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            mc[c] = c < n_split ? ld_cluster_f32(peer[c] + L::kMergeM + r * 4) : -INFINITY;
            lc[c] = c < n_split ? ld_cluster_f32(peer[c] + L::kMergeM + (kAtcRows + r) * 4) : 0.f;
        }
        float mm = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; ++c) mm = fmaxf(mm, mc[c]);
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {            // CTAs in rank order: a fixed summation order
            const float scale = expf(mc[c] - mm);   // a CTA without tiles: e^(-inf) = 0
            lsum += lc[c] * scale;
            weight[c * kAtcRows + tid] = scale;
        }
        weight[8 * kAtcRows + tid] = lsum;
    }
    __syncthreads();
    // Then the outputs, four columns per item and consecutive threads along a row (remote
    // reads and global stores are contiguous runs); two items per thread at a time so that
    // up to 16 remote 16-byte loads are in flight.
    constexpr int kBatch = 2, kGroups = D / 4;
    for (int base = 0; base < rows_per * kGroups; base += kBatch * kAtcThreads) {
        float4 x[kBatch][8];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int idx = base + b * kAtcThreads + tid;
            const int rl = idx / kGroups, g = idx % kGroups;
            const uint32_t off = (uint32_t)((split * rows_per + rl) * L::kMergeStride + 4 * g) * 4;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                x[b][c] = (c < n_split && rl < rows_per) ? ld_cluster_f32x4(peer[c] + off) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int idx = base + b * kAtcThreads + tid;
            const int rl = idx / kGroups, g = idx % kGroups;
            const int row = row0 + split * rows_per + rl;
            if (rl >= rows_per || row >= seq_len) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float w = weight[c * kAtcRows + rl];
                acc.x += x[b][c].x * w;
                acc.y += x[b][c].y * w;
                acc.z += x[b][c].z * w;
                acc.w += x[b][c].w * w;
            }
            const float lsum = weight[8 * kAtcRows + rl];
            *reinterpret_cast<float4*>(out + (size_t)row * D + 4 * g) =
                make_float4(__fdiv_rn(acc.x, lsum), __fdiv_rn(acc.y, lsum), __fdiv_rn(acc.z, lsum), __fdiv_rn(acc.w, lsum));
        }
    }
    ATC_STAMP(5);
    cluster_sync();                           // nobody leaves while a peer reads its memory
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)L::kCols) : "memory");
    }
    ATC_STAMP(6);
}

}  // namespace feather
