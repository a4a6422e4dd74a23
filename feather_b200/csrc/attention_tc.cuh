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
// Mapping.  A CTA owns 128 query rows = the 128 lanes of tensor memory.  It is eight worker
// warps and one issuing warp.  Two worker threads share a row (warps w and w + 4 reach the
// same 32 lanes): each takes half of a tile's keys and half of the output columns, and
// both read all 64 scores of the row for its maximum, so the softmax needs no shuffles
// and no exchange.  The key tiles of one query block are split over the 1 .. 8 CTAs of a
// thread-block cluster (contiguous ranges, as many CTAs as still run in one wave),
// each with its own running maximum, sum and output; at the end every CTA leaves its
// partial result in its own shared memory and the cluster merges them through distributed
// shared memory (out = sum_c O_c 2^(m_c - m) / sum_c l_c 2^(m_c - m), CTAs in rank order),
// each CTA writing its share of the 128 rows.  No global scratch, no atomics, deterministic.
//
// Tensor memory: columns 0..63 hold S = Q K^T of the current tile, columns 64..64+d-1 the
// output, which P V accumulates into; before P(i) V(i) is issued each worker has multiplied
// its half row of the output by alpha = 2^(old maximum - new maximum) (tcgen05.ld / .st),
// which is the reference's acc * alpha + P V.  A warp skips that when none of its rows saw
// a new maximum (alpha is exactly 1 then).
//
// Per key tile i there is ONE CTA barrier.  Before it a worker
//   1. waits for S(i) and for P(i-1) V(i-1) (mbarriers the tensor core arrives on),
//   2. reads its scores (tcgen05.ld 32x32b), runs the online softmax -- the maximum lives in
//      the exponent's scale, m2 = max * log2(e) / sqrt(d), so a probability is one FMA and
//      one ex2, the FMAs and the sums two at a time in the packed FP32 forms -- and stores
//      its FP16 probabilities as the A operand of the second product,
//   3. rescales its half row of the output;
// behind it one lane of the issuing warp issues S(i+1) (kind::f8f6f4: the tensor core reads
// the E5M2 codes themselves, d / 32 instructions) and then P(i) V(i) (kind::f16, 4
// instructions), each followed by a tcgen05.commit, and starts the copies of tile i+2:
// two tensor-map copies (cp.async.bulk.tensor.2d), K into the swizzled operand layout and
// V as stored, which count their bytes on the buffer's mbarrier; rows past seq_len arrive
// as zeros.  The workers meanwhile
//   4. wait for the codes of tile i+1 and spread its V to FP16 (an E5M2 code is the high
//      byte of an FP16 number) in the layout the second product reads.
// K codes, V codes and V as FP16 are double-buffered; P and S are not (their readers have
// finished by the time they are written again, see the loop).  No worker thread touches
// global memory inside the loop.
//
// Shared-memory operand layouts (16-byte units; LBO / SBO of the matrix descriptor):
//   * Q, K (K-major, 1 byte per element): rows of d bytes as they are in global memory, the
//     16-byte units of a row swizzled over d bytes (128-, 64- or 32-byte swizzle) by the
//     tensor-map copy and un-swizzled by the tensor core; 8-row groups 8 d bytes apart
//     (SBO), a step of 32 codes along the contraction is 32 bytes further along the row;
//   * P (K-major FP16, no swizzle): [16-byte unit along the contraction][row][16 B]: rows are
//     16 B apart (an 8-row core matrix is 128 contiguous bytes, SBO = 128) and the units
//     along the contraction are 128 * 16 B apart (LBO);
//   * V (MN-major FP16: the model dimension runs fastest, as V is stored): a core matrix
//     is 8 keys x 8 columns (128 B, key rows 16 B apart); column groups follow 144 B apart
//     (SBO; the odd 16 B keep the conversion's stores free of bank conflicts) and key
//     groups (d / 8) * 144 B apart (LBO).
//
// Rows of 256 codes are two swizzled 128-byte column segments per operand and one CTA per
// SM.  Rows of 512 codes need 64 + 512 tensor-memory columns, more than an SM has: a pair of
// CTAs in the cluster shares the query block, both compute the same S and P, each multiplies
// P with its half of V's columns and owns that half of the output; with Q at 64 KB their K
// tile is single-buffered (the copy of the next tile waits for S of the current one).
//
// Every wait is bounded (mbar_wait raises the status word and gives up after the limit);
// a CTA that gave up still walks every CTA and cluster barrier and frees its tensor
// memory.  Shared memory per CTA is sized so that the CTAs resident on one SM never ask
// for more than its 512 tensor-memory columns.
#pragma once
#include <cuda.h>           // CUtensorMap and its enumerations (types only: nothing of libcuda is linked)
#include "gemv_ring.cuh"   // mbarrier wrappers, bounded waits

namespace feather {

constexpr int kAtcRows = 128;      // queries per CTA = lanes of tensor memory
constexpr int kAtcWorkers = 256;    // two threads per query row: each takes half the keys and half the columns
constexpr int kAtcThreads = kAtcWorkers + 32;   // ... and a warp that issues the tensor-core instructions
constexpr int kAtcTile = 64;       // keys per step (the reference's tile, attention.py:9)

template <int D>
struct AtcLayout {
    // Rows of 512 codes: the output's columns are split over a pair of CTAs (kHalves = 2):
    // both compute the same S and P, each multiplies P with its half of V's columns.
    static constexpr int kHalves = D > 256 ? 2 : 1;
    static constexpr int kDo = D / kHalves;                    // output columns of a CTA
    static constexpr int kKBufs = D > 256 ? 1 : 2;             // 512 codes: no room for a second K tile
    static constexpr int kQ = 0;                               // [128][D] codes, 16-byte units swizzled
    static constexpr int kQBytes = kAtcRows * D;
    static constexpr int kK = kQ + kQBytes;                    // kKBufs x [64][D], swizzled like Q
    static constexpr int kKBytes = kAtcTile * D;
    static constexpr int kVraw = kK + kKBufs * kKBytes;        // 2 x [64][kDo] codes
    static constexpr int kVrawBytes = kAtcTile * kDo;
    static constexpr int kV = kVraw + 2 * kVrawBytes;          // 2 x FP16, see above
    static constexpr int kVSbo = 144;
    static constexpr int kVLbo = (kDo / 8) * kVSbo;
    static constexpr int kVBytes = (kAtcTile / 8) * kVLbo;
    static constexpr int kP = kV + 2 * kVBytes;                // [8][128][16 B] FP16
    static constexpr int kPBytes = kAtcRows * kAtcTile * 2;
    static constexpr int kBar = kP + kPBytes;                  // mbarriers: S, P V; tensor-memory base; K x 2, V codes x 2
    static constexpr int kTileBytes = kBar + 64;
    // Operand rows are swizzled over kSeg = min(D, 128) bytes; rows wider than 128 bytes are
    // held as D / 128 column segments, one swizzled [rows][128 B] region after the other.
    // kSwizzle is the descriptor's layout type, kGroup the 8-row group stride (SBO); the
    // tensor maps that fill the regions use the same swizzle.
    static constexpr int kSeg = D < 128 ? D : 128;             // bytes of a row per segment
    static constexpr int kSegs = D / kSeg;
    static constexpr uint32_t kSwizzle = kSeg == 128 ? 2u : kSeg == 64 ? 4u : 6u;   // 128 B, 64 B, 32 B
    static constexpr uint32_t kGroup = 8 * kSeg;
    // the merge reuses the operand space: O as [128][kDo + 4] floats (the odd 16 B keep a
    // thread-per-row's 16-byte stores free of bank conflicts), then m[128] and the two threads' l[2][128]
    static constexpr int kMergeStride = kDo + 4;
    static constexpr int kMergeM = kAtcRows * kMergeStride * 4;
    static constexpr int kMergeBytes = kMergeM + 3 * kAtcRows * 4;
    static_assert(kMergeBytes <= kBar, "the merge buffer must not reach the barriers");
    static constexpr int kCols = kDo > 128 ? 512 : kDo > 64 ? 256 : 128;   // tensor-memory columns: 64 (S) + kDo (P V)
    // at most 512 / kCols CTAs of this kernel per SM: ask for more than 1 / (that + 1) of 227 KiB
    static constexpr int kMinBytes = (227 * 1024) / (512 / kCols + 1) + 1024;
    static constexpr int kBytes = kTileBytes > kMinBytes ? kTileBytes : kMinBytes;
};

// ---- tcgen05 / tensor-map copy / cluster wrappers ----
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
// The same for a K-major operand whose rows are swizzled (layout type in bits 61-63: 2, 4, 6
// for 128, 64, 32 bytes): the leading offset is not used (1), `group` is the stride between
// 8-row groups, and a step along the contraction inside a row adds its bytes to addr.
__device__ __forceinline__ uint64_t tc_desc_swizzled(uint32_t addr, uint32_t group, uint32_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(group >> 4) << 32) | (1ull << 46) |
           ((uint64_t)layout << 61);
}
// One box of a 2-D tensor map (x: bytes along a row, y: row) into this CTA's shared memory,
// completion counted in bytes on `bar`.  x must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Instruction descriptors: FP32 accumulator (bits 4-5 = 1), operand formats (bits 7-9 and
// 10-12: E5M2 = 1 for kind::f8f6f4, FP16 = 0 for kind::f16), B MN-major (bit 16), N / 8 (bits
// 17-22), M / 16 (bits 24-28).
constexpr uint32_t kAtcIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((kAtcTile / 8) << 17) | ((kAtcRows / 16) << 24);
template <int D>
constexpr uint32_t kAtcIdescPV = (1u << 4) | (1u << 16) | ((uint32_t)(D / 8) << 17) | ((kAtcRows / 16) << 24);   // D: columns of the product

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
// This thread's lane of tensor memory, N = 16 or 32 consecutive columns from taddr.
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&r)[N]) {
    static_assert(N == 16 || N == 32, "16 or 32 columns");
    uint32_t x[N];
    if constexpr (N == 32)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]),
              "=r"(x[8]), "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15]),
              "=r"(x[16]), "=r"(x[17]), "=r"(x[18]), "=r"(x[19]), "=r"(x[20]), "=r"(x[21]), "=r"(x[22]), "=r"(x[23]),
              "=r"(x[24]), "=r"(x[25]), "=r"(x[26]), "=r"(x[27]), "=r"(x[28]), "=r"(x[29]), "=r"(x[30]), "=r"(x[31])
            : "r"(taddr) : "memory");
    else
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]),
              "=r"(x[8]), "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15])
            : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < N; ++i) r[i] = __uint_as_float(x[i]);
}
// The same lane and columns, written.
template <int N>
__device__ __forceinline__ void tmem_st(uint32_t taddr, const float (&r)[N]) {
    static_assert(N == 16 || N == 32, "16 or 32 columns");
    uint32_t x[N];
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = __float_as_uint(r[i]);
    if constexpr (N == 32)
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
            :: "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7]),
               "r"(x[8]), "r"(x[9]), "r"(x[10]), "r"(x[11]), "r"(x[12]), "r"(x[13]), "r"(x[14]), "r"(x[15]),
               "r"(x[16]), "r"(x[17]), "r"(x[18]), "r"(x[19]), "r"(x[20]), "r"(x[21]), "r"(x[22]), "r"(x[23]),
               "r"(x[24]), "r"(x[25]), "r"(x[26]), "r"(x[27]), "r"(x[28]), "r"(x[29]), "r"(x[30]), "r"(x[31]),
               "r"(taddr) : "memory");
    else
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
            :: "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7]),
               "r"(x[8]), "r"(x[9]), "r"(x[10]), "r"(x[11]), "r"(x[12]), "r"(x[13]), "r"(x[14]), "r"(x[15]),
               "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Two FP32 operations in one instruction (the lanes round like the scalar forms).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// CTA barrier with an OR over a predicate; the worker warps and the issuing warp meet in it
// from different places in the code.
__device__ __forceinline__ bool cta_sync_or(bool pred) {
    uint32_t r;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.or.pred q, 0, p; selp.u32 %0, 1, 0, q; }"
                 : "=r"(r) : "r"((uint32_t)pred) : "memory");
    return r != 0;
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
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float4 x) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"r"(addr), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float x) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(x) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float x;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x) : "r"(addr) : "memory");
    return x;
}

// Host side: a row-major matrix of `rows` x d bytes as a 2-D tensor map with boxes of
// box_bytes x box_rows (swizzled over box_bytes = 32, 64 or 128, or not swizzled and up to
// 256 bytes wide); elements
// outside the matrix read as zeros.  False if the driver does not offer the encoder or
// refuses the arguments (base 16-byte aligned, d a multiple of 16).
typedef CUresult (*AtcEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline AtcEncodeTiled atc_encoder() {
    static const AtcEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<AtcEncodeTiled>(p);
    }();
    return fn;
}
inline bool atc_make_map(CUtensorMap* map, const void* base, int d, long long rows, int box_bytes, int box_rows,
                         bool swizzled) {
    const AtcEncodeTiled encode = atc_encoder();
    if (!encode) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)d};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t steps[2] = {1, 1};
    const CUtensorMapSwizzle sw = !swizzled         ? CU_TENSOR_MAP_SWIZZLE_NONE
                                  : box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : box_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                                                     : CU_TENSOR_MAP_SWIZZLE_32B;
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, steps,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// D = codes per row: 32, 64, 128, 256 or 512.  Grid (splits, query blocks * kHalves), cluster
// (splits, kHalves, 1) with kHalves = 2 for 512 codes (the pair shares a query block), else 1;
// 288 threads, AtcLayout<D>::kBytes of dynamic shared memory.  map_q, map_k, map_v: the
// seq_len x D byte matrices as 2-D tensor maps with boxes of kSeg x 128, kSeg x 64 (swizzled)
// and kDo x 64 (not swizzled) bytes x rows (atc_make_map above); rows past seq_len read as
// zeros.
template <int D>
__global__ void __launch_bounds__(kAtcThreads, D > 128 ? 1 : D > 64 ? 2 : 3)   // CTAs per SM, see AtcLayout::kCols
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, float* __restrict__ out, int seq_len,
                    unsigned int* status) {
    extern __shared__ __align__(1024) unsigned char atc_smem[];
    using L = AtcLayout<D>;
    constexpr int DO = L::kDo;                    // output columns of this CTA
    constexpr int DH = DO / 2;                    // output columns per thread
    constexpr int KH = kAtcTile / 2;              // keys per thread
    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (kAtcRows - 1);         // this thread's query row = lane of tensor memory
    const int half = tid >> 7;                    // ... and which half of the keys and columns
    const int n_split = (int)gridDim.x, split = (int)blockIdx.x;
    const int row0 = (int)(blockIdx.y / L::kHalves) * kAtcRows;
    const int col0 = (int)(blockIdx.y % L::kHalves) * DO;      // this CTA's first output column
    const uint32_t sbase = smem_u32(atc_smem);
    const uint32_t bar_s = sbase + L::kBar, bar_o = bar_s + 8;
    const uint32_t bar_k = bar_s + 32, bar_v = bar_s + 48;     // + 8: the second buffer's
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may be scheduled as SMs free up
    if (sbase & 1023u) {                          // the swizzled operands want 1 KiB alignment (every CTA alike)
        if (tid == 0) atomicOr(status, 2u);
        return;
    }

    // this CTA's key tiles: a contiguous range
    const int tiles = (seq_len + kAtcTile - 1) / kAtcTile;
    const int per = (tiles + n_split - 1) / n_split;
    const int t_begin = min(split * per, tiles);
    const int n = min(tiles, t_begin + per) - t_begin;

    // One lane of the issuing warp does everything asynchronous.  The codes of key tile t
    // arrive by tensor-map copies that count their bytes on mbarriers: K into the swizzled
    // operand layout (buffer and phase of tile t: t % 2 and t / 2 with two buffers, 0 and t
    // with one), this CTA's columns of V as stored (buffer t % 2, phase t / 2).
    auto k_bar = [&](int t) { return bar_k + (L::kKBufs == 2 ? 8 * (t & 1) : 0); };
    auto k_parity = [&](int t) { return (uint32_t)((L::kKBufs == 2 ? t >> 1 : t) & 1); };
    auto k_at = [&](int t) { return sbase + L::kK + (L::kKBufs == 2 ? (t & 1) * L::kKBytes : 0); };
    auto load_k = [&](int t, uint32_t more_bytes = 0) {
        mbar_arrive_expect_tx(k_bar(t), L::kKBytes + more_bytes);
#pragma unroll
        for (int g = 0; g < L::kSegs; ++g)
            tma_load_2d(k_at(t) + g * (kAtcTile * L::kSeg), &map_k, g * L::kSeg, (t_begin + t) * kAtcTile, k_bar(t));
    };
    auto load_v = [&](int t) {
        mbar_arrive_expect_tx(bar_v + 8 * (t & 1), L::kVrawBytes);
        tma_load_2d(sbase + L::kVraw + (t & 1) * L::kVrawBytes, &map_v, col0, (t_begin + t) * kAtcTile, bar_v + 8 * (t & 1));
    };
    constexpr int kIssuer = kAtcWorkers / 32;     // the issuing warp: it also owns the tensor-memory allocation
    if (warp == kIssuer) {
        if ((tid & 31) == 0) {
            mbar_init(bar_s, 1);
            mbar_init(bar_o, 1);
            mbar_init(bar_k, 1);
            mbar_init(bar_k + 8, 1);
            mbar_init(bar_v, 1);
            mbar_init(bar_v + 8, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            // Launched with programmatic stream serialization, the grid may start while the
            // kernel before it in the stream still runs: nothing of global memory is read
            // before that kernel has completed (Q, K, V may be its results) ...
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (n > 0) {                          // the first copies leave before anything else is set up
                load_k(0, L::kQBytes);            // Q rides on the first K tile's barrier
#pragma unroll
                for (int g = 0; g < L::kSegs; ++g)
                    tma_load_2d(sbase + L::kQ + g * (kAtcRows * L::kSeg), &map_q, g * L::kSeg, row0, k_bar(0));
                load_v(0);
                if (n > 1) {
                    if (L::kKBufs == 2) load_k(1);
                    load_v(1);
                }
            }
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sbase + L::kBar + 16), "r"((uint32_t)L::kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(atc_smem + L::kBar + 16);
    // a warp reaches the 32 lanes of its quarter: warps w and w + 4 share lanes 32 (w % 4) ..
    const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    // The products: S = Q K^T of a tile (d / 32 instructions of 32 codes each: 32 bytes further
    // along the swizzled rows) and P V (4 instructions of 16 keys, two key groups, each).
    auto issue_qk = [&](int t) {
#pragma unroll
        for (int j = 0; j < D / 32; ++j) {
            constexpr int kPer = L::kSeg / 32;    // steps per column segment
            tc_mma<true>(tmem,
                         tc_desc_swizzled(sbase + L::kQ + (j / kPer) * (kAtcRows * L::kSeg) + (j % kPer) * 32,
                                          L::kGroup, L::kSwizzle),
                         tc_desc_swizzled(k_at(t) + (j / kPer) * (kAtcTile * L::kSeg) + (j % kPer) * 32,
                                          L::kGroup, L::kSwizzle),
                         kAtcIdescQK, j > 0);
        }
        tc_commit(bar_s);
    };
    auto issue_pv = [&](int buf, bool accumulate) {
#pragma unroll
        for (int j = 0; j < kAtcTile / 16; ++j)
            tc_mma<false>(tmem + kAtcTile,
                          tc_desc(sbase + L::kP + j * 2 * (kAtcRows * 16), kAtcRows * 16, 128),
                          tc_desc(sbase + L::kV + buf * L::kVBytes + j * 2 * L::kVLbo, L::kVLbo, L::kVSbo),
                          kAtcIdescPV<DO>, accumulate || j > 0);
        tc_commit(bar_o);
    };
    // V codes -> FP16 (8 codes -> one 16-byte unit) in the layout P V reads.
    auto spread_v = [&](int buf) {
#pragma unroll
        for (int u = tid; u < kAtcTile * (DO / 8); u += kAtcWorkers) {
            const int ng = u % (DO / 8), key = u / (DO / 8);
            const uint2 w = *reinterpret_cast<const uint2*>(atc_smem + L::kVraw + buf * L::kVrawBytes + key * DO + ng * 8);
            uint4 h;
            decode_word_h2<kE5M2>(w.x, h.x, h.y);
            decode_word_h2<kE5M2>(w.y, h.z, h.w);
            *reinterpret_cast<uint4*>(atc_smem + L::kV + buf * L::kVBytes + (key >> 3) * L::kVLbo + ng * L::kVSbo +
                                      (key & 7) * 16) = h;
        }
    };

    // The output accumulates in tensor memory (columns 64 .. 64 + D - 1): P(i) V(i) adds to
    // it, and before that product is issued each thread has multiplied its half row by
    // alpha = e^(old maximum - new maximum), as the reference's acc * alpha + P V does.
    // The running maximum lives in the exponent's own scale: m2 = max(score) * log2(e) /
    // sqrt(d), so that e^(score / sqrt(d) - max) is one FMA and one ex2 per score.  l sums
    // this thread's half of the keys only; the halves meet in the merge.
    float m2 = -INFINITY, l = 0.f;
    const float scale2 = 1.4426950408889634f / sqrtf((float)D);
    bool ok = true;
    constexpr int CH = 16;                        // output columns per tensor-memory load or store (32 at a time spill registers)
    const uint32_t tmem_o = tmem_row + kAtcTile + DH * half;

    // The loop has ONE CTA barrier per tile.  At the barrier of tile i every worker has
    // stored its part of P(i), rescaled its part of the output, stored its part of V(i + 1)
    // as FP16 (second half of the previous trip) and has seen its copies of tile i + 1's
    // codes land; behind the barrier the issuing warp issues S(i + 1) = Q K(i + 1)^T and then
    // P(i) V(i), so that the tensor core has the next scores ready when the workers come
    // back from their copies.
    if (warp == kIssuer) {
        // ---- the issuing warp: the workers' tile barriers, one lane issues behind each ----
        bool okk = true;
        if (n > 0 && (tid & 31) == 0) {
            okk = mbar_wait(k_bar(0), k_parity(0), status);
            issue_qk(0);
            if (L::kKBufs == 1 && n > 1) {        // the one K buffer is free once S(0) is done
                okk = mbar_wait(bar_s, 0, status) && okk;
                load_k(1);
            }
        }
        __syncwarp();
        for (int i = 0; i < n; ++i) {
            if (cta_sync_or(false)) break;
            if ((tid & 31) == 0) {
                tc_fence_after();
                if (i + 1 < n) {
                    okk = mbar_wait(k_bar(i + 1), k_parity(i + 1), status) && okk;
                    issue_qk(i + 1);
                }
                issue_pv(i & 1, i > 0);
                // tile i + 2's codes go where tile i's were: S(i) and the spread of V(i) are done with them
                if (i + 2 < n) {
                    load_v(i + 2);
                    if (L::kKBufs == 1) okk = mbar_wait(bar_s, (uint32_t)((i + 1) & 1), status) && okk;   // S(i + 1) done
                    load_k(i + 2);
                }
            }
            __syncwarp();
        }
    } else {
        if (n > 0) {
            ok = mbar_wait(bar_v, 0, status);
            spread_v(0);
        }

        for (int i = 0; i < n; ++i) {
            const int buf = i & 1;
            // ---- S(i) is ready; P(i - 1) V(i - 1) has completed: P and the output are ours ----
            ok = mbar_wait(bar_s, (uint32_t)(i & 1), status) && ok;
            if (i > 0) ok = mbar_wait(bar_o, (uint32_t)((i - 1) & 1), status) && ok;
            tc_fence_after();
            float s[KH];                          // this thread's 32 keys; the other 32 only feed the maximum
            float mx4[4];
            {
                float other[KH];
                tmem_ld<KH>(tmem_row + KH * (half ^ 1), other);
#pragma unroll
                for (int j = 0; j < 4; ++j) mx4[j] = other[j];
#pragma unroll
                for (int j = 4; j < KH; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], other[j]);
            }
            tmem_ld<KH>(tmem_row + KH * half, s);
#pragma unroll
            for (int j = 0; j < KH; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float mn2 = fmaxf(m2, mx * scale2);
            const float alpha = ex2_approx(m2 - mn2);
            // pairs of scores through the packed FP32 forms: one FMA and one add per two scores
            const uint64_t scale_pair = f2_pack(scale2, scale2), minus_max = f2_pack(-mn2, -mn2);
            uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};      // four pairs of partial sums (+0.0f bits)
#pragma unroll
            for (int u = 0; u < KH / 8; ++u) {
                uint32_t p[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    float a0, a1;
                    f2_unpack(f2_fma(f2_pack(s[8 * u + 2 * x], s[8 * u + 2 * x + 1]), scale_pair, minus_max), a0, a1);
                    const float e0 = ex2_approx(a0), e1 = ex2_approx(a1);
                    sum2[x] = f2_add(sum2[x], f2_pack(e0, e1));
                    const __half2 h = __floats2half2_rn(e0, e1);
                    p[x] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(atc_smem + L::kP + (half * (KH / 8) + u) * (kAtcRows * 16) + row * 16) =
                    make_uint4(p[0], p[1], p[2], p[3]);
            }
            {
                float lo, hi;
                f2_unpack(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])), lo, hi);
                l = l * alpha + (lo + hi);
            }
            m2 = mn2;
            // ---- output *= alpha, unless no row of this warp saw a new maximum (alpha = 1 everywhere) ----
            if (i > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) {
#pragma unroll
                for (int c = 0; c < DH / CH; ++c) {
                    float acc[CH];
                    tmem_ld<CH>(tmem_o + CH * c, acc);
                    const uint64_t alpha_pair = f2_pack(alpha, alpha);
#pragma unroll
                    for (int x = 0; x < CH; x += 2) f2_unpack(f2_mul(f2_pack(acc[x], acc[x + 1]), alpha_pair), acc[x], acc[x + 1]);
                    tmem_st<CH>(tmem_o + CH * c, acc);
                }
                tmem_wait_st();
            }
            fence_proxy_async_smem();             // P(i) and V(i + 1) as FP16: visible to the tensor core
            tc_fence_before();
            if (cta_sync_or(!ok)) break;
            if (i + 1 < n) {                      // P(i - 1) V(i - 1), the last reader of that half, has completed
                ok = mbar_wait(bar_v + 8 * (buf ^ 1), (uint32_t)(((i + 1) >> 1) & 1), status) && ok;
                spread_v(buf ^ 1);
            }
        }
        if (n > 0 && ok) ok = mbar_wait(bar_o, (uint32_t)((n - 1) & 1), status);
        tc_fence_after();
    }
    // ---- partial result to shared memory (the operands are no longer read), merge over the cluster ----
    float* mo = reinterpret_cast<float*>(atc_smem);
    if (warp != kIssuer) {
#pragma unroll
        for (int c = 0; c < DH / CH; ++c) {
            float acc[CH];
            if (n > 0) {
                tmem_ld<CH>(tmem_o + CH * c, acc);
            } else {
#pragma unroll
                for (int x = 0; x < CH; ++x) acc[x] = 0.f;
            }
#pragma unroll
            for (int x = 0; x < CH; x += 4)
                *reinterpret_cast<float4*>(mo + row * L::kMergeStride + DH * half + CH * c + x) =
                    make_float4(acc[x], acc[x + 1], acc[x + 2], acc[x + 3]);
        }
        if (half == 0) mo[L::kMergeM / 4 + row] = m2;
        mo[L::kMergeM / 4 + (1 + half) * kAtcRows + row] = l;
    }
    tc_fence_before();
    cluster_sync();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // ... and nothing is written (it may write `out` too)
    // Every CTA merges its share of the 128 rows (128 / n_split, rounded up): four columns
    // per item, consecutive threads along a row (remote reads and global stores are
    // contiguous runs).  A thread reads the n_split maxima and sums of its row and the
    // n_split pieces of its item and weighs them with 2^(m_c - m), CTAs in rank order.
    const int rows_per = (kAtcRows + n_split - 1) / n_split;          // the last CTA may own fewer
    const int rows_here = max(0, min(rows_per, kAtcRows - split * rows_per));
    uint32_t peer[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)               // the CTAs with this CTA's columns: cluster rank = split + n_split * column half
        peer[c] = map_cluster(sbase, (uint32_t)(min(c, n_split - 1) + n_split * (int)(blockIdx.y % L::kHalves)));
    constexpr int kGroups = DO / 4;
    if (n_split == 1) {
        // nothing to merge: this CTA's own rows, plain shared-memory loads
        const float* mo_l = mo + L::kMergeM / 4 + kAtcRows;
        for (int idx = tid; idx < kAtcRows * kGroups && warp != kIssuer; idx += kAtcWorkers) {
            const int rr = idx / kGroups, g = idx % kGroups;
            if (row0 + rr >= seq_len) break;
            const float lsum = mo_l[rr] + mo_l[kAtcRows + rr];
            const float4 x = *reinterpret_cast<const float4*>(mo + rr * L::kMergeStride + 4 * g);
            *reinterpret_cast<float4*>(out + (size_t)(row0 + rr) * D + col0 + 4 * g) =
                make_float4(__fdiv_rn(x.x, lsum), __fdiv_rn(x.y, lsum), __fdiv_rn(x.z, lsum), __fdiv_rn(x.w, lsum));
        }
    }
    for (int idx = tid; idx < rows_here * kGroups && warp != kIssuer && n_split > 1; idx += kAtcWorkers) {
        const int rl = idx / kGroups, g = idx % kGroups;
        const int rr = split * rows_per + rl;             // row of the query block
        // every remote load of the item leaves before the first is used: one round trip
        float w[8], la[8], lb[8];
        float4 x[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < n_split) {
                w[c] = ld_cluster_f32(peer[c] + L::kMergeM + rr * 4);
                la[c] = ld_cluster_f32(peer[c] + L::kMergeM + (kAtcRows + rr) * 4);
                lb[c] = ld_cluster_f32(peer[c] + L::kMergeM + (2 * kAtcRows + rr) * 4);
                x[c] = ld_cluster_f32x4(peer[c] + (uint32_t)(rr * L::kMergeStride + 4 * g) * 4);
            } else {
                w[c] = -INFINITY;
                la[c] = lb[c] = 0.f;
                x[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (row0 + rr >= seq_len) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; ++c) mm = fmaxf(mm, w[c]);
        float lsum = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float wc = ex2_approx(w[c] - mm);       // a CTA without tiles: 2^(-inf) = 0
            lsum += (la[c] + lb[c]) * wc;
            acc.x += x[c].x * wc;
            acc.y += x[c].y * wc;
            acc.z += x[c].z * wc;
            acc.w += x[c].w * wc;
        }
        *reinterpret_cast<float4*>(out + (size_t)(row0 + rr) * D + col0 + 4 * g) =
            make_float4(__fdiv_rn(acc.x, lsum), __fdiv_rn(acc.y, lsum), __fdiv_rn(acc.z, lsum), __fdiv_rn(acc.w, lsum));
    }
    cluster_sync();                           // nobody leaves while a peer reads its memory
    if (warp == kIssuer) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)L::kCols) : "memory");
    }
}

}  // namespace feather
