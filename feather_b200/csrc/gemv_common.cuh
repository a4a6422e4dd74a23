// Device helpers shared by the GEMV and dot kernels: streaming loads, the FP16
// pair decode, the mixed-precision FMA and the warp reductions.
#pragma once
#include "fp8_codec.cuh"

namespace feather {

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

// acc += a.lo * b.lo ; acc2 += a.hi * b.hi   (FP16 operands, FP32 accumulate)
__device__ __forceinline__ void fma_h2(uint32_t a, uint32_t b, float& acc_lo, float& acc_hi) {
    asm("{ .reg .b16 a0, a1, b0, b1;\n"
        "  mov.b32 {a0, a1}, %2; mov.b32 {b0, b1}, %3;\n"
        "  fma.rn.f32.f16 %0, a0, b0, %0;\n"
        "  fma.rn.f32.f16 %1, a1, b1, %1; }"
        : "+f"(acc_lo), "+f"(acc_hi) : "r"(a), "r"(b));
}

// Decode the four codes of a word to two FP16 pairs (same pairing for the
// matrix and the vector): E5M2 lo=(c0,c1) hi=(c2,c3); E4M3 lo=(c0,c2) hi=(c1,c3).
template <int MODE>
__device__ __forceinline__ void decode_word_h2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    if (MODE == kE5M2) {
        lo = prmt(w, 0u, 0x1404u);
        hi = prmt(w, 0u, 0x3424u);
    } else {
        lo = e4m3_pair_to_h2(w << 8);
        hi = e4m3_pair_to_h2(w);
    }
}

// One 16-byte chunk of a row (16 codes) times the matching 16 vector values
// (va, vb: eight FP16 pairs in decode_word_h2's pairing) into four accumulators.
template <int MODE>
__device__ __forceinline__ void fma_chunk(const uint4 mw, const uint4 va, const uint4 vb,
                                          float (&acc)[4]) {
    uint32_t lo, hi;
    decode_word_h2<MODE>(mw.x, lo, hi);
    fma_h2(lo, va.x, acc[0], acc[1]);
    fma_h2(hi, va.y, acc[2], acc[3]);
    decode_word_h2<MODE>(mw.y, lo, hi);
    fma_h2(lo, va.z, acc[0], acc[1]);
    fma_h2(hi, va.w, acc[2], acc[3]);
    decode_word_h2<MODE>(mw.z, lo, hi);
    fma_h2(lo, vb.x, acc[0], acc[1]);
    fma_h2(hi, vb.y, acc[2], acc[3]);
    decode_word_h2<MODE>(mw.w, lo, hi);
    fma_h2(lo, vb.z, acc[0], acc[1]);
    fma_h2(hi, vb.w, acc[2], acc[3]);
}

// Sum RW per-lane values over the warp with a halving butterfly: after it, the
// lanes with lane % (32/RW) == 0 hold the total of row lane / (32/RW) in v[0].
template <int RW>
__device__ __forceinline__ void warp_reduce_rows(float (&v)[RW], int lane) {
    int o = 16;
#pragma unroll
    for (int n = RW; n > 1; n >>= 1, o >>= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
        }
    }
    for (; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xFFFFFFFFu, v[0], o);
}

// How long a bounded wait may go without progress before it gives up: 2 s
// unless the host changed it (feather_set_wait_limit_ms).  One copy per kernel
// image that includes this header; the library has one.
__device__ unsigned long long g_wait_limit_ns = 2000000000ull;
#define kWaitLimitNs g_wait_limit_ns

// Sticky status word: bit 0 / 1 / 2 raised by a bounded wait that gave up
// (ring stage / peer rank / chain dependency), bit 8 by a bounds guard of a
// -DFEATHER_DEBUG_BOUNDS build.  Read and cleared by feather_device_status().
__device__ unsigned int g_wait_status;

// Debug builds (-DFEATHER_DEBUG_BOUNDS, the stand-in for a memory checker):
// every global-memory index the GEMV kernels form is checked against its
// buffer; a bad one raises bit 8 of the status word and the access is skipped.
// Release builds compile the guard away.
__device__ __forceinline__ bool bounds_ok(bool ok) {
#ifdef FEATHER_DEBUG_BOUNDS
    if (!ok) atomicOr(&g_wait_status, 0x100u);
    return ok;
#else
    (void)ok;
    return true;
#endif
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// System-scope relaxed accesses for the epoch flags.  Ordering comes from ONE
// system-scope fence before the flag stores (release pattern) and one after the
// flag loads (acquire pattern): a release store per peer would pay a full
// system fence per peer, which at eight ranks cost more than the whole exchange.
__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// 16-byte accesses that are neither cached in L1 nor reordered by the
// compiler, for (value, tag) pairs that a peer GPU writes and this GPU polls.
// An aligned 8-byte half of such a store arrives whole, so a pair whose tag
// matches carries its value.
__device__ __forceinline__ void st_volatile_v4(float* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const float* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Column-sharded GEMV with the all-reduce fused behind it (gemv_rows_kernel,
// ALLREDUCE = true): where every rank's inbox and flag block live, as mapped
// into this process.  An inbox is two halves used by alternate calls; a half
// holds one slot per rank, a slot one (sum, call number) pair per row, M rounded
// up to a multiple of 16 rows.
constexpr int kMaxArRanks = 16;
constexpr int kArTicketWord = 16;  // flag-block word: CTAs of the running call that have finished
constexpr int kArEpochWord = 17;   // flag-block word: number of all-reduce calls completed so far
struct AllReduceArgs {
    float* inbox[kMaxArRanks];           // rank p's inbox
    unsigned int* flags[kMaxArRanks];    // rank p's flag block (only this rank's own is used)
    float* result;                       // this rank's reduced output, M floats
    long long half;                      // floats per half of an inbox
    int rank, world;
};

}  // namespace feather
