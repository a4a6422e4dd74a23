// C ABI of libfeather_b200.so (declared in include/feather_b200.h): argument
// checks, launch geometry and the encode / decode kernels.  The GEMV and dot
// kernels live in gemv_kernels.cuh / dot_kernels.cuh.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>

#include "../../include/feather_b200.h"
#include "attention_kernels.cuh"
#include "attention_tc.cuh"
#include "dot_kernels.cuh"
#include "fp8_codec.cuh"
#include "gemv_chain.cuh"
#include "gemv_kernels.cuh"
#include "gemv_multi.cuh"
#include "gemv_multi_tc.cuh"
#include "gemv_mma.cuh"
#include "gemv_ring.cuh"

namespace feather {

// ------------------------------------------------------------ tuning -------
// Knobs for A/B runs in benchmarks, never needed for correct results.  Set by
// feather_set_tuning("key=value,key=value") or, once, from the environment
// variable FEATHER_KERNEL when the library first touches a device.
//   ring_pre_kb      KiB of a CTA's first rows the ring kernel asks L2 for ahead
//                    of its stream-order wait (0 = none)
//   rows_pre         1: the warp-owned-rows kernel does the same for its first batch
//   dot_unroll       16-byte loads per operand a dot thread keeps in flight (1, 2, 4)
//   dot_ctas_per_sm  grid of the dot kernel, in CTAs per SM
//   ring_pre_kb_e4m3 the same for E4M3 matrices; -1 = 64 KiB for matrices up to 128 MiB,
//                    none above (measured: the decode-bound kernel loses there)
//   dot_ring         0: register-load dot kernel only; 1, 2, 3: long aligned operands take the
//                    bulk-copy ring kernel with 6 x 32 KiB, 3 x 64 KiB or 12 x 16 KiB stages
//   dot_pre_kb       KiB the dot ring kernel asks L2 for ahead of its stream-order wait
//   attn_tc          attention with 32 .. 512 codes per row: 0 the register-fed mma.sync
//                    kernel, 1 the tcgen05 kernel from 1024 / 1024 / 256 / 128 / 128 queries
//                    up, 2 the tcgen05 kernel always
//   multi_tc         E5M2 GEMV against several vectors, large matrices with rows of a multiple of
//                    128 codes: 1 the tcgen05 kernel (16 vectors per pass), 0 the mma.sync kernel
struct Tuning {
    std::atomic<int> ring_pre_kb{128};
    std::atomic<int> rows_pre{1};
    std::atomic<int> dot_unroll{4};
    std::atomic<int> dot_ctas_per_sm{6};
    std::atomic<int> dot_ring{2};
    std::atomic<int> dot_pre_kb{64};
    std::atomic<int> ring_pre_kb_e4m3{-1};
    std::atomic<int> attn_tc{1};
    std::atomic<int> multi_tc{1};
};
static Tuning g_tune;

static int apply_tuning(const char* spec) {
    if (!spec) return FEATHER_ERR_BAD_ARG;
    const char* p = spec;
    while (*p) {
        while (*p == ',' || *p == ' ') ++p;
        if (!*p) break;
        const char* eq = strchr(p, '=');
        if (!eq) return FEATHER_ERR_BAD_ARG;
        const size_t klen = (size_t)(eq - p);
        char* end = nullptr;
        const long val = strtol(eq + 1, &end, 10);
        if (end == eq + 1 || (*end && *end != ',' && *end != ' ')) return FEATHER_ERR_BAD_ARG;
        auto is = [&](const char* k) { return strlen(k) == klen && strncmp(p, k, klen) == 0; };
        if (is("ring_pre_kb") && val >= 0 && val <= 16384) g_tune.ring_pre_kb = (int)val;
        else if (is("rows_pre") && (val == 0 || val == 1)) g_tune.rows_pre = (int)val;
        else if (is("dot_unroll") && (val == 1 || val == 2 || val == 4)) g_tune.dot_unroll = (int)val;
        else if (is("dot_ctas_per_sm") && val >= 1 && val <= 16) g_tune.dot_ctas_per_sm = (int)val;
        else if (is("dot_ring") && val >= 0 && val <= 3) g_tune.dot_ring = (int)val;
        else if (is("dot_pre_kb") && val >= 0 && val <= 16384) g_tune.dot_pre_kb = (int)val;
        else if (is("ring_pre_kb_e4m3") && val >= -1 && val <= 16384) g_tune.ring_pre_kb_e4m3 = (int)val;
        else if (is("attn_tc") && val >= 0 && val <= 2) g_tune.attn_tc = (int)val;
        else if (is("multi_tc") && (val == 0 || val == 1)) g_tune.multi_tc = (int)val;
        else return FEATHER_ERR_BAD_ARG;
        p = end;
    }
    return FEATHER_OK;
}

// ------------------------------------------------------------ encode -------
// One thread per 16 elements: 128-bit loads of the source, one 128-bit store
// of sixteen codes (feather/packers/fp8.py:123-134: element 4k + i goes to
// byte i of word k, i.e. the packed buffer is the code stream in element
// order).
template <int MODE>
__device__ __forceinline__ uint32_t pack4(float a, float b, float c, float d) {
    return encode_f32<MODE>(a) | (encode_f32<MODE>(b) << 8) | (encode_f32<MODE>(c) << 16) |
           (encode_f32<MODE>(d) << 24);
}

// fp16 -> fp32 widening is exact, but the hardware conversion may hand back a
// canonical NaN; the sign is therefore taken from the fp16 bits themselves
// (the reference keeps the sign of a NaN: 0xFE / 0xFF codes).
template <int MODE>
__device__ __forceinline__ uint32_t encode_h(uint32_t h16) {
    const float x = __half2float(__ushort_as_half((unsigned short)h16));
    const uint32_t u = (__float_as_uint(x) & 0x7FFFFFFFu) | ((h16 & 0x8000u) << 16);
    return MODE == kE5M2 ? encode_e5m2(u) : encode_e4m3(u);
}

template <int MODE>
__device__ __forceinline__ uint32_t pack4_h(uint2 h) {  // four fp16 values
    return encode_h<MODE>(h.x & 0xFFFFu) | (encode_h<MODE>(h.x >> 16) << 8) |
           (encode_h<MODE>(h.y & 0xFFFFu) << 16) | (encode_h<MODE>(h.y >> 16) << 24);
}

// fp16 -> E5M2 on two values at once.  For a non-NaN fp16 bit pattern h the
// code is RNE of the low byte:  (h + 0x7F + ((h >> 8) & 1)) >> 8  (a mantissa
// carry walks into the exponent, 0x7BFF.. rounds to inf 0x7C).  Both halves of
// a 32-bit word are rounded with one add; no carry can cross from the low half
// to the high half unless the low half is a negative NaN, and words that hold
// a NaN take the scalar path.  The two codes end up in bytes 1 and 3.
__device__ __forceinline__ uint32_t round_e5m2_pair(uint32_t w) {
    return w + 0x007F007Fu + ((w >> 8) & 0x00010001u);
}
__device__ __forceinline__ uint32_t has_nan_pair(uint32_t w) {  // bit 15 / 31 set for a NaN half
    return ((w & 0x7FFF7FFFu) + 0x03FF03FFu) & 0x80008000u;
}

template <int MODE, bool F32>
__global__ void __launch_bounds__(256)
encode_vec_kernel(const void* __restrict__ src, uint4* __restrict__ dst, long long n_groups) {
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    uint4 o;
    if (F32) {
        const float4* s = reinterpret_cast<const float4*>(src) + g * 4;
        const float4 a = __ldcs(s), b = __ldcs(s + 1), c = __ldcs(s + 2), d = __ldcs(s + 3);
        o.x = pack4<MODE>(a.x, a.y, a.z, a.w);
        o.y = pack4<MODE>(b.x, b.y, b.z, b.w);
        o.z = pack4<MODE>(c.x, c.y, c.z, c.w);
        o.w = pack4<MODE>(d.x, d.y, d.z, d.w);
    } else {
        const uint4* s = reinterpret_cast<const uint4*>(src) + g * 2;
        const uint4 a = __ldcs(s), b = __ldcs(s + 1);
        if (MODE == kE5M2) {
            const uint32_t nan = has_nan_pair(a.x) | has_nan_pair(a.y) | has_nan_pair(a.z) |
                                 has_nan_pair(a.w) | has_nan_pair(b.x) | has_nan_pair(b.y) |
                                 has_nan_pair(b.z) | has_nan_pair(b.w);
            if (nan == 0u) {  // the usual case: sixteen values, two per integer add
                o.x = prmt(round_e5m2_pair(a.x), round_e5m2_pair(a.y), 0x7531u);
                o.y = prmt(round_e5m2_pair(a.z), round_e5m2_pair(a.w), 0x7531u);
                o.z = prmt(round_e5m2_pair(b.x), round_e5m2_pair(b.y), 0x7531u);
                o.w = prmt(round_e5m2_pair(b.z), round_e5m2_pair(b.w), 0x7531u);
                dst[g] = o;
                return;
            }
        }
        o.x = pack4_h<MODE>(make_uint2(a.x, a.y));
        o.y = pack4_h<MODE>(make_uint2(a.z, a.w));
        o.z = pack4_h<MODE>(make_uint2(b.x, b.y));
        o.w = pack4_h<MODE>(make_uint2(b.z, b.w));
    }
    dst[g] = o;
}

// One thread per word, element loads: unaligned buffers and the ragged tail
// (elements past n_elems encode as code 0, fp8.py:200-204).
template <int MODE, bool F32>
__global__ void __launch_bounds__(256)
encode_word_kernel(const void* __restrict__ src, uint32_t* __restrict__ dst, long long first_word,
                   long long n_words, long long n_elems) {
    const long long w = first_word + (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= n_words) return;
    uint32_t code[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long e = w * 4 + i;
        if (e >= n_elems) code[i] = 0u;
        else if (F32) code[i] = encode_f32<MODE>(reinterpret_cast<const float*>(src)[e]);
        else code[i] = encode_h<MODE>(reinterpret_cast<const unsigned short*>(src)[e]);
    }
    dst[w] = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
}

// ------------------------------------------------------------ decode -------
template <int MODE, bool IEEE>
__device__ __forceinline__ float4 decode4(uint32_t w) {
    if (MODE == kE4M3 && IEEE)
        return make_float4(decode_e4m3_ieee(w & 0xFF), decode_e4m3_ieee((w >> 8) & 0xFF),
                           decode_e4m3_ieee((w >> 16) & 0xFF), decode_e4m3_ieee(w >> 24));
    return decode_word_ordered<MODE>(w);  // E5M2: both semantics coincide
}

// One packed word per thread and step, eight steps in flight: the word loads of a
// warp are one 128-byte line, its float4 stores one 512-byte run.  Measured on B200, 2^26
// codes to FP32 (67 MB read, 268 MB written): steps a whole grid apart 62.2 us; consecutive
// lines per warp, four per trip 58.6 us, eight 55.6 us (16 CTAs per SM) / 54.6 us (32 per
// SM or one trip per warp), sixteen 55.3 us; 8 CTAs per SM 61 - 63 us.  RELU: the
// reference's ReLU-on-unpack (feather/routines/activations.py:8-29), max(0, x)
// with the compiled kernel's semantics of max: a NaN code gives 0, -0 gives +0.
constexpr int kDecodeLines = 8;   // 128-byte lines of codes a warp takes per trip
template <int MODE, bool IEEE, bool RELU>
__global__ void __launch_bounds__(256)
decode_kernel(const uint32_t* __restrict__ src, float* __restrict__ dst, long long n_elems) {
    const long long n_words = (n_elems + 3) >> 2;
    const bool vec = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    // A warp takes eight consecutive 128-byte lines of codes per trip (lane l the words l,
    // l + 32, ... of them) and writes 4 KB of consecutive floats, a CTA 32 KB: long runs per
    // open DRAM page.
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    constexpr int U = kDecodeLines;
    for (long long base = warp * (32 * U); base < n_words; base += warps * (32 * U)) {
        uint32_t x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long w = base + 32 * u + lane;
            x[u] = w < n_words ? __ldg(src + w) : 0u;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long w = base + 32 * u + lane;
            if (w >= n_words) break;
            float4 f = decode4<MODE, IEEE>(x[u]);
            if (RELU) f = make_float4(fmaxf(0.f, f.x), fmaxf(0.f, f.y), fmaxf(0.f, f.z), fmaxf(0.f, f.w));
            const long long e = w * 4;
            if (vec && e + 4 <= n_elems) {
                __stcs(reinterpret_cast<float4*>(dst) + w, f);
            } else {
                const float y[4] = {f.x, f.y, f.z, f.w};
                for (int i = 0; i < 4 && e + i < n_elems; ++i) dst[e + i] = y[i];
            }
        }
    }
}

// ------------------------------------------------------------ host side ----
struct DeviceInfo {
    std::atomic<int> state{0};  // 0 unknown, 1 ok, -1 wrong architecture
    int sm_count = 0;
};
static DeviceInfo g_dev[64];

static int device_info(const DeviceInfo** info) {
    static std::once_flag env_once;
    std::call_once(env_once, [] {
        if (const char* spec = getenv("FEATHER_KERNEL")) apply_tuning(spec);  // a bad spec is ignored
    });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FEATHER_ERR_LAUNCH;
    DeviceInfo& d = g_dev[dev];
    int st = d.state.load(std::memory_order_acquire);
    if (st == 0) {
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return FEATHER_ERR_LAUNCH;
        d.sm_count = sms;
        st = (major == 10) ? 1 : -1;
        d.state.store(st, std::memory_order_release);
    }
    *info = &d;
    return st == 1 ? FEATHER_OK : FEATHER_ERR_ARCH;
}

static inline bool aligned(const void* p, uintptr_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

static inline int launch_status() {
    return cudaGetLastError() == cudaSuccess ? FEATHER_OK : FEATHER_ERR_LAUNCH;
}

template <int MODE, bool F32>
static int encode_launch(const void* src, uint32_t* dst, long long n, cudaStream_t s) {
    const long long n_words = (n + 3) / 4;
    long long vec_groups = 0;
    if (aligned(src, 16) && aligned(dst, 16)) vec_groups = n / 16;
    if (vec_groups > 0) {
        const long long blocks = (vec_groups + 255) / 256;
        encode_vec_kernel<MODE, F32><<<(unsigned)blocks, 256, 0, s>>>(
            src, reinterpret_cast<uint4*>(dst), vec_groups);
    }
    const long long rest = n_words - vec_groups * 4;
    if (rest > 0) {
        const long long blocks = (rest + 255) / 256;
        encode_word_kernel<MODE, F32><<<(unsigned)blocks, 256, 0, s>>>(src, dst, vec_groups * 4,
                                                                         n_words, n);
    }
    return launch_status();
}

// g_wait_status (gemv_common.cuh): the sticky status word of the device.
static int status_word(unsigned int** ptr) {
    static std::atomic<unsigned int*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FEATHER_ERR_LAUNCH;
    unsigned int* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_wait_status) != cudaSuccess)
            return FEATHER_ERR_LAUNCH;
        cached[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    return FEATHER_OK;
}

// Launch geometry.
//   ring kernel (large matrices): 16 consumer warps x 1 row, 4 KiB of a row per
//   bulk copy, 3 stages of 64 KiB, FP16 vector tile of 16384 codes, 1 CTA/SM.
//   rows kernel (small and mid-size): 8 warps per CTA, each warp owns 1, 2 or 4 rows.
constexpr int kRingCW = 16, kRingRW = 1, kRingCL = 8, kRingStages = 3, kRingTile = 16384;

template <typename K>
static int ensure_smem(K kernel, int smem, std::atomic<unsigned long long>& configured) {
    int devid = 0;
    if (cudaGetDevice(&devid) != cudaSuccess) return FEATHER_ERR_LAUNCH;
    if (!((configured.load(std::memory_order_acquire) >> devid) & 1ull)) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess)
            return FEATHER_ERR_LAUNCH;
        configured.fetch_or(1ull << devid, std::memory_order_release);
    }
    return FEATHER_OK;
}

// Bytes of a CTA's first rows the ring kernel asks L2 for ahead of its
// stream-order wait.  Measured on B200, back-to-back calls: E5M2 gains ~1 us per
// call with 64-128 KiB (more than 512 KiB per CTA overflows L2 and loses); E4M3,
// bound by decode issue, gains on matrices up to 128 MiB and loses above.
static int ring_pre_bytes(int mode, long long M, long long N) {
    if (mode == kE5M2) return g_tune.ring_pre_kb.load(std::memory_order_relaxed) * 1024;
    const int e4 = g_tune.ring_pre_kb_e4m3.load(std::memory_order_relaxed);
    if (e4 >= 0) return e4 * 1024;
    return M * N <= (128ll << 20) ? 64 * 1024 : 0;
}

template <int MODE, bool FUSED, bool EARLY = false>
static int gemv_ring_launch(const uint32_t* m, const uint32_t* v, float* out, long long M,
                            long long N, const DeviceInfo& dev, cudaStream_t s,
                            const ShardArgs& shard) {
    using G = RingGeometry<kRingCW, kRingRW, kRingCL, kRingStages, kRingTile>;
    auto kernel = gemv_ring_kernel<MODE, kRingCW, kRingRW, kRingCL, kRingStages, kRingTile, 1, false,
                                   FUSED, EARLY>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, G::kSmemBytes, configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    long long grid = dev.sm_count;
    const long long max_useful = (M + G::kTaskRows - 1) / G::kTaskRows;
    if (grid > max_useful) grid = max_useful;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(FUSED ? G::kThreadsFused : G::kThreads);
    cfg.dynamicSmemBytes = G::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const unsigned char*>(m),
                                             v, out, (int)M, (int)(N / 16), status,
                                             ring_pre_bytes(MODE, M, N), shard);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

// Shapes the bulk-copy ring kernel takes: 16-byte aligned rows, rows long
// enough for 4 KiB copies, and at least two full tasks for every SM.
static bool ring_eligible(const void* m, long long M, long long N, const DeviceInfo& dev) {
    return (N % 16 == 0) && aligned(m, 16) && N >= 4096 &&
           M >= 2ll * dev.sm_count * kRingCW * kRingRW;
}

template <int MODE, int RW, int U, bool EARLY>
static int gemv_rows_launch(const uint32_t* m, const uint32_t* v, float* out, long long M,
                            long long N, cudaStream_t s, int out_code = -1) {
    auto kernel = gemv_rows_kernel<MODE, RW, U, EARLY, false>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, gemv_rows_smem_bytes(kRowsTileCodes), configured)) return st;
    const long long rows_per_cta = (kRowsThreads / 32) * RW;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((M + rows_per_cta - 1) / rows_per_cta));
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = gemv_rows_smem_bytes((int)(N > kRowsTileCodes ? kRowsTileCodes : N));
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const uint4*>(m), v, out,
                                             (int)M, (int)(N / 16), out_code, NoAllReduce{},
                                             static_cast<unsigned int*>(nullptr),
                                             g_tune.rows_pre.load(std::memory_order_relaxed));
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

// Column-sharded GEMV with the all-reduce in the kernel's epilogue.  Its CTAs
// wait for the peers' CTAs of the same index, so the whole grid must be resident
// at once: FEATHER_ERR_TOO_LARGE when it is not.
template <int MODE, int RW, int U>
static int gemv_allreduce_launch(const uint32_t* m, const uint32_t* v, long long M, long long N,
                                 const AllReduceArgs& ar, const DeviceInfo& dev, cudaStream_t s) {
    auto kernel = gemv_rows_kernel<MODE, RW, U, true, true>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, gemv_rows_smem_bytes(kRowsTileCodes), configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    const long long rows_per_cta = (kRowsThreads / 32) * RW;
    const long long grid = (M + rows_per_cta - 1) / rows_per_cta;
    const int smem = gemv_rows_smem_bytes((int)(N > kRowsTileCodes ? kRowsTileCodes : N));
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRowsThreads, smem) != cudaSuccess)
        return FEATHER_ERR_LAUNCH;
    if (grid > (long long)per_sm * dev.sm_count) return FEATHER_ERR_TOO_LARGE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const uint4*>(m), v,
                                             static_cast<float*>(nullptr), (int)M, (int)(N / 16), -1, ar,
                                             status, 0);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

// out_code < 0: `out` receives M FP32 sums.  out_code = kE5M2 / kE4M3: `out`
// receives ceil(M / 4) packed words of the sums encoded to that format; the
// warp-owned-rows kernel encodes in its epilogue, the other kernels write the
// sums to `workspace` (M floats) and the encoder runs behind them.
template <int MODE>
static int gemv_launch(const uint32_t* m, const uint32_t* v, float* out, long long M, long long N,
                       const DeviceInfo& dev, cudaStream_t s, bool static_matrix = false,
                       int out_code = -1, float* workspace = nullptr) {
    const bool vec_ok = (N % 16 == 0) && aligned(m, 16);
    const bool ring = ring_eligible(m, M, N, dev);
    if (ring || !vec_ok) {
        float* sums = out_code < 0 ? out : workspace;
        if (!sums) return FEATHER_ERR_WORKSPACE;
        int st;
        if (ring) {
            st = static_matrix
                     ? gemv_ring_launch<MODE, false, true>(m, v, sums, M, N, dev, s, ShardArgs{})
                     : gemv_ring_launch<MODE, false>(m, v, sums, M, N, dev, s, ShardArgs{});
        } else {
            const long long blocks = (M + 7) / 8;  // 8 warps per CTA, one row per warp
            const long long cap = (long long)dev.sm_count * 8;
            gemv_general_kernel<MODE><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(
                m, v, sums, (int)M, (int)(N / 4));
            st = launch_status();
        }
        if (st != FEATHER_OK || out_code < 0) return st;
        uint32_t* words = reinterpret_cast<uint32_t*>(out);
        return out_code == kE5M2 ? encode_launch<kE5M2, true>(sums, words, M, s)
                                 : encode_launch<kE4M3, true>(sums, words, M, s);
    }
    // warp-owned rows: as many rows per warp as still leaves ~16 warps per SM
    const long long warps_wanted = (long long)dev.sm_count * 16;
    if (M >= 4 * warps_wanted)
        return static_matrix ? gemv_rows_launch<MODE, 4, 2, true>(m, v, out, M, N, s, out_code)
                             : gemv_rows_launch<MODE, 4, 2, false>(m, v, out, M, N, s, out_code);
    if (M >= 2 * warps_wanted)
        return static_matrix ? gemv_rows_launch<MODE, 2, 4, true>(m, v, out, M, N, s, out_code)
                             : gemv_rows_launch<MODE, 2, 4, false>(m, v, out, M, N, s, out_code);
    return static_matrix ? gemv_rows_launch<MODE, 1, 4, true>(m, v, out, M, N, s, out_code)
                         : gemv_rows_launch<MODE, 1, 4, false>(m, v, out, M, N, s, out_code);
}

template <int MODE, int NB, bool EARLY>
static int gemv_multi_launch(const uint32_t* m, const uint32_t* v, float* out, long long M,
                             long long N, int B, cudaStream_t s) {
    auto kernel = gemv_multi_kernel<MODE, NB, EARLY>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, gemv_multi_smem_bytes(kRowsTileCodes, NB), configured)) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((M + 15) / 16));
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = gemv_multi_smem_bytes((int)(N > kRowsTileCodes ? kRowsTileCodes : N), NB);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const uint4*>(m), v, out,
                                             (int)M, (int)(N / 16), B);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

template <int MODE, bool EARLY>
static int gemv_mma_launch(const uint32_t* m, const uint32_t* v, float* out, long long M, long long N,
                           int B, const DeviceInfo& dev, cudaStream_t s) {
    auto kernel = gemv_mma_kernel<MODE, EARLY>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, kMmaSmemBytes, configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    // 16-row groups a CTA works on at a time: the count (at most 8, two warps each)
    // that leaves the fewest idle SM-slots over the waves of the persistent grid;
    // ties go to the larger count (more of the matrix in flight per SM)
    const long long groups = (M + 15) / 16;
    int gpc = 1;
    double best = 0.0;
    for (int c = 1; c <= kMmaMaxGroups; ++c) {
        const long long passes = (groups + c - 1) / c;
        const long long waves = (passes + dev.sm_count - 1) / dev.sm_count;
        const double eff = (double)groups / (double)(waves * dev.sm_count * c);
        if (eff >= best - 1e-9) { best = eff; gpc = c; }
    }
    const long long passes = (groups + gpc - 1) / gpc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(passes < dev.sm_count ? passes : dev.sm_count));
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = kMmaSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const uint4*>(m), v, out,
                                             (int)M, (int)(N / 16), B, gpc, status);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

// E5M2, rows of a multiple of 128 codes, 16-byte aligned operands: up to 16 vectors per pass
// on the tcgen05 kernel.  One CTA per SM, its rows walked in equal blocks of at most 128.
static int gemv_multi_tc_launch(const uint32_t* m, const uint32_t* v, float* out, long long M, long long N,
                                int nb, const DeviceInfo& dev, cudaStream_t s) {
    auto kernel = gemv_multi_tc_kernel;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, kMtcSmemBytes, configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    long long grid = dev.sm_count;
    if (grid > (M + 15) / 16) grid = (M + 15) / 16;
    const long long rows_cta = (M + grid - 1) / grid;
    const long long n_blk = (rows_cta + kMtcSlotRows - 1) / kMtcSlotRows;
    const long long blk_rows = (rows_cta + n_blk - 1) / n_blk;
    CUtensorMap map_m, map_v;
    if (!atc_make_map(&map_m, m, (int)N, M, kMtcBox, (int)blk_rows, true) ||
        !atc_make_map(&map_v, v, (int)N, nb, kMtcBox, kMtcVectors, true))
        return FEATHER_ERR_LAUNCH;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kMtcThreads);
    cfg.dynamicSmemBytes = kMtcSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, map_m, map_v, out, (int)M, (int)N, nb, (int)rows_cta,
                                             (int)blk_rows, (int)n_blk, status);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

template <int MODE>
static int gemv_multi_dispatch(const uint32_t* m, const uint32_t* v, float* out, long long M,
                               long long N, int B, const DeviceInfo& dev, cudaStream_t s,
                               bool static_matrix) {
    const long long n_words = N / 4;
    if ((N % 16) || !aligned(m, 16)) {  // ragged rows: one single-vector GEMV per vector
        for (int b = 0; b < B; ++b)
            if (int st = gemv_launch<MODE>(m, v + b * n_words, out + (long long)b * M, M, N, dev, s,
                                           static_matrix))
                return st;
        return FEATHER_OK;
    }
    if (MODE == kE5M2 && M >= 64ll * dev.sm_count && N % kMtcStep == 0 && N <= 0x7FFFFFFF && aligned(v, 16) &&
        atc_encoder() && g_tune.multi_tc.load(std::memory_order_relaxed)) {
        // large E5M2 matrices: the tensor core reads the codes themselves, 16 vectors per pass
        for (int b0 = 0; b0 < B; b0 += kMtcVectors) {
            const int nb = B - b0 < kMtcVectors ? B - b0 : kMtcVectors;
            const int st = nb == 1 ? gemv_launch<MODE>(m, v + b0 * n_words, out + (long long)b0 * M, M, N, dev, s,
                                                       static_matrix)
                                   : gemv_multi_tc_launch(m, v + b0 * n_words, out + (long long)b0 * M, M, N, nb, dev, s);
            if (st) return st;
        }
        return FEATHER_OK;
    }
    if (M >= 64ll * dev.sm_count) {
        // large matrices: tensor-core kernel, up to eight vectors per pass
        for (int b0 = 0; b0 < B; b0 += kMmaVectors) {
            const int nb = B - b0 < kMmaVectors ? B - b0 : kMmaVectors;
            const uint32_t* vb = v + b0 * n_words;
            float* ob = out + (long long)b0 * M;
            int st;
            if (nb == 1) st = gemv_launch<MODE>(m, vb, ob, M, N, dev, s, static_matrix);
            else st = static_matrix ? gemv_mma_launch<MODE, true>(m, vb, ob, M, N, nb, dev, s)
                                    : gemv_mma_launch<MODE, false>(m, vb, ob, M, N, nb, dev, s);
            if (st) return st;
        }
        return FEATHER_OK;
    }
    for (int b0 = 0; b0 < B; b0 += 4) {  // up to four vectors per pass over the matrix
        const int nb = B - b0 < 4 ? B - b0 : 4;
        const uint32_t* vb = v + b0 * n_words;
        float* ob = out + (long long)b0 * M;
        int st;
        if (nb == 1)
            st = gemv_launch<MODE>(m, vb, ob, M, N, dev, s, static_matrix);
        else if (nb == 2)
            st = static_matrix ? gemv_multi_launch<MODE, 2, true>(m, vb, ob, M, N, nb, s)
                               : gemv_multi_launch<MODE, 2, false>(m, vb, ob, M, N, nb, s);
        else
            st = static_matrix ? gemv_multi_launch<MODE, 4, true>(m, vb, ob, M, N, nb, s)
                               : gemv_multi_launch<MODE, 4, false>(m, vb, ob, M, N, nb, s);
        if (st) return st;
    }
    return FEATHER_OK;
}

template <int D>
static int attention_launch(const uint32_t* q, const uint32_t* k, const uint32_t* v, float* out,
                            long long seq_len, const DeviceInfo& dev, cudaStream_t s) {
    const long long grid = (seq_len + 15) / 16;   // one CTA per 16 queries
    if (D > 128) {
        // wide rows: D / 128 warps per CTA, each owning 128 columns
        constexpr int kSplits = D > 128 ? D / 128 : 1;
        attention_e5m2_kernel<D, kSplits><<<(unsigned)grid, 32 * kSplits, kSplits * 1024 * sizeof(float), s>>>(
            q, k, v, out, (int)seq_len);
        return launch_status();
    }
    // 1, 2, 4 or 8 warps per CTA split the key tiles, so that short sequences still put a
    // few warps on every scheduler (4 per SM); the merge buffer stays within the 48 KiB of
    // shared memory a kernel gets without asking
    const long long tiles = (seq_len + kAttnTile - 1) / kAttnTile;
    int warps = 1;
    while (warps < 8 && grid * warps < 8ll * dev.sm_count && 2 * warps <= tiles &&
           2 * warps * (16 * D + 32) * sizeof(float) <= 48 * 1024)
        warps <<= 1;
    const size_t smem = warps > 1 ? (size_t)warps * (16 * D + 32) * sizeof(float) : 0;
    attention_e5m2_kernel<(D > 128 ? 128 : D), 1><<<(unsigned)grid, 32 * warps, smem, s>>>(q, k, v, out,
                                                                                         (int)seq_len);
    return launch_status();
}

// The tcgen05 kernel: 128 queries per CTA, the key tiles of a query block split over a
// cluster of 1 .. 8 CTAs (rows of 512 codes: times the pair of CTAs that split the output's columns).
template <int D>
static int attention_tc_launch(const uint32_t* q, const uint32_t* k, const uint32_t* v, float* out,
                               long long seq_len, const DeviceInfo& dev, cudaStream_t s) {
    using L = AtcLayout<D>;
    auto kernel = attention_tc_kernel<D>;
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, L::kBytes, configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    const long long blocks = (seq_len + kAtcRows - 1) / kAtcRows;
    const long long tiles = (seq_len + kAtcTile - 1) / kAtcTile;
    // as many CTAs per query block as still run in one wave (1 CTA per SM with rows of 256
    // codes, 2 with 128, 3 with narrower ones), at most 8 (a portable cluster) and at least
    // 2 tiles each
    const long long per_sm = D > 128 ? 1 : D > 64 ? 2 : 3;
    long long splits = per_sm * dev.sm_count / (blocks * L::kHalves);
    if (splits > 8 / L::kHalves) splits = 8 / L::kHalves;
    if (splits > tiles / 2) splits = tiles / 2;
    if (splits < 1) splits = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)splits, (unsigned)(blocks * L::kHalves));
    cfg.blockDim = dim3(kAtcThreads);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = L::kHalves;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CUtensorMap map_q, map_k, map_v;
    if (!atc_make_map(&map_q, q, D, seq_len, L::kSeg, kAtcRows, true) ||
        !atc_make_map(&map_k, k, D, seq_len, L::kSeg, kAtcTile, true) ||
        !atc_make_map(&map_v, v, D, seq_len, L::kDo, kAtcTile, false))
        return attention_launch<D>(q, k, v, out, seq_len, dev, s);   // no encoder in this driver: the other kernel
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, map_q, map_k, map_v, out, (int)seq_len, status);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

template <int D>
static int attention_any(const uint32_t* q, const uint32_t* k, const uint32_t* v, float* out,
                         long long seq_len, const DeviceInfo& dev, cudaStream_t s) {
    const int tc = g_tune.attn_tc.load(std::memory_order_relaxed);
    // Measured on B200: below these lengths the register-fed kernel (16 queries per CTA, no
    // cluster, no tensor-memory allocation) is as fast or faster.
    constexpr long long kFrom = D >= 256 ? 128 : D >= 128 ? 256 : 1024;
    // the grid's second dimension is at most 65535; the tensor maps want 16-byte alignment
    if (tc && (tc == 2 || seq_len >= kFrom) && seq_len <= 32767ll * kAtcRows && aligned(q, 16) &&
        aligned(k, 16) && aligned(v, 16))
        return attention_tc_launch<D>(q, k, v, out, seq_len, dev, s);
    return attention_launch<D>(q, k, v, out, seq_len, dev, s);
}

// Decode (optionally through ReLU) n_elems codes: a grid of up to 32 CTAs per SM,
// each warp walking runs of eight 128-byte lines.
static int decode_launch(const uint32_t* src, float* dst, long long n_elems, int mode, bool ieee,
                         bool relu, const DeviceInfo& dev, cudaStream_t s) {
    const long long n_words = (n_elems + 3) / 4;
    long long blocks = (n_words + kDecodeLines * 256 - 1) / (kDecodeLines * 256);
    const long long cap = (long long)dev.sm_count * 32;
    if (blocks > cap) blocks = cap;
    const unsigned g = (unsigned)blocks;
    if (mode == FEATHER_MODE_E5M2) {
        if (relu) decode_kernel<kE5M2, false, true><<<g, 256, 0, s>>>(src, dst, n_elems);
        else decode_kernel<kE5M2, false, false><<<g, 256, 0, s>>>(src, dst, n_elems);
    } else if (relu) {
        decode_kernel<kE4M3, false, true><<<g, 256, 0, s>>>(src, dst, n_elems);
    } else if (ieee) {
        decode_kernel<kE4M3, true, false><<<g, 256, 0, s>>>(src, dst, n_elems);
    } else {
        decode_kernel<kE4M3, false, false><<<g, 256, 0, s>>>(src, dst, n_elems);
    }
    return launch_status();
}

// One launch of the dot kernel.  The grid is CTAs-per-SM x SMs, never more CTAs
// than fit the GPU at once (the kernel walks the operands grid-strided, so a
// second wave would only add imbalance), than there is work for, or than
// `max_ctas` partial-sum slots.
template <int MODE, bool VEC, int UNROLL>
static int dot_launch_as(const uint32_t* a, const uint32_t* b, float* out, unsigned int* ticket,
                         float* partial, long long n_words, long long max_ctas,
                         const DeviceInfo& dev, cudaStream_t s) {
    auto kernel = dot_kernel<MODE, VEC, UNROLL>;
    static std::atomic<int> resident[64];
    int devid = 0;
    if (cudaGetDevice(&devid) != cudaSuccess || devid < 0 || devid >= 64) return FEATHER_ERR_LAUNCH;
    int per_sm = resident[devid].load(std::memory_order_acquire);
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kDotThreads, 0) != cudaSuccess ||
            per_sm < 1)
            return FEATHER_ERR_LAUNCH;
        resident[devid].store(per_sm, std::memory_order_release);
    }
    const int want = g_tune.dot_ctas_per_sm.load(std::memory_order_relaxed);
    long long grid = (long long)dev.sm_count * (want < per_sm ? want : per_sm);
    const long long need = (n_words / 4 + kDotThreads - 1) / kDotThreads;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    if (grid > max_ctas) grid = max_ctas;
    kernel<<<(unsigned)grid, kDotThreads, 0, s>>>(a, b, out, ticket, partial, n_words);
    return launch_status();
}

// Long operands: the bulk-copy ring kernel, one CTA per SM.
template <int MODE, int STAGES, int STAGE_CHUNKS>
static int dot_ring_launch(const uint32_t* a, const uint32_t* b, float* out, unsigned int* ticket,
                           float* partial, long long n_words, long long max_ctas,
                           const DeviceInfo& dev, cudaStream_t s) {
    auto kernel = dot_ring_kernel<MODE, STAGES, STAGE_CHUNKS>;
    constexpr int kSmem = dot_ring_smem_bytes(STAGES, STAGE_CHUNKS);
    static std::atomic<unsigned long long> configured{0};
    if (int st = ensure_smem(kernel, kSmem, configured)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    long long grid = dev.sm_count;
    if (grid > max_ctas) grid = max_ctas;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kDotRingThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a, b, out, ticket, partial, n_words, status,
                                             g_tune.dot_pre_kb.load(std::memory_order_relaxed) * 1024);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

template <int MODE>
static int dot_launch_any(const uint32_t* a, const uint32_t* b, float* out, unsigned int* ticket,
                          float* partial, long long n_words, long long max_ctas,
                          const DeviceInfo& dev, cudaStream_t s) {
    if (!(aligned(a, 16) && aligned(b, 16)))
        return dot_launch_as<MODE, false, 1>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
    // at least four full stages for every CTA of the ring kernel
    const int ring = g_tune.dot_ring.load(std::memory_order_relaxed);
    if (ring && (n_words >> 2) >= 8192ll * dev.sm_count) {
        if (ring == 2) return dot_ring_launch<MODE, 3, 2048>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
        if (ring == 3) return dot_ring_launch<MODE, 12, 512>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
        return dot_ring_launch<MODE, 6, 1024>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
    }
    switch (g_tune.dot_unroll.load(std::memory_order_relaxed)) {
        case 1: return dot_launch_as<MODE, true, 1>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
        case 2: return dot_launch_as<MODE, true, 2>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
        default: return dot_launch_as<MODE, true, 4>(a, b, out, ticket, partial, n_words, max_ctas, dev, s);
    }
}

template <int MODE>
static int dot_launch(const uint32_t* a, const uint32_t* b, float* out, void* workspace,
                      long long n_words, const DeviceInfo& dev, cudaStream_t s) {
    unsigned int* ticket = reinterpret_cast<unsigned int*>(workspace);
    float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 16);
    return dot_launch_any<MODE>(a, b, out, ticket, partial, n_words, kDotMaxCtas, dev, s);
}

// ---------------------------------------------------- dot without allocation --
// Scratch of feather_dot_fp8_static: the ticket counter (first 16 bytes) and one
// partial sum per CTA.  It lives in the library image, so every GPU that loads
// the library holds these few KiB until the process exits, and every call on a
// device shares it.
constexpr int kStaticDotSlots = 1024;                 // CTAs (= partial sums) at most
constexpr long long kStaticDotMaxWords = 1ll << 28;   // 1 GiB of codes per operand
constexpr int kStaticDotPartialOffset = 256;
static __device__ __align__(256) unsigned char g_dot_scratch[kStaticDotPartialOffset + 4 * kStaticDotSlots];

// Device address of g_dot_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not a pointer a kernel could
// use, so the address is asked for once per device (with that device current)
// and remembered.
static int static_dot_scratch(unsigned char** ptr) {
    static std::atomic<unsigned char*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FEATHER_ERR_LAUNCH;
    unsigned char* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dot_scratch) != cudaSuccess || !p)
            return FEATHER_ERR_LAUNCH;
        cached[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    return FEATHER_OK;
}

template <int MODE>
static int dot_static_launch(const uint32_t* a, const uint32_t* b, float* out, long long n_words,
                             const DeviceInfo& dev, cudaStream_t s) {
    unsigned char* scratch = nullptr;
    if (int st = static_dot_scratch(&scratch)) return st;
    // The array keeps whatever the previous call left.  The partial sums are
    // all rewritten before they are read; the ticket must start at zero.
    if (cudaMemsetAsync(scratch, 0, 16, s) != cudaSuccess) return FEATHER_ERR_LAUNCH;
    unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch);
    float* partial = reinterpret_cast<float*>(scratch + kStaticDotPartialOffset);
    // the same kernel and grid as feather_dot_fp8 (a B200's grid stays below the
    // slot count), hence the same bits
    return dot_launch_any<MODE>(a, b, out, ticket, partial, n_words, kStaticDotSlots, dev, s);
}

}  // namespace feather

using namespace feather;

extern "C" {

int feather_version(void) { return 300; /* 0.3.0: + GEMV chain in one launch, split-phase sharded GEMV, ring dot */ }

#ifdef FEATHER_RING_STAMPS
// Diagnostic build only: copy the timer stamps of the last 16 gemv_ring_kernel launches
// (16 x 160 x 8 uint64, see gemv_ring.cuh) to host memory; synchronises the device.
extern "C" int feather_debug_ring_stamps(void* host_dst) {
    if (!host_dst) return FEATHER_ERR_BAD_ARG;
    if (cudaDeviceSynchronize() != cudaSuccess) return FEATHER_ERR_LAUNCH;
    return cudaMemcpyFromSymbol(host_dst, g_ring_stamps, sizeof(g_ring_stamps)) == cudaSuccess
               ? FEATHER_OK : FEATHER_ERR_LAUNCH;
}
#endif

int feather_debug_bounds(void) {
#ifdef FEATHER_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

const char* feather_strerror(int status) {
    switch (status) {
        case FEATHER_OK: return "success";
        case FEATHER_ERR_BAD_ARG: return "bad argument (null pointer, negative size, or N not a multiple of 4)";
        case FEATHER_ERR_MISALIGNED: return "pointer is not aligned as the entry point requires";
        case FEATHER_ERR_MODE: return "unknown mode, source dtype or decode semantics";
        case FEATHER_ERR_ARCH: return "current device is not a compute-capability 10.x (B200) GPU";
        case FEATHER_ERR_LAUNCH: return "CUDA reported an error at launch";
        case FEATHER_ERR_WORKSPACE: return "workspace is missing or too small";
        case FEATHER_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case FEATHER_ERR_BOUNDS: return "debug build: a kernel formed an index outside its buffer (access skipped)";
        case FEATHER_ERR_TOO_LARGE: return "size exceeds what this entry point covers (built-in scratch, inbox, resident grid or model dimension)";
        default: return "unknown feather status";
    }
}

int feather_encode_fp8(const void* src, int src_dtype, uint32_t* dst, int64_t n_elems, int mode,
                       void* stream) {
    if (n_elems < 0) return FEATHER_ERR_BAD_ARG;
    if ((mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) ||
        (src_dtype != FEATHER_SRC_F16 && src_dtype != FEATHER_SRC_F32))
        return FEATHER_ERR_MODE;
    if (n_elems == 0) return FEATHER_OK;
    if (!src || !dst) return FEATHER_ERR_BAD_ARG;
    if (!aligned(src, src_dtype == FEATHER_SRC_F16 ? 2 : 4) || !aligned(dst, 4))
        return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mode == FEATHER_MODE_E5M2)
        return src_dtype == FEATHER_SRC_F32 ? encode_launch<kE5M2, true>(src, dst, n_elems, s)
                                            : encode_launch<kE5M2, false>(src, dst, n_elems, s);
    return src_dtype == FEATHER_SRC_F32 ? encode_launch<kE4M3, true>(src, dst, n_elems, s)
                                        : encode_launch<kE4M3, false>(src, dst, n_elems, s);
}

int feather_decode_fp8(const uint32_t* src, float* dst, int64_t n_elems, int mode, int semantics,
                       void* stream) {
    if (n_elems < 0) return FEATHER_ERR_BAD_ARG;
    if ((mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) ||
        (semantics != FEATHER_DECODE_KERNEL && semantics != FEATHER_DECODE_IEEE))
        return FEATHER_ERR_MODE;
    if (n_elems == 0) return FEATHER_OK;
    if (!src || !dst) return FEATHER_ERR_BAD_ARG;
    if (!aligned(src, 4) || !aligned(dst, 4)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return decode_launch(src, dst, n_elems, mode, semantics == FEATHER_DECODE_IEEE, false, *dev, s);
}

int feather_attention_fp8_e5m2(const uint32_t* q, const uint32_t* k, const uint32_t* v, float* out,
                               int64_t seq_len, int64_t h_dim_words, void* stream) {
    if (seq_len < 0 || h_dim_words <= 0 || seq_len > 0x7FFFFFFF / 512) return FEATHER_ERR_BAD_ARG;
    if (seq_len == 0) return FEATHER_OK;
    if (!q || !k || !v || !out) return FEATHER_ERR_BAD_ARG;
    if (!aligned(q, 4) || !aligned(k, 4) || !aligned(v, 4) || !aligned(out, 16)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (h_dim_words) {
        case 4: return attention_launch<16>(q, k, v, out, seq_len, *dev, s);
        case 8: return attention_any<32>(q, k, v, out, seq_len, *dev, s);
        case 16: return attention_any<64>(q, k, v, out, seq_len, *dev, s);
        case 32: return attention_any<128>(q, k, v, out, seq_len, *dev, s);
        case 64: return attention_any<256>(q, k, v, out, seq_len, *dev, s);
        case 128: return attention_any<512>(q, k, v, out, seq_len, *dev, s);
        default: return h_dim_words > 128 ? FEATHER_ERR_TOO_LARGE : FEATHER_ERR_BAD_ARG;
    }
}

int feather_relu_fp8(const uint32_t* src, float* dst, int64_t n_elems, int mode, void* stream) {
    if (n_elems < 0) return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    if (n_elems == 0) return FEATHER_OK;
    if (!src || !dst) return FEATHER_ERR_BAD_ARG;
    if (!aligned(src, 4) || !aligned(dst, 4)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    return decode_launch(src, dst, n_elems, mode, false, true, *dev, static_cast<cudaStream_t>(stream));
}

int feather_gemv_fp8(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                     int mode, void* stream) {
    return feather_gemv_fp8_ex(m, v, out, M, N, mode, 0u, stream);
}

int feather_gemv_fp8_ex(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                        int mode, uint32_t flags, void* stream) {
    if (flags & ~(uint32_t)FEATHER_GEMV_STATIC_MATRIX) return FEATHER_ERR_BAD_ARG;
    if (M < 0 || N < 0 || (N & 3) || M > 0x7FFFFFFF || N > 0x7FFFFFFFll * 4) return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    if (M == 0) return FEATHER_OK;
    if (!out || (N > 0 && (!m || !v))) return FEATHER_ERR_BAD_ARG;
    if (!aligned(m, 4) || !aligned(v, 4) || !aligned(out, 4)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0)
        return cudaMemsetAsync(out, 0, sizeof(float) * (size_t)M, s) == cudaSuccess
                   ? FEATHER_OK : FEATHER_ERR_LAUNCH;
    const bool static_matrix = (flags & FEATHER_GEMV_STATIC_MATRIX) != 0;
    return mode == FEATHER_MODE_E5M2 ? gemv_launch<kE5M2>(m, v, out, M, N, *dev, s, static_matrix)
                                     : gemv_launch<kE4M3>(m, v, out, M, N, *dev, s, static_matrix);
}

int feather_gemv_fp8_multi(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                           int B, int mode, uint32_t flags, void* stream) {
    if (flags & ~(uint32_t)FEATHER_GEMV_STATIC_MATRIX) return FEATHER_ERR_BAD_ARG;
    if (M < 0 || N < 0 || (N & 3) || M > 0x7FFFFFFF || N > 0x7FFFFFFFll * 4 || B < 0 || B > 64)
        return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    if (M == 0 || B == 0) return FEATHER_OK;
    if (!out || (N > 0 && (!m || !v))) return FEATHER_ERR_BAD_ARG;
    if (!aligned(m, 4) || !aligned(v, 4) || !aligned(out, 4)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0)
        return cudaMemsetAsync(out, 0, sizeof(float) * (size_t)M * B, s) == cudaSuccess
                   ? FEATHER_OK : FEATHER_ERR_LAUNCH;
    const bool static_matrix = (flags & FEATHER_GEMV_STATIC_MATRIX) != 0;
    return mode == FEATHER_MODE_E5M2
               ? gemv_multi_dispatch<kE5M2>(m, v, out, M, N, B, *dev, s, static_matrix)
               : gemv_multi_dispatch<kE4M3>(m, v, out, M, N, B, *dev, s, static_matrix);
}

int64_t feather_gemv_fp8_packed_workspace_bytes(int64_t M, int64_t N) {
    if (M <= 0 || N <= 0 || (N & 3)) return 0;
    const DeviceInfo* dev;
    if (device_info(&dev)) return 4 * M;
    return ((N & 15) || ring_eligible(nullptr, M, N, *dev)) ? 4 * M : 0;
}

int feather_gemv_fp8_packed(const uint32_t* m, const uint32_t* v, uint32_t* out_words,
                            void* workspace, int64_t M, int64_t N, int mode, int out_mode,
                            uint32_t flags, void* stream) {
    if (flags & ~(uint32_t)FEATHER_GEMV_STATIC_MATRIX) return FEATHER_ERR_BAD_ARG;
    if (M < 0 || N < 0 || (N & 3) || M > 0x7FFFFFFF || N > 0x7FFFFFFFll * 4) return FEATHER_ERR_BAD_ARG;
    if ((mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) ||
        (out_mode != FEATHER_MODE_E5M2 && out_mode != FEATHER_MODE_E4M3))
        return FEATHER_ERR_MODE;
    if (M == 0) return FEATHER_OK;
    if (!out_words || (N > 0 && (!m || !v))) return FEATHER_ERR_BAD_ARG;
    if (!aligned(m, 4) || !aligned(v, 4) || !aligned(out_words, 4) || !aligned(workspace, 4))
        return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0)  // empty rows sum to +0, which encodes as code 0 in both formats
        return cudaMemsetAsync(out_words, 0, 4 * (size_t)((M + 3) / 4), s) == cudaSuccess
                   ? FEATHER_OK : FEATHER_ERR_LAUNCH;
    const bool static_matrix = (flags & FEATHER_GEMV_STATIC_MATRIX) != 0;
    float* out = reinterpret_cast<float*>(out_words);
    float* ws = static_cast<float*>(workspace);
    const int out_code = out_mode == FEATHER_MODE_E5M2 ? kE5M2 : kE4M3;
    return mode == FEATHER_MODE_E5M2
               ? gemv_launch<kE5M2>(m, v, out, M, N, *dev, s, static_matrix, out_code, ws)
               : gemv_launch<kE4M3>(m, v, out, M, N, *dev, s, static_matrix, out_code, ws);
}

// Base address of the cudaMalloc allocation that contains `ptr` (the driver's
// cuMemGetAddressRange, reached through the runtime so libcuda is not linked).
static int allocation_base(const void* ptr, const void** base) {
    typedef int (*get_range_fn)(unsigned long long*, size_t*, unsigned long long);
    static std::atomic<get_range_fn> cached{nullptr};
    get_range_fn fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !sym)
            return FEATHER_ERR_LAUNCH;
        fn = reinterpret_cast<get_range_fn>(sym);
        cached.store(fn, std::memory_order_release);
    }
    unsigned long long b = 0;
    size_t size = 0;
    if (fn(&b, &size, (unsigned long long)(uintptr_t)ptr) != 0) return FEATHER_ERR_BAD_ARG;
    *base = reinterpret_cast<const void*>((uintptr_t)b);
    return FEATHER_OK;
}

int feather_ipc_export(const void* ptr, void* handle64, int64_t* offset) {
    if (!ptr || !handle64 || !offset) return FEATHER_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    const void* base = nullptr;
    if (int st = allocation_base(ptr, &base)) return st;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void*>(base)) != cudaSuccess) {
        cudaGetLastError();
        return FEATHER_ERR_LAUNCH;
    }
    memcpy(handle64, &h, 64);
    *offset = (int64_t)((const char*)ptr - (const char*)base);
    return FEATHER_OK;
}

int feather_ipc_open(const void* handle64, int64_t offset, void** mapped) {
    if (!handle64 || !mapped || offset < 0) return FEATHER_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* base = nullptr;
    // opened with the CONSUMER's device current: the runtime maps the peer's
    // allocation for this device and turns peer access on
    if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !base) {
        cudaGetLastError();
        return FEATHER_ERR_LAUNCH;
    }
    // the mapping must resolve to device memory from this device's point of view
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, base) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        cudaIpcCloseMemHandle(base);
        return FEATHER_ERR_LAUNCH;
    }
    *mapped = (char*)base + offset;
    return FEATHER_OK;
}

int feather_ipc_close(void* mapped, int64_t offset) {
    if (!mapped || offset < 0) return FEATHER_ERR_BAD_ARG;
    if (cudaIpcCloseMemHandle((char*)mapped - offset) != cudaSuccess) {
        cudaGetLastError();
        return FEATHER_ERR_LAUNCH;
    }
    return FEATHER_OK;
}

int feather_enable_peer_access(int peer_device) {
    int dev = 0, can = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return FEATHER_ERR_LAUNCH;
    if (peer_device == dev) return FEATHER_OK;
    if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess || !can) return FEATHER_ERR_BAD_ARG;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();  // not an error for us: clear the sticky code
        return FEATHER_OK;
    }
    return e == cudaSuccess ? FEATHER_OK : FEATHER_ERR_LAUNCH;
}

int feather_gemv_fp8_sharded_supported(int64_t rows_local, int64_t N) {
    const DeviceInfo* dev;
    if (device_info(&dev)) return 0;
    return rows_local > 0 && rows_local <= 0x7FFFFFFF && N > 0 && N <= 0x7FFFFFFFll * 4 &&
           ring_eligible(nullptr, rows_local, N, *dev) ? 1 : 0;
}

int feather_gemv_fp8_sharded(const uint32_t* m_local, const uint32_t* v, int64_t rows_local,
                             int64_t N, int mode, float* const* peer_out,
                             uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                             void* stream) {
    return feather_gemv_fp8_sharded_ex(m_local, v, rows_local, N, mode, peer_out, peer_flags, rank, world,
                                       epoch, 0u, nullptr, stream);
}

int feather_gemv_fp8_sharded_ex(const uint32_t* m_local, const uint32_t* v, int64_t rows_local,
                                int64_t N, int mode, float* const* peer_out,
                                uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                                uint32_t flags, uint64_t* stamps, void* stream) {
    if (flags & ~(uint32_t)(FEATHER_GEMV_STATIC_MATRIX | FEATHER_SHARDED_NO_WAIT)) return FEATHER_ERR_BAD_ARG;
    if (rows_local <= 0 || N <= 0 || (N & 3) || rows_local > 0x7FFFFFFF || !peer_out || !peer_flags ||
        world < 1 || world > kMaxShardRanks || rank < 0 || rank >= world || epoch == 0 || !m_local || !v)
        return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    if (!aligned(v, 4) || !aligned(stamps, 8)) return FEATHER_ERR_MISALIGNED;
    if (!ring_eligible(m_local, rows_local, N, *dev)) return FEATHER_ERR_BAD_ARG;
    ShardArgs sh = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_out[p] || !peer_flags[p]) return FEATHER_ERR_BAD_ARG;
        if (!aligned(peer_out[p], 4) || !aligned(peer_flags[p], 4)) return FEATHER_ERR_MISALIGNED;
        sh.out[p] = peer_out[p];
        sh.flags[p] = peer_flags[p];
    }
    sh.row_offset = (long long)rank * rows_local;
    sh.rank = rank;
    sh.world = world;
    sh.epoch = epoch;
    sh.no_wait = (flags & FEATHER_SHARDED_NO_WAIT) ? 1 : 0;
    sh.stamps = reinterpret_cast<unsigned long long*>(stamps);
    {   // rows per CTA as the kernel will split them (grid = min(SMs, tasks))
        long long grid = dev->sm_count;
        const long long tasks = (rows_local + kRingCW * kRingRW - 1) / (kRingCW * kRingRW);
        if (grid > tasks) grid = tasks;
        sh.staged = (rows_local + grid - 1) / grid <= kShardStageRows ? 1 : 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* mine = peer_out[rank] + sh.row_offset;
    const bool early = (flags & FEATHER_GEMV_STATIC_MATRIX) != 0;
    if (mode == FEATHER_MODE_E5M2)
        return early ? gemv_ring_launch<kE5M2, true, true>(m_local, v, mine, rows_local, N, *dev, s, sh)
                     : gemv_ring_launch<kE5M2, true>(m_local, v, mine, rows_local, N, *dev, s, sh);
    return early ? gemv_ring_launch<kE4M3, true, true>(m_local, v, mine, rows_local, N, *dev, s, sh)
                 : gemv_ring_launch<kE4M3, true>(m_local, v, mine, rows_local, N, *dev, s, sh);
}

int feather_gemv_fp8_sharded_wait(uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                                  uint64_t* stamps, void* stream) {
    if (!peer_flags || world < 1 || world > kMaxShardRanks || rank < 0 || rank >= world || epoch == 0 ||
        !peer_flags[rank])
        return FEATHER_ERR_BAD_ARG;
    if (!aligned(peer_flags[rank], 4) || !aligned(stamps, 8)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, shard_wait_kernel,
                                             static_cast<const unsigned int*>(peer_flags[rank]), world,
                                             (unsigned int)epoch, status,
                                             reinterpret_cast<unsigned long long*>(stamps));
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

int feather_gemv_fp8_allreduce(const uint32_t* m_local, const uint32_t* v_local, float* result,
                               int64_t M, int64_t N_local, int mode, float* const* peer_inbox,
                               int64_t inbox_floats, uint32_t* const* peer_flags, int rank,
                               int world, void* stream) {
    if (M <= 0 || N_local <= 0 || (N_local & 15) || M > 0x7FFFFFFF || N_local > 0x7FFFFFFF ||
        !peer_inbox || !peer_flags || world < 1 || world > kMaxShardRanks || rank < 0 ||
        rank >= world || !m_local || !v_local || !result)
        return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    const int64_t half = (inbox_floats / 2) & ~(int64_t)3;      // floats, 16-byte granular
    const int64_t slot = 2 * ((M + 15) / 16 * 16);              // (sum, tag) pairs of one rank
    if (half < (int64_t)world * slot) return FEATHER_ERR_TOO_LARGE;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    if (!aligned(m_local, 16) || !aligned(v_local, 4) || !aligned(result, 4))
        return FEATHER_ERR_MISALIGNED;
    AllReduceArgs ar = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_inbox[p] || !peer_flags[p]) return FEATHER_ERR_BAD_ARG;
        if (!aligned(peer_inbox[p], 16) || !aligned(peer_flags[p], 4)) return FEATHER_ERR_MISALIGNED;
        ar.inbox[p] = peer_inbox[p];
        ar.flags[p] = peer_flags[p];
    }
    ar.result = result;
    ar.half = half;
    ar.rank = rank;
    ar.world = world;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // one row per warp while that keeps the grid resident, else two
    const bool one = M < 2ll * dev->sm_count * 16;
    int st = FEATHER_ERR_TOO_LARGE;
    if (mode == FEATHER_MODE_E5M2) {
        if (one) st = gemv_allreduce_launch<kE5M2, 1, 4>(m_local, v_local, M, N_local, ar, *dev, s);
        if (st == FEATHER_ERR_TOO_LARGE)
            st = gemv_allreduce_launch<kE5M2, 2, 4>(m_local, v_local, M, N_local, ar, *dev, s);
    } else {
        if (one) st = gemv_allreduce_launch<kE4M3, 1, 4>(m_local, v_local, M, N_local, ar, *dev, s);
        if (st == FEATHER_ERR_TOO_LARGE)
            st = gemv_allreduce_launch<kE4M3, 2, 4>(m_local, v_local, M, N_local, ar, *dev, s);
    }
    return st;
}

int feather_set_wait_limit_ms(int milliseconds) {
    if (milliseconds < 1 || milliseconds > 600000) return FEATHER_ERR_BAD_ARG;
    const unsigned long long ns = (unsigned long long)milliseconds * 1000000ull;
    return cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns)) == cudaSuccess ? FEATHER_OK
                                                                                : FEATHER_ERR_LAUNCH;
}

// ------------------------------------------------------- GEMV chain ----------
// Plan buffer in device memory: [ticket + one counter per op, padded to 16 bytes | ops].
static inline int64_t chain_counter_bytes(int64_t n_ops) { return ((n_ops + 1) * 4 + 15) / 16 * 16; }

int64_t feather_gemv_chain_plan_bytes(int32_t n_ops) {
    if (n_ops <= 0) return 0;
    return chain_counter_bytes(n_ops) + (int64_t)n_ops * (int64_t)sizeof(ChainOp);
}

int feather_gemv_chain_plan(const feather_chain_op* ops, int32_t n_ops, void* plan, int64_t plan_bytes,
                            void* stream) {
    static_assert(sizeof(feather_chain_op) == sizeof(ChainOp), "public and device op records match");
    if (!ops || n_ops <= 0 || !plan) return FEATHER_ERR_BAD_ARG;
    if (plan_bytes < feather_gemv_chain_plan_bytes(n_ops)) return FEATHER_ERR_WORKSPACE;
    if (!aligned(plan, 16)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    const int grid = dev->sm_count;   // the launch's grid: the row split is planned for it
    std::unique_ptr<ChainOp[]> host(new (std::nothrow) ChainOp[n_ops]);
    if (!host) return FEATHER_ERR_LAUNCH;
    int n_ar = 0;   // all-reduced ops so far: an op's inbox region is its index among them
    for (int i = 0; i < n_ops; ++i) {
        const feather_chain_op& o = ops[i];
        if (o.M <= 0 || o.N <= 0 || (o.N & 15) || !o.m || !o.v || !o.out) return FEATHER_ERR_BAD_ARG;
        if (o.N > kChainTile) return FEATHER_ERR_TOO_LARGE;
        if ((o.mode != FEATHER_MODE_E5M2 && o.mode != FEATHER_MODE_E4M3) ||
            (o.out_mode != -1 && o.out_mode != FEATHER_MODE_E5M2 && o.out_mode != FEATHER_MODE_E4M3))
            return FEATHER_ERR_MODE;
        if (o.wait_op < -1 || o.wait_op >= i) return FEATHER_ERR_BAD_ARG;   // only EARLIER ops
        if (!aligned(o.m, 16) || !aligned(o.v, 16) || !aligned(o.out, 4)) return FEATHER_ERR_MISALIGNED;
        ChainOp& d = host[i];
        d.m = static_cast<const unsigned char*>(static_cast<const void*>(o.m));
        d.v = o.v;
        d.out = o.out;
        d.M = o.M;
        d.N = o.N;
        const int mode = o.mode == FEATHER_MODE_E5M2 ? kE5M2 : kE4M3;
        const int out_sel = o.out_mode < 0 ? 0 : 1 + (o.out_mode == FEATHER_MODE_E5M2 ? kE5M2 : kE4M3);
        if (o.allreduce != 0 && o.allreduce != 1) return FEATHER_ERR_BAD_ARG;
        d.flags = mode | (out_sel << 1) | (o.allreduce ? (++n_ar) << 4 : 0);
        d.wait_op = o.wait_op;
        d.rows_q = ((o.M + kChainCW - 1) / kChainCW) / grid;
        d.rot = (int)(((long long)i * kChainRotate) % grid);
    }
    for (int i = 0; i < n_ops; ++i)
        if (host[i].wait_op >= 0) host[host[i].wait_op].flags |= 8;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char* base = static_cast<char*>(plan);
    const int64_t cb = chain_counter_bytes(n_ops);
    if (cudaMemsetAsync(base, 0, (size_t)cb, s) != cudaSuccess ||
        cudaMemcpyAsync(base + cb, host.get(), sizeof(ChainOp) * (size_t)n_ops, cudaMemcpyHostToDevice, s) !=
            cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)   // the host copy of the table is released on return
        return FEATHER_ERR_LAUNCH;
    return FEATHER_OK;
}

static int chain_launch(const void* plan, int32_t n_ops, uint32_t flags, const ChainArArgs& ar,
                        void* stream) {
    if (flags & ~(uint32_t)FEATHER_GEMV_STATIC_MATRIX) return FEATHER_ERR_BAD_ARG;
    if (!plan || n_ops <= 0) return FEATHER_ERR_BAD_ARG;
    if (!aligned(plan, 16)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    const bool early = (flags & FEATHER_GEMV_STATIC_MATRIX) != 0;
    auto kernel = early ? gemv_chain_kernel<true> : gemv_chain_kernel<false>;
    static std::atomic<unsigned long long> configured[2];
    if (int st = ensure_smem(kernel, kChainSmemBytes, configured[early ? 1 : 0])) return st;
    char* base = static_cast<char*>(const_cast<void*>(plan));
    unsigned int* done = reinterpret_cast<unsigned int*>(base);
    const ChainOp* ops = reinterpret_cast<const ChainOp*>(base + chain_counter_bytes(n_ops));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dev->sm_count);   // one CTA per SM: resident at once
    cfg.blockDim = dim3(kChainThreads);
    cfg.dynamicSmemBytes = kChainSmemBytes;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ops, (int)n_ops, done, status, ar);
    return e == cudaSuccess ? launch_status() : FEATHER_ERR_LAUNCH;
}

int feather_gemv_chain_fp8(const void* plan, int32_t n_ops, uint32_t flags, void* stream) {
    return chain_launch(plan, n_ops, flags, ChainArArgs{}, stream);
}

int64_t feather_gemv_chain_inbox_floats(int32_t n_allreduce_ops, int32_t max_allreduce_rows, int world) {
    if (n_allreduce_ops <= 0 || max_allreduce_rows <= 0 || world < 1) return 0;
    const int64_t rows_cap = ((int64_t)max_allreduce_rows + 15) / 16 * 16;
    return 2 /* call parities */ * (int64_t)n_allreduce_ops * world * rows_cap * 2 /* (sum, tag) */;
}

int feather_gemv_chain_fp8_tp(const void* plan, int32_t n_ops, uint32_t flags, int32_t n_allreduce_ops,
                              int32_t max_allreduce_rows, float* const* peer_inbox, int64_t inbox_floats,
                              uint32_t* const* peer_flags, int rank, int world, void* stream) {
    if (n_allreduce_ops < 0 || max_allreduce_rows < 0 || !peer_inbox || !peer_flags || world < 1 ||
        world > kMaxArRanks || rank < 0 || rank >= world)
        return FEATHER_ERR_BAD_ARG;
    if (n_allreduce_ops > 0 &&
        inbox_floats < feather_gemv_chain_inbox_floats(n_allreduce_ops, max_allreduce_rows, world))
        return FEATHER_ERR_TOO_LARGE;
    ChainArArgs ar = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_inbox[p] || !peer_flags[p]) return FEATHER_ERR_BAD_ARG;
        if (!aligned(peer_inbox[p], 16) || !aligned(peer_flags[p], 4)) return FEATHER_ERR_MISALIGNED;
        ar.inbox[p] = peer_inbox[p];
        ar.flags[p] = peer_flags[p];
    }
    ar.rank = rank;
    ar.world = world;
    ar.n_ar = n_allreduce_ops;
    ar.rows_cap = (max_allreduce_rows + 15) / 16 * 16;
    return chain_launch(plan, n_ops, flags, ar, stream);
}

int feather_set_tuning(const char* spec) { return apply_tuning(spec); }

int feather_device_status(void* stream) {
    unsigned int* status = nullptr;
    if (int st = status_word(&status)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned int host = 0;
    if (cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
        return FEATHER_ERR_LAUNCH;
    if (host == 0) return FEATHER_OK;
    if (cudaMemsetAsync(status, 0, sizeof(host), s) != cudaSuccess) return FEATHER_ERR_LAUNCH;
    return (host & 0x100u) ? FEATHER_ERR_BOUNDS : FEATHER_ERR_TIMEOUT;
}

int64_t feather_dot_workspace_bytes(int64_t n_words) {
    (void)n_words;  // one partial slot per CTA of the largest grid, plus the ticket
    return kDotWorkspaceBytes;
}

int feather_dot_fp8(const uint32_t* a, const uint32_t* b, float* out, void* workspace,
                    int64_t n_words, int mode, void* stream) {
    if (n_words < 0) return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    if (!out || (n_words > 0 && (!a || !b))) return FEATHER_ERR_BAD_ARG;
    if (!workspace) return FEATHER_ERR_WORKSPACE;
    if (!aligned(a, 4) || !aligned(b, 4) || !aligned(out, 4) || !aligned(workspace, 16))
        return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return mode == FEATHER_MODE_E5M2 ? dot_launch<kE5M2>(a, b, out, workspace, n_words, *dev, s)
                                     : dot_launch<kE4M3>(a, b, out, workspace, n_words, *dev, s);
}

int64_t feather_dot_fp8_static_max_words(void) { return kStaticDotMaxWords; }

int feather_dot_fp8_static(const uint32_t* a, const uint32_t* b, float* out, int64_t n_words,
                           int mode, void* stream) {
    if (n_words < 0) return FEATHER_ERR_BAD_ARG;
    if (mode != FEATHER_MODE_E5M2 && mode != FEATHER_MODE_E4M3) return FEATHER_ERR_MODE;
    if (n_words > kStaticDotMaxWords) return FEATHER_ERR_TOO_LARGE;
    if (!out || (n_words > 0 && (!a || !b))) return FEATHER_ERR_BAD_ARG;
    if (!aligned(a, 4) || !aligned(b, 4) || !aligned(out, 4)) return FEATHER_ERR_MISALIGNED;
    const DeviceInfo* dev;
    if (int st = device_info(&dev)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return mode == FEATHER_MODE_E5M2 ? dot_static_launch<kE5M2>(a, b, out, n_words, *dev, s)
                                     : dot_static_launch<kE4M3>(a, b, out, n_words, *dev, s);
}

}  // extern "C"
