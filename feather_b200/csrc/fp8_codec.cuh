// FP8 encode / decode device functions shared by every kernel of the library.
//
// Encode is bit-exact with the reference packer, which casts with ml_dtypes
// (feather/packers/fp8.py:109-120): one round-to-nearest-even step from the
// source value, E5M2 overflow -> +-inf (0x7C), E5M2 NaN -> 0x7E | sign, E4M3
// overflow / inf / NaN -> 0x7F | sign, subnormals kept.
//
// Decode follows the reference KERNELS (feather/routines/gemv.py:31-34 and
// gemv.py:83-88), not IEEE: E5M2 is the fp16 whose bits are code << 8; E4M3 is
// the fp16  sign<<15 | ((e+8)*(e>0))<<10 | m<<7 , so exponent-0 codes give
// +-m * 2^-17 and 0x7F / 0xFF give +-480.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace feather {

enum : int { kE5M2 = 0, kE4M3 = 1 };

// ---------------------------------------------------------------- encode ---
// fp32 bit pattern -> E5M2 code.  Normal range: re-bias the exponent
// (127 -> 15) and round the 21 dropped mantissa bits to nearest-even in
// integer arithmetic; a mantissa carry walks into the exponent by itself.
// Below 2^-14 the code is RNE(|x| * 2^16), obtained by adding 2^7 in fp32 (one
// ulp of [2^7, 2^8) is 2^-16, and the adder rounds to nearest-even).
__device__ __forceinline__ uint32_t encode_e5m2(uint32_t u) {
    const uint32_t sign = (u >> 24) & 0x80u;
    const uint32_t a = u & 0x7FFFFFFFu;
    uint32_t mag;
    if (a >= 0x38800000u) {  // |x| >= 2^-14, inf and NaN included
        const uint32_t t = a - 0x38000000u;
        mag = (t + 0x000FFFFFu + ((t >> 21) & 1u)) >> 21;
        mag = min(mag, 0x7Cu);            // overflow and inf -> inf
        if (a > 0x7F800000u) mag = 0x7Eu; // NaN, any payload
    } else {
        mag = __float_as_uint(__fadd_rn(__uint_as_float(a), 128.0f)) - 0x43000000u;
    }
    return mag | sign;
}

// fp32 bit pattern -> E4M3 (fn) code.  Same scheme with bias 7 / 3 mantissa
// bits; below 2^-6 the code is RNE(|x| * 2^9) (add 2^14).  Everything that
// rounds above 0x7E (from 464 exclusive), inf and NaN give 0x7F.
__device__ __forceinline__ uint32_t encode_e4m3(uint32_t u) {
    const uint32_t sign = (u >> 24) & 0x80u;
    const uint32_t a = u & 0x7FFFFFFFu;
    uint32_t mag;
    if (a >= 0x3C800000u) {  // |x| >= 2^-6
        const uint32_t t = a - 0x3C000000u;
        mag = (t + 0x0007FFFFu + ((t >> 20) & 1u)) >> 20;
        mag = min(mag, 0x7Fu);
    } else {
        mag = __float_as_uint(__fadd_rn(__uint_as_float(a), 16384.0f)) - 0x46800000u;
    }
    return mag | sign;
}

template <int MODE>
__device__ __forceinline__ uint32_t encode_f32(float x) {
    return MODE == kE5M2 ? encode_e5m2(__float_as_uint(x)) : encode_e4m3(__float_as_uint(x));
}

// ---------------------------------------------------------------- decode ---
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t h2) {
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

// E4M3 kernel decode of two codes sitting in the HIGH byte of each 16-bit half
// of `x` (low bytes are ignored).  Returns the two fp16 results packed.
//   t  = sign | (code & 0x7F) << 7     fp16 with exponent field e, mantissa m<<7
//      = value / 256 when e > 0, and exactly the value (m * 2^-17, an fp16
//        subnormal) when e == 0.
//   hz = t * 1.0 with flush-to-zero     drops exactly the e == 0 lanes
//   r  = hz * 255 + t                   256 t for e > 0, t for e == 0; every
//                                       result is representable, so exact.
__device__ __forceinline__ uint32_t e4m3_pair_to_h2(uint32_t x) {
    const uint32_t t = (x & 0x80008000u) | ((x >> 1) & 0x3F803F80u);
    uint32_t hz, r;
    asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(hz) : "r"(t), "r"(0x3C003C00u));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(hz), "r"(0x5BF85BF8u), "r"(t));
    return r;
}

// Decode the four codes of one word.  The pairing is chosen per mode so that
// each pair costs the fewest instructions:
//   E5M2: lo = (c0, c1), hi = (c2, c3)
//   E4M3: lo = (c0, c2), hi = (c1, c3)
// Callers lay the vector operand out in the same order (pair_order()).
template <int MODE>
__device__ __forceinline__ void decode_word(uint32_t w, float2& lo, float2& hi) {
    if (MODE == kE5M2) {
        lo = h2_to_f2(prmt(w, 0u, 0x1404u));  // (c0 << 8) | (c1 << 24)
        hi = h2_to_f2(prmt(w, 0u, 0x3424u));  // (c2 << 8) | (c3 << 24)
    } else {
        lo = h2_to_f2(e4m3_pair_to_h2(w << 8));  // c0, c2 in the high bytes
        hi = h2_to_f2(e4m3_pair_to_h2(w));       // c1, c3 in the high bytes
    }
}

// Element order of decode_word's outputs: (lo.x, lo.y, hi.x, hi.y) hold codes
// pair_order<MODE>(0..3).
template <int MODE>
__device__ __forceinline__ int pair_order(int i) {
    return MODE == kE5M2 ? i : ((i & 1) << 1 | (i >> 1));
}

// Decode one word to four floats in ELEMENT order (c0, c1, c2, c3).
template <int MODE>
__device__ __forceinline__ float4 decode_word_ordered(uint32_t w) {
    float2 lo, hi;
    decode_word<MODE>(w, lo, hi);
    return MODE == kE5M2 ? make_float4(lo.x, lo.y, hi.x, hi.y)
                         : make_float4(lo.x, hi.x, lo.y, hi.y);
}

// IEEE E4M3 (fn) value of a code, as the reference CPU unpacker returns it
// (feather/packers/fp8.py:366-391): exponent-0 codes are m * 2^-9, 0x7F/0xFF
// are NaN.  Off the hot path; plain arithmetic.
__device__ __forceinline__ float decode_e4m3_ieee(uint32_t c) {
    const uint32_t e = (c >> 3) & 0xFu, m = c & 7u;
    float v;
    if ((c & 0x7Fu) == 0x7Fu) v = __uint_as_float(0x7FC00000u);
    else if (e == 0) v = (float)m * 0.001953125f;  // 2^-9
    else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (c & 0x80u) ? -v : v;
}

}  // namespace feather
