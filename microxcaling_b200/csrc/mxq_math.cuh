// Device-side arithmetic of the MX / elementwise quantizers (sm_100a).
//
// Every routine here produces exactly the value of the reference's
// quantize_elemwise / quantize_mx_elem (mx/cpp/quantize.cuh:88-177) and
// mx_get_shared_scale (mx/cpp/shared_exp.cuh:27-49), but none of them follows
// that code's shift-and-reassemble structure.  Two formulations are used:
//
//  * round_grid_*: the hot one.  A number x is rounded to the grid of a small
//    floating-point format (P significand bits, minimum normal exponent emin)
//    by adding and subtracting a power of two c whose unit in the last place is
//    the grid spacing at x: 2^(max(exponent(x), emin) - (P-1)).  The addition
//    itself performs the rounding, in the hardware's round-to-nearest-even or
//    round-toward-zero mode; round-half-away is a toward-zero addition at half
//    the spacing followed by an integer (+1, clear low bit) on the result bits.
//    c's exponent field is an integer max and add on x's exponent field, so the
//    whole thing is a handful of integer/float instructions with no branches.
//  * round_generic: exact integer rounding of the 24-bit significand; handles
//    every (bits <= 24, exp_bits <= 8) format and every input, and is used for
//    the wide formats the add-subtract trick does not cover.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <string.h>
#include <math.h>

namespace mxq {

enum : int { RN_AWAY = 0, RZ = 1, RN_EVEN = 2, DITHER = 3 };
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

constexpr uint32_t kNaN = 0x7fc00000u;
constexpr uint32_t kInf = 0x7f800000u;

// Launch-constant description of the element format, in the *scaled* domain
// (block maximum mapped next to the format's largest exponent).
struct ElemFmt {
    uint32_t emin_field;   // (emin + 127) << 23, emin = smallest normal exponent
    uint32_t k_field;      // exponent-field offset of the rounding constant
    float    max_norm;     // largest magnitude of the format
    float    smul;         // 2^(k_field >> 23)
    int      ebits;        // 0 = fixed-point "int" format
    int      mbits;        // sign + significand bits (implicit one included)
    int      emax_elem;    // unbiased exponent of max_norm
};

__host__ __device__ inline int fmt_emin(int ebits) { return ebits == 0 ? 0 : 2 - (1 << (ebits - 1)); }

__host__ inline ElemFmt make_fmt(int ebits, int mbits, float max_norm, int mode) {
    ElemFmt f;
    const int P = mbits - 1;
    f.emin_field = (uint32_t)(fmt_emin(ebits) + 127) << 23;
    f.k_field = (uint32_t)((mode == RN_AWAY ? 23 : 24) - P) << 23;
    f.max_norm = max_norm;
    f.smul = ldexpf(1.0f, (mode == RN_AWAY ? 23 : 24) - P);
    f.ebits = ebits;
    f.mbits = mbits;
    uint32_t u;
    memcpy(&u, &max_norm, 4);
    const int e = (int)((u >> 23) & 0xff);
    f.emax_elem = e == 0 ? -126 : e - 127;
    return f;
}

// |v| (finite, bits `a`) rounded to the format grid and saturated at max_norm.
// Preconditions: 2 <= P <= 12, exponent(v) <= 127 - 24 (true in the scaled
// domain, where |v| < 2^(emax_elem+1) <= 2^17).
template <int MODE>
__device__ __forceinline__ float round_grid_abs(uint32_t a, const uint32_t emin_field,
                                                const uint32_t k_field, const float max_norm) {
    const uint32_t ea = a & 0x7f800000u;
    const uint32_t cb = max(ea, emin_field) + k_field;
    const float c = __uint_as_float(cb);
    const float av = __uint_as_float(a);
    float r;
    if (MODE == RN_EVEN) {
        r = __fadd_rn(av, c) - c;
    } else if (MODE == RZ) {
        r = __fadd_rz(av, c) - c;
    } else {
        uint32_t t = __float_as_uint(__fadd_rz(av, c));
        t = (t + 1u) & ~1u;
        r = __uint_as_float(t) - c;
    }
    return fminf(r, max_norm);
}

// The same rounding applied directly to an unscaled magnitude ax = |x| of a
// source with at most 11 significand bits (bf16, fp16): the grid is the element
// format's grid multiplied by the block scale, so the smallest-normal constant
// `cmin` = 2^(emin + s) * scale and the saturation bound are per-block values
// and no multiply into or out of the scaled domain is needed.  `smul` = 2^s,
// s = 24-P, so that the rounding constant c = max(ax * 2^s, cmin) has an ulp
// equal to the grid spacing at ax.  c only has to lie in that binade and be an
// even multiple of the spacing; with a narrow source ax * 2^s qualifies (its low
// significand bits are zero and ax + c cannot leave the binade), which keeps the
// computation on the FMA pipe.
//   even:       RN(ax + c) - c
//   floor:      RZ(ax + c) - c
//   half-away:  RN(ax * (1 + 2^-12) + c) - c.  ax / spacing has at most 11
//               significant bits, so the relative nudge is smaller than the
//               distance of any non-tie from the next half-way point yet turns
//               every exact tie into a round-up.
// Returns the rounded, unsaturated magnitude.  Valid when cmin and ax * 2^s are
// normal finite floats (the caller checks the block's exponent range and
// otherwise uses the scaled-domain routine above).
template <int MODE>
__device__ __forceinline__ float round_unscaled_abs(float ax, const float cmin, const float smul) {
    const float c = fmaxf(ax * smul, cmin);
    if (MODE == RN_EVEN) return __fadd_rn(ax, c) - c;
    if (MODE == RZ) return __fadd_rz(ax, c) - c;
    return __fmaf_rn(ax, 1.000244140625f, c) - c;
}

// Biased exponent (0..255) of the block scale from the bits of the block's
// absolute maximum; 255 = NaN scale, 0 = 2^-127.
__device__ __forceinline__ int scale_exp_from_absmax(uint32_t amax_bits, int emax_elem, int scale_emax) {
    int E = (int)(amax_bits >> 23);                  // amax_bits has no sign
    if (E != 255) E -= emax_elem;
    const int ub = E - 127;
    if (ub > scale_emax) E = 255;
    else if (ub < -scale_emax) E = 127 - scale_emax;
    return E;
}

// 2^(E-127) as a float for E in [0, 254]; E == 0 is the subnormal 2^-127.
__device__ __forceinline__ float pow2_from_field(int E) {
    return __uint_as_float(E == 0 ? 0x00400000u : ((uint32_t)E << 23));
}
// 2^(127-E): the exact reciprocal of the above (E == 254 gives 2^-127).
__device__ __forceinline__ float inv_pow2_from_field(int E) {
    return __uint_as_float(E == 254 ? 0x00400000u : ((uint32_t)(254 - E) << 23));
}

// Exact integer rounding of one fp32 value to (bits, exp_bits); any format with
// bits <= 24, exp_bits <= 8.  Inf stays Inf, NaN stays NaN, zero stays +0,
// a negative value that rounds to zero gives -0.
__device__ __forceinline__ float round_generic(float x, int bits, int exp_bits, float max_norm,
                                               int mode, bool saturate, bool allow_denorm,
                                               float noise = 0.f) {
    const uint32_t u = __float_as_uint(x);
    const uint32_t a = u & 0x7fffffffu;
    const uint32_t sgn = u & 0x80000000u;
    if (a == 0) return 0.0f;
    if (a > kInf) return __uint_as_float(kNaN);
    if (a == kInf) return x;
    const bool is_int = exp_bits == 0;
    const int P = bits - 1;
    const int emin = fmt_emin(exp_bits);
    const int ef = (int)(a >> 23);
    uint32_t sig = a & 0x7fffffu;
    int lsb, ue;
    if (ef == 0) { lsb = -149; ue = -127; }
    else { sig |= 0x800000u; lsb = ef - 150; ue = ef - 127; }
    if (!is_int && !allow_denorm && ue < emin) return __uint_as_float(sgn);
    const int qe = max(ue, emin) - (P - 1);
    const int sh = qe - lsb;                          // >= 0 because bits <= 24
    uint32_t r;
    if (mode == DITHER) {
        // floor(|x|/quantum + noise) with the sum rounded to fp32 first, as
        // torch.floor(torch.abs(A) + rand_A) does (mx/elemwise_ops.py:57-59).
        const float w = ldexpf((float)sig, -min(sh, 60));
        r = (uint32_t)floorf(__fadd_rn(w, noise));
    } else if (sh == 0) {
        r = sig;
    } else if (sh > 25) {
        r = 0;
    } else {
        const uint32_t q = sig >> sh;
        const uint32_t rem = sig & ((1u << sh) - 1u);
        const uint32_t half = 1u << (sh - 1);
        r = q;
        if (mode == RN_AWAY) r += (rem >= half);
        else if (mode == RN_EVEN) r += (rem > half) || (rem == half && (q & 1u));
    }
    if (r == 0) return __uint_as_float(sgn);
    float v = ldexpf((float)r, qe);
    if (v > max_norm) v = (is_int || saturate) ? max_norm : __uint_as_float(kInf);
    return __uint_as_float(__float_as_uint(v) | sgn);
}

// ---- storage types ---------------------------------------------------------
template <int DT> struct Store;
template <> struct Store<DT_F32> {
    using T = float;
    static __device__ __forceinline__ float load(const T& v) { return v; }
    static __device__ __forceinline__ T make(float v) { return v; }
};
template <> struct Store<DT_F16> {
    using T = __half;
    static __device__ __forceinline__ float load(const T& v) { return __half2float(v); }
    static __device__ __forceinline__ T make(float v) { return __float2half_rn(v); }
};
template <> struct Store<DT_BF16> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float load(const T& v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T make(float v) { return __float2bfloat16_rn(v); }
};

// Element code (one byte) of an already-rounded scaled value, in an fp8
// container: e5m2 for the e5m2 format, e4m3 for e4m3 and for every narrower
// float format (each e3m2 / e2m3 / e2m1 value is also an e4m3 value, so the
// container changes no product).  Fixed-point formats use two's complement
// with (mbits-2) fractional bits.  The conversions are exact because the input
// already lies on the target grid.
__device__ __forceinline__ uint32_t encode2_e4m3(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t encode2_e5m2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// Packed bfloat16 arithmetic: one correctly rounded (nearest-even) result per lane.  For a product that is
// the fp32 product of the two operands (exact: 8 x 8 significant bits) rounded to bfloat16, for a sum it
// equals the fp32 sum rounded again (the fp32 sum is exact unless the operands are more than 15 binades
// apart, and then it is nowhere near a bfloat16 rounding midpoint) -- i.e. what a framework computes for
// bfloat16 tensors, at one instruction per two elements instead of two unpacks, two operations and a pack.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Two values rounded to a 6- or 4-bit element format by the hardware conversion (nearest-even on the
// format's grid, subnormals included, saturating at its largest value), then widened to e4m3 code bytes;
// the two widening conversions are exact because every value of the narrow formats is an e4m3 value.
__device__ __forceinline__ uint32_t encode2_via_e3m2(float lo, float hi) {
    uint16_t r;
    asm("{\n\t.reg .b16 t;\n\t.reg .b32 f;\n\tcvt.rn.satfinite.e3m2x2.f32 t, %1, %2;\n\tcvt.rn.f16x2.e3m2x2 f, t;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 %0, f;\n\t}" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t encode2_via_e2m3(float lo, float hi) {
    uint16_t r;
    asm("{\n\t.reg .b16 t;\n\t.reg .b32 f;\n\tcvt.rn.satfinite.e2m3x2.f32 t, %1, %2;\n\tcvt.rn.f16x2.e2m3x2 f, t;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 %0, f;\n\t}" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t encode2_via_e2m1(float lo, float hi) {
    uint16_t r;
    asm("{\n\t.reg .b8 t;\n\t.reg .b32 f;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.rn.f16x2.e2m1x2 f, t;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 %0, f;\n\t}" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t encode1(float q, int ebits, int mbits) {
    if (ebits == 0) return (uint32_t)(__float2int_rn(ldexpf(q, mbits - 2)) & 0xff);
    return (ebits == 5 ? encode2_e5m2(q, 0.f) : encode2_e4m3(q, 0.f)) & 0xffu;
}

}  // namespace mxq
