// Host (CPU) twins of the two quantizers: the same results as the GPU kernels
// for tensors that live in ordinary host memory, computed on the host cores.
// They take the place of the reference's quantize_mx_func_cpp and
// quantize_elemwise_func_cpp (mx/cpp/funcs.cpp:23-98, 117-149), which loop
// over the tensor in one thread; here rows of blocks are spread over OpenMP
// threads.  The arithmetic is the exact integer rounding of the significand
// (the formulation of round_generic in mxq_math.cuh) written for the host.
// Nothing here touches a GPU.
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif
#include "../../include/mxq.h"

namespace {

inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

constexpr uint32_t kNaNBits = 0x7fc00000u, kInfBits = 0x7f800000u;

// ---- storage types <-> fp32 (conversions written out so that no device header is needed) ----
inline float half_to_float(uint16_t h) {
    const uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) return u2f(s) == 0.0f && m == 0 ? u2f(s) : copysignf(ldexpf((float)m, -24), u2f(s | 0x3f800000u));
    if (e == 31) return u2f(s | kInfBits | (m << 13));
    return u2f(s | ((e + 112u) << 23) | (m << 13));
}
inline uint16_t float_to_half_rn(float f) {
    const uint32_t u = f2u(f), s = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > kInfBits) return (uint16_t)(s | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(s | 0x7c00u);                  // >= 65536: Inf (65520 rounds below)
    if (a < 0x33000000u) return (uint16_t)s;                                // < 2^-25: zero
    const int e = (int)(a >> 23) - 127;
    uint32_t sig = (a & 0x7fffffu) | 0x800000u;
    const int sh = e < -14 ? 13 + (-14 - e) : 13;                           // bits dropped
    const uint32_t q = sig >> sh, rem = sig & ((1u << sh) - 1u), half = 1u << (sh - 1);
    uint32_t r = q + ((rem > half) || (rem == half && (q & 1u)));
    uint32_t out = e < -14 ? r : (((uint32_t)(e + 15) << 10) + (r - 0x400u));   // a carry walks into the exponent
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(s | out);
}
inline float bf16_to_float(uint16_t h) { return u2f((uint32_t)h << 16); }
inline uint16_t float_to_bf16_rn(float f) {
    const uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > kInfBits) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

inline float load_elem(const void* p, int dt, int64_t i) {
    if (dt == MXQ_F32) return reinterpret_cast<const float*>(p)[i];
    const uint16_t h = reinterpret_cast<const uint16_t*>(p)[i];
    return dt == MXQ_F16 ? half_to_float(h) : bf16_to_float(h);
}
inline void store_elem(void* p, int dt, int64_t i, float v) {
    if (dt == MXQ_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<uint16_t*>(p)[i] = dt == MXQ_F16 ? float_to_half_rn(v) : float_to_bf16_rn(v);
}

inline int fmt_emin(int ebits) { return ebits == 0 ? 0 : 2 - (1 << (ebits - 1)); }

// One fp32 value rounded to (bits, exp_bits): exact integer rounding of the
// 24-bit significand.  Inf stays Inf, NaN stays NaN, zero gives +0, a negative
// value that rounds to zero gives -0.
inline float round_elem(float x, int bits, int exp_bits, float max_norm, int mode, bool saturate, bool allow_denorm,
                        float noise) {
    const uint32_t u = f2u(x), a = u & 0x7fffffffu, sgn = u & 0x80000000u;
    if (a == 0) return 0.0f;
    if (a > kInfBits) return u2f(kNaNBits);
    if (a == kInfBits) return x;
    const bool is_int = exp_bits == 0;
    const int P = bits - 1, emin = fmt_emin(exp_bits), ef = (int)(a >> 23);
    uint32_t sig = a & 0x7fffffu;
    int lsb, ue;
    if (ef == 0) { lsb = -149; ue = -127; }
    else { sig |= 0x800000u; lsb = ef - 150; ue = ef - 127; }
    if (!is_int && !allow_denorm && ue < emin) return u2f(sgn);
    const int qe = std::max(ue, emin) - (P - 1);
    const int sh = qe - lsb;
    uint32_t r;
    if (mode == MXQ_ROUND_DITHER) {
        const float w = ldexpf((float)sig, -std::min(sh, 60));
        r = (uint32_t)floorf(w + noise);
    } else if (sh == 0) {
        r = sig;
    } else if (sh > 25) {
        r = 0;
    } else {
        const uint32_t q = sig >> sh, rem = sig & ((1u << sh) - 1u), half = 1u << (sh - 1);
        r = q;
        if (mode == MXQ_ROUND_NEAREST) r += (rem >= half);
        else if (mode == MXQ_ROUND_EVEN) r += (rem > half) || (rem == half && (q & 1u));
    }
    if (r == 0) return u2f(sgn);
    float v = ldexpf((float)r, qe);
    if (v > max_norm) v = (is_int || saturate) ? max_norm : u2f(kInfBits);
    return u2f(f2u(v) | sgn);
}

inline int threads_for(int nthreads) {
#ifdef _OPENMP
    return nthreads > 0 ? nthreads : omp_get_max_threads();
#else
    (void)nthreads;
    return 1;
#endif
}

}  // namespace

extern "C" int mxq_cpu_quantize_elemwise(const void* in, void* out, int in_dtype, int out_dtype, int64_t n, int bits,
                                         int exp_bits, float max_norm, int rmode, int saturate_normals,
                                         int allow_denorm, const void* noise, int nthreads) {
    if (n < 0 || (n > 0 && (!in || !out))) return MXQ_ERR_BAD_ARG;
    if (in_dtype < MXQ_F32 || in_dtype > MXQ_BF16 || out_dtype < MXQ_F32 || out_dtype > MXQ_BF16) return MXQ_ERR_BAD_ARG;
    if (bits < 2 || bits > 24 || exp_bits < 0 || exp_bits > 8) return MXQ_ERR_BAD_ARG;
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_DITHER) return MXQ_ERR_BAD_ARG;
    if (rmode == MXQ_ROUND_DITHER && !noise) return MXQ_ERR_BAD_ARG;
    const float* nz = reinterpret_cast<const float*>(noise);
    const int nt = threads_for(nthreads);
    (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; ++i)
        store_elem(out, out_dtype, i,
                   round_elem(load_elem(in, in_dtype, i), bits, exp_bits, max_norm, rmode, saturate_normals != 0,
                              allow_denorm != 0, nz ? nz[i] : 0.0f));
    return MXQ_OK;
}

extern "C" int mxq_cpu_quantize_mx(const void* in, void* out, int dtype, int64_t pre, int64_t axis_len, int64_t post,
                                   int block, int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                                   int flush_fp32_subnorms, int rmode, const void* noise, int nthreads) {
    if (pre < 0 || axis_len < 0 || post < 0) return MXQ_ERR_BAD_ARG;
    if (pre == 0 || axis_len == 0 || post == 0) return MXQ_OK;
    if (!in || !out || dtype < MXQ_F32 || dtype > MXQ_BF16) return MXQ_ERR_BAD_ARG;
    if (scale_bits < 1 || scale_bits > 8 || elem_mbits < 2 || elem_mbits > 24 || elem_ebits < 0 || elem_ebits > 8)
        return MXQ_ERR_BAD_ARG;
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_DITHER) return MXQ_ERR_BAD_ARG;
    if (rmode == MXQ_ROUND_DITHER && !noise) return MXQ_ERR_BAD_ARG;
    const int64_t blk = block > 0 ? block : axis_len;
    const int64_t nblk = (axis_len + blk - 1) / blk;
    const int scale_emax = (1 << (scale_bits - 1)) - 1;
    const uint32_t mn_bits = f2u(elem_max_norm);
    const int mn_e = (int)((mn_bits >> 23) & 0xff);
    const int emax_elem = mn_e == 0 ? -126 : mn_e - 127;
    const float* nz = reinterpret_cast<const float*>(noise);
    const int64_t tiles = pre * nblk;                 // one tile = the `post` blocks at (p, b)
    const int nt = threads_for(nthreads);
    (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t t = 0; t < tiles; ++t) {
        const int64_t p = t / nblk, b = t % nblk;
        const int64_t k0 = b * blk, k1 = std::min(k0 + blk, axis_len);
        for (int64_t j = 0; j < post; ++j) {
            const int64_t base = p * axis_len * post + j;
            uint32_t m = 0;
            for (int64_t k = k0; k < k1; ++k) m = std::max(m, f2u(load_elem(in, dtype, base + k * post)) & 0x7fffffffu);
            // biased exponent of the shared scale: 255 = NaN block, clamped to scale_bits
            int E = (int)(m >> 23);
            if (E != 255) E -= emax_elem;
            if (E - 127 > scale_emax) E = 255;
            else if (E - 127 < -scale_emax) E = 127 - scale_emax;
            const bool nan_blk = E == 255;
            const bool dead = nan_blk || (flush_fp32_subnorms && (m >> 23) == 0);
            const float scale = nan_blk ? u2f(kNaNBits) : u2f(E == 0 ? 0x00400000u : ((uint32_t)E << 23));
            const float inv = dead ? 0.0f : u2f(E == 254 ? 0x00400000u : ((uint32_t)(254 - E) << 23));
            for (int64_t k = k0; k < k1; ++k) {
                const int64_t idx = base + k * post;
                const float x = load_elem(in, dtype, idx);
                const float v = dead ? 0.0f : x * inv;             // exact: power-of-two scaling
                float q = round_elem(v, elem_mbits, elem_ebits, elem_max_norm, rmode, true, true, nz ? nz[idx] : 0.0f);
                q = u2f((f2u(q) & 0x7fffffffu) | (f2u(x) & 0x80000000u));   // the sign of x survives a result of zero
                store_elem(out, dtype, idx, q * scale);
            }
        }
    }
    return MXQ_OK;
}
