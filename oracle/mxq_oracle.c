/*
 * mxq_oracle.c -- CPU restatement of microxcaling's quantization math.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are
 * compared with; nothing in the shipped library links, loads or calls it.
 * It may be used by the test-suite, by the smoke test and by the benchmark's
 * cpu-baseline leg, and by nothing else.
 *
 * Parity status: PINNED.  The functions below are checked against
 *   - the reference's own known-answer vectors (mx/tests/test_fp8_e4m3_fix.py,
 *     test_e5m0_scale.py, test_corners_mx.py, test_corners_elemwise.py,
 *     test_quantize_elemwise.py, test_formats.py),
 *   - outputs of the reference's pure-PyTorch CPU path (custom_cuda=False)
 *     recorded as fixtures, and
 *   - the reference's C++ math headers compiled unmodified (oracle/_ref).
 *
 * The arithmetic is written as exact integer rounding of the fp32 significand
 * (my own formulation); each routine names the reference lines it restates.
 * Paths are relative to the reference project root.
 */
#include <stdint.h>
#include <string.h>
#include <math.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { MXO_F32 = 0, MXO_F16 = 1, MXO_BF16 = 2 };
enum { MXO_RN_AWAY = 0, MXO_RZ = 1, MXO_RN_EVEN = 2 };   /* mx/formats.py:12-19 */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- storage conversions (mx/cpp/common.cuh:183-196 `as_float`, and the
 *      `(T)` casts in mx/cpp/mx.cuh:88,154) ---------------------------------- */
static inline float bf16_to_f(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline uint16_t f_to_bf16(float f) {          /* round-to-nearest-even */
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float f16_to_f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f_to_f16(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

static inline float load_as_f(const void* p, int dtype, int64_t i) {
    switch (dtype) {
        case MXO_F32:  return ((const float*)p)[i];
        case MXO_F16:  return f16_to_f(((const uint16_t*)p)[i]);
        default:       return bf16_to_f(((const uint16_t*)p)[i]);
    }
}
static inline void store_from_f(void* p, int dtype, int64_t i, float v) {
    switch (dtype) {
        case MXO_F32:  ((float*)p)[i] = v; break;
        case MXO_F16:  ((uint16_t*)p)[i] = f_to_f16(v); break;
        default:       ((uint16_t*)p)[i] = f_to_bf16(v); break;
    }
}

/*
 * Round one fp32 value to a (bits, exp_bits) element format.
 *
 * Restates quantize_elemwise (mx/cpp/quantize.cuh:88-155) together with
 * shift_right_round_mantissa / shift_left_mantissa (quantize.cuh:15-80), and
 * agrees with _quantize_elemwise_core (mx/elemwise_ops.py:82-170):
 *   bits      sign + significand bits (implicit one included); ints: total bits
 *   exp_bits  0 means a sign-magnitude fixed-point "int" format with bias 1
 *   mode      0 half-away-from-zero, 1 toward zero, 2 half-to-even
 * The value is written as sig * 2^lsb with an integer significand, the target
 * quantum is 2^(max(exponent, emin) - (P-1)), and sig is divided by the quantum
 * with exact integer rounding.  Magnitudes above max_norm saturate (ints, or
 * saturate != 0) or become infinity.  Inf stays Inf and NaN stays NaN
 * (elemwise_ops.py:160-163).  A negative value that rounds to zero gives -0,
 * as sign(A)*floor(...) does in elemwise_ops.py:63.
 */
float mxo_round_elem(float x, int bits, int exp_bits, float max_norm,
                     int mode, int saturate, int allow_denorm)
{
    const uint32_t u = f2u(x);
    const uint32_t a = u & 0x7fffffffu;
    const uint32_t sgn = u & 0x80000000u;
    if (a == 0) return 0.0f;                         /* quantize.cuh:99 */
    if (a > 0x7f800000u) return u2f(0x7fc00000u);     /* NaN */
    if (a == 0x7f800000u) return x;                  /* +-Inf kept */

    const int is_int = (exp_bits == 0);
    const int P = bits - 1;                          /* significand bits */
    const int emin = is_int ? 0 : 2 - (1 << (exp_bits - 1));
    const int efield = (int)(a >> 23);
    uint64_t sig = a & 0x7fffffu;
    int lsb;                                         /* value = sig * 2^lsb */
    int ue;                                          /* exponent used for the binade */
    if (efield == 0) { lsb = -149; ue = -127; }      /* fp32 subnormal: quantize.cuh:124-127 */
    else { sig |= 0x800000u; lsb = efield - 150; ue = efield - 127; }

    if (!is_int && !allow_denorm && ue < emin)       /* quantize.cuh:113-115 */
        return u2f(sgn);

    const int qe = (ue > emin ? ue : emin) - (P - 1);
    int sh = qe - lsb;                               /* bits to drop, >= 0 for bits <= 24 */
    uint64_t r;
    if (sh <= 0) r = sig << (-sh);
    else if (sh > 40) r = 0;
    else {
        const uint64_t q = sig >> sh;
        const uint64_t rem = sig & (((uint64_t)1 << sh) - 1);
        const uint64_t half = (uint64_t)1 << (sh - 1);
        r = q;
        if (mode == MXO_RN_AWAY) { if (rem >= half) r = q + 1; }
        else if (mode == MXO_RN_EVEN) { if (rem > half || (rem == half && (q & 1))) r = q + 1; }
        /* MXO_RZ: truncate */
    }
    if (r == 0) return u2f(sgn);
    float v = ldexpf((float)r, qe);                  /* exact: r < 2^25, result >= 2^-149 */
    if (v > max_norm)                                /* quantize.cuh:147-152 */
        v = (is_int || saturate) ? max_norm : INFINITY;
    return u2f(f2u(v) | sgn);
}

/* Power-of-two block scale from the block's absolute maximum.
 * Restates mx_get_shared_scale / clamp_shared_exp (mx/cpp/shared_exp.cuh:9-49)
 * and the scale path of _quantize_mx (mx/mx_ops.py:267-283).  Returns the
 * biased scale exponent (0..255; 255 = NaN scale, 0 = 2^-127) and the float. */
int mxo_scale_exp(float absmax, int scale_bits, float max_norm, float* scale_out)
{
    int E = (int)((f2u(absmax) >> 23) & 0xffu);      /* common.cuh:146-154 */
    const uint32_t mn = f2u(max_norm);
    int elem_emax = (int)((mn >> 23) & 0xffu);
    elem_emax = (elem_emax == 0) ? -126 : elem_emax - 127;
    if (E != 255) E -= elem_emax;                    /* shared_exp.cuh:33-36 */
    const int smax = scale_bits ? (1 << (scale_bits - 1)) - 1 : 255;
    const int ub = E - 127;
    if (ub > smax) E = 255;                          /* overflow: NaN scale */
    else if (ub < -smax) E = 127 - smax;             /* underflow: smallest scale */
    if (scale_out) {
        const uint32_t mant = (E == 0 || E == 255) ? 0x400000u : 0u;  /* shared_exp.cuh:41-45 */
        *scale_out = u2f(((uint32_t)E << 23) | mant);
    }
    return E;
}

static inline float absmax_nan(float m, float v) {   /* mx.cuh:76-79,131-139 */
    const float a = fabsf(v);
    return (a > m || isnan(a)) ? a : m;
}

/* One MX element given its block scale: quantize_mx_elem (quantize.cuh:160-177). */
static inline float mx_elem(float x, float scale, int flush, int ebits, int mbits,
                            float max_norm, int mode)
{
    const float si = flush ? 0.0f : x / scale;
    const float so = mxo_round_elem(si, mbits, ebits, max_norm, mode, 1, 1);
    float o = so * scale;
    if (isnan(o)) o = u2f(0x7fc00000u);
    return o;
}

/*
 * MX fake-quantization of a contiguous [pre, axis_len, post] tensor in blocks
 * of `block` consecutive elements along the middle axis (ragged tail allowed).
 * Restates quantize_mx_by_tile_cuda_kernel (mx/cpp/mx.cuh:98-158) and
 * quantize_mx_cpp (mx/cpp/funcs.h:61-100); equals _quantize_mx with
 * custom_cuda=False (mx/mx_ops.py:173-298) numerically.
 * Optional outputs: codes (one byte per element, OCP MX element encodings;
 * int8 as two's complement of value*64) and scales (one E8M0 byte per block,
 * laid out [pre, nblocks, post]).
 */
int mxo_quantize_mx(const void* in, void* out, uint8_t* codes, uint8_t* scales,
                    int dtype, int64_t pre, int64_t axis_len, int64_t post,
                    int block, int scale_bits, int ebits, int mbits, float max_norm,
                    int flush_subnorms, int mode, int nthreads)
{
    if (block <= 0) block = (int)axis_len;
    if (axis_len == 0 || pre == 0 || post == 0) return 0;
    const int64_t nblk = (axis_len + block - 1) / block;
    const int64_t ntiles = pre * nblk * post;
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#endif
    (void)nthreads;
    #pragma omp parallel for num_threads(nthreads) schedule(static)
    for (int64_t t = 0; t < ntiles; ++t) {
        const int64_t j = t % post;
        const int64_t b = (t / post) % nblk;
        const int64_t i = t / (post * nblk);
        const int64_t k0 = b * block;
        const int64_t k1 = (k0 + block < axis_len) ? k0 + block : axis_len;
        const int64_t base = i * axis_len * post + j;
        float m = 0.0f;
        for (int64_t k = k0; k < k1; ++k)
            m = absmax_nan(m, load_as_f(in, dtype, base + k * post));
        const int Emax = (int)((f2u(m) >> 23) & 0xffu);
        const int flush = (Emax == 0 && flush_subnorms);   /* mx.cuh:82,142 */
        float scale;
        const int E = mxo_scale_exp(m, scale_bits, max_norm, &scale);
        if (scales) scales[t] = (uint8_t)E;
        for (int64_t k = k0; k < k1; ++k) {
            const int64_t idx = base + k * post;
            const float x = load_as_f(in, dtype, idx);
            const float o = mx_elem(x, scale, flush, ebits, mbits, max_norm, mode);
            if (out) store_from_f(out, dtype, idx, o);
            if (codes) {
                extern uint8_t mxo_encode_elem(float q, int ebits, int mbits);
                const float si = flush ? 0.0f : x / scale;
                const float q = mxo_round_elem(si, mbits, ebits, max_norm, mode, 1, 1);
                codes[idx] = mxo_encode_elem(q, ebits, mbits);
            }
        }
    }
    return 0;
}

/* Bit encoding of an already-quantized scaled element (OCP Microscaling v1.0
 * element formats: sign | exponent | mantissa, bias 2^(ebits-1)-1; MXINT8 is
 * two's complement with 6 fractional bits).  NaN encodes as the format's NaN
 * when it has one (e5m2 0x7f, e4m3 0x7f) and as 0 otherwise. */
uint8_t mxo_encode_elem(float q, int ebits, int mbits)
{
    const uint32_t u = f2u(q);
    const uint32_t a = u & 0x7fffffffu;
    const int P = mbits - 1;
    if (ebits == 0) {                                /* fixed point, P-1 fractional bits */
        if (a > 0x7f800000u) return 0;
        int v = (int)lrintf(ldexpf(q, P - 1));
        return (uint8_t)(v & ((1 << mbits) - 1));
    }
    const int M = P - 1;                             /* explicit mantissa bits */
    const uint8_t s = (uint8_t)((u >> 31) << (ebits + M));
    if (a > 0x7f800000u) return (ebits >= 4) ? (uint8_t)((1u << (ebits + M)) - 1) : 0;
    if (a == 0) return s;
    const int bias = (1 << (ebits - 1)) - 1;
    int ue = (int)(a >> 23) - 127;
    uint32_t frac = a & 0x7fffffu;
    int efield, mant;
    if (ue + bias >= 1) { efield = ue + bias; mant = (int)(frac >> (23 - M)); }
    else {                                           /* target subnormal */
        const int sh = 1 - (ue + bias);
        efield = 0;
        mant = (int)((frac | 0x800000u) >> (23 - M + sh));
    }
    return (uint8_t)(s | (efield << M) | mant);
}

/* Decode of the above, times 2^(E-127).  E == 255 gives NaN. */
float mxo_decode_elem(uint8_t code, int ebits, int mbits, int E)
{
    if (E == 255) return u2f(0x7fc00000u);
    const int P = mbits - 1;
    float v;
    if (ebits == 0) {
        int iv = code & ((1 << mbits) - 1);
        if (iv & (1 << (mbits - 1))) iv -= (1 << mbits);
        v = ldexpf((float)iv, -(P - 1));
    } else {
        const int M = P - 1;
        const int bias = (1 << (ebits - 1)) - 1;
        const int sgn = (code >> (ebits + M)) & 1;
        const int ef = (code >> M) & ((1 << ebits) - 1);
        const int mant = code & ((1 << M) - 1);
        if (ef == 0) v = ldexpf((float)mant, 1 - bias - M);
        else v = ldexpf((float)(mant | (1 << M)), ef - bias - M);
        if (sgn) v = -v;
    }
    return ldexpf(v, E - 127);
}

/* Elementwise format rounding of n values: quantize_tensor (mx/cpp/funcs.cpp:100-115)
 * / quantize_elemwise_cuda_kernel (mx/cpp/elemwise.cuh:14-35). */
int mxo_quantize_elemwise(const void* in, void* out, int in_dtype, int out_dtype,
                          int64_t n, int bits, int exp_bits, float max_norm, int mode,
                          int saturate, int allow_denorm, int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#endif
    (void)nthreads;
    #pragma omp parallel for num_threads(nthreads) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float x = load_as_f(in, in_dtype, i);
        store_from_f(out, out_dtype, i,
                     mxo_round_elem(x, bits, exp_bits, max_norm, mode, saturate, allow_denorm));
    }
    return 0;
}

/* Inner-dimension reductions of an fp32 [rows, inner] matrix:
 * reduce_sum_inner_dim / reduce_max_inner_dim (mx/cpp/reduce.cu:15-89). The
 * reference test compares them with torch.sum / torch.max at 1e-6 relative
 * (mx/tests/test_reduce.py:17-46); the sum here accumulates in double. */
int mxo_reduce_sum_inner(const float* in, float* out, int64_t rows, int64_t inner, int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#endif
    (void)nthreads;
    #pragma omp parallel for num_threads(nthreads) schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0.0;
        for (int64_t c = 0; c < inner; ++c) s += in[r * inner + c];
        out[r] = (float)s;
    }
    return 0;
}
int mxo_reduce_max_inner(const float* in, float* out, int64_t rows, int64_t inner, int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#endif
    (void)nthreads;
    #pragma omp parallel for num_threads(nthreads) schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float m = -INFINITY;
        for (int64_t c = 0; c < inner; ++c) { const float v = in[r * inner + c]; if (v > m || isnan(v)) m = v; }
        out[r] = m;
    }
    return 0;
}

/*
 * Emulated MX GEMM: C[b] = A[b] (M x K, row-major) * B[b]^T (B stored N x K,
 * row-major), both operands already fake-quantized fp32, accumulated in double.
 * This is what F.linear / torch.matmul / torch.bmm compute on the dequantized
 * operands in mx/linear.py:86, mx/matmul.py:86 and mx/bmm.py:59, with the
 * accumulation order removed (double accumulation is exact to well below one
 * fp32 ulp for these sizes).  Optional sum of |a*b| per output supports an
 * accumulation-order error bound.
 */
int mxo_gemm_nt(const float* A, const float* B, double* C, double* Cabs,
                int64_t batch, int64_t M, int64_t N, int64_t K, int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#endif
    (void)nthreads;
    #pragma omp parallel for num_threads(nthreads) schedule(static) collapse(2)
    for (int64_t b = 0; b < batch; ++b)
    for (int64_t i = 0; i < M; ++i) {
        const float* a = A + (b * M + i) * K;
        for (int64_t j = 0; j < N; ++j) {
            const float* w = B + (b * N + j) * K;
            double s = 0.0, sa = 0.0;
            for (int64_t k = 0; k < K; ++k) { const double p = (double)a[k] * (double)w[k]; s += p; sa += fabs(p); }
            C[(b * M + i) * N + j] = s;
            if (Cabs) Cabs[(b * M + i) * N + j] = sa;
        }
    }
    return 0;
}

int mxo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
