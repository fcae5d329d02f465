// MX block quantization kernels (sm_100a) and their C entry point.
//
// Three kernels share one per-element routine:
//   mx_lastaxis_kernel  blocks along the contiguous axis: each thread owns one
//                       16-byte vector, the block maximum is a butterfly of
//                       warp shuffles over the lanes that share a block, the
//                       tensor is read once and written once.
//   mx_strided_kernel   blocks along an outer axis (stride `post`): each thread
//                       owns an 8-byte column strip and keeps all rows of the
//                       block in registers, so the column maxima need no
//                       communication and the input is read exactly once.  The
//                       same kernel can write the packed operand transposed
//                       (blocked axis innermost), which is the layout the
//                       backward GEMMs need.
//   mx_generic_kernel   one thread per block, any shape / block size / mode;
//                       used for ragged, unaligned or very wide cases.
// HBM-bound: the arithmetic per element is one multiply into the scaled
// domain, the add-subtract grid rounding of mxq_math.cuh, one multiply back.
#pragma once
#include "mxq_common.cuh"
#include "vector_math.cuh"
#include <algorithm>
#include <cstring>

namespace mxq {

// Division of a 32-bit number by a launch-invariant divisor: one multiply-high
// and two shifts instead of the long software division sequence.
struct FastDiv {
    uint32_t d, m, s1, s2;
    __host__ void set(uint32_t div) {
        d = div ? div : 1;
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        m = (uint32_t)((((1ull << l) - d) << 32) / d + 1);
        s1 = l < 1 ? l : 1;
        s2 = l > 0 ? l - 1 : 0;
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const {
        const uint32_t t = __umulhi(m, n);
        return (t + ((n - t) >> s1)) >> s2;
    }
};

struct MxArgs {
    const void* in;
    const void* in2;        // second input of a fused prologue (SiLU(in) * in2), else unused
    const uint16_t* sig_table;   // sigmoid chain of every bfloat16 bit pattern (fused prologue only)
    void* out;
    uint8_t* codes;
    uint8_t* scales;
    const float* noise;
    int64_t pre, axis_len, post;
    int64_t nblk;
    int block;
    int scale_emax;
    int flush;
    int mode;
    int transposed;
    int sf_gemm;            // scales in the 512-byte chunk layout of the GEMM
    int64_t sf_rpb;         // rows per batch element for that layout
    FastDiv div_nblk;       // last-axis kernels: block index -> (row, block in row)
    FastDiv div_rpb;        // row -> (batch, row in batch)
    ElemFmt fmt;
    // unscaled fast path of the bf16 kernels (set_fast_consts)
    uint32_t fp_e_lo, fp_e_span;   // usable iff (exponent field of the block maximum - fp_e_lo) <= fp_e_span
    uint32_t fp_cmin_base;         // bits of cmin   = fp_cmin_base + (E << 23)
    uint32_t fp_maxn_base;         // bits of maxn   = fp_maxn_base + (E << 23)
    uint32_t fp_mp_base;           // packed bf16 maxn pair = fp_mp_base + E * 0x00800080
    int direct;                    // element rounding by hardware conversion (see code_quad_direct): 0 no, 1 the format is its
                                   // own container (fp8_e4m3 / fp8_e5m2), 2 fp6_e3m2, 3 fp6_e2m3, 4 fp4_e2m1 (e4m3 container)
};

// The unscaled fast path needs its per-block constants to be normal, finite
// floats and the scale exponent to need no clamping; both hold when the block
// maximum's exponent field lies in one launch-constant interval, computed here.
__host__ inline void set_fast_consts(MxArgs& a) {
    const int emin_f = (int)(a.fmt.emin_field >> 23);
    // rounding constants sit at the full grid spacing in every mode (k_field is one less for half-away)
    const int kf_f = (int)(a.fmt.k_field >> 23) + (a.mode == RN_AWAY ? 1 : 0);
    const int ee = a.fmt.emax_elem;
    int lo = 48, hi = 200;
    lo = std::max(lo, 127 - a.scale_emax + ee);          // scale exponent not clamped
    hi = std::min(hi, 127 + a.scale_emax + ee);
    lo = std::max(lo, 1 - emin_f - kf_f + 127 + ee);      // cmin normal and finite
    hi = std::min(hi, 253 - emin_f - kf_f + 127 + ee);
    uint32_t mn;
    memcpy(&mn, &a.fmt.max_norm, 4);
    const int mp_half = (int)(mn >> 16) - (127 << 7);
    if (lo > hi || mp_half < 0 || (mn & 0xffffu) != 0) { a.fp_e_lo = 0xffffff00u; a.fp_e_span = 0; }
    else { a.fp_e_lo = (uint32_t)lo; a.fp_e_span = (uint32_t)(hi - lo); }
    a.fp_cmin_base = ((uint32_t)(emin_f + kf_f) << 23) - (127u << 23);
    a.fp_maxn_base = mn - (127u << 23);
    a.fp_mp_base = (uint32_t)(mp_half < 0 ? 0 : mp_half) * 0x10001u;
    const auto is = [&](int e, int m, float mx) { return a.fmt.ebits == e && a.fmt.mbits == m && a.fmt.max_norm == mx; };
    a.direct = (is(4, 5, 448.0f) || is(5, 4, 57344.0f)) ? 1 : is(3, 4, 28.0f) ? 2 : is(2, 5, 7.5f) ? 3 : is(2, 3, 6.0f) ? 4 : 0;
}

// Last-axis kernels: byte index of the scale of linear block index `blk`
// (row-major over [rows, nblk]); 32-bit arithmetic with invariant divisors.
__device__ __forceinline__ int64_t scale_index_last(const MxArgs& a, uint32_t blk) {
    if (!a.sf_gemm) return blk;
    const uint32_t row_all = a.div_nblk.div(blk);
    const uint32_t b = blk - row_all * (uint32_t)a.nblk;
    const uint32_t batch = a.div_rpb.div(row_all);
    const uint32_t row = row_all - batch * (uint32_t)a.sf_rpb;
    const int64_t r128 = (a.sf_rpb + 127) >> 7, kb4 = (a.nblk + 3) >> 2;
    return ((batch * r128 + (row >> 7)) * kb4 + (b >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (b & 3);
}

// Byte index of the scale of block b of (pre index p, post index j).
__device__ __forceinline__ int64_t scale_index(const MxArgs& a, int64_t p, int64_t b, int64_t j) {
    if (a.sf_gemm) {
        int64_t batch, row;
        if (a.transposed) { batch = p; row = j; }
        else { batch = p / a.sf_rpb; row = p % a.sf_rpb; }
        const int64_t r128 = (a.sf_rpb + 127) >> 7, kb4 = (a.nblk + 3) >> 2;
        return ((batch * r128 + (row >> 7)) * kb4 + (b >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (b & 3);
    }
    return a.transposed ? (p * a.post + j) * a.nblk + b : (p * a.nblk + b) * a.post + j;
}

// Per-block constants derived from the block's absolute maximum.
struct BlockScale {
    float scale;   // 2^(E-127), NaN when the block is NaN
    float inv;     // 2^(127-E), 0 when the block is flushed or NaN
    int E;
};

__device__ __forceinline__ BlockScale block_scale(uint32_t amax_bits, const MxArgs& a) {
    BlockScale s;
    const int E = scale_exp_from_absmax(amax_bits, a.fmt.emax_elem, a.scale_emax);
    const bool nan_blk = (E == 255);
    const bool flush = a.flush && (amax_bits >> 23) == 0;
    s.E = E;
    s.scale = nan_blk ? __uint_as_float(kNaN) : pow2_from_field(E);
    s.inv = (nan_blk || flush) ? 0.0f : inv_pow2_from_field(E);
    return s;
}

// x (fp32 bits) -> scaled rounded magnitude q (>= 0); the dequantized bits are
// (q * scale) | sign.
template <int MODE>
__device__ __forceinline__ float quant_abs(uint32_t xb, const BlockScale& s, const ElemFmt& f) {
    const float v = __uint_as_float(xb & 0x7fffffffu) * s.inv;
    return round_grid_abs<MODE>(__float_as_uint(v), f.emin_field, f.k_field, f.max_norm);
}

// Per-block constants of the unscaled fast path (see round_unscaled_abs), from
// the exponent field (0..255) of the block maximum.  Blocks outside the usable
// interval (tiny or huge maxima, zero, NaN/Inf, flushed) are marked !ok and go
// through a compact scaled-domain loop instead; their E is not meaningful.
struct FastBlock {
    float cmin;      // 2^(emin + s) * scale
    float maxn;      // max_norm * scale
    float inv;       // 1 / scale, for the element codes
    uint32_t E;      // biased scale exponent (E8M0 byte)
    bool ok;
};

__device__ __forceinline__ FastBlock fast_block(uint32_t eraw, const MxArgs& a) {
    FastBlock f;
    f.ok = (eraw - a.fp_e_lo) <= a.fp_e_span;
    f.E = eraw - (uint32_t)a.fmt.emax_elem;
    const uint32_t e23 = f.E << 23;
    f.cmin = __uint_as_float(a.fp_cmin_base + e23);
    f.maxn = __uint_as_float(a.fp_maxn_base + e23);
    f.inv = __uint_as_float((254u << 23) - e23);
    return f;
}

__device__ __forceinline__ uint32_t pack_codes4(const float* q, const uint32_t* xb, const ElemFmt& f) {
    // four signed scaled values -> four code bytes (little endian)
    float s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = __uint_as_float(__float_as_uint(q[i]) | (xb[i] & 0x80000000u));
    if (f.ebits == 0) {
        uint32_t r = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) r |= (uint32_t)(__float2int_rn(ldexpf(s[i], f.mbits - 2)) & 0xff) << (8 * i);
        return r;
    }
    if (f.ebits == 5) return encode2_e5m2(s[0], s[1]) | (encode2_e5m2(s[2], s[3]) << 16);
    return encode2_e4m3(s[0], s[1]) | (encode2_e4m3(s[2], s[3]) << 16);
}

// ---------------------------------------------------------------------------
// last-axis kernel
// ---------------------------------------------------------------------------
constexpr int kLastThreads = 256;
constexpr int kLastUnroll = 4;

template <int DT, int MODE, bool WANT_DQ, bool WANT_CODES>
__global__ void __launch_bounds__(kLastThreads)
mx_lastaxis_kernel(const MxArgs a, const int64_t nvec, const int lanes_per_block) {
    using IO = VecIO<DT, 16>;
    constexpr int N = IO::N;
    const int64_t tile = (int64_t)kLastThreads * kLastUnroll;
    for (int64_t base = (int64_t)blockIdx.x * tile; base < nvec; base += (int64_t)gridDim.x * tile) {
        uint32_t xb[kLastUnroll][N];
        bool live[kLastUnroll];
#pragma unroll
        for (int u = 0; u < kLastUnroll; ++u) {
            const int64_t v = base + (int64_t)u * kLastThreads + threadIdx.x;
            live[u] = v < nvec;
            if (live[u]) IO::load(a.in, v * N, xb[u]);
            else {
#pragma unroll
                for (int i = 0; i < N; ++i) xb[u][i] = 0;
            }
        }
#pragma unroll
        for (int u = 0; u < kLastUnroll; ++u) {
            const int64_t v = base + (int64_t)u * kLastThreads + threadIdx.x;
            uint32_t m = 0;
#pragma unroll
            for (int i = 0; i < N; ++i) m = max(m, xb[u][i] & 0x7fffffffu);   // NaN bits compare largest
            for (int s = 1; s < lanes_per_block; s <<= 1)
                m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
            const BlockScale bs = block_scale(m, a);
            float q[N];
#pragma unroll
            for (int i = 0; i < N; ++i) q[i] = quant_abs<MODE>(xb[u][i], bs, a.fmt);
            if (!live[u]) continue;
            if (WANT_CODES) {
                uint32_t c[N / 4];
#pragma unroll
                for (int i = 0; i < N / 4; ++i) c[i] = pack_codes4(&q[4 * i], &xb[u][4 * i], a.fmt);
                if (N == 4) *reinterpret_cast<uint32_t*>(a.codes + v * N) = c[0];
                else *reinterpret_cast<uint2*>(a.codes + v * N) = make_uint2(c[0], c[N / 4 - 1]);
                if ((threadIdx.x & (lanes_per_block - 1)) == 0)
                    a.scales[scale_index_last(a, (uint32_t)(v / lanes_per_block))] = (uint8_t)bs.E;
            }
            if (WANT_DQ) {
                uint32_t ob[N];
#pragma unroll
                for (int i = 0; i < N; ++i)
                    ob[i] = __float_as_uint(q[i] * bs.scale) | (xb[u][i] & 0x80000000u);
                IO::store(a.out, v * N, ob);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// strided-axis kernel: thread = 8-byte column strip x up to 32 rows
// ---------------------------------------------------------------------------
constexpr int kStrThreads = 128;
constexpr int kMaxRows = 32;

template <int DT, int MODE, bool WANT_DQ, bool WANT_CODES>
__global__ void __launch_bounds__(kStrThreads)
mx_strided_kernel(const MxArgs a, const int64_t col_tiles, const int64_t ntiles) {
    using IO = VecIO<DT, 8>;
    constexpr int N = IO::N;
    const int64_t cols_per_cta = (int64_t)kStrThreads * N;
    for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int64_t ct = t % col_tiles;
        const int64_t pb = t / col_tiles;                 // pre * nblk index
        const int64_t b = pb % a.nblk;
        const int64_t p = pb / a.nblk;
        const int64_t col = ct * cols_per_cta + (int64_t)threadIdx.x * N;
        if (col >= a.post) continue;
        const int64_t row0 = b * a.block;
        const int rows = (int)min((int64_t)a.block, a.axis_len - row0);
        const int64_t base = (p * a.axis_len + row0) * a.post + col;
        uint32_t xb[kMaxRows][N];
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r) {
            if (r < rows) IO::load(a.in, base + (int64_t)r * a.post, xb[r]);
            else {
#pragma unroll
                for (int i = 0; i < N; ++i) xb[r][i] = 0;
            }
        }
        uint32_t m[N];
#pragma unroll
        for (int i = 0; i < N; ++i) m[i] = 0;
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r)
#pragma unroll
            for (int i = 0; i < N; ++i) m[i] = max(m[i], xb[r][i] & 0x7fffffffu);
        BlockScale bs[N];
#pragma unroll
        for (int i = 0; i < N; ++i) bs[i] = block_scale(m[i], a);

        if (WANT_CODES) {
#pragma unroll
            for (int i = 0; i < N; ++i) a.scales[scale_index(a, p, b, col + i)] = (uint8_t)bs[i].E;
        }
        // transposed codes: 32 bytes per column, rows innermost
        uint32_t tc[N][kMaxRows / 4];
#pragma unroll
        for (int r4 = 0; r4 < kMaxRows / 4; ++r4) {
            float q[4][N];
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
                const int r = r4 * 4 + rr;
#pragma unroll
                for (int i = 0; i < N; ++i) q[rr][i] = quant_abs<MODE>(xb[r][i], bs[i], a.fmt);
                if (WANT_DQ && r < rows) {
                    uint32_t ob[N];
#pragma unroll
                    for (int i = 0; i < N; ++i)
                        ob[i] = __float_as_uint(q[rr][i] * bs[i].scale) | (xb[r][i] & 0x80000000u);
                    IO::store(a.out, base + (int64_t)r * a.post, ob);
                }
                if (WANT_CODES && !a.transposed && r < rows) {
                    // row-major codes: N bytes per thread per row
                    float qq[4]; uint32_t xx[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { qq[i] = q[rr][i < N ? i : 0]; xx[i] = xb[r][i < N ? i : 0]; }
                    const uint32_t c = pack_codes4(qq, xx, a.fmt);
                    if (N == 4) *reinterpret_cast<uint32_t*>(a.codes + base + (int64_t)r * a.post) = c;
                    else *reinterpret_cast<uint16_t*>(a.codes + base + (int64_t)r * a.post) = (uint16_t)c;
                }
            }
            if (WANT_CODES && a.transposed) {
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    float qq[4]; uint32_t xx[4];
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) { qq[rr] = q[rr][i]; xx[rr] = xb[r4 * 4 + rr][i]; }
                    tc[i][r4] = pack_codes4(qq, xx, a.fmt);
                }
            }
        }
        if (WANT_CODES && a.transposed) {
            // [pre, post, nblk*block]: the block's bytes are contiguous
            const int64_t padded = a.nblk * a.block;
#pragma unroll
            for (int i = 0; i < N; ++i) {
                uint8_t* dst = a.codes + (p * a.post + col + i) * padded + row0;
                if (a.block == kMaxRows && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(tc[i][0], tc[i][1], tc[i][2], tc[i][3]);
                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(tc[i][4], tc[i][5], tc[i][6], tc[i][7]);
                } else {
                    for (int r = 0; r < a.block; ++r) dst[r] = (uint8_t)(tc[i][r >> 2] >> (8 * (r & 3)));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// bf16 kernels: operate on packed pairs.  The block maximum is taken on the
// packed 16-bit magnitudes (one AND and one two-lane max per two elements), the
// results are bf16 values so their upper halves are packed back with one byte
// permute, and saturation and sign are applied to the packed pair.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t vmax_u16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// running maximum of two packed bf16 magnitudes: max(m, |w|) per lane, NaN-propagating
__device__ __forceinline__ uint32_t amax_bf16x2(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmax.NaN.bf16x2 %0, %1, t;\n\t}" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
// min(m, |w|) per packed bf16 lane (m, w not NaN)
__device__ __forceinline__ uint32_t amin_bf16x2(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmin.bf16x2 %0, %1, t;\n\t}" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t vmin_u16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// two bf16 elements (word w) -> two dequantized bf16 elements, fast path.
// lo/hi constants may differ (strided kernel: adjacent columns).
// PRE_CLAMP: saturation is applied to the packed magnitudes before rounding
// (max_norm * scale is a grid point and rounding is monotonic, so this equals
// saturating afterwards) and r_lo / r_hi return saturated magnitudes; otherwise
// the packed result is saturated and r_lo / r_hi are not.  The first form is
// cheaper but keeps a second copy of the inputs alive, which only the kernels
// with few registers in flight can afford.
template <int MODE, bool PRE_CLAMP>
__device__ __forceinline__ uint32_t quant_pair_bf16(uint32_t w, float cmin_lo, float cmin_hi,
                                                    uint32_t maxn_pair, const ElemFmt& f,
                                                    float& r_lo, float& r_hi) {
    // the fast path rounds at the full grid spacing in every mode (f.smul is half of that for half-away)
    const float smul = MODE == RN_AWAY ? f.smul * 2.0f : f.smul;
    if (PRE_CLAMP) {
        const uint32_t ax = amin_bf16x2(maxn_pair, w);
        r_lo = round_unscaled_abs<MODE>(__uint_as_float(ax << 16), cmin_lo, smul);
        r_hi = round_unscaled_abs<MODE>(__uint_as_float(ax & 0xffff0000u), cmin_hi, smul);
        return __byte_perm(__float_as_uint(r_lo), __float_as_uint(r_hi), 0x7632) | (w & 0x80008000u);
    }
    r_lo = round_unscaled_abs<MODE>(fabsf(__uint_as_float(w << 16)), cmin_lo, smul);
    r_hi = round_unscaled_abs<MODE>(fabsf(__uint_as_float(w & 0xffff0000u)), cmin_hi, smul);
    uint32_t p = __byte_perm(__float_as_uint(r_lo), __float_as_uint(r_hi), 0x7632);
    p = vmin_u16x2(p, maxn_pair);
    return p | (w & 0x80008000u);
}

// Code container of the packed operand, fixed at compile time in the bf16
// kernels so that only one conversion is emitted.
// CK_E4M3N: e4m3 container of a narrower element format (fp6 / fp4) whose rounding the hardware
// conversions do (MxArgs::direct says which); only the packing-only kernels are built with it.
enum : int { CK_NONE = 0, CK_E4M3 = 1, CK_E5M2 = 2, CK_E4M3N = 3 };

// two scaled magnitudes + the signs of the source pair w -> two code bytes (lo element in bits 0..7)
template <int CK>
__device__ __forceinline__ uint32_t code_pair(float q_lo, float q_hi, uint32_t w) {
    const float sl = __uint_as_float(__float_as_uint(q_lo) | ((w << 16) & 0x80000000u));
    const float sh = __uint_as_float(__float_as_uint(q_hi) | (w & 0x80000000u));
    return CK == CK_E5M2 ? encode2_e5m2(sl, sh) : encode2_e4m3(sl, sh);
}
// four scaled magnitudes + the signs of the two source pairs -> four code bytes:
// the sign bits are moved into place for all four bytes at once
template <int CK>
__device__ __forceinline__ uint32_t code_quad(float q0, float q1, float q2, float q3, uint32_t w01, uint32_t w23) {
    const uint32_t lo = CK == CK_E5M2 ? encode2_e5m2(q0, q1) : encode2_e4m3(q0, q1);
    const uint32_t hi = CK == CK_E5M2 ? encode2_e5m2(q2, q3) : encode2_e4m3(q2, q3);
    return __byte_perm(lo, hi, 0x5410) | (__byte_perm(w01, w23, 0x7531) & 0x80808080u);
}

// Codes straight from the hardware conversion when only the packed operand is wanted, for the formats
// the conversion instructions know (fp8_e4m3 and fp8_e5m2, which are their own container; fp6_e3m2,
// fp6_e2m3 and fp4_e2m1, narrowed and then widened exactly to an e4m3 byte): cvt.rn.satfinite rounds
// the scaled value to the format's grid (subnormals included) to nearest-even and saturates at max_norm,
// which is the element rounding of MX in 'even' mode; for 'nearest' (ties away from zero) the scale factor carries a relative
// nudge of 2^-12, which turns every exact tie into a round-up and moves nothing else (a bfloat16 source
// has 8 significant bits, so x / spacing is never within 2^-8 of a half-way point without being on it).
// c = 2^-s (exact reciprocal of the block scale) or 2^-s * (1 + 2^-12); the products are exact in fp32
// (8 x 13 significant bits).  The sign travels through the conversion.  Two pairs -> four code bytes.
// KIND as in MxArgs::direct (1: the container itself, 2 fp6_e3m2, 3 fp6_e2m3, 4 fp4_e2m1)
template <int CK, int KIND>
__device__ __forceinline__ uint32_t direct_pair(float lo, float hi) {
    if (CK == CK_E5M2) return encode2_e5m2(lo, hi);
    if (CK != CK_E4M3N) return encode2_e4m3(lo, hi);
    return KIND == 2 ? encode2_via_e3m2(lo, hi) : KIND == 3 ? encode2_via_e2m3(lo, hi) : encode2_via_e2m1(lo, hi);
}
template <int CK, int KIND>
__device__ __forceinline__ uint32_t code_quad_direct_k(uint32_t w01, uint32_t w23, float c0, float c1, float c2, float c3) {
    const float v0 = __uint_as_float(w01 << 16) * c0, v1 = __uint_as_float(w01 & 0xffff0000u) * c1;
    const float v2 = __uint_as_float(w23 << 16) * c2, v3 = __uint_as_float(w23 & 0xffff0000u) * c3;
    return __byte_perm(direct_pair<CK, KIND>(v0, v1), direct_pair<CK, KIND>(v2, v3), 0x5410);
}
// one decision on the narrow format per call, not per pair (it is warp-uniform but the compiler keeps it a branch)
template <int CK>
__device__ __forceinline__ uint32_t code_quad_direct(uint32_t w01, uint32_t w23, float c0, float c1, float c2, float c3,
                                                     int kind) {
    if (CK != CK_E4M3N) return code_quad_direct_k<CK, 1>(w01, w23, c0, c1, c2, c3);
    if (kind == 2) return code_quad_direct_k<CK, 2>(w01, w23, c0, c1, c2, c3);
    if (kind == 3) return code_quad_direct_k<CK, 3>(w01, w23, c0, c1, c2, c3);
    return code_quad_direct_k<CK, 4>(w01, w23, c0, c1, c2, c3);
}
// eight elements (four packed pairs) scaled by one factor -> eight code bytes
template <int CK>
__device__ __forceinline__ uint2 code_oct_direct(const uint32_t* w, float c, int kind) {
    if (CK != CK_E4M3N)
        return make_uint2(code_quad_direct_k<CK, 1>(w[0], w[1], c, c, c, c), code_quad_direct_k<CK, 1>(w[2], w[3], c, c, c, c));
    if (kind == 2)
        return make_uint2(code_quad_direct_k<CK, 2>(w[0], w[1], c, c, c, c), code_quad_direct_k<CK, 2>(w[2], w[3], c, c, c, c));
    if (kind == 3)
        return make_uint2(code_quad_direct_k<CK, 3>(w[0], w[1], c, c, c, c), code_quad_direct_k<CK, 3>(w[2], w[3], c, c, c, c));
    return make_uint2(code_quad_direct_k<CK, 4>(w[0], w[1], c, c, c, c), code_quad_direct_k<CK, 4>(w[2], w[3], c, c, c, c));
}
// whether a kernel built for container CK rounds its elements with the conversions
template <bool WANT_DQ, int CK, int MODE>
__device__ __forceinline__ bool use_direct(const MxArgs& a) {
    if (WANT_DQ || CK == CK_NONE || MODE == RZ) return false;
    return CK == CK_E4M3N ? true : a.direct == 1;
}
// the factor c of a block: bits of 2^-s with the 2^-12 nudge in the mantissa for half-away rounding
template <int MODE>
__device__ __forceinline__ float direct_factor(float inv) {
    return MODE == RN_AWAY ? __uint_as_float(__float_as_uint(inv) | 0x800u) : inv;
}

// code-byte sinks of the slow path
struct StridedBytes {                    // global memory, element r at p[r * s]
    uint8_t* p;
    int64_t s;
    __device__ __forceinline__ void operator()(int r, uint8_t v) const { p[r * s] = v; }
};
struct StagedBytes {                     // one column of the transposed staging tile (see mx_strided_bf16_kernel)
    uint8_t* tile;
    int chunk0;                          // logical 16-byte chunk index of row 0
    int swz;
    __device__ __forceinline__ void operator()(int r, uint8_t v) const {
        tile[(((chunk0 + (r >> 4)) ^ swz) << 4) + (r & 15)] = v;
    }
};

template <int MODE, int CK, typename CodeSink>
__device__ __forceinline__ void bf16_block_slow(const MxArgs& a, const uint16_t* in, int64_t first, int64_t stride,
                                                int rows, uint32_t amax, const CodeSink sink, int pad_to) {
    const BlockScale bs = block_scale(amax, a);
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
    if (amax == 0) {                       // a block of (signed) zeros passes through
#pragma unroll 1
        for (int r = 0; r < rows; ++r) {
            const uint16_t x = in[first + r * stride];
            if (out) out[first + r * stride] = x;
            if (CK != CK_NONE) sink(r, (uint8_t)((x >> 8) & 0x80u));
        }
        if (CK != CK_NONE) {
#pragma unroll 1
            for (int r = rows; r < pad_to; ++r) sink(r, 0);
        }
        return;
    }
#pragma unroll 1
    for (int r = 0; r < rows; ++r) {
        const uint32_t xb = (uint32_t)in[first + r * stride] << 16;
        const float q = quant_abs<MODE>(xb, bs, a.fmt);
        if (out) out[first + r * stride] = (uint16_t)((__float_as_uint(q * bs.scale) | (xb & 0x80000000u)) >> 16);
        if (CK != CK_NONE) sink(r, (uint8_t)code_pair<CK>(q, 0.f, xb >> 16));
    }
    if (CK != CK_NONE) {
#pragma unroll 1
        for (int r = rows; r < pad_to; ++r) sink(r, 0);
    }
}

constexpr int kLastBfThreads = 256;
constexpr int kLastBfUnroll = 4;

// A warp owns 2 KB of consecutive input (4 x 32 lanes x 16 bytes); a block of 32
// elements is shared by `lanes_per_block` neighbouring lanes.  `row_local`: every
// warp's 32 blocks lie in one row of the GEMM scale layout (4 lanes per block and
// a multiple of 32 blocks per row), so the scale index is computed once per thread.
// PRO = 1: the value that is quantized is SiLU(in) * in2, computed per element
// as the bfloat16 vector chain of the gated feed-forward block (sigmoid chain,
// gate * sigmoid, then the product with in2, each step rounded to bfloat16)
// instead of being loaded: the activation tensor is never written to memory.
// Codes and scales only.  The sigmoid chain is a pure function of the 16 input
// bits, so it is read from a 64 Ki-entry table (built once per device by running
// the chain itself on every bit pattern) held in shared memory; the kernel is
// then persistent, 1024 threads per SM, one table load per CTA.
constexpr int kSwigluThreads = 1024;

template <int MODE, bool WANT_DQ, int CK, int PRO, bool FULL>
__device__ __forceinline__ void lastaxis_bf16_tile_impl(const MxArgs& a, const int64_t nvec, const int lanes_per_block,
                                                        const int row_local, const int64_t tile_base,
                                                        const uint16_t* sig_tab) {
    const int lane_shift = 31 - __clz(lanes_per_block);
    const int64_t base = tile_base + (threadIdx.x >> 5) * (32 * kLastBfUnroll) + (threadIdx.x & 31);
    uint4 raw[kLastBfUnroll];
    bool live[kLastBfUnroll];
#pragma unroll
    for (int u = 0; u < kLastBfUnroll; ++u) {
        const int64_t v = base + u * 32;
        live[u] = FULL || v < nvec;
        raw[u] = live[u] ? __ldg(reinterpret_cast<const uint4*>(a.in) + v) : make_uint4(0, 0, 0, 0);
    }
    if (PRO == 1) {
#pragma unroll
        for (int u = 0; u < kLastBfUnroll; ++u) {
            const int64_t v = base + u * 32;
            const uint4 up4 = live[u] ? __ldg(reinterpret_cast<const uint4*>(a.in2) + v) : make_uint4(0, 0, 0, 0);
            const uint32_t g[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            const uint32_t up[4] = {up4.x, up4.y, up4.z, up4.w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t s2 = (uint32_t)sig_tab[g[i] & 0xffffu] | ((uint32_t)sig_tab[g[i] >> 16] << 16);
                o[i] = mul_bf16x2(mul_bf16x2(g[i], s2), up[i]);    // gate * sigmoid, rounded, then * up, rounded
            }
            raw[u] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    int64_t sidx0 = 0;
    if (CK != CK_NONE && row_local) sidx0 = scale_index_last(a, (uint32_t)(base >> 2));
    // Straight-line form of the common packing-only case (whole tile inside the tensor, blocks of 32, one
    // scale row per warp, elements rounded by the conversion instructions): taken when every block of the
    // warp's four vectors has a fast-path maximum (one vote), so the hot path has no divergent branch.
    if (FULL && lanes_per_block == 4 && row_local && use_direct<WANT_DQ, CK, MODE>(a)) {
        uint32_t mx[kLastBfUnroll];
        bool ok = true;
#pragma unroll
        for (int u = 0; u < kLastBfUnroll; ++u) {
            const uint32_t m2 = amax_bf16x2(amax_bf16x2(amax_bf16x2(raw[u].x & 0x7fff7fffu, raw[u].y), raw[u].z), raw[u].w);
            uint32_t m = max(m2 & 0xffffu, m2 >> 16);
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
            mx[u] = m >> 7;
            ok = ok && ((mx[u] - a.fp_e_lo) <= a.fp_e_span);
        }
        if (__all_sync(0xffffffffu, ok)) {
            const bool lead = (threadIdx.x & 3) == 0;
            uint2* codes = reinterpret_cast<uint2*>(a.codes) + base;
#pragma unroll
            for (int u = 0; u < kLastBfUnroll; ++u) {
                const uint32_t E = mx[u] - (uint32_t)a.fmt.emax_elem;
                if (lead) a.scales[sidx0 + u * 1024] = (uint8_t)E;
                const float cf = direct_factor<MODE>(__uint_as_float((254u << 23) - (E << 23)));
                const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                codes[u * 32] = code_oct_direct<CK>(w, cf, a.direct);
            }
            return;
        }
    }
#pragma unroll
    for (int u = 0; u < kLastBfUnroll; ++u) {
        const int64_t v = base + u * 32;
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        uint32_t m2 = amax_bf16x2(amax_bf16x2(amax_bf16x2(w[0] & 0x7fff7fffu, w[1]), w[2]), w[3]);
        uint32_t m = max(m2 & 0xffffu, m2 >> 16);
        if (lanes_per_block == 4) {                                  // blocks of 32: the usual case, unrolled
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
        } else {
            for (int s = 1; s < lanes_per_block; s <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
        }
        const FastBlock fb = fast_block(m >> 7, a);
        if (CK != CK_NONE && live[u] && (threadIdx.x & (lanes_per_block - 1)) == 0) {
            // 8 blocks further along the row = two 512-byte chunks of the GEMM scale layout
            const int64_t sidx = row_local ? sidx0 + u * 1024 : scale_index_last(a, (uint32_t)(v >> lane_shift));
            a.scales[sidx] = (uint8_t)(fb.ok ? fb.E : (uint32_t)scale_exp_from_absmax(m << 16, a.fmt.emax_elem, a.scale_emax));
        }
        if (!fb.ok) {
            if (PRO == 1) {
                // the values exist only in registers: scaled-domain rounding of the 8 elements, unrolled
                if (live[u]) {
                    const BlockScale bs = block_scale(m << 16, a);
                    uint32_t c[2] = {0, 0};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t xb = (i & 1) ? (w[i >> 1] & 0xffff0000u) : (w[i >> 1] << 16);
                        const float q = quant_abs<MODE>(xb, bs, a.fmt);
                        c[i >> 2] |= (code_pair<CK>(q, 0.f, xb >> 16) & 0xffu) << (8 * (i & 3));
                    }
                    reinterpret_cast<uint2*>(a.codes)[v] = make_uint2(c[0], c[1]);
                }
            } else if (live[u]) {
                bf16_block_slow<MODE, CK>(a, reinterpret_cast<const uint16_t*>(a.in), v * 8, 1, 8, m << 16,
                                          StridedBytes{CK != CK_NONE ? a.codes + v * 8 : nullptr, 1}, 8);
            }
            continue;
        }
        if (use_direct<WANT_DQ, CK, MODE>(a)) {
            if (live[u]) {
                const float cf = direct_factor<MODE>(fb.inv);
                reinterpret_cast<uint2*>(a.codes)[v] = code_oct_direct<CK>(w, cf, a.direct);
            }
            continue;
        }
        const uint32_t mp = a.fp_mp_base + fb.E * 0x00800080u;
        uint32_t o[4];
        float q[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = quant_pair_bf16<MODE, true>(w[i], fb.cmin, fb.cmin, mp, a.fmt, q[2 * i], q[2 * i + 1]);
        if (!live[u]) continue;
        if (WANT_DQ) reinterpret_cast<uint4*>(a.out)[v] = make_uint4(o[0], o[1], o[2], o[3]);
        if (CK != CK_NONE) {
            uint32_t c[2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                c[i] = code_quad<CK>(q[4 * i] * fb.inv, q[4 * i + 1] * fb.inv, q[4 * i + 2] * fb.inv, q[4 * i + 3] * fb.inv,
                                     w[2 * i], w[2 * i + 1]);
            reinterpret_cast<uint2*>(a.codes)[v] = make_uint2(c[0], c[1]);
        }
    }
}

// FULL tiles (every vector inside the tensor) run without bounds predicates.
template <int MODE, bool WANT_DQ, int CK, int PRO>
__device__ __forceinline__ void lastaxis_bf16_tile(const MxArgs& a, const int64_t nvec, const int lanes_per_block,
                                                   const int row_local, const int64_t tile_base,
                                                   const uint16_t* sig_tab) {
    if (tile_base + (int64_t)blockDim.x * kLastBfUnroll <= nvec)
        lastaxis_bf16_tile_impl<MODE, WANT_DQ, CK, PRO, true>(a, nvec, lanes_per_block, row_local, tile_base, sig_tab);
    else
        lastaxis_bf16_tile_impl<MODE, WANT_DQ, CK, PRO, false>(a, nvec, lanes_per_block, row_local, tile_base, sig_tab);
}

template <int MODE, bool WANT_DQ, int CK, int PRO = 0>
__global__ void __launch_bounds__(PRO ? kSwigluThreads : kLastBfThreads)
mx_lastaxis_bf16_kernel(const MxArgs a, const int64_t nvec, const int lanes_per_block, const int row_local) {
    static_assert(PRO == 0 || (!WANT_DQ && CK != CK_NONE), "the fused prologue produces the packed operand only");
    if (PRO == 0) {
        lastaxis_bf16_tile<MODE, WANT_DQ, CK, 0>(a, nvec, lanes_per_block, row_local,
                                                 (int64_t)blockIdx.x * (kLastBfThreads * kLastBfUnroll), nullptr);
    } else {
        extern __shared__ uint4 sig_tab_smem[];
        const uint4* src = reinterpret_cast<const uint4*>(a.sig_table);
        for (int i = threadIdx.x; i < 65536 * 2 / 16; i += kSwigluThreads) sig_tab_smem[i] = __ldg(src + i);
        __syncthreads();
        const int64_t per_tile = (int64_t)kSwigluThreads * kLastBfUnroll;
        const int64_t ntiles = (nvec + per_tile - 1) / per_tile;
        for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x)
            lastaxis_bf16_tile<MODE, WANT_DQ, CK, PRO>(a, nvec, lanes_per_block, row_local, t * per_tile,
                                                       reinterpret_cast<const uint16_t*>(sig_tab_smem));
    }
}

constexpr int kStrBfThreads = 128;

// One thread owns 4 adjacent columns of one block (up to 32 rows).
// TRANSPOSED (only with codes, block == 32): codes and scales are written with
// the blocked axis innermost.  A thread walks four consecutive blocks of its
// columns; the code bytes of two blocks at a time are staged in shared memory as
// a [512 columns][64 bytes] tile and written out by the whole CTA, four lanes per
// output row, so that a warp's store covers eight 64-byte segments instead of 32
// scattered 16-byte ones.  The tile is addressed in 16-byte chunks,
// chunk(c, j) = (4c + j) ^ ((c >> 2) & 7), which keeps both the per-column
// writes and the row-major readout free of bank conflicts.  In the GEMM scale
// layout the four scale bytes of a column are one 32-bit word.
// BPT: consecutive blocks a thread walks in the transposed form: 4, or 1 for tensors so small that four would
// leave most SMs without a CTA (the operands of an attention head).
template <int MODE, bool WANT_DQ, int CK, bool TRANSPOSED, int BPT = 4>
__global__ void __launch_bounds__(kStrBfThreads, (CK == CK_NONE && !TRANSPOSED) ? 6 : 4)
mx_strided_bf16_kernel(const MxArgs a, const int64_t col_tiles, const int64_t nbgrp) {
    constexpr int kBlocksPerThread = TRANSPOSED ? BPT : 1;
    __shared__ uint4 stage[TRANSPOSED ? kStrBfThreads * 4 * 4 : 1];
    // Columns are numbered across the leading axis: g = p * post + col.  A CTA owns 512 consecutive such
    // columns (four per thread; post % 4 == 0 keeps a thread's four inside one p), so tensors whose `post` is
    // short (the 128-wide heads of an attention block) still fill every thread.
    const int tid = threadIdx.x;
    const int64_t t = blockIdx.x;
    const int64_t ct = t % col_tiles;
    const int64_t bg = t / col_tiles;
    const int64_t g0 = ct * (kStrBfThreads * 4);
    const int64_t gcol = g0 + (int64_t)tid * 4;
    const int64_t gcols = a.pre * a.post;
    const bool active = gcol < gcols;
    if (!TRANSPOSED && !active) return;
    const int64_t p = active ? gcol / a.post : 0;
    const int64_t col = active ? gcol - p * a.post : 0;
    const uint16_t* in = reinterpret_cast<const uint16_t*>(a.in);
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
    const int64_t padded = a.nblk * a.block;
    uint32_t sf_word[4] = {0, 0, 0, 0};
#pragma unroll 1
    for (int bb = 0; bb < kBlocksPerThread; ++bb) {
        const int64_t b = bg * kBlocksPerThread + bb;
        if (b >= a.nblk) break;                                            // uniform over the CTA
        if (active) {
            const int64_t row0 = b * a.block;
            const int rows = (int)min((int64_t)a.block, a.axis_len - row0);
            const int64_t base = (p * a.axis_len + row0) * a.post + col;       // element index
            uint2 raw[kMaxRows];
            const bool full = rows == kMaxRows;                                // a ragged last block goes the slow way
            if (full) {
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r)
                    raw[r] = __ldg(reinterpret_cast<const uint2*>(in + base + (int64_t)r * a.post));
            } else {
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r)
                    raw[r] = r < rows ? __ldg(reinterpret_cast<const uint2*>(in + base + (int64_t)r * a.post)) : make_uint2(0, 0);
            }
            uint32_t m0 = 0, m1 = 0;
#pragma unroll
            for (int r = 0; r < kMaxRows; ++r) {
                m0 = amax_bf16x2(m0, raw[r].x);
                m1 = amax_bf16x2(m1, raw[r].y);
            }
            const uint32_t eraw[4] = {(m0 >> 7) & 0xffu, m0 >> 23, (m1 >> 7) & 0xffu, m1 >> 23};
            FastBlock fb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) fb[i] = fast_block(eraw[i], a);
            const bool all_ok = full && fb[0].ok && fb[1].ok && fb[2].ok && fb[3].ok;
            if (CK != CK_NONE) {
                uint32_t E[4] = {fb[0].E, fb[1].E, fb[2].E, fb[3].E};
                if (!all_ok) {
                    const uint32_t amax[4] = {m0 << 16, m0 & 0xffff0000u, m1 << 16, m1 & 0xffff0000u};
#pragma unroll
                    for (int i = 0; i < 4; ++i) E[i] = (uint32_t)scale_exp_from_absmax(amax[i], a.fmt.emax_elem, a.scale_emax);
                }
                if (TRANSPOSED && a.sf_gemm) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) sf_word[i] |= (E[i] & 0xffu) << (8 * bb);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) a.scales[scale_index(a, p, b, col + i)] = (uint8_t)E[i];
                }
            }
            if (!all_ok) {
#pragma unroll 1
                for (int i = 0; i < 4; ++i) {
                    const uint32_t mm = (i & 2) ? m1 : m0;
                    const uint32_t am = (i & 1) ? (mm & 0xffff0000u) : (mm << 16);
                    if (TRANSPOSED)
                        bf16_block_slow<MODE, CK>(a, in, base + i, a.post, rows, am,
                                                  StagedBytes{reinterpret_cast<uint8_t*>(stage),
                                                              (tid * 4 + i) * 4 + (bb & 1) * 2, tid & 7}, kMaxRows);
                    else
                        bf16_block_slow<MODE, CK>(a, in, base + i, a.post, rows, am,
                                                  StridedBytes{CK != CK_NONE ? a.codes + base + i : nullptr, a.post}, rows);
                }
            } else {
                const uint32_t mp0 = a.fp_mp_base + ((fb[0].E | (fb[1].E << 16)) << 7);
                const uint32_t mp1 = a.fp_mp_base + ((fb[2].E | (fb[3].E << 16)) << 7);
                const bool direct = use_direct<WANT_DQ, CK, MODE>(a);
                float inv[4] = {fb[0].inv, fb[1].inv, fb[2].inv, fb[3].inv};
                if (direct) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) inv[i] = direct_factor<MODE>(inv[i]);
                }
                uint32_t tc[4][4];                 // transposed codes: [column][4 rows per word], 16 rows
#pragma unroll
                for (int r4 = 0; r4 < kMaxRows / 4; ++r4) {
                    uint32_t c4[4];
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) {
                        const int r = r4 * 4 + rr;
                        if (!WANT_DQ && CK != CK_NONE && MODE != RZ && direct) {
                            c4[rr] = code_quad_direct<CK>(raw[r].x, raw[r].y, inv[0], inv[1], inv[2], inv[3], a.direct);
                            if (!TRANSPOSED)
                                *reinterpret_cast<uint32_t*>(a.codes + base + (int64_t)r * a.post) = c4[rr];
                            continue;
                        }
                        float q[4];
                        const uint32_t o0 = quant_pair_bf16<MODE, false>(raw[r].x, fb[0].cmin, fb[1].cmin, mp0, a.fmt, q[0], q[1]);
                        const uint32_t o1 = quant_pair_bf16<MODE, false>(raw[r].y, fb[2].cmin, fb[3].cmin, mp1, a.fmt, q[2], q[3]);
                        if (WANT_DQ)
                            *reinterpret_cast<uint2*>(out + base + (int64_t)r * a.post) = make_uint2(o0, o1);
                        if (CK != CK_NONE) {
                            c4[rr] = code_quad<CK>(fminf(q[0], fb[0].maxn) * inv[0], fminf(q[1], fb[1].maxn) * inv[1],
                                                   fminf(q[2], fb[2].maxn) * inv[2], fminf(q[3], fb[3].maxn) * inv[3], raw[r].x, raw[r].y);
                            if (!TRANSPOSED)
                                *reinterpret_cast<uint32_t*>(a.codes + base + (int64_t)r * a.post) = c4[rr];
                        }
                    }
                    if (CK != CK_NONE && TRANSPOSED) {
                        // 4 rows x 4 columns of code bytes -> one word per column (rows innermost)
                        const uint32_t t0 = __byte_perm(c4[0], c4[1], 0x5140), t1 = __byte_perm(c4[2], c4[3], 0x5140);
                        const uint32_t u0 = __byte_perm(c4[0], c4[1], 0x7362), u1 = __byte_perm(c4[2], c4[3], 0x7362);
                        tc[0][r4 & 3] = __byte_perm(t0, t1, 0x5410);
                        tc[1][r4 & 3] = __byte_perm(t0, t1, 0x7632);
                        tc[2][r4 & 3] = __byte_perm(u0, u1, 0x5410);
                        tc[3][r4 & 3] = __byte_perm(u0, u1, 0x7632);
                        if ((r4 & 3) == 3) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int chunk = (tid * 4 + i) * 4 + (bb & 1) * 2 + (r4 >> 2);
                                stage[chunk ^ (tid & 7)] = make_uint4(tc[i][0], tc[i][1], tc[i][2], tc[i][3]);
                            }
                        }
                    }
                }
            }
        }
        if (CK != CK_NONE && TRANSPOSED && ((bb & 1) || bb + 1 >= kBlocksPerThread || b + 1 >= a.nblk)) {
            // write out the staged pair of blocks: 4 lanes per output row.  A warp stages and writes only its own
            // 128 columns, so the warps of a CTA never wait for one another and drift out of lock-step.
            __syncwarp();
            const int nchunk = ((bb & 1) + 1) * 2;
            const int64_t k0 = (bg * kBlocksPerThread + (bb & ~1)) * kMaxRows;
            const int id0 = (tid & ~31) * 16 + (tid & 31);
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int id = id0 + it * 32;
                const int c = id >> 2, j = id & 3;
                if (g0 + c < gcols && j < nchunk)
                    *reinterpret_cast<uint4*>(a.codes + (g0 + c) * padded + k0 + j * 16) =
                        stage[id ^ ((id >> 4) & 7)];
            }
            __syncwarp();
        }
    }
    if (CK != CK_NONE && TRANSPOSED && a.sf_gemm && active) {
        const int64_t b0 = bg * kBlocksPerThread;
        const int nb = (int)min((int64_t)kBlocksPerThread, a.nblk - b0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint8_t* dst = a.scales + scale_index(a, p, b0, col + i);
            if (kBlocksPerThread == 4 && nb == 4) *reinterpret_cast<uint32_t*>(dst) = sf_word[i];
            else for (int k = 0; k < nb; ++k) dst[k] = (uint8_t)(sf_word[i] >> (8 * k));
        }
    }
}

// ---------------------------------------------------------------------------
// generic kernel: one thread per block of the tensor
// ---------------------------------------------------------------------------
template <int DT>
__global__ void mx_generic_kernel(const MxArgs a, const int64_t ntiles) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= ntiles) return;
    const int64_t j = t % a.post;
    const int64_t b = (t / a.post) % a.nblk;
    const int64_t p = t / (a.post * a.nblk);
    const int64_t k0 = b * a.block;
    const int64_t k1 = min(k0 + a.block, a.axis_len);
    const int64_t base = p * a.axis_len * a.post + j;
    uint32_t m = 0;
    for (int64_t k = k0; k < k1; ++k)
        m = max(m, __float_as_uint(load1<DT>(a.in, base + k * a.post)) & 0x7fffffffu);
    const BlockScale bs = block_scale(m, a);
    const bool dead = bs.inv == 0.0f;               // NaN block or flushed block
    if (a.scales) a.scales[scale_index(a, p, b, j)] = (uint8_t)bs.E;
    const int64_t padded = a.nblk * a.block;
    for (int64_t k = k0; k < k0 + a.block; ++k) {
        if (k >= k1) {                              // padding of a ragged transposed block
            if (a.codes && a.transposed) a.codes[(p * a.post + j) * padded + k] = 0;
            continue;
        }
        const int64_t idx = base + k * a.post;
        const float x = load1<DT>(a.in, idx);
        const float v = dead ? 0.0f : x * bs.inv;   // exact: power-of-two scaling
        float q = round_generic(v, a.fmt.mbits, a.fmt.ebits, a.fmt.max_norm, a.mode, true, true,
                                a.noise ? a.noise[idx] : 0.f);
        // keep the sign of x on results that rounded to zero
        q = __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(x) & 0x80000000u));
        if (a.out) store1<DT>(a.out, idx, q * bs.scale);
        if (a.codes) {
            const uint8_t c = (uint8_t)encode1(q, a.fmt.ebits, a.fmt.mbits);
            if (a.transposed) a.codes[(p * a.post + j) * padded + k] = c;
            else a.codes[idx] = c;
        }
    }
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------
template <int DT, int MODE>
static int launch_last(const MxArgs& a, int64_t nvec, int lanes, cudaStream_t st) {
    const int64_t tile = (int64_t)kLastThreads * kLastUnroll;
    const int64_t need = (nvec + tile - 1) / tile;
    const int grid = (int)std::min<int64_t>(need, (int64_t)sm_count() * 16);
    if (a.out && a.codes) mx_lastaxis_kernel<DT, MODE, true, true><<<grid, kLastThreads, 0, st>>>(a, nvec, lanes);
    else if (a.codes) mx_lastaxis_kernel<DT, MODE, false, true><<<grid, kLastThreads, 0, st>>>(a, nvec, lanes);
    else mx_lastaxis_kernel<DT, MODE, true, false><<<grid, kLastThreads, 0, st>>>(a, nvec, lanes);
    return check_launch();
}

template <int DT, int MODE>
static int launch_strided(const MxArgs& a, cudaStream_t st) {
    constexpr int N = VecIO<DT, 8>::N;
    const int64_t col_tiles = (a.post + (int64_t)kStrThreads * N - 1) / ((int64_t)kStrThreads * N);
    const int64_t ntiles = col_tiles * a.pre * a.nblk;
    const int grid = (int)std::min<int64_t>(ntiles, (int64_t)sm_count() * 64);
    if (a.out && a.codes) mx_strided_kernel<DT, MODE, true, true><<<grid, kStrThreads, 0, st>>>(a, col_tiles, ntiles);
    else if (a.codes) mx_strided_kernel<DT, MODE, false, true><<<grid, kStrThreads, 0, st>>>(a, col_tiles, ntiles);
    else mx_strided_kernel<DT, MODE, true, false><<<grid, kStrThreads, 0, st>>>(a, col_tiles, ntiles);
    return check_launch();
}

template <int MODE>
static int launch_last_bf16(const MxArgs& a, int64_t nvec, int lanes, cudaStream_t st) {
    const int64_t tile = (int64_t)kLastBfThreads * kLastBfUnroll;
    const int64_t grid = (nvec + tile - 1) / tile;
    if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
    const unsigned g = (unsigned)grid;
    const bool e5 = a.fmt.ebits == 5;
    const int rl = a.sf_gemm && lanes == 4 && a.nblk % 32 == 0;
    if (!a.codes) mx_lastaxis_bf16_kernel<MODE, true, CK_NONE><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    else if (a.out && e5) mx_lastaxis_bf16_kernel<MODE, true, CK_E5M2><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    else if (a.out) mx_lastaxis_bf16_kernel<MODE, true, CK_E4M3><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    else if (e5) mx_lastaxis_bf16_kernel<MODE, false, CK_E5M2><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    else if (MODE != RZ && a.direct >= 2) mx_lastaxis_bf16_kernel<MODE, false, CK_E4M3N><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    else mx_lastaxis_bf16_kernel<MODE, false, CK_E4M3><<<g, kLastBfThreads, 0, st>>>(a, nvec, lanes, rl);
    return check_launch();
}

template <int MODE, bool WANT_DQ, int CK, bool TR>
static int launch_strided_bf16_one(const MxArgs& a, cudaStream_t st) {
    const int64_t col_tiles = (a.pre * a.post + (int64_t)kStrBfThreads * 4 - 1) / ((int64_t)kStrBfThreads * 4);
    if (TR && !WANT_DQ && col_tiles * ((a.nblk + 3) / 4) < 2 * (int64_t)sm_count()) {
        // a small operand: one block per thread, four times the CTAs
        mx_strided_bf16_kernel<MODE, WANT_DQ, CK, TR, 1><<<(unsigned)(col_tiles * a.nblk), kStrBfThreads, 0, st>>>(a, col_tiles, a.nblk);
        return check_launch();
    }
    const int64_t nbgrp = TR ? (a.nblk + 3) / 4 : a.nblk;
    const int64_t grid = col_tiles * nbgrp;
    if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
    mx_strided_bf16_kernel<MODE, WANT_DQ, CK, TR><<<(unsigned)grid, kStrBfThreads, 0, st>>>(a, col_tiles, nbgrp);
    return check_launch();
}

template <int MODE>
static int launch_strided_bf16(const MxArgs& a, cudaStream_t st) {
    const bool e5 = a.fmt.ebits == 5;
    if (!a.codes) return launch_strided_bf16_one<MODE, true, CK_NONE, false>(a, st);
    if (a.transposed) {
        if (a.out) return e5 ? launch_strided_bf16_one<MODE, true, CK_E5M2, true>(a, st)
                             : launch_strided_bf16_one<MODE, true, CK_E4M3, true>(a, st);
        if (!e5 && MODE != RZ && a.direct >= 2) return launch_strided_bf16_one<MODE, false, CK_E4M3N, true>(a, st);
        return e5 ? launch_strided_bf16_one<MODE, false, CK_E5M2, true>(a, st)
                  : launch_strided_bf16_one<MODE, false, CK_E4M3, true>(a, st);
    }
    if (a.out) return e5 ? launch_strided_bf16_one<MODE, true, CK_E5M2, false>(a, st)
                         : launch_strided_bf16_one<MODE, true, CK_E4M3, false>(a, st);
    if (!e5 && MODE != RZ && a.direct >= 2) return launch_strided_bf16_one<MODE, false, CK_E4M3N, false>(a, st);
    return e5 ? launch_strided_bf16_one<MODE, false, CK_E5M2, false>(a, st)
              : launch_strided_bf16_one<MODE, false, CK_E4M3, false>(a, st);
}

template <int DT>
int dispatch_dt(const MxArgs& a, cudaStream_t st) {
    constexpr int N16 = VecIO<DT, 16>::N;
    constexpr int N8 = VecIO<DT, 8>::N;
    const int64_t total = a.pre * a.axis_len * a.post;
    const int P = a.fmt.mbits - 1;
    const bool fast_math = a.mode <= RN_EVEN && P >= 1 && P <= 12 && a.fmt.ebits <= 5;
    const bool pow2 = (a.block & (a.block - 1)) == 0;
    const bool ptrs16 = aligned16(a.in) && (!a.out || aligned16(a.out)) && (!a.codes || aligned8(a.codes));
    const bool ptrs8 = aligned8(a.in) && (!a.out || aligned8(a.out)) && (!a.codes || aligned8(a.codes));

    if (fast_math && a.post == 1 && pow2 && a.block >= N16 && a.block <= 32 * N16 &&
        a.axis_len % a.block == 0 && ptrs16 && !a.transposed && total / a.block <= 0xffffffffLL) {
        const int lanes = a.block / N16;
        const int64_t nvec = total / N16;
        if (DT == DT_BF16 && P <= 8 && (!a.codes || a.fmt.ebits != 0)) {
            switch (a.mode) {
                case RN_AWAY: return launch_last_bf16<RN_AWAY>(a, nvec, lanes, st);
                case RZ:      return launch_last_bf16<RZ>(a, nvec, lanes, st);
                default:      return launch_last_bf16<RN_EVEN>(a, nvec, lanes, st);
            }
        }
        switch (a.mode) {
            case RN_AWAY: return launch_last<DT, RN_AWAY>(a, nvec, lanes, st);
            case RZ:      return launch_last<DT, RZ>(a, nvec, lanes, st);
            default:      return launch_last<DT, RN_EVEN>(a, nvec, lanes, st);
        }
    }
    if (fast_math && a.post > 1 && a.block <= kMaxRows && a.post % N8 == 0 && ptrs8) {
        if (DT == DT_BF16 && P <= 8 && a.block == kMaxRows && (!a.codes || (a.fmt.ebits != 0 && (!a.transposed || aligned16(a.codes)) && (!a.sf_gemm || !a.scales || (reinterpret_cast<uintptr_t>(a.scales) & 3u) == 0)))) {
            switch (a.mode) {
                case RN_AWAY: return launch_strided_bf16<RN_AWAY>(a, st);
                case RZ:      return launch_strided_bf16<RZ>(a, st);
                default:      return launch_strided_bf16<RN_EVEN>(a, st);
            }
        }
        switch (a.mode) {
            case RN_AWAY: return launch_strided<DT, RN_AWAY>(a, st);
            case RZ:      return launch_strided<DT, RZ>(a, st);
            default:      return launch_strided<DT, RN_EVEN>(a, st);
        }
    }
    const int64_t ntiles = a.pre * a.nblk * a.post;
    const int threads = 128;
    const int64_t grid = (ntiles + threads - 1) / threads;
    if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
    mx_generic_kernel<DT><<<(unsigned)grid, threads, 0, st>>>(a, ntiles);
    return check_launch();
}

}  // namespace mxq
