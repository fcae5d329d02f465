// Elementwise format rounding (bfloatX / fpX / arbitrary eXmY) for sm_100a.
//
// One streaming kernel: each thread converts eight consecutive elements per
// step (16- or 32-byte vector loads and stores), grid sized from the SM count.
// Formats with eight exponent bits (the bfloat family, which is what the MX
// layers use between GEMMs) share fp32's exponent layout, subnormals included,
// so rounding is an integer add-and-mask on the raw bits; every other format
// goes through the exact integer routine of mxq_math.cuh.
#include "mxq_common.cuh"
#include <algorithm>
#include <cstring>

namespace mxq {

struct EwArgs {
    const void* in;
    void* out;
    const float* noise;
    int64_t n;
    int bits, exp_bits;
    float max_norm;
    int mode;
    int saturate, allow_denorm;
    uint32_t drop;          // low bits removed (8-exponent-bit path)
    uint32_t max_bits;      // bit pattern of max_norm
};

// fp32 bit pattern -> rounded fp32 bit pattern, formats with 8 exponent bits
template <int MODE>
__device__ __forceinline__ uint32_t round_bf_family(uint32_t u, const EwArgs& a) {
    const uint32_t mag = u & 0x7fffffffu;
    const uint32_t sgn = u & 0x80000000u;
    if (mag >= kInf) return mag > kInf ? kNaN : u;
    if (!a.allow_denorm && mag < 0x00800000u) return mag == 0 ? 0u : sgn;
    const uint32_t mask = (1u << a.drop) - 1u;
    uint32_t r = mag;
    if (MODE == RN_AWAY) r += 1u << (a.drop - 1);
    else if (MODE == RN_EVEN) r += (mask >> 1) + ((mag >> a.drop) & 1u);
    r &= ~mask;
    if (r > a.max_bits) r = a.saturate ? a.max_bits : kInf;
    return (r == 0 && mag == 0) ? 0u : (r | sgn);
}

template <int IN_DT, int N> struct Load8;
template <> struct Load8<DT_F32, 8> {
    static __device__ __forceinline__ void run(const void* p, int64_t e, uint32_t (&b)[8]) {
        uint32_t lo[4], hi[4];
        VecIO<DT_F32, 16>::load(p, e, lo);
        VecIO<DT_F32, 16>::load(p, e + 4, hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) { b[i] = lo[i]; b[4 + i] = hi[i]; }
    }
};
template <> struct Load8<DT_BF16, 8> {
    static __device__ __forceinline__ void run(const void* p, int64_t e, uint32_t (&b)[8]) { VecIO<DT_BF16, 16>::load(p, e, b); }
};
template <> struct Load8<DT_F16, 8> {
    static __device__ __forceinline__ void run(const void* p, int64_t e, uint32_t (&b)[8]) { VecIO<DT_F16, 16>::load(p, e, b); }
};

template <int OUT_DT> __device__ __forceinline__ void store8(void* p, int64_t e, const uint32_t (&b)[8]);
template <> __device__ __forceinline__ void store8<DT_F32>(void* p, int64_t e, const uint32_t (&b)[8]) {
    float* o = reinterpret_cast<float*>(p) + e;
    reinterpret_cast<uint4*>(o)[0] = make_uint4(b[0], b[1], b[2], b[3]);
    reinterpret_cast<uint4*>(o)[1] = make_uint4(b[4], b[5], b[6], b[7]);
}
template <> __device__ __forceinline__ void store8<DT_BF16>(void* p, int64_t e, const uint32_t (&b)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(b[2 * i]), __uint_as_float(b[2 * i + 1]));
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p) + e) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ void store8<DT_F16>(void* p, int64_t e, const uint32_t (&b)[8]) {
    VecIO<DT_F16, 16>::store(p, e, b);
}

// PATH 0: 8-exponent-bit integer rounding; PATH 1: exact generic routine
template <int IN_DT, int OUT_DT, int PATH, int MODE>
__device__ __forceinline__ uint32_t ew_one(uint32_t u, const EwArgs& a, int64_t idx) {
    if (PATH == 0) return round_bf_family<MODE>(u, a);
    return __float_as_uint(round_generic(__uint_as_float(u), a.bits, a.exp_bits, a.max_norm, a.mode,
                                         a.saturate != 0, a.allow_denorm != 0,
                                         a.noise ? a.noise[idx] : 0.f));
}

constexpr int kEwThreads = 256;

template <int IN_DT, int OUT_DT, int PATH, int MODE>
__global__ void __launch_bounds__(kEwThreads)
ew_vec_kernel(const EwArgs a, const int64_t nvec8) {
    const int64_t stride = (int64_t)gridDim.x * kEwThreads;
    for (int64_t v = (int64_t)blockIdx.x * kEwThreads + threadIdx.x; v < nvec8; v += stride) {
        uint32_t b[8];
        Load8<IN_DT, 8>::run(a.in, v * 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = ew_one<IN_DT, OUT_DT, PATH, MODE>(b[i], a, v * 8 + i);
        store8<OUT_DT>(a.out, v * 8, b);
    }
}

template <int IN_DT, int OUT_DT, int PATH, int MODE>
__global__ void ew_scalar_kernel(const EwArgs a, const int64_t first, const int64_t n) {
    const int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t u = __float_as_uint(load1<IN_DT>(a.in, i));
    store1<OUT_DT>(a.out, i, __uint_as_float(ew_one<IN_DT, OUT_DT, PATH, MODE>(u, a, i)));
}

// bf16 -> bf16 for bfloat-family targets: the rounding acts on the bf16 bit
// pattern itself (drop16 = low mantissa bits removed, 0 = nothing to round), two
// elements per 32-bit operation.  Vectors that hold Inf/NaN (or subnormals when
// those are flushed) take the per-element routine.
__device__ __forceinline__ uint32_t vmaxu2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t vminu2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

constexpr int kEwBfUnroll = 4;

template <int MODE>
__global__ void __launch_bounds__(kEwThreads)
ew_bf16_pairs_kernel(const EwArgs a, const int64_t nvec, const uint32_t drop16, const uint32_t cap16) {
    const int64_t base = (int64_t)blockIdx.x * (kEwThreads * kEwBfUnroll);
    uint4 raw[kEwBfUnroll];
    bool live[kEwBfUnroll];
#pragma unroll
    for (int u = 0; u < kEwBfUnroll; ++u) {
        const int64_t v = base + (int64_t)u * kEwThreads + threadIdx.x;
        live[u] = v < nvec;
        raw[u] = live[u] ? __ldg(reinterpret_cast<const uint4*>(a.in) + v) : make_uint4(0, 0, 0, 0);
    }
    const uint32_t mask = ((1u << drop16) - 1u) * 0x10001u;
    const uint32_t half = drop16 ? (1u << (drop16 - 1)) * 0x10001u : 0u;
    const uint32_t cap = cap16 * 0x10001u;
#pragma unroll
    for (int u = 0; u < kEwBfUnroll; ++u) {
        if (!live[u]) continue;
        const int64_t v = base + (int64_t)u * kEwThreads + threadIdx.x;
        uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        uint32_t mag[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) mag[i] = w[i] & 0x7fff7fffu;
        const uint32_t mx = vmaxu2(vmaxu2(mag[0], mag[1]), vmaxu2(mag[2], mag[3]));
        const bool special = (mx & 0xffffu) >= 0x7f80u || (mx >> 16) >= 0x7f80u || !a.allow_denorm;
        uint32_t o[4];
        if (!special) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t r = mag[i];
                if (MODE == RN_AWAY) r += half;
                else if (MODE == RN_EVEN) r += (half - (drop16 ? 0x10001u : 0u)) + ((mag[i] >> drop16) & (drop16 ? 0x10001u : 0u));
                r &= ~mask;
                r = vminu2(r, cap);                     // overflow -> Inf pattern, or max_norm when saturating
                o[i] = r | (w[i] & 0x80008000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t lo = round_bf_family<MODE>(w[i] << 16, a);
                const uint32_t hi = round_bf_family<MODE>(w[i] & 0xffff0000u, a);
                o[i] = __byte_perm(lo, hi, 0x7632);
            }
        }
        reinterpret_cast<uint4*>(a.out)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// fp32 -> bfloat16 storage, round to nearest even, subnormals kept, overflow to Inf: the cast
// `A.to(torch.bfloat16)` the reference takes for bfloat = 16, round = 'even' (mx/elemwise_ops.py:248-251).
// The hardware conversion is that rounding; NaN results are rewritten to the quiet NaN torch's cast
// produces (0x7fc0).  A thread converts four groups of eight elements, all eight 16-byte loads issued
// before the first use.
constexpr int kCastUnroll = 4;
__global__ void __launch_bounds__(kEwThreads)
ew_f32_to_bf16_rne_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, const int64_t nvec) {
    const int64_t base = (int64_t)blockIdx.x * (kEwThreads * kCastUnroll);
    uint4 lo[kCastUnroll], hi[kCastUnroll];
    bool live[kCastUnroll];
#pragma unroll
    for (int u = 0; u < kCastUnroll; ++u) {
        const int64_t v = base + (int64_t)u * kEwThreads + threadIdx.x;
        live[u] = v < nvec;
        lo[u] = live[u] ? __ldg(in + 2 * v) : make_uint4(0, 0, 0, 0);
        hi[u] = live[u] ? __ldg(in + 2 * v + 1) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kCastUnroll; ++u) {
        if (!live[u]) continue;
        const uint32_t f[8] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1]));
            uint32_t p = *reinterpret_cast<const uint32_t*>(&h);
            const uint32_t q = p & 0x7fff7fffu;
            if (((q + 0x007f007fu) & 0x80008000u) != 0) {      // a half above 0x7f80: NaN
                if ((q & 0xffffu) > 0x7f80u) p = (p & 0xffff0000u) | 0x7fc0u;
                if ((q >> 16) > 0x7f80u) p = (p & 0x0000ffffu) | 0x7fc00000u;
            }
            w[i] = p;
        }
        out[base + (int64_t)u * kEwThreads + threadIdx.x] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <int MODE>
static int launch_ew_bf16_pairs(const EwArgs& a, cudaStream_t st) {
    // bits = P + 1 with P significand bits; bf16 carries 8, so 8 - P low bits go
    const int P = a.bits - 1;
    const uint32_t drop16 = P >= 8 ? 0u : (uint32_t)(8 - P);
    const uint32_t cap16 = a.saturate ? (a.max_bits >> 16) : 0x7f80u;
    const int64_t nvec = a.n / 8;
    if (nvec > 0) {
        const int64_t tile = (int64_t)kEwThreads * kEwBfUnroll;
        const int64_t grid = (nvec + tile - 1) / tile;
        if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
        ew_bf16_pairs_kernel<MODE><<<(unsigned)grid, kEwThreads, 0, st>>>(a, nvec, drop16, cap16);
    }
    const int64_t first = nvec * 8;
    if (first < a.n) ew_scalar_kernel<DT_BF16, DT_BF16, 0, MODE><<<1, 128, 0, st>>>(a, first, a.n);
    return check_launch();
}

template <int IN_DT, int OUT_DT, int PATH, int MODE>
static int launch_ew(const EwArgs& a, cudaStream_t st) {
    const bool vec_ok = aligned16(a.in) && aligned16(a.out);
    const int64_t nvec8 = vec_ok ? a.n / 8 : 0;
    if (nvec8 > 0) {
        const int64_t need = (nvec8 + kEwThreads - 1) / kEwThreads;
        const int grid = (int)std::min<int64_t>(need, (int64_t)sm_count() * 32);
        ew_vec_kernel<IN_DT, OUT_DT, PATH, MODE><<<grid, kEwThreads, 0, st>>>(a, nvec8);
    }
    const int64_t first = nvec8 * 8;
    if (first < a.n) {
        const int64_t rest = a.n - first;
        const int64_t grid = (rest + 127) / 128;
        if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
        ew_scalar_kernel<IN_DT, OUT_DT, PATH, MODE><<<(unsigned)grid, 128, 0, st>>>(a, first, a.n);
    }
    return check_launch();
}

template <int IN_DT, int OUT_DT>
static int dispatch_path(const EwArgs& a, cudaStream_t st) {
    // the packed bf16 path takes "above max_norm" to mean "rounded past the top of the grid", which
    // holds when max_norm is the largest finite value of the format (what _get_max_norm gives)
    const int p_bits = a.bits - 1;
    const uint32_t grid_top = 0x7f7f0000u & ~(((p_bits >= 8 ? 0u : (1u << (8 - p_bits)) - 1u)) << 16);
    if (IN_DT == DT_BF16 && OUT_DT == DT_BF16 && a.exp_bits == 8 && a.mode <= RN_EVEN && a.bits >= 2 &&
        a.max_bits == grid_top && aligned16(a.in) && aligned16(a.out)) {
        switch (a.mode) {
            case RN_AWAY: return launch_ew_bf16_pairs<RN_AWAY>(a, st);
            case RZ:      return launch_ew_bf16_pairs<RZ>(a, st);
            default:      return launch_ew_bf16_pairs<RN_EVEN>(a, st);
        }
    }
    if (IN_DT == DT_F32 && OUT_DT == DT_BF16 && a.exp_bits == 8 && a.bits == 9 && a.mode == RN_EVEN && a.allow_denorm &&
        !a.saturate && a.max_bits == 0x7f7f0000u && aligned16(a.in) && aligned16(a.out) && a.n >= 8) {
        const int64_t nvec = a.n / 8;
        const int64_t tile = (int64_t)kEwThreads * kCastUnroll;
        const int64_t grid = (nvec + tile - 1) / tile;
        if (grid > 0x7fffffffLL) return MXQ_ERR_TOO_LARGE;
        ew_f32_to_bf16_rne_kernel<<<(unsigned)grid, kEwThreads, 0, st>>>(reinterpret_cast<const uint4*>(a.in),
                                                                         reinterpret_cast<uint4*>(a.out), nvec);
        if (nvec * 8 < a.n) ew_scalar_kernel<DT_F32, DT_BF16, 0, RN_EVEN><<<1, 128, 0, st>>>(a, nvec * 8, a.n);
        return check_launch();
    }
    if (a.exp_bits == 8 && a.mode <= RN_EVEN) {
        switch (a.mode) {
            case RN_AWAY: return launch_ew<IN_DT, OUT_DT, 0, RN_AWAY>(a, st);
            case RZ:      return launch_ew<IN_DT, OUT_DT, 0, RZ>(a, st);
            default:      return launch_ew<IN_DT, OUT_DT, 0, RN_EVEN>(a, st);
        }
    }
    return launch_ew<IN_DT, OUT_DT, 1, 0>(a, st);
}

}  // namespace mxq

extern "C" int mxq_quantize_elemwise(const void* in, void* out, int in_dtype, int out_dtype, int64_t n,
                                     int bits, int exp_bits, float max_norm, int rmode,
                                     int saturate_normals, int allow_denorm, const void* noise,
                                     void* stream) {
    using namespace mxq;
    if (n < 0) return MXQ_ERR_BAD_ARG;
    if (n == 0) return MXQ_OK;
    if (!in || !out) return MXQ_ERR_BAD_ARG;
    if (bits < 2 || bits > 24 || exp_bits < 0 || exp_bits > 8) return MXQ_ERR_BAD_ARG;  // funcs.cpp:209
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_DITHER) return MXQ_ERR_BAD_ARG;
    if (rmode == MXQ_ROUND_DITHER && !noise) return MXQ_ERR_BAD_ARG;
    EwArgs a;
    a.in = in; a.out = out; a.noise = (const float*)noise; a.n = n;
    a.bits = bits; a.exp_bits = exp_bits; a.max_norm = max_norm; a.mode = rmode;
    a.saturate = saturate_normals != 0; a.allow_denorm = allow_denorm != 0;
    a.drop = (uint32_t)(24 - (bits - 1));
    memcpy(&a.max_bits, &max_norm, 4);
    cudaStream_t st = (cudaStream_t)stream;
#define MXQ_EW_CASE(I, O) if (in_dtype == I && out_dtype == O) return dispatch_path<I, O>(a, st)
    MXQ_EW_CASE(DT_F32, DT_F32);
    MXQ_EW_CASE(DT_BF16, DT_BF16);
    MXQ_EW_CASE(DT_F16, DT_F16);
    MXQ_EW_CASE(DT_F32, DT_BF16);
    MXQ_EW_CASE(DT_F32, DT_F16);
    MXQ_EW_CASE(DT_BF16, DT_F32);
    MXQ_EW_CASE(DT_F16, DT_F32);
#undef MXQ_EW_CASE
    return MXQ_ERR_UNSUPPORTED;
}
