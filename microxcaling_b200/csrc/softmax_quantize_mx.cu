// Softmax over the last dimension fused with the MX packing of the
// probabilities (sm_100a).
//
// In an attention block the reference computes P = softmax(S) as a chain of
// vector operations, each rounded to bfloat16 (mx/softmax.py:18-41), and the
// product P V then MX-quantizes P along its last axis as the left operand
// (mx/bmm.py:40-59, mx/matmul.py:68-86).  Here one warp keeps a row of S in
// registers, runs the same chain (max, subtract, exp, sum, divide; the same fp32
// operations and bfloat16 roundings as mxq_softmax_bf16) and then quantizes the
// row's 32-element blocks where they sit: the block maximum is a butterfly over
// the four lanes that share a block, the element rounding is the packed-pair
// routine of the last-axis MX kernel.  Written: one code byte per probability
// and the E8M0 scales (GEMM chunk layout), and the bfloat16 probabilities
// themselves when the caller wants them.  S is read once; P is never re-read.
#include "quantize_mx_impl.cuh"
#include <math_constants.h>

namespace mxq {

// Persistent CTAs of 32 warps, one per SM.  Shared memory: the exp table (d <= 0 always, so the sign
// bit is dropped: 32 Ki entries, 64 KB) and one 4 KB landing buffer per warp, into which the warp's NEXT
// row streams (cp.async) while the current one is processed in registers, so every warp always has a row
// in flight and the kernel is not exposed to memory latency.
constexpr int kSqThreads = 1024;
constexpr int kSqWarps = kSqThreads / 32;
constexpr int kSqTabEntries = 32768;
constexpr int kSqTabBytes = kSqTabEntries * 2;
constexpr int kSqRowBytes = 4096;          // rows of up to 2048 bfloat16
constexpr int kSqSmemBytes = kSqTabBytes + kSqWarps * kSqRowBytes;
constexpr int kSqMaxVec = 8;              // 16-byte chunks per lane

__device__ __forceinline__ float sq_nan_max(float a, float b) { return (b > a || b != b) ? b : a; }
__device__ __forceinline__ uint32_t max_nan_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// a - b per packed bfloat16 lane, one rounding (to nearest even).  Equal to the fp32 subtraction of the two
// values followed by the rounding to bfloat16: that subtraction is exact unless the exponents are more than
// 16 apart, and then either way the result is the operand of larger magnitude.
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// CK == CK_NONE: softmax only (probabilities to a.out); otherwise also (or only, !WANT_P) the MX packing.
// UNI: the row length is a multiple of 256, so a 16-byte chunk index lane + 32 k is inside the row for all
// lanes of a warp or for none: the bounds checks are warp-uniform branches (no divergence bookkeeping).
template <int MODE, int CK, bool WANT_P, bool UNI>
__global__ void __launch_bounds__(kSqThreads, 1)
softmax_rows_kernel(const MxArgs a, const uint16_t* __restrict__ table, const int64_t rows, const int cols) {
    extern __shared__ uint4 sq_smem[];
    // the non-negative half of the table (exp of -|d|): entry i of the full table's upper half
    for (int i = threadIdx.x; i < kSqTabBytes / 16; i += kSqThreads)
        sq_smem[i] = __ldg(reinterpret_cast<const uint4*>(table + 32768) + i);
    __syncthreads();
    const uint16_t* tab = reinterpret_cast<const uint16_t*>(sq_smem);
    const uint16_t* x = reinterpret_cast<const uint16_t*>(a.in);
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nchunk = cols >> 3;
    auto inside = [&](int k, int lane_) { return UNI ? 32 * k < nchunk : lane_ + 32 * k < nchunk; };
    const int64_t warps = (int64_t)gridDim.x * kSqWarps;
    uint4* rowbuf = sq_smem + kSqTabBytes / 16 + warp * (kSqRowBytes / 16);
    const uint32_t rowbuf_s = (uint32_t)__cvta_generic_to_shared(rowbuf);
    const int64_t r128 = (a.sf_rpb + 127) >> 7, kb4 = (a.nblk + 3) >> 2;

    int64_t row = (int64_t)blockIdx.x * kSqWarps + warp;
    if (row < rows) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
        if (UNI) {
#pragma unroll 1
            for (int k = 0; k < (nchunk >> 5); ++k) cp_async16(rowbuf_s + (lane + 32 * k) * 16, xr + lane + 32 * k);
        } else {
            for (int c = lane; c < nchunk; c += 32) cp_async16(rowbuf_s + c * 16, xr + c);
        }
    }
    cp_async_commit();
    for (; row < rows; row += warps) {
        cp_async_wait_all();
        __syncwarp();
        uint32_t w[kSqMaxVec][4];
        uint32_t m2 = 0xff80ff80u;                                  // (-inf, -inf)
#pragma unroll
        for (int k = 0; k < kSqMaxVec; ++k) {
            const int c = lane + 32 * k;
            if (inside(k, lane)) {
                const uint4 v = rowbuf[c];
                w[k][0] = v.x; w[k][1] = v.y; w[k][2] = v.z; w[k][3] = v.w;
                m2 = max_nan_bf16x2(max_nan_bf16x2(m2, v.x), max_nan_bf16x2(v.y, max_nan_bf16x2(v.z, v.w)));
            }
        }
        __syncwarp();                                               // every lane has its chunks: the buffer is free
        if (row + warps < rows) {
            const uint4* xn = reinterpret_cast<const uint4*>(x + (row + warps) * cols);
            if (UNI) {
#pragma unroll 1
                for (int k = 0; k < (nchunk >> 5); ++k) cp_async16(rowbuf_s + (lane + 32 * k) * 16, xn + lane + 32 * k);
            } else {
                for (int c = lane; c < nchunk; c += 32) cp_async16(rowbuf_s + c * 16, xn + c);
            }
        }
        cp_async_commit();
        float m = sq_nan_max(bf_lo(m2), bf_hi(m2));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) m = sq_nan_max(m, __shfl_xor_sync(0xffffffffu, m, s));
        const uint32_t mb = __float_as_uint(m) >> 16;
        const uint32_t mm2 = mb | (mb << 16);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t dmax2 = 0;                                         // packed maximum of |d|
        const char* tabb = reinterpret_cast<const char*>(tab);
#pragma unroll
        for (int k = 0; k < kSqMaxVec; ++k) {
            if (inside(k, lane)) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t d2 = sub_bf16x2(w[k][i], mm2) & 0x7fff7fffu;       // |d|: d <= 0 (NaN stays NaN)
                    dmax2 = vmax_u16x2(dmax2, d2);
                    const uint32_t off2 = d2 << 1;                  // byte offsets into the table, one per lane
                    const uint32_t e_lo = *reinterpret_cast<const uint16_t*>(tabb + (off2 & 0xffffu));
                    const uint32_t e_hi = *reinterpret_cast<const uint16_t*>(tabb + (off2 >> 16));
                    const uint32_t e2 = __byte_perm(e_lo, e_hi, 0x5410);
                    acc[i] += bf_lo(e2);
                    acc[i] += bf_hi(e2);
                    w[k][i] = e2;
                }
            }
        }
        float accs = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        uint32_t dmax = max(dmax2 & 0xffffu, dmax2 >> 16);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            accs += __shfl_xor_sync(0xffffffffu, accs, s);
            dmax = max(dmax, __shfl_xor_sync(0xffffffffu, dmax, s));
        }
        // A nonzero e below 2^-115 (exponent field under 12) can only come from |d| > 79.5 (pattern 0x429f).
        // Rows with such a |d| (masked scores at -inf among them) are searched for one: packed minimum of
        // (e - 1), zeros wrap to the top.
        uint32_t tmin = 0xffffu;
        if (dmax >= 0x429fu) {
            uint32_t tiny = 0xffffffffu;
#pragma unroll
            for (int k = 0; k < kSqMaxVec; ++k) {
                if (inside(k, lane)) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) tiny = vmin_u16x2(tiny, w[k][i] - 0x00010001u);
                }
            }
            tmin = min(tiny & 0xffffu, tiny >> 16);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) tmin = min(tmin, __shfl_xor_sync(0xffffffffu, tmin, s));
        }
        const float sum = rb(accs);
        const float rsum = __frcp_rn(sum);
        // e / sum is computed as e * (1 / sum) with 1 / sum correctly rounded: e and sum have 8 significant bits
        // each, so e / sum is never a bfloat16 rounding midpoint and stays at least 2^-17 (relative) away from
        // one, far more than the 2^-23 error of the product.  Only quotients in bfloat16's subnormal range
        // (e < 2^-115, i.e. a nonzero e with an exponent field below 12) need the exact division; such rows
        // are detected through `tmin` and take the slow form for all their elements.
        const bool exact_div = tmin < (12u << 7);
        int64_t srow = 0;
        if (CK != CK_NONE) {
            if (a.sf_gemm) {
                const int64_t batch = row / a.sf_rpb, rr = row - batch * a.sf_rpb;
                srow = ((batch * r128 + (rr >> 7)) * kb4) * 512 + (rr & 31) * 16 + ((rr & 127) >> 5) * 4;
            } else {
                srow = row * a.nblk;
            }
        }
#pragma unroll
        for (int k = 0; k < kSqMaxVec; ++k) {
            const int c = lane + 32 * k;
            if (32 * k >= nchunk) break;                           // warp-uniform: nothing left in this row
            // all 32 lanes take part in the shuffles below; lanes past the row carry zeros
            uint32_t p[4] = {0, 0, 0, 0};
            if (UNI || c < nchunk) {
                if (!exact_div) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) p[i] = rb2(bf_lo(w[k][i]) * rsum, bf_hi(w[k][i]) * rsum);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) p[i] = rb2(__fdiv_rn(bf_lo(w[k][i]), sum), __fdiv_rn(bf_hi(w[k][i]), sum));
                }
                if (WANT_P) reinterpret_cast<uint4*>(out + row * cols)[c] = make_uint4(p[0], p[1], p[2], p[3]);
            }
            if (CK == CK_NONE) continue;
            // ---- MX packing of the 8 probabilities this lane holds (block = 4 neighbouring lanes) ----
            // probabilities are non-negative (or NaN, whose patterns sort above every number): integer maxima
            const uint32_t b2 = vmax_u16x2(vmax_u16x2(p[0], p[1]), vmax_u16x2(p[2], p[3])) & 0x7fff7fffu;
            uint32_t bm = max(b2 & 0xffffu, b2 >> 16);
            bm = max(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            bm = max(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
            const FastBlock fb = fast_block(bm >> 7, a);
            // one vote per chunk: when every block of the warp's chunk has a fast-path maximum the packing is
            // straight-line code (no divergent branch)
            const bool all_fast = use_direct<false, CK == CK_NONE ? CK_E4M3 : CK, MODE>(a) &&
                                  __all_sync(0xffffffffu, fb.ok || (!UNI && c >= nchunk));
            if (!UNI && c >= nchunk) continue;
            const int blk = c >> 2;
            if (all_fast) {
                if ((lane & 3) == 0)
                    a.scales[a.sf_gemm ? srow + (int64_t)(blk >> 2) * 512 + (blk & 3) : srow + blk] = (uint8_t)fb.E;
                reinterpret_cast<uint2*>(a.codes + row * cols)[c] =
                    code_oct_direct<CK == CK_NONE ? CK_E4M3 : CK>(p, direct_factor<MODE>(fb.inv), a.direct);
                continue;
            }
            if ((lane & 3) == 0) {
                const int64_t sidx = a.sf_gemm ? srow + (int64_t)(blk >> 2) * 512 + (blk & 3) : srow + blk;
                a.scales[sidx] = (uint8_t)(fb.ok ? fb.E : (uint32_t)scale_exp_from_absmax(bm << 16, a.fmt.emax_elem, a.scale_emax));
            }
            uint32_t cw[2] = {0, 0};
            if (fb.ok && use_direct<false, CK == CK_NONE ? CK_E4M3 : CK, MODE>(a)) {
                const float cf = direct_factor<MODE>(fb.inv);
                const uint2 c8 = code_oct_direct<CK == CK_NONE ? CK_E4M3 : CK>(p, cf, a.direct);
                cw[0] = c8.x; cw[1] = c8.y;
            } else if (fb.ok) {
                const uint32_t mp = a.fp_mp_base + fb.E * 0x00800080u;
                float q[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) (void)quant_pair_bf16<MODE, true>(p[i], fb.cmin, fb.cmin, mp, a.fmt, q[2 * i], q[2 * i + 1]);
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    cw[i] = code_quad<CK == CK_NONE ? CK_E4M3 : CK>(q[4 * i] * fb.inv, q[4 * i + 1] * fb.inv, q[4 * i + 2] * fb.inv,
                                                                    q[4 * i + 3] * fb.inv, p[2 * i], p[2 * i + 1]);
            } else {
                // tiny, zero or NaN block maximum: scaled-domain rounding
                const BlockScale bs = block_scale(bm << 16, a);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t xb = (i & 1) ? (p[i >> 1] & 0xffff0000u) : (p[i >> 1] << 16);
                    const float q = quant_abs<MODE>(xb, bs, a.fmt);
                    cw[i >> 2] |= (code_pair<CK == CK_NONE ? CK_E4M3 : CK>(q, 0.f, xb >> 16) & 0xffu) << (8 * (i & 3));
                }
            }
            reinterpret_cast<uint2*>(a.codes + row * cols)[c] = make_uint2(cw[0], cw[1]);
        }
    }
    cp_async_wait_all();
}

template <int MODE, int CK, bool WANT_P, bool UNI>
static int launch_softmax_rows_uni(const MxArgs& a, const uint16_t* table, int64_t rows, int cols, cudaStream_t st) {
    auto k = softmax_rows_kernel<MODE, CK, WANT_P, UNI>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSqSmemBytes) != cudaSuccess) {
        cudaGetLastError();
        return MXQ_ERR_CUDA;
    }
    const int64_t ctas = (rows + kSqWarps - 1) / kSqWarps;
    k<<<(unsigned)std::min<int64_t>(ctas, sm_count()), kSqThreads, kSqSmemBytes, st>>>(a, table, rows, cols);
    return check_launch();
}

template <int MODE, int CK, bool WANT_P>
static int launch_softmax_rows_one(const MxArgs& a, const uint16_t* table, int64_t rows, int cols, cudaStream_t st) {
    return cols % 256 == 0 ? launch_softmax_rows_uni<MODE, CK, WANT_P, true>(a, table, rows, cols, st)
                           : launch_softmax_rows_uni<MODE, CK, WANT_P, false>(a, table, rows, cols, st);
}

template <int MODE>
static int launch_softmax_quantize(const MxArgs& a, const uint16_t* table, int64_t rows, int cols, cudaStream_t st) {
    const bool e5 = a.fmt.ebits == 5;
    const bool narrow = !e5 && MODE != RZ && a.direct >= 2;           // fp6 / fp4: see CK_E4M3N
    if (a.out) return e5 ? launch_softmax_rows_one<MODE, CK_E5M2, true>(a, table, rows, cols, st)
                         : narrow ? launch_softmax_rows_one<MODE, CK_E4M3N, true>(a, table, rows, cols, st)
                                  : launch_softmax_rows_one<MODE, CK_E4M3, true>(a, table, rows, cols, st);
    return e5 ? launch_softmax_rows_one<MODE, CK_E5M2, false>(a, table, rows, cols, st)
              : narrow ? launch_softmax_rows_one<MODE, CK_E4M3N, false>(a, table, rows, cols, st)
                       : launch_softmax_rows_one<MODE, CK_E4M3, false>(a, table, rows, cols, st);
}

// Softmax alone through the same kernel (called by mxq_softmax_bf16 for large inputs).
int softmax_rows_large(const void* x, void* out, int64_t rows, int64_t cols, cudaStream_t st) {
    const uint16_t* table = exp_table();
    if (!table) return MXQ_ERR_CUDA;
    MxArgs a;
    memset(&a, 0, sizeof(a));
    a.in = x; a.out = out;
    a.pre = rows; a.axis_len = cols; a.post = 1; a.block = 32; a.nblk = cols / 32; a.sf_rpb = rows;
    return launch_softmax_rows_one<RN_EVEN, CK_NONE, true>(a, table, rows, (int)cols, st);
}
}  // namespace mxq

extern "C" int mxq_softmax_quantize_mx(const void* x, void* probs, void* codes, void* scales, int64_t rows, int64_t cols,
                                       int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                                       int flush_fp32_subnorms, int rmode, int flags, int64_t sf_rows_per_batch,
                                       void* stream) {
    using namespace mxq;
    if (rows < 0 || cols < 0) return MXQ_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return MXQ_OK;
    if (!x || !codes || !scales) return MXQ_ERR_BAD_ARG;
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_EVEN) return MXQ_ERR_UNSUPPORTED;
    if (scale_bits < 0 || scale_bits > 8) return MXQ_ERR_BAD_ARG;
    if (elem_ebits < 1 || elem_ebits > 5 || elem_mbits < 3 || elem_mbits > 8) return MXQ_ERR_UNSUPPORTED;   // fp formats with a one-byte container
    if (cols % 32 != 0 || cols > kSqMaxVec * 256 || (flags & MXQ_CODES_TRANSPOSED)) return MXQ_ERR_UNSUPPORTED;
    if (!aligned16(x) || (probs && !aligned16(probs)) || !aligned8(codes)) return MXQ_ERR_ALIGN;
    MxArgs a;
    a.in = x; a.in2 = nullptr; a.sig_table = nullptr; a.out = probs; a.codes = (uint8_t*)codes; a.scales = (uint8_t*)scales;
    a.noise = nullptr;
    a.pre = rows; a.axis_len = cols; a.post = 1;
    a.block = 32;
    a.nblk = cols / 32;
    if (scale_bits == 0) scale_bits = 8;
    a.scale_emax = (1 << (scale_bits - 1)) - 1;
    a.flush = flush_fp32_subnorms != 0;
    a.mode = rmode;
    a.transposed = 0;
    a.sf_gemm = (flags & MXQ_SCALES_GEMM_LAYOUT) != 0;
    a.sf_rpb = sf_rows_per_batch > 0 ? sf_rows_per_batch : rows;
    a.div_nblk.set((uint32_t)a.nblk);
    a.div_rpb.set((uint32_t)std::min<int64_t>(a.sf_rpb, 0xffffffffLL));
    a.fmt = make_fmt(elem_ebits, elem_mbits, elem_max_norm, rmode);
    set_fast_consts(a);
    g_launch_count[1].fetch_add(1, std::memory_order_relaxed);
    const uint16_t* table = exp_table();
    if (!table) return MXQ_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    switch (rmode) {
        case RN_AWAY: return launch_softmax_quantize<RN_AWAY>(a, table, rows, (int)cols, st);
        case RZ:      return launch_softmax_quantize<RZ>(a, table, rows, (int)cols, st);
        default:      return launch_softmax_quantize<RN_EVEN>(a, table, rows, (int)cols, st);
    }
}
