// Fused bfloat16 vector chains (sm_100a): SiLU (optionally times a second
// tensor) and RMSNorm.
//
// The reference builds these layers from single vector operations, each
// followed by a rounding to the bfloat format (mx/vector_ops.py:1-130,
// mx/activations.py:418-455, mx/layernorm.py:98-200); on bfloat16 CUDA tensors
// with bfloat = 16 every such step is one elementwise kernel over the whole
// tensor that computes in fp32 and rounds the result to bfloat16
// (round-to-nearest-even).  The kernels here run the same chain of fp32
// operations and bfloat16 roundings per element in registers, so a layer reads
// its inputs once and writes its outputs once: HBM-bound streaming kernels,
// 16-byte accesses, grid sized from the SM count.
#include "mxq_common.cuh"
#include "vector_math.cuh"
#include <cuda_bf16.h>
#include <algorithm>
#include <mutex>
#include <math_constants.h>

namespace mxq {

// Tables over all 65536 bfloat16 bit patterns, built on first use by the very operations they replace:
// WHICH = 0: the sigmoid chain of silu_chain; WHICH = 1: exp rounded to bfloat16 (the softmax numerator).
template <int WHICH>
__global__ void build_table_kernel(uint16_t* tab) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    const float q = __uint_as_float(i << 16);
    float s, y;
    if (WHICH == 0) silu_chain(q, s, y);
    else s = rb(expf(q));
    tab[i] = (uint16_t)(__float_as_uint(s) >> 16);
}

template <int WHICH>
static const uint16_t* bf16_table() {
    static uint16_t* tabs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tabs[dev]) {
        uint16_t* t = nullptr;
        if (cudaMalloc(&t, 65536 * sizeof(uint16_t)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        build_table_kernel<WHICH><<<65536 / 256, 256>>>(t);
        if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(0) != cudaSuccess) { cudaFree(t); return nullptr; }
        tabs[dev] = t;
    }
    return tabs[dev];
}

const uint16_t* sigmoid_table() { return bf16_table<0>(); }
const uint16_t* exp_table() { return bf16_table<1>(); }
int softmax_rows_large(const void* x, void* out, int64_t rows, int64_t cols, cudaStream_t st);

constexpr int kVecThreads = 256;

template <bool HAS_UP, bool WANT_SIG>
__global__ void __launch_bounds__(kVecThreads)
silu_bf16_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out,
                 uint4* __restrict__ sig, const int64_t nvec, const int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kVecThreads;
    for (int64_t v = (int64_t)blockIdx.x * kVecThreads + threadIdx.x; v < nvec; v += stride) {
        const uint4 g4 = __ldg(gate + v);
        uint4 u4 = make_uint4(0, 0, 0, 0);
        if (HAS_UP) u4 = __ldg(up + v);
        const uint32_t g[4] = {g4.x, g4.y, g4.z, g4.w};
        const uint32_t u[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t o[4], sg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float s0, y0, s1, y1;
            silu_chain(bf_lo(g[i]), s0, y0);
            silu_chain(bf_hi(g[i]), s1, y1);
            if (HAS_UP) { y0 = rb(y0 * bf_lo(u[i])); y1 = rb(y1 * bf_hi(u[i])); }
            o[i] = pack_bf(y0, y1);
            sg[i] = pack_bf(s0, s1);
        }
        out[v] = make_uint4(o[0], o[1], o[2], o[3]);
        if (WANT_SIG) sig[v] = make_uint4(sg[0], sg[1], sg[2], sg[3]);
    }
    // ragged tail (n not a multiple of 8): one thread per element
    const int64_t t = nvec * 8 + (int64_t)blockIdx.x * kVecThreads + threadIdx.x;
    if (t < n) {
        const uint16_t* g = reinterpret_cast<const uint16_t*>(gate);
        float s, y;
        silu_chain(__uint_as_float((uint32_t)g[t] << 16), s, y);
        if (HAS_UP) y = rb(y * __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(up)[t] << 16));
        reinterpret_cast<uint16_t*>(out)[t] = (uint16_t)(__float_as_uint(y) >> 16);
        if (WANT_SIG) reinterpret_cast<uint16_t*>(sig)[t] = (uint16_t)(__float_as_uint(s) >> 16);
    }
}

// The same chain for large tensors: the sigmoid part is a pure function of the 16 input bits
// and is read from the table of sigmoid_table() held in shared memory (persistent CTAs, one
// table load each); the multiplications and their roundings are done as above.
constexpr int kTabThreads = 1024;
constexpr int kTabBytes = 65536 * 2;

template <bool HAS_UP, bool WANT_SIG>
__global__ void __launch_bounds__(kTabThreads)
silu_tab_bf16_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out,
                     uint4* __restrict__ sig, const uint16_t* __restrict__ table, const int64_t nvec) {
    extern __shared__ uint4 tab_smem[];
    for (int i = threadIdx.x; i < kTabBytes / 16; i += kTabThreads) tab_smem[i] = __ldg(reinterpret_cast<const uint4*>(table) + i);
    __syncthreads();
    const uint16_t* tab = reinterpret_cast<const uint16_t*>(tab_smem);
    const int64_t stride = (int64_t)gridDim.x * kTabThreads;
    for (int64_t v = (int64_t)blockIdx.x * kTabThreads + threadIdx.x; v < nvec; v += stride) {
        const uint4 g4 = __ldg(gate + v);
        uint4 u4 = make_uint4(0, 0, 0, 0);
        if (HAS_UP) u4 = __ldg(up + v);
        const uint32_t g[4] = {g4.x, g4.y, g4.z, g4.w};
        const uint32_t u[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t o[4], sg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t b0 = tab[g[i] & 0xffffu], b1 = tab[g[i] >> 16];
            sg[i] = b0 | (b1 << 16);
            uint32_t y = mul_bf16x2(g[i], sg[i]);                   // gate * sigmoid, rounded
            if (HAS_UP) y = mul_bf16x2(y, u[i]);                    // ... * up, rounded
            o[i] = y;
        }
        out[v] = make_uint4(o[0], o[1], o[2], o[3]);
        if (WANT_SIG) sig[v] = make_uint4(sg[0], sg[1], sg[2], sg[3]);
    }
}

template <bool HAS_UP, bool WANT_SIG>
static int launch_silu_tab(const uint4* g, const uint4* u, uint4* o, uint4* s, const uint16_t* table, int64_t nvec,
                           cudaStream_t st) {
    auto kern = silu_tab_bf16_kernel<HAS_UP, WANT_SIG>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTabBytes) != cudaSuccess) {
        cudaGetLastError();
        return MXQ_ERR_CUDA;
    }
    const unsigned grid = (unsigned)std::min<int64_t>((nvec + kTabThreads - 1) / kTabThreads, sm_count());
    kern<<<grid, kTabThreads, kTabBytes, st>>>(g, u, o, s, table, nvec);
    return check_launch();
}

// RMSNorm of one row per CTA (mx/layernorm.py:113-125):
//   ms = mean(x*x), r = 1/sqrt(ms + eps), xn = x * r, y = w * xn + b
// with a bfloat16 rounding after every operation; the row sum is accumulated in
// fp32 and rounded once, like a library reduction.  The row is read twice, the
// second time from cache.
constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bf16_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                    uint16_t* __restrict__ out, uint16_t* __restrict__ xnorm, uint16_t* __restrict__ rinv,
                    const int64_t rows, const int64_t hidden, const float inv_hidden, const float eps) {
    __shared__ float part[kNormThreads / 32];
    __shared__ float r_shared;
    const bool vec = (hidden & 7) == 0;
    // rows of up to kNormKeep * 256 vectors stay in registers between the two passes (one read of x)
    constexpr int kNormKeep = 4;
    const bool keep = vec && hidden / 8 <= (int64_t)kNormKeep * kNormThreads;
    uint4 kept[kNormKeep];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint16_t* xr = x + row * hidden;
        float acc = 0.f;
        if (keep) {
            const uint4* xv0 = reinterpret_cast<const uint4*>(xr);
#pragma unroll
            for (int k = 0; k < kNormKeep; ++k) {
                const int64_t i = threadIdx.x + (int64_t)k * kNormThreads;
                kept[k] = i < hidden / 8 ? __ldg(xv0 + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int k = 0; k < kNormKeep; ++k) {
                const uint32_t q[4] = {kept[k].x, kept[k].y, kept[k].z, kept[k].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t sq = mul_bf16x2(q[j], q[j]);
                    acc += bf_lo(sq);
                    acc += bf_hi(sq);
                }
            }
        } else if (vec) {
            const uint4* xv = reinterpret_cast<const uint4*>(xr);
            for (int64_t i = threadIdx.x; i < hidden / 8; i += kNormThreads) {
                const uint4 v = __ldg(xv + i);
                const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t sq = mul_bf16x2(q[k], q[k]);
                    acc += bf_lo(sq);
                    acc += bf_hi(sq);
                }
            }
        } else {
            for (int64_t i = threadIdx.x; i < hidden; i += kNormThreads) {
                const float v = __uint_as_float((uint32_t)xr[i] << 16);
                acc += rb(v * v);
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.f;
#pragma unroll
            for (int k = 0; k < kNormThreads / 32; ++k) tot += part[k];
            const float sum = rb(tot);
            const float ms = rb(sum * inv_hidden);           // division by a host scalar = multiply by its reciprocal
            const float t = rb(ms + eps);
            const float r = rb(sqrtf(t));
            const float ri = rb(__frcp_rn(r));               // = 1.0f / r (both correctly rounded)
            r_shared = ri;
            if (rinv) rinv[row] = (uint16_t)(__float_as_uint(ri) >> 16);
        }
        __syncthreads();
        const float ri = r_shared;
        const uint32_t ri2 = (__float_as_uint(ri) >> 16) * 0x10001u;         // (ri, ri) as a packed pair
        uint16_t* orow = out + row * hidden;
        uint16_t* nrow = xnorm ? xnorm + row * hidden : nullptr;
        if (vec) {
            const uint4* xv = reinterpret_cast<const uint4*>(xr);
            const uint4* wv = reinterpret_cast<const uint4*>(w);
            const uint4* bv = reinterpret_cast<const uint4*>(b);
            const int64_t nv = hidden / 8;
#pragma unroll 1
            for (int64_t i = threadIdx.x, k = 0; i < nv; i += kNormThreads, ++k) {
                uint4 v;
                if (keep) v = k == 0 ? kept[0] : k == 1 ? kept[1] : k == 2 ? kept[2] : kept[3];
                else v = __ldg(xv + i);
                const uint4 ww = __ldg(wv + i);
                uint4 bb = make_uint4(0, 0, 0, 0);
                if (b) bb = __ldg(bv + i);
                const uint32_t q[4] = {v.x, v.y, v.z, v.w}, wq[4] = {ww.x, ww.y, ww.z, ww.w}, bq[4] = {bb.x, bb.y, bb.z, bb.w};
                uint32_t o[4], nn[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t n2 = mul_bf16x2(q[k], ri2);
                    uint32_t y2 = mul_bf16x2(wq[k], n2);
                    if (b) y2 = add_bf16x2(y2, bq[k]);
                    o[k] = y2;
                    nn[k] = n2;
                }
                reinterpret_cast<uint4*>(orow)[i] = make_uint4(o[0], o[1], o[2], o[3]);
                if (nrow) reinterpret_cast<uint4*>(nrow)[i] = make_uint4(nn[0], nn[1], nn[2], nn[3]);
            }
        } else {
            for (int64_t i = threadIdx.x; i < hidden; i += kNormThreads) {
                const float n0 = rb(__uint_as_float((uint32_t)xr[i] << 16) * ri);
                float y0 = rb(__uint_as_float((uint32_t)w[i] << 16) * n0);
                if (b) y0 = rb(y0 + __uint_as_float((uint32_t)b[i] << 16));
                orow[i] = (uint16_t)(__float_as_uint(y0) >> 16);
                if (nrow) nrow[i] = (uint16_t)(__float_as_uint(n0) >> 16);
            }
        }
        __syncthreads();                                      // part / r_shared are reused by the next row
    }
}

// Softmax over the last dimension, one warp per row kept in registers
// (mx/softmax.py:18-41): m = max(x), d = x - m, e = exp(d) (or exp2), s = sum(e),
// y = e / s with a bfloat16 rounding after every step; the row sum is accumulated
// in fp32 and rounded once.  Rows of up to kSmMaxVec * 256 elements.
constexpr int kSmThreads = 256;
constexpr int kSmMaxVec = 8;

__device__ __forceinline__ float nan_max(float a, float b) { return (b > a || b != b) ? b : a; }   // NaN wins, like torch.max

// Small inputs and exp2; large inputs run the persistent kernel of softmax_quantize_mx.cu (exp from a table,
// rows prefetched into shared memory).  The division e / s is done as e * (1/s) with 1/s correctly rounded: e
// and s have 8 significant bits each, so e / s is never a bfloat16 rounding midpoint and stays at least 2^-17
// (relative) away from one, far more than the 2^-23 error of the product, hence the bfloat16 result is the one
// of the exact division; quotients that would round in bfloat16's subnormal range take the exact division.
template <bool EXP2>
__global__ void __launch_bounds__(kSmThreads)
softmax_bf16_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, const int64_t rows, const int cols) {
    constexpr int kThreads = kSmThreads;
    const int lane = threadIdx.x & 31;
    const int nchunk = cols >> 3;
    const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
    for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
        uint32_t w[kSmMaxVec][4];
        float m = -CUDART_INF_F;
#pragma unroll
        for (int k = 0; k < kSmMaxVec; ++k) {
            const int c = lane + 32 * k;
            if (c < nchunk) {
                const uint4 v = __ldg(xr + c);
                w[k][0] = v.x; w[k][1] = v.y; w[k][2] = v.z; w[k][3] = v.w;
#pragma unroll
                for (int i = 0; i < 4; ++i) { m = nan_max(m, bf_lo(w[k][i])); m = nan_max(m, bf_hi(w[k][i])); }
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, s));
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < kSmMaxVec; ++k) {
            if (lane + 32 * k < nchunk) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t d2 = rb2(bf_lo(w[k][i]) - m, bf_hi(w[k][i]) - m);
                    const float d0 = bf_lo(d2), d1 = bf_hi(d2);
                    const uint32_t e2 = rb2(EXP2 ? exp2f(d0) : expf(d0), EXP2 ? exp2f(d1) : expf(d1));
                    acc += bf_lo(e2);
                    acc += bf_hi(e2);
                    w[k][i] = e2;
                }
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
        const float sum = rb(acc);
        const float rsum = __frcp_rn(sum);
        uint4* orow = reinterpret_cast<uint4*>(out + row * cols);
#pragma unroll
        for (int k = 0; k < kSmMaxVec; ++k) {
            const int c = lane + 32 * k;
            if (c < nchunk) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float e0 = bf_lo(w[k][i]), e1 = bf_hi(w[k][i]);
                    const float q0 = fabsf(e0) < 1e-30f ? __fdiv_rn(e0, sum) : e0 * rsum;
                    const float q1 = fabsf(e1) < 1e-30f ? __fdiv_rn(e1, sum) : e1 * rsum;
                    o[i] = rb2(q0, q1);
                }
                orow[c] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

}  // namespace mxq

extern "C" int mxq_silu_bf16(const void* gate, const void* up, void* out, void* sig, int64_t n, void* stream) {
    using namespace mxq;
    if (n < 0) return MXQ_ERR_BAD_ARG;
    if (n == 0) return MXQ_OK;
    if (!gate || !out) return MXQ_ERR_BAD_ARG;
    if (!aligned16(gate) || !aligned16(out) || (up && !aligned16(up)) || (sig && !aligned16(sig))) return MXQ_ERR_BAD_ARG;
    const int64_t nvec = n / 8;
    const int64_t want = std::max<int64_t>((nvec + kVecThreads - 1) / kVecThreads, ((n - nvec * 8) + kVecThreads - 1) / kVecThreads);
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)sm_count() * 16));
    cudaStream_t st = (cudaStream_t)stream;
    const uint4 *g = (const uint4*)gate, *u = (const uint4*)up;
    uint4 *o = (uint4*)out, *s = (uint4*)sig;
    if (n % 8 == 0 && n >= (int64_t)1 << 22) {
        // large tensors: table-driven kernel (one 128 KB table load per SM pays off)
        const uint16_t* table = sigmoid_table();
        if (table) {
            if (up && sig) return launch_silu_tab<true, true>(g, u, o, s, table, nvec, st);
            if (up) return launch_silu_tab<true, false>(g, u, o, s, table, nvec, st);
            if (sig) return launch_silu_tab<false, true>(g, u, o, s, table, nvec, st);
            return launch_silu_tab<false, false>(g, u, o, s, table, nvec, st);
        }
    }
    if (up && sig) silu_bf16_kernel<true, true><<<grid, kVecThreads, 0, st>>>(g, u, o, s, nvec, n);
    else if (up) silu_bf16_kernel<true, false><<<grid, kVecThreads, 0, st>>>(g, u, o, s, nvec, n);
    else if (sig) silu_bf16_kernel<false, true><<<grid, kVecThreads, 0, st>>>(g, u, o, s, nvec, n);
    else silu_bf16_kernel<false, false><<<grid, kVecThreads, 0, st>>>(g, u, o, s, nvec, n);
    return check_launch();
}

extern "C" int mxq_rmsnorm_bf16(const void* x, const void* weight, const void* bias, void* out, void* x_norm,
                                void* rms_inv, int64_t rows, int64_t hidden, float eps, void* stream) {
    using namespace mxq;
    if (rows < 0 || hidden < 0) return MXQ_ERR_BAD_ARG;
    if (rows == 0 || hidden == 0) return MXQ_OK;
    if (!x || !weight || !out) return MXQ_ERR_BAD_ARG;
    if ((hidden & 7) == 0 && (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (bias && !aligned16(bias)) ||
                              (x_norm && !aligned16(x_norm))))
        return MXQ_ERR_BAD_ARG;
    const unsigned grid = (unsigned)std::min<int64_t>(rows, (int64_t)0x7fffffff);
    rmsnorm_bf16_kernel<<<grid, kNormThreads, 0, (cudaStream_t)stream>>>(
        (const uint16_t*)x, (const uint16_t*)weight, (const uint16_t*)bias, (uint16_t*)out, (uint16_t*)x_norm,
        (uint16_t*)rms_inv, rows, hidden, 1.0f / (float)hidden, eps);
    return check_launch();
}

extern "C" int mxq_softmax_bf16(const void* x, void* out, int64_t rows, int64_t cols, int use_exp2, void* stream) {
    using namespace mxq;
    if (rows < 0 || cols < 0) return MXQ_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return MXQ_OK;
    if (!x || !out) return MXQ_ERR_BAD_ARG;
    if (cols % 8 != 0 || cols > kSmMaxVec * 256) return MXQ_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(out)) return MXQ_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const uint16_t* xs = (const uint16_t*)x;
    uint16_t* os = (uint16_t*)out;
    if (!use_exp2 && rows * cols >= ((int64_t)1 << 22)) {
        // large inputs: the persistent kernel with the exp table and row prefetch (softmax_quantize_mx.cu)
        const int rc = softmax_rows_large(x, out, rows, cols, st);
        if (rc == MXQ_OK) return rc;
        cudaGetLastError();
    }
    const int64_t ctas = (rows + kSmThreads / 32 - 1) / (kSmThreads / 32);
    const unsigned grid = (unsigned)std::min<int64_t>(ctas, (int64_t)sm_count() * 8);
    if (use_exp2) softmax_bf16_kernel<true><<<grid, kSmThreads, 0, st>>>(xs, os, rows, (int)cols);
    else softmax_bf16_kernel<false><<<grid, kSmThreads, 0, st>>>(xs, os, rows, (int)cols);
    return check_launch();
}
