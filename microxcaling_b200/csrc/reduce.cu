// Innermost-dimension sum / max of an fp32 [rows, inner] matrix (sm_100a).
//
// HBM-bound streaming reduction, one pass, no atomics and no zero-initialised
// output (the reference accumulates rows wider than 1024 with atomics into a
// zeroed buffer, mx/cpp/reduce.cuh:55-81).  Work split by row width:
//   inner <= 1024 : one warp per row, 16-byte loads, shuffle tree;
//   inner  > 1024 : one CTA per row, per-warp partials combined in shared memory.
#include "mxq_common.cuh"
#include <algorithm>
#include <cstring>
#include <math_constants.h>

namespace mxq {

template <bool IS_MAX> struct Op;
template <> struct Op<false> {
    static __device__ __forceinline__ float init() { return 0.f; }
    static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
template <> struct Op<true> {
    static __device__ __forceinline__ float init() { return -CUDART_INF_F; }
    // NaN-propagating max, like torch.max
    static __device__ __forceinline__ float apply(float a, float b) { return (b > a || b != b) ? b : a; }
};

template <bool IS_MAX>
__device__ __forceinline__ float row_partial(const float* row, int64_t inner, int lane, int nlanes, bool vec) {
    float acc = Op<IS_MAX>::init();
    if (vec) {
        const int64_t n4 = inner / 4;
        for (int64_t i = lane; i < n4; i += nlanes) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(row) + i);
            acc = Op<IS_MAX>::apply(acc, v.x); acc = Op<IS_MAX>::apply(acc, v.y);
            acc = Op<IS_MAX>::apply(acc, v.z); acc = Op<IS_MAX>::apply(acc, v.w);
        }
        for (int64_t i = n4 * 4 + lane; i < inner; i += nlanes) acc = Op<IS_MAX>::apply(acc, __ldg(row + i));
    } else {
        for (int64_t i = lane; i < inner; i += nlanes) acc = Op<IS_MAX>::apply(acc, __ldg(row + i));
    }
    return acc;
}

template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = Op<IS_MAX>::apply(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}

constexpr int kRedThreads = 256;

template <bool IS_MAX>
__global__ void __launch_bounds__(kRedThreads)
reduce_warp_rows_kernel(const float* in, float* out, int64_t rows, int64_t inner, bool vec) {
    const int warps_per_cta = kRedThreads / 32;
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows;
         r += (int64_t)gridDim.x * warps_per_cta) {
        float v = row_partial<IS_MAX>(in + r * inner, inner, lane, 32, vec);
        v = warp_reduce<IS_MAX>(v);
        if (lane == 0) out[r] = v;
    }
}

template <bool IS_MAX>
__global__ void __launch_bounds__(kRedThreads)
reduce_cta_rows_kernel(const float* in, float* out, int64_t rows, int64_t inner, bool vec) {
    __shared__ float part[kRedThreads / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float v = row_partial<IS_MAX>(in + r * inner, inner, threadIdx.x, kRedThreads, vec);
        v = warp_reduce<IS_MAX>(v);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x < 32) {
            float w = threadIdx.x < kRedThreads / 32 ? part[threadIdx.x] : Op<IS_MAX>::init();
            w = warp_reduce<IS_MAX>(w);
            if (threadIdx.x == 0) out[r] = w;
        }
        __syncthreads();
    }
}

template <bool IS_MAX>
static int reduce_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream) {
    if (rows < 0 || inner < 0) return MXQ_ERR_BAD_ARG;
    if (rows == 0) return MXQ_OK;
    if (!in || !out || inner == 0) return MXQ_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = aligned16(in) && (inner % 4 == 0);
    if (inner <= 1024) {
        const int64_t need = (rows + kRedThreads / 32 - 1) / (kRedThreads / 32);
        const int grid = (int)std::min<int64_t>(need, (int64_t)sm_count() * 32);
        reduce_warp_rows_kernel<IS_MAX><<<grid, kRedThreads, 0, st>>>((const float*)in, (float*)out, rows, inner, vec);
    } else {
        const int grid = (int)std::min<int64_t>(rows, (int64_t)sm_count() * 16);
        reduce_cta_rows_kernel<IS_MAX><<<grid, kRedThreads, 0, st>>>((const float*)in, (float*)out, rows, inner, vec);
    }
    return check_launch();
}

}  // namespace mxq

extern "C" int mxq_reduce_sum_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream) {
    return mxq::reduce_inner<false>(in, out, rows, inner, stream);
}
extern "C" int mxq_reduce_max_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream) {
    return mxq::reduce_inner<true>(in, out, rows, inner, stream);
}

// ---------------------------------------------------------------------------
// Sum of n fp32 slabs of equal size, added in slab order (the reduction step
// after a scattering GEMM: slab s holds the partial sums rank s produced).
// ---------------------------------------------------------------------------
namespace mxq {
constexpr int kSumThreads = 256;
__global__ void __launch_bounds__(kSumThreads)
sum_slabs_kernel(const float4* __restrict__ slabs, float4* __restrict__ out, const int n_slabs, const int64_t vec_per_slab) {
    const int64_t stride = (int64_t)gridDim.x * kSumThreads;
    for (int64_t i = (int64_t)blockIdx.x * kSumThreads + threadIdx.x; i < vec_per_slab; i += stride) {
        float4 acc = __ldg(slabs + i);
        for (int s = 1; s < n_slabs; ++s) {
            const float4 v = __ldg(slabs + (int64_t)s * vec_per_slab + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        out[i] = acc;
    }
}
}  // namespace mxq

extern "C" int mxq_sum_slabs_f32(const void* slabs, int n_slabs, int64_t elems_per_slab, void* out, void* stream) {
    using namespace mxq;
    if (n_slabs <= 0 || elems_per_slab < 0) return MXQ_ERR_BAD_ARG;
    if (elems_per_slab == 0) return MXQ_OK;
    if (!slabs || !out) return MXQ_ERR_BAD_ARG;
    if (elems_per_slab % 4 != 0 || !aligned16(slabs) || !aligned16(out)) return MXQ_ERR_ALIGN;
    const int64_t nvec = elems_per_slab / 4;
    const unsigned grid = (unsigned)std::min<int64_t>((nvec + kSumThreads - 1) / kSumThreads, (int64_t)sm_count() * 16);
    sum_slabs_kernel<<<grid, kSumThreads, 0, (cudaStream_t)stream>>>((const float4*)slabs, (float4*)out, n_slabs, nvec);
    return check_launch();
}
