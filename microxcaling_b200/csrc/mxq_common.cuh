// Shared host/device helpers of the library: status codes, vector load/store
// of the three storage types, launch-size helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include "mxq_math.cuh"
#include "../../include/mxq.h"

namespace mxq {

// The GPU this pool targets has 148 SMs; grids of the persistent kernels are
// sized from the queried SM count, this is only the fallback.
constexpr int kDefaultSMs = 148;

// SM count of the current device, cached per device index.  The cache holds
// plain ints written with the same value by every thread that races on a
// first use, so it needs no lock.
inline int sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kDefaultSMs;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = kDefaultSMs;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// SMs the persistent GEMM kernels may occupy (mxq_gemm_sm_budget); 0 = every SM of the device.
extern std::atomic<int> g_gemm_sm_budget;
inline int gemm_sms() {
    const int all = sm_count(), b = g_gemm_sm_budget.load(std::memory_order_relaxed);
    return (b > 0 && b < all) ? b : all;
}

// Launch statistics of this process (mxq_launch_count): 0 = block-scaled GEMMs, 1 = MX quantizations.
extern std::atomic<int64_t> g_launch_count[2];

inline int check_launch() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MXQ_OK : MXQ_ERR_CUDA;
}

// ---- BYTES-wide vector of storage type DT, unpacked to fp32 bit patterns ---
template <int DT, int BYTES> struct VecIO;

template <int BYTES> struct VecIO<DT_F32, BYTES> {
    static constexpr int N = BYTES / 4;
    static constexpr int ESZ = 4;
    static __device__ __forceinline__ void load(const void* base, int64_t elem, uint32_t (&b)[N]) {
        if (BYTES == 16) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + elem));
            b[0] = v.x; b[1] = v.y; b[N > 2 ? 2 : 0] = v.z; b[N > 3 ? 3 : 0] = v.w;
        } else {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const float*>(base) + elem));
            b[0] = v.x; b[1] = v.y;
        }
    }
    static __device__ __forceinline__ void store(void* base, int64_t elem, const uint32_t (&b)[N]) {
        if (BYTES == 16)
            *reinterpret_cast<uint4*>(reinterpret_cast<float*>(base) + elem) =
                make_uint4(b[0], b[1], b[N > 2 ? 2 : 0], b[N > 3 ? 3 : 0]);
        else
            *reinterpret_cast<uint2*>(reinterpret_cast<float*>(base) + elem) = make_uint2(b[0], b[1]);
    }
};

template <int BYTES> struct VecIO<DT_BF16, BYTES> {
    static constexpr int N = BYTES / 2;
    static constexpr int ESZ = 2;
    static __device__ __forceinline__ void load(const void* base, int64_t elem, uint32_t (&b)[N]) {
        uint32_t w[BYTES / 4];
        if (BYTES == 16) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + elem));
            w[0] = v.x; w[1] = v.y; w[BYTES / 4 > 2 ? 2 : 0] = v.z; w[BYTES / 4 > 3 ? 3 : 0] = v.w;
        } else {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + elem));
            w[0] = v.x; w[1] = v.y;
        }
#pragma unroll
        for (int i = 0; i < BYTES / 4; ++i) { b[2 * i] = w[i] << 16; b[2 * i + 1] = w[i] & 0xffff0000u; }
    }
    // Quantized results of bf16 inputs are bf16 values: keeping the upper
    // halves is exact (and maps the canonical NaN to a bf16 NaN).
    static __device__ __forceinline__ void store(void* base, int64_t elem, const uint32_t (&b)[N]) {
        uint32_t w[BYTES / 4];
#pragma unroll
        for (int i = 0; i < BYTES / 4; ++i) w[i] = __byte_perm(b[2 * i], b[2 * i + 1], 0x7632);
        if (BYTES == 16)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + elem) =
                make_uint4(w[0], w[1], w[BYTES / 4 > 2 ? 2 : 0], w[BYTES / 4 > 3 ? 3 : 0]);
        else
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + elem) = make_uint2(w[0], w[1]);
    }
};

template <int BYTES> struct VecIO<DT_F16, BYTES> {
    static constexpr int N = BYTES / 2;
    static constexpr int ESZ = 2;
    static __device__ __forceinline__ void load(const void* base, int64_t elem, uint32_t (&b)[N]) {
        uint32_t w[BYTES / 4];
        if (BYTES == 16) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + elem));
            w[0] = v.x; w[1] = v.y; w[BYTES / 4 > 2 ? 2 : 0] = v.z; w[BYTES / 4 > 3 ? 3 : 0] = v.w;
        } else {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + elem));
            w[0] = v.x; w[1] = v.y;
        }
#pragma unroll
        for (int i = 0; i < BYTES / 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            b[2 * i] = __float_as_uint(f.x); b[2 * i + 1] = __float_as_uint(f.y);
        }
    }
    // The cast back to half rounds to nearest even, as the reference's
    // `(T)` cast does (mx/cpp/mx.cuh:88); values above 65504 become Inf.
    static __device__ __forceinline__ void store(void* base, int64_t elem, const uint32_t (&b)[N]) {
        uint32_t w[BYTES / 4];
#pragma unroll
        for (int i = 0; i < BYTES / 4; ++i) {
            const __half2 h = __floats2half2_rn(__uint_as_float(b[2 * i]), __uint_as_float(b[2 * i + 1]));
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        if (BYTES == 16)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + elem) =
                make_uint4(w[0], w[1], w[BYTES / 4 > 2 ? 2 : 0], w[BYTES / 4 > 3 ? 3 : 0]);
        else
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + elem) = make_uint2(w[0], w[1]);
    }
};

// scalar access (generic kernels)
template <int DT> __device__ __forceinline__ float load1(const void* base, int64_t i) {
    return Store<DT>::load(reinterpret_cast<const typename Store<DT>::T*>(base)[i]);
}
template <int DT> __device__ __forceinline__ void store1(void* base, int64_t i, float v) {
    reinterpret_cast<typename Store<DT>::T*>(base)[i] = Store<DT>::make(v);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }
inline int dtype_size(int dt) { return dt == DT_F32 ? 4 : 2; }

}  // namespace mxq
