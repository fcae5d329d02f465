// Forward of an MX linear layer with pre-packed weights as one C call:
//   y[M,N] = round( MX(x)[M,K] * W[N,K]^T (+ bias) )
// The activations are MX-quantized along K into a packed operand (codes and
// E8M0 scales) held in a caller-provided workspace, then multiplied on the
// block-scaled tensor cores with the output rounding fused.  This is the
// sequence mx/linear.py:62-96 performs on every forward call, minus the weight
// quantization, which an inference caller does once.
#include <algorithm>
#include <initializer_list>
#include <mutex>
#include "mxq_common.cuh"

namespace mxq {
int gemm_mx_with_status(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                        void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int a_fmt, int b_fmt,
                        int out_dtype, int out_bfloat_bits, int out_round, const void* bias, int tile_n,
                        int* status_word, void* stream, void* const* dests = nullptr, int n_dests = 0,
                        int64_t rows_per_dest = 0);

static inline int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

// Layout of the workspace: [0, 256) status word, then codes, then scales.
struct LinearWs {
    int* status;
    uint8_t* codes;
    uint8_t* scales;
    int64_t scale_bytes;
    int64_t total;
};

static LinearWs carve(void* base, int64_t M, int64_t K) {
    LinearWs w;
    uint8_t* p = reinterpret_cast<uint8_t*>(base);
    w.status = reinterpret_cast<int*>(p);
    w.codes = p + 256;
    w.scale_bytes = mxq_sf_bytes(1, M, K);
    w.scales = w.codes + align256(M * K);
    w.total = 256 + align256(M * K) + align256(w.scale_bytes);
    return w;
}

static int linear_fwd_impl(const void* x, int x_dtype, int64_t M, int64_t K, int a_ebits, int a_mbits,
                           float a_max_norm, int a_round, int scale_bits, int flush, const void* w_codes,
                           const void* w_scales, int64_t N, int w_fmt, void* y, int y_dtype, int out_bfloat_bits,
                           int out_round, const void* bias, void* ws_base, void* stream) {
    const LinearWs w = carve(ws_base, M, K);
    cudaStream_t st = (cudaStream_t)stream;
    // scale bytes of padding rows are never written by the quantizer: start them (and the status word) at zero
    if (cudaMemsetAsync(w.status, 0, 256, st) != cudaSuccess) return MXQ_ERR_CUDA;
    if (cudaMemsetAsync(w.scales, 0, (size_t)w.scale_bytes, st) != cudaSuccess) return MXQ_ERR_CUDA;
    int rc = mxq_quantize_mx(x, nullptr, w.codes, w.scales, x_dtype, M, K, 1, 32, scale_bits, a_ebits, a_mbits,
                             a_max_norm, flush, a_round, nullptr, MXQ_SCALES_GEMM_LAYOUT, M, stream);
    if (rc) return rc;
    return gemm_mx_with_status(w.codes, w.scales, w_codes, w_scales, y, 1, M, N, K, a_ebits == 5 ? 1 : 0, w_fmt,
                               y_dtype, out_bfloat_bits, out_round, bias, 0, w.status, stream);
}

static int check_linear_args(const void* x, int64_t M, int64_t K, const void* w_codes, const void* w_scales,
                             int64_t N, void* y, int a_ebits, int a_mbits) {
    if (M < 0 || N < 0 || K < 0) return MXQ_ERR_BAD_ARG;
    if (!x || !w_codes || !w_scales || !y) return MXQ_ERR_BAD_ARG;
    if (K == 0 || K % 128 != 0) return MXQ_ERR_UNSUPPORTED;
    if (a_ebits < 2 || a_ebits > 5 || a_mbits > 5) return MXQ_ERR_UNSUPPORTED;   // needs an fp8 container
    return MXQ_OK;
}
}  // namespace mxq

extern "C" int64_t mxq_linear_workspace_bytes(int64_t M, int64_t K) {
    if (M < 0 || K < 0) return -1;
    return mxq::carve(nullptr, M, K).total;
}

extern "C" int mxq_linear_fwd(const void* x, int x_dtype, int64_t M, int64_t K, int a_ebits, int a_mbits,
                              float a_max_norm, int a_round, int scale_bits, int flush_fp32_subnorms,
                              const void* w_codes, const void* w_scales, int64_t N, int w_fmt, void* y, int y_dtype,
                              int out_bfloat_bits, int out_round, const void* bias, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    using namespace mxq;
    const int rc = check_linear_args(x, M, K, w_codes, w_scales, N, y, a_ebits, a_mbits);
    if (rc) return rc;
    if (M == 0 || N == 0) return MXQ_OK;
    if (!workspace || !aligned16(workspace) || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return MXQ_ERR_ALIGN;
    if (workspace_bytes < carve(nullptr, M, K).total) return MXQ_ERR_TOO_LARGE;
    return linear_fwd_impl(x, x_dtype, M, K, a_ebits, a_mbits, a_max_norm, a_round, scale_bits, flush_fp32_subnorms,
                           w_codes, w_scales, N, w_fmt, y, y_dtype, out_bfloat_bits, out_round, bias, workspace, stream);
}

// ---------------------------------------------------------------------------
// Variant for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the time they need a
// linear layer: a serving process that reserved all device memory for its own
// pools at start-up has nothing left to hand out, and a caller inside a
// latency-bound loop cannot afford the device-wide synchronisation an
// allocation implies.  Such callers also often have no spare buffer to pass as
// the workspace of mxq_linear_fwd.  mxq_linear_fwd_static therefore keeps the
// packed activations and the status word in a fixed array that is part of the
// library image: every GPU that loads libmxq.so holds kLinearStaticBytes of
// device memory for it until the process exits.
//
// In host code `g_linear_scratch` is only a handle for the device symbol, not
// an address a kernel could use; the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and passed on.
// ---------------------------------------------------------------------------
namespace mxq {
constexpr int64_t kLinearStaticMaxElems = int64_t(32) << 20;          // ceil(M/128)*128 * K
constexpr int64_t kLinearStaticBytes = 256 + kLinearStaticMaxElems + kLinearStaticMaxElems / 32;
static __device__ __align__(256) unsigned char g_linear_scratch[kLinearStaticBytes];

static void* linear_static_base(int* rc_out) {
    static void* base[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *rc_out = MXQ_ERR_CUDA; return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!base[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_linear_scratch) != cudaSuccess || !p) { *rc_out = MXQ_ERR_CUDA; return nullptr; }
        base[dev] = p;
    }
    *rc_out = MXQ_OK;
    return base[dev];
}
}  // namespace mxq

extern "C" int64_t mxq_linear_static_max_elems(void) { return mxq::kLinearStaticMaxElems; }

extern "C" int mxq_linear_fwd_static(const void* x, int x_dtype, int64_t M, int64_t K, int a_ebits, int a_mbits,
                                     float a_max_norm, int a_round, int scale_bits, int flush_fp32_subnorms,
                                     const void* w_codes, const void* w_scales, int64_t N, int w_fmt, void* y,
                                     int y_dtype, int out_bfloat_bits, int out_round, const void* bias,
                                     void* stream) {
    using namespace mxq;
    int rc = check_linear_args(x, M, K, w_codes, w_scales, N, y, a_ebits, a_mbits);
    if (rc) return rc;
    if (M == 0 || N == 0) return MXQ_OK;
    const int64_t m_pad = (M + 127) / 128 * 128;
    if (m_pad > kLinearStaticMaxElems / K) return MXQ_ERR_TOO_LARGE;   // ceil(M/128)*128*K beyond the fixed array
    void* base = linear_static_base(&rc);
    if (!base) return rc;
    // The array belongs to the CURRENT device.  A caller whose current device is not the one x and y live
    // on would hand the kernels another GPU's address: refuse that instead of launching.
    int cur = -1;
    cudaPointerAttributes pa;
    if (cudaGetDevice(&cur) != cudaSuccess) return MXQ_ERR_CUDA;
    for (const void* p : {x, (const void*)y, w_codes}) {
        if (cudaPointerGetAttributes(&pa, p) != cudaSuccess) { cudaGetLastError(); return MXQ_ERR_CUDA; }
        if (pa.type == cudaMemoryTypeDevice && pa.device != cur) return MXQ_ERR_BAD_ARG;
    }
    // The array still holds the previous call's packed activations; linear_fwd_impl zeroes the
    // status word and the scale region (its padding rows are read but never written) before use.
    return linear_fwd_impl(x, x_dtype, M, K, a_ebits, a_mbits, a_max_norm, a_round, scale_bits, flush_fp32_subnorms,
                           w_codes, w_scales, N, w_fmt, y, y_dtype, out_bfloat_bits, out_round, bias, base, stream);
}

extern "C" int mxq_linear_static_status(void) {
    int rc = 0;
    void* base = mxq::linear_static_base(&rc);
    if (!base) return rc;
    int v = 0;
    if (cudaMemcpy(&v, base, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MXQ_ERR_CUDA;
    return v;
}
