// SiLU(gate) * up fused into the MX packing of the product (sm_100a).
//
// In a gated feed-forward block the reference computes silu(gate), multiplies
// by up (mx/activations.py:418-439, mx/simd_ops.py:189-237: one elementwise
// kernel per vector operation) and then MX-quantizes the product along the
// hidden axis as the left operand of the down projection (mx/linear.py:75-83).
// Here the last-axis MX kernel computes the product in registers, with the same
// fp32 operations and bfloat16 roundings, and writes only the packed operand
// (1 code byte per element + E8M0 scales): 4 B read + 1 1/32 B written per
// element instead of 4 + 2 written, 2 read, 1 1/32 written.
#include "quantize_mx_impl.cuh"

namespace mxq {
template <int MODE>
static int launch_swiglu(const MxArgs& a, int64_t nvec, cudaStream_t st) {
    const int64_t tile = (int64_t)kSwigluThreads * kLastBfUnroll;
    const int64_t ntiles = (nvec + tile - 1) / tile;
    const unsigned grid = (unsigned)std::min<int64_t>(ntiles, sm_count());       // persistent: one CTA per SM
    const int rl = a.sf_gemm && a.nblk % 32 == 0;
    constexpr int kTabBytes = 65536 * 2;
    auto k5 = mx_lastaxis_bf16_kernel<MODE, false, CK_E5M2, 1>;
    auto k4 = mx_lastaxis_bf16_kernel<MODE, false, CK_E4M3, 1>;
    auto kern = a.fmt.ebits == 5 ? k5 : k4;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTabBytes) != cudaSuccess) {
        cudaGetLastError();
        return MXQ_ERR_CUDA;
    }
    kern<<<grid, kSwigluThreads, kTabBytes, st>>>(a, nvec, 4, rl);
    return check_launch();
}
}  // namespace mxq

extern "C" int mxq_swiglu_quantize_mx(const void* gate, const void* up, void* codes, void* scales, int64_t rows,
                                      int64_t K, int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                                      int flush_fp32_subnorms, int rmode, int flags, int64_t sf_rows_per_batch,
                                      void* stream) {
    using namespace mxq;
    if (rows < 0 || K < 0) return MXQ_ERR_BAD_ARG;
    if (rows == 0 || K == 0) return MXQ_OK;
    if (!gate || !up || !codes || !scales) return MXQ_ERR_BAD_ARG;
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_EVEN) return MXQ_ERR_UNSUPPORTED;
    if (scale_bits < 0 || scale_bits > 8) return MXQ_ERR_BAD_ARG;
    if (elem_ebits < 1 || elem_ebits > 5 || elem_mbits < 3 || elem_mbits > 8) return MXQ_ERR_UNSUPPORTED;   // fp formats with a one-byte container
    if (K % 32 != 0 || (flags & MXQ_CODES_TRANSPOSED)) return MXQ_ERR_UNSUPPORTED;
    if (!aligned16(gate) || !aligned16(up) || !aligned8(codes)) return MXQ_ERR_ALIGN;
    if (rows * (K / 32) > 0xffffffffLL) return MXQ_ERR_TOO_LARGE;
    MxArgs a;
    a.sig_table = sigmoid_table();
    if (!a.sig_table) return MXQ_ERR_CUDA;
    a.in = gate; a.in2 = up; a.out = nullptr; a.codes = (uint8_t*)codes; a.scales = (uint8_t*)scales; a.noise = nullptr;
    a.pre = rows; a.axis_len = K; a.post = 1;
    a.block = 32;
    a.nblk = K / 32;
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
    const int64_t nvec = rows * K / 8;
    cudaStream_t st = (cudaStream_t)stream;
    switch (rmode) {
        case RN_AWAY: return launch_swiglu<RN_AWAY>(a, nvec, st);
        case RZ:      return launch_swiglu<RZ>(a, nvec, st);
        default:      return launch_swiglu<RN_EVEN>(a, nvec, st);
    }
}
