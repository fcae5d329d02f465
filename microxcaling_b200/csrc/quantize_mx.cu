// C entry point of MX block quantization; the kernels live in
// quantize_mx_impl.cuh and are instantiated per storage type in
// quantize_mx_{f32,f16,bf16}.cu.
#include "quantize_mx_impl.cuh"
namespace mxq {
extern template int dispatch_dt<DT_F32>(const MxArgs&, cudaStream_t);
extern template int dispatch_dt<DT_F16>(const MxArgs&, cudaStream_t);
extern template int dispatch_dt<DT_BF16>(const MxArgs&, cudaStream_t);
}  // namespace mxq

extern "C" int mxq_quantize_mx(const void* in, void* out, void* codes, void* scales, int dtype,
                               int64_t pre, int64_t axis_len, int64_t post, int block,
                               int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                               int flush_fp32_subnorms, int rmode, const void* noise, int flags,
                               int64_t sf_rows_per_batch, void* stream) {
    using namespace mxq;
    if (pre < 0 || axis_len < 0 || post < 0) return MXQ_ERR_BAD_ARG;
    if (pre == 0 || axis_len == 0 || post == 0) return MXQ_OK;        // empty tensor: nothing to do
    if (!in || (!out && !codes)) return MXQ_ERR_BAD_ARG;
    if (codes && !scales) return MXQ_ERR_BAD_ARG;
    if (dtype < MXQ_F32 || dtype > MXQ_BF16) return MXQ_ERR_BAD_ARG;
    if (rmode < MXQ_ROUND_NEAREST || rmode > MXQ_ROUND_DITHER) return MXQ_ERR_BAD_ARG;
    if (rmode == MXQ_ROUND_DITHER && !noise) return MXQ_ERR_BAD_ARG;
    if (scale_bits < 0 || scale_bits > 8) return MXQ_ERR_BAD_ARG;
    if (elem_mbits < 2 || elem_mbits > 25 || elem_ebits < 0 || elem_ebits > 8) return MXQ_ERR_BAD_ARG;
    if (codes && elem_mbits > 8) return MXQ_ERR_UNSUPPORTED;           // no one-byte container
    if (block <= 0 || block > axis_len) block = (int)std::min<int64_t>(axis_len, 0x7fffffff);
    MxArgs a;
    a.in = in; a.in2 = nullptr; a.sig_table = nullptr; a.out = out; a.codes = (uint8_t*)codes; a.scales = (uint8_t*)scales;
    a.noise = (const float*)noise;
    a.pre = pre; a.axis_len = axis_len; a.post = post;
    a.block = block;
    a.nblk = (axis_len + block - 1) / block;
    if (scale_bits == 0) scale_bits = 8;                               // mx/mx_ops.py:320-323
    a.scale_emax = (1 << (scale_bits - 1)) - 1;
    a.flush = flush_fp32_subnorms != 0;
    a.mode = rmode;
    a.transposed = (flags & MXQ_CODES_TRANSPOSED) != 0;
    a.sf_gemm = (flags & MXQ_SCALES_GEMM_LAYOUT) != 0;
    a.sf_rpb = sf_rows_per_batch > 0 ? sf_rows_per_batch : (a.transposed ? post : pre);
    if (a.sf_gemm && (block != 32 || (!a.transposed && post != 1))) return MXQ_ERR_UNSUPPORTED;
    a.div_nblk.set((uint32_t)std::min<int64_t>(a.nblk, 0xffffffffLL));
    a.div_rpb.set((uint32_t)std::min<int64_t>(a.sf_rpb, 0xffffffffLL));
    a.fmt = make_fmt(elem_ebits, elem_mbits, elem_max_norm, rmode);
    set_fast_consts(a);
    g_launch_count[1].fetch_add(1, std::memory_order_relaxed);
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case MXQ_F32: return dispatch_dt<DT_F32>(a, st);
        case MXQ_F16: return dispatch_dt<DT_F16>(a, st);
        default:      return dispatch_dt<DT_BF16>(a, st);
    }
}
