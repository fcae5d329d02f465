// Forward and backward of an MX linear layer as one C call each (training form: the weight is
// quantized in the call, as the reference does on every forward, mx/linear.py:40-96, and the two
// gradient products of mx/linear.py:103-200 are formed in one call).  The calls only chain the
// library's own kernels on the caller's stream -- four MX packings and two block-scaled GEMMs for
// the backward pass -- with their packed operands in a caller-provided workspace, so a training
// step costs two library calls instead of nine operator calls on the host side.
#include <algorithm>
#include "mxq_common.cuh"

namespace mxq {
int gemm_mx_with_status(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                        void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int a_fmt, int b_fmt,
                        int out_dtype, int out_bfloat_bits, int out_round, const void* bias, int tile_n,
                        int* status_word, void* stream, void* const* dests = nullptr, int n_dests = 0,
                        int64_t rows_per_dest = 0);

static inline int64_t up256(int64_t v) { return (v + 255) & ~int64_t(255); }

// One packed [rows, K] operand inside a workspace.
struct PackedSlot {
    uint8_t* codes;
    uint8_t* scales;
    int64_t scale_bytes;
    bool ragged;            // scale chunks have padding bytes the quantizer does not write
};
static PackedSlot carve_slot(uint8_t*& p, int64_t rows, int64_t K) {
    PackedSlot s;
    s.codes = p;
    p += up256(rows * K);
    s.scale_bytes = mxq_sf_bytes(1, rows, K);
    s.scales = p;
    p += up256(s.scale_bytes);
    s.ragged = (rows % 128) != 0 || (K % 128) != 0;
    return s;
}

static bool fmt_ok(const mxq_elem_format* f) {
    return f && f->ebits >= 2 && f->ebits <= 5 && f->mbits >= 3 && f->mbits <= 5 && f->round >= MXQ_ROUND_NEAREST &&
           f->round <= MXQ_ROUND_EVEN;
}

// x [rows, K] (contraction last) or [K, rows] (transposed: contraction along axis 0) -> slot
static int pack_into(const PackedSlot& s, const void* x, int dtype, int64_t rows, int64_t K, bool contraction_last,
                     const mxq_elem_format* f, int scale_bits, int flush, cudaStream_t st) {
    if (s.ragged && cudaMemsetAsync(s.scales, 0, (size_t)s.scale_bytes, st) != cudaSuccess) return MXQ_ERR_CUDA;
    if (contraction_last)
        return mxq_quantize_mx(x, nullptr, s.codes, s.scales, dtype, rows, K, 1, 32, scale_bits, f->ebits, f->mbits,
                               f->max_norm, flush, f->round, nullptr, MXQ_SCALES_GEMM_LAYOUT, rows, st);
    return mxq_quantize_mx(x, nullptr, s.codes, s.scales, dtype, 1, K, rows, 32, scale_bits, f->ebits, f->mbits,
                           f->max_norm, flush, f->round, nullptr, MXQ_SCALES_GEMM_LAYOUT | MXQ_CODES_TRANSPOSED, 0, st);
}
}  // namespace mxq

extern "C" int64_t mxq_linear_train_workspace_bytes(int64_t M, int64_t K, int64_t N) {
    if (M < 0 || K < 0 || N < 0) return -1;
    using namespace mxq;
    // the backward pass holds four operands: go^T [N, M], x^T [K, M], go [M, N], w^T [K, N]
    auto slot = [](int64_t rows, int64_t k) { return up256(rows * k) + up256(mxq_sf_bytes(1, rows, k)); };
    const int64_t bwd = slot(N, M) + slot(K, M) + slot(M, N) + slot(K, N);
    const int64_t fwd = slot(M, K) + slot(N, K);
    return 256 + std::max(bwd, fwd);
}

extern "C" int mxq_linear_fwd_train(const void* x, const void* w, int dtype, int64_t M, int64_t K, int64_t N,
                                    const mxq_elem_format* a_fmt, const mxq_elem_format* w_fmt, int scale_bits,
                                    int flush_fp32_subnorms, void* y, int y_dtype, int out_bfloat_bits, int out_round,
                                    const void* bias, void* workspace, int64_t workspace_bytes, void* stream) {
    using namespace mxq;
    if (M < 0 || K < 0 || N < 0) return MXQ_ERR_BAD_ARG;
    if (M == 0 || N == 0) return MXQ_OK;
    if (!x || !w || !y || !workspace || !fmt_ok(a_fmt) || !fmt_ok(w_fmt)) return MXQ_ERR_BAD_ARG;
    if (K == 0 || K % 32 != 0) return MXQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
    if (workspace_bytes < mxq_linear_train_workspace_bytes(M, K, N)) return MXQ_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* p = reinterpret_cast<uint8_t*>(workspace);
    int* status = reinterpret_cast<int*>(p);
    p += 256;
    if (cudaMemsetAsync(status, 0, 256, st) != cudaSuccess) return MXQ_ERR_CUDA;
    const PackedSlot sx = carve_slot(p, M, K), sw = carve_slot(p, N, K);
    int rc = pack_into(sx, x, dtype, M, K, true, a_fmt, scale_bits, flush_fp32_subnorms, st);
    if (rc) return rc;
    rc = pack_into(sw, w, dtype, N, K, true, w_fmt, scale_bits, flush_fp32_subnorms, st);
    if (rc) return rc;
    return gemm_mx_with_status(sx.codes, sx.scales, sw.codes, sw.scales, y, 1, M, N, K, a_fmt->ebits == 5 ? 1 : 0,
                               w_fmt->ebits == 5 ? 1 : 0, y_dtype, out_bfloat_bits, out_round, bias, 0, status, stream);
}

extern "C" int mxq_linear_bwd(const void* grad_out, const void* x, const void* w, int dtype, int64_t M, int64_t K,
                              int64_t N, const mxq_elem_format* go_fmt_gw, const mxq_elem_format* x_fmt_gw,
                              const mxq_elem_format* go_fmt_gi, const mxq_elem_format* w_fmt_gi, int scale_bits,
                              int flush_fp32_subnorms, void* grad_x, void* grad_w, int g_dtype, int out_bfloat_bits,
                              int round_grad_input, int round_grad_weight, void* workspace, int64_t workspace_bytes,
                              void* stream) {
    using namespace mxq;
    if (M < 0 || K < 0 || N < 0) return MXQ_ERR_BAD_ARG;
    if (M == 0 || N == 0 || K == 0) return MXQ_OK;
    if (!grad_out || !x || !w || !workspace || (!grad_x && !grad_w)) return MXQ_ERR_BAD_ARG;
    if (!fmt_ok(go_fmt_gw) || !fmt_ok(x_fmt_gw) || !fmt_ok(go_fmt_gi) || !fmt_ok(w_fmt_gi)) return MXQ_ERR_BAD_ARG;
    // contraction lengths: M (tokens) for grad_weight, N (out_features) for grad_input; the strided packing
    // kernels of the transposed operands want 8-byte aligned rows
    if (M % 32 != 0 || N % 32 != 0 || K % 4 != 0) return MXQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
    if (workspace_bytes < mxq_linear_train_workspace_bytes(M, K, N)) return MXQ_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* p = reinterpret_cast<uint8_t*>(workspace);
    int* status = reinterpret_cast<int*>(p);
    p += 256;
    if (cudaMemsetAsync(status, 0, 256, st) != cudaSuccess) return MXQ_ERR_CUDA;
    const PackedSlot s_got = carve_slot(p, N, M), s_xt = carve_slot(p, K, M), s_go = carve_slot(p, M, N),
                     s_wt = carve_slot(p, K, N);
    int rc;
    if (grad_w) {
        // grad_weight [N, K] = MX(go)^T MX(x), blocks along the token axis
        rc = pack_into(s_got, grad_out, dtype, N, M, false, go_fmt_gw, scale_bits, flush_fp32_subnorms, st);
        if (rc) return rc;
        rc = pack_into(s_xt, x, dtype, K, M, false, x_fmt_gw, scale_bits, flush_fp32_subnorms, st);
        if (rc) return rc;
        rc = gemm_mx_with_status(s_got.codes, s_got.scales, s_xt.codes, s_xt.scales, grad_w, 1, N, K, M,
                                 go_fmt_gw->ebits == 5 ? 1 : 0, x_fmt_gw->ebits == 5 ? 1 : 0, g_dtype, out_bfloat_bits,
                                 round_grad_weight, nullptr, 0, status, stream);
        if (rc) return rc;
    }
    if (grad_x) {
        // grad_input [M, K] = MX(go) MX(w), blocks along out_features
        rc = pack_into(s_go, grad_out, dtype, M, N, true, go_fmt_gi, scale_bits, flush_fp32_subnorms, st);
        if (rc) return rc;
        rc = pack_into(s_wt, w, dtype, K, N, false, w_fmt_gi, scale_bits, flush_fp32_subnorms, st);
        if (rc) return rc;
        rc = gemm_mx_with_status(s_go.codes, s_go.scales, s_wt.codes, s_wt.scales, grad_x, 1, M, K, N,
                                 go_fmt_gi->ebits == 5 ? 1 : 0, w_fmt_gi->ebits == 5 ? 1 : 0, g_dtype, out_bfloat_bits,
                                 round_grad_input, nullptr, 0, status, stream);
        if (rc) return rc;
    }
    return MXQ_OK;
}

// ---------------------------------------------------------------------------
// One batched MX product as one call: C[b] = op(A[b]) op(B[b]), both operands MX-quantized along the
// contraction axis in the call (mx/matmul.py:68-86, mx/bmm.py:40-59).  A is [batch, M, K] or, with
// a_trans, [batch, K, M]; B is [batch, K, N] or, with b_trans, [batch, N, K].  A may arrive already
// packed (a_codes / a_scales in the GEMM layout, e.g. probabilities packed by mxq_softmax_quantize_mx);
// `a` is then not read.
// ---------------------------------------------------------------------------
namespace mxq {
static int pack_batched(uint8_t* codes, uint8_t* scales, int64_t scale_bytes, const void* x, int dtype, int64_t batch,
                        int64_t rows, int64_t K, bool contraction_last, const mxq_elem_format* f, int scale_bits,
                        int flush, cudaStream_t st) {
    if (((rows % 128) != 0 || (K % 128) != 0) && cudaMemsetAsync(scales, 0, (size_t)scale_bytes, st) != cudaSuccess)
        return MXQ_ERR_CUDA;
    if (contraction_last)
        return mxq_quantize_mx(x, nullptr, codes, scales, dtype, batch * rows, K, 1, 32, scale_bits, f->ebits, f->mbits,
                               f->max_norm, flush, f->round, nullptr, MXQ_SCALES_GEMM_LAYOUT, rows, st);
    return mxq_quantize_mx(x, nullptr, codes, scales, dtype, batch, K, rows, 32, scale_bits, f->ebits, f->mbits,
                           f->max_norm, flush, f->round, nullptr, MXQ_SCALES_GEMM_LAYOUT | MXQ_CODES_TRANSPOSED, 0, st);
}
}  // namespace mxq

extern "C" int64_t mxq_matmul_workspace_bytes(int64_t batch, int64_t M, int64_t K, int64_t N) {
    if (batch < 0 || M < 0 || K < 0 || N < 0) return -1;
    using namespace mxq;
    return 256 + up256(batch * M * K) + up256(mxq_sf_bytes(batch, M, K)) + up256(batch * N * K) +
           up256(mxq_sf_bytes(batch, N, K));
}

extern "C" int mxq_matmul_fwd(const void* a, const void* b, int dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                              int a_trans, int b_trans, const mxq_elem_format* a_fmt, const mxq_elem_format* b_fmt,
                              int scale_bits, int flush_fp32_subnorms, const void* a_codes, const void* a_scales,
                              void* c, int c_dtype, int out_bfloat_bits, int out_round, const void* bias,
                              void* workspace, int64_t workspace_bytes, void* stream) {
    using namespace mxq;
    if (batch < 0 || M < 0 || K < 0 || N < 0) return MXQ_ERR_BAD_ARG;
    if (batch == 0 || M == 0 || N == 0) return MXQ_OK;
    const bool a_packed = a_codes != nullptr;
    if ((!a && !a_packed) || (a_packed && !a_scales) || !b || !c || !workspace || !fmt_ok(a_fmt) || !fmt_ok(b_fmt))
        return MXQ_ERR_BAD_ARG;
    if (K == 0 || K % 32 != 0) return MXQ_ERR_UNSUPPORTED;
    // the strided packing kernels of a transposed operand want 8-byte aligned rows
    if ((a_trans && !a_packed && M % 4 != 0) || (!b_trans && N % 4 != 0)) return MXQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
    if (workspace_bytes < mxq_matmul_workspace_bytes(batch, M, K, N)) return MXQ_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* p = reinterpret_cast<uint8_t*>(workspace);
    int* status = reinterpret_cast<int*>(p);
    p += 256;
    if (cudaMemsetAsync(status, 0, 256, st) != cudaSuccess) return MXQ_ERR_CUDA;
    uint8_t* ac = p;            p += up256(batch * M * K);
    const int64_t a_sf = mxq_sf_bytes(batch, M, K);
    uint8_t* as = p;            p += up256(a_sf);
    uint8_t* bc = p;            p += up256(batch * N * K);
    const int64_t b_sf = mxq_sf_bytes(batch, N, K);
    uint8_t* bs = p;
    int rc;
    if (!a_packed) {
        rc = pack_batched(ac, as, a_sf, a, dtype, batch, M, K, !a_trans, a_fmt, scale_bits, flush_fp32_subnorms, st);
        if (rc) return rc;
    }
    rc = pack_batched(bc, bs, b_sf, b, dtype, batch, N, K, b_trans != 0, b_fmt, scale_bits, flush_fp32_subnorms, st);
    if (rc) return rc;
    return gemm_mx_with_status(a_packed ? a_codes : ac, a_packed ? a_scales : as, bc, bs, c, batch, M, N, K,
                               a_fmt->ebits == 5 ? 1 : 0, b_fmt->ebits == 5 ? 1 : 0, c_dtype, out_bfloat_bits, out_round,
                               bias, 0, status, stream);
}

