/*
 * mxq.h -- C ABI of libmxq.so, the sm_100a back-end of the MX quantization path.
 *
 * This boundary takes the place of the pybind module the reference JIT-builds
 * in mx/custom_extensions.py:11-19 (exported functions: mx/cpp/funcs.cpp:234-242).
 * Differences in convention, all deliberate:
 *   - plain pointers and sizes, no tensor types; the caller owns every buffer
 *     (the reference allocates its result with torch::empty_like);
 *   - every call takes the CUDA stream to launch on (the reference launches on
 *     the legacy default stream, mx/cpp/mx.cu:58,170,230);
 *   - errors come back as a negative status, the process is never exited
 *     (the reference's gpuErrchk calls exit(), mx/cpp/common.cuh:247-255);
 *   - nothing here allocates device memory unless stated.
 * All pointers are device pointers on the current device unless stated.
 */
#ifndef MXQ_H
#define MXQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define MXQ_OK               0
#define MXQ_ERR_BAD_ARG     -1   /* null pointer, negative size, unknown enum */
#define MXQ_ERR_UNSUPPORTED -2   /* a valid request this build has no kernel for */
#define MXQ_ERR_CUDA        -3   /* a CUDA runtime / driver call failed */
#define MXQ_ERR_ALIGN       -4   /* pointer or size not aligned as the call requires */
#define MXQ_ERR_TOO_LARGE   -5   /* size beyond a documented maximum */
#define MXQ_ERR_DEVICE      -6   /* a kernel reported a device-side time-out or fault word */

/* storage types of tensors */
#define MXQ_F32  0
#define MXQ_F16  1
#define MXQ_BF16 2

/* rounding modes: 0..2 are the reference's RoundingMode enum
 * (mx/formats.py:12-19, mx/cpp/common.cuh:128-132); 3 is the PyTorch-only
 * 'dither' mode of mx/elemwise_ops.py:57-59 and needs a noise tensor. */
#define MXQ_ROUND_NEAREST 0      /* ties away from zero */
#define MXQ_ROUND_FLOOR   1      /* toward zero */
#define MXQ_ROUND_EVEN    2      /* ties to even */
#define MXQ_ROUND_DITHER  3      /* floor(|x|/quantum + noise) */

/* flags of mxq_quantize_mx */
#define MXQ_CODES_TRANSPOSED 1   /* write codes/scales with the blocked axis innermost */
#define MXQ_SCALES_GEMM_LAYOUT 2  /* write scales in the chunk layout mxq_gemm_mx reads (block must be 32) */

const char* mxq_status_string(int status);
int mxq_version(void);
/* Launches made by this process so far: what = 0 block-scaled GEMMs (through any entry point),
 * what = 1 MX quantizations (mxq_quantize_mx and the fused packing entry points, the ones inside
 * the composite linear calls included).  For tests and accounting; no reference counterpart. */
int64_t mxq_launch_count(int what);

/* SMs the persistent GEMM kernels of this process occupy from the next launch on: sms > 0 sets the
 * budget (values at or above the device's SM count mean all of them), 0 restores "all", a negative
 * value only reads.  Returns the previous setting.  A caller that runs a collective beside a GEMM
 * leaves the collective's CTAs room this way; results do not depend on it.  No reference counterpart. */
int mxq_gemm_sm_budget(int sms);

/*
 * Device buffers shared between the processes of one node (no reference
 * counterpart), the destinations of mxq_gemm_mx_scatter.  mxq_peer_alloc
 * allocates `bytes` on the current device and fills a 64-byte handle another
 * process passes to mxq_peer_open WITH ITS OWN DEVICE CURRENT; the pointer it
 * gets is valid for kernels of that device.  Close every mapping before the
 * owner frees the buffer.
 */
int mxq_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int mxq_peer_free(void* ptr);
int mxq_peer_open(const void* handle64, void** ptr);
int mxq_peer_close(void* ptr);

/*
 * MX block fake-quantization, optionally also emitting the packed operand.
 * Replaces quantize_mx_by_tile_func_cuda (mx/cpp/funcs.cpp:177-197) and
 * quantize_mx_func_cuda (funcs.cpp:154-175; the caller no longer computes the
 * per-block maximum).
 *
 * The tensor is contiguous [pre, axis_len, post]; blocks of `block` consecutive
 * elements along the middle axis share one power-of-two scale (block <= 0: one
 * block spans the axis; a ragged last block is allowed).
 *   in        input, `dtype`
 *   out       dequantized result, same dtype and shape, or NULL
 *   codes     one byte per element or NULL: the quantized element in an fp8
 *             container (e5m2 for elem_ebits == 5, otherwise e4m3, which holds
 *             every e4m3 / e3m2 / e2m3 / e2m1 value exactly); fixed-point
 *             formats are two's complement with (elem_mbits - 2) fraction bits.
 *             Layout [pre, axis_len, post], or with MXQ_CODES_TRANSPOSED
 *             [pre, post, axis_len_padded] where axis_len_padded = nblocks*block
 *             (padding bytes are zero).
 *   scales    one E8M0 byte per block (biased exponent, 255 = NaN) or NULL;
 *             layout [pre, nblocks, post], transposed: [pre, post, nblocks].
 *             Required when codes is given.
 *   scale_bits, elem_ebits, elem_mbits, elem_max_norm, flush_fp32_subnorms,
 *   rmode     as in the reference signature
 *   noise     fp32 uniform [0,1) tensor of the input's shape for
 *             MXQ_ROUND_DITHER, else NULL
 *   flags     MXQ_CODES_TRANSPOSED, MXQ_SCALES_GEMM_LAYOUT
 *   sf_rows_per_batch  only with MXQ_SCALES_GEMM_LAYOUT: the operand is seen as
 *             [batch, rows, K] with K the blocked axis.  Not transposed
 *             (post == 1): the pre axis is batch * rows and this gives rows
 *             (0: one batch).  Transposed: batch = pre, rows = post.  The scale
 *             of (batch b, row r, block k) is byte
 *               ((b*ceil(rows/128) + r/128) * ceil(nblocks/4) + k/4) * 512
 *                 + (r%32)*16 + ((r%128)/32)*4 + k%4
 *             of the scales buffer (mxq_sf_bytes gives its size); bytes of
 *             padding rows / blocks are not written.
 */
int mxq_quantize_mx(const void* in, void* out, void* codes, void* scales, int dtype,
                    int64_t pre, int64_t axis_len, int64_t post, int block,
                    int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                    int flush_fp32_subnorms, int rmode, const void* noise, int flags,
                    int64_t sf_rows_per_batch, void* stream);

/*
 * Elementwise rounding to a (bits, exp_bits) format.  Replaces
 * quantize_elemwise_func_cuda (mx/cpp/funcs.cpp:199-217); bits <= 24.
 * in_dtype and out_dtype may differ (fp32 in, bf16 out is the
 * `A.to(torch.bfloat16)` shortcut of mx/elemwise_ops.py:248-251).
 */
int mxq_quantize_elemwise(const void* in, void* out, int in_dtype, int out_dtype, int64_t n,
                          int bits, int exp_bits, float max_norm, int rmode,
                          int saturate_normals, int allow_denorm, const void* noise,
                          void* stream);

/*
 * The two quantizers for tensors in HOST memory (use pinned memory: pageable
 * memory makes the copies synchronous).  Same arguments as the device entry
 * points, plus a device workspace of mxq_host_workspace_bytes() bytes
 * (256-byte aligned).  The tensor is processed in chunks of whole blocks on
 * three internal streams (created on first use, kept until exit) so that the
 * host->device copy, the kernel and the device->host copy of different chunks
 * overlap; the work is ordered after what `stream` holds at the call, and
 * `stream` waits for it.  The reference's counterpart for host tensors is its
 * single-threaded C++ loop, quantize_mx_func_cpp / quantize_elemwise_func_cpp
 * (mx/cpp/funcs.cpp:23-149).  Codes / scales outputs and 'dither' are not
 * offered here.
 */
int mxq_quantize_mx_host(const void* h_in, void* h_out, int dtype, int64_t pre, int64_t axis_len,
                         int64_t post, int block, int scale_bits, int elem_ebits, int elem_mbits,
                         float elem_max_norm, int flush_fp32_subnorms, int rmode, void* workspace,
                         int64_t workspace_bytes, void* stream);
int mxq_quantize_elemwise_host(const void* h_in, void* h_out, int in_dtype, int out_dtype, int64_t n,
                               int bits, int exp_bits, float max_norm, int rmode, int saturate_normals,
                               int allow_denorm, void* workspace, int64_t workspace_bytes, void* stream);
int64_t mxq_host_workspace_bytes(void);

/*
 * The two quantizers on the HOST cores, for tensors in ordinary host memory
 * (no GPU is touched).  Replace quantize_mx_func_cpp (mx/cpp/funcs.cpp:23-98,
 * loop mx/cpp/funcs.h:61-100) and quantize_elemwise_func_cpp
 * (mx/cpp/funcs.cpp:117-149), which the reference calls for CPU tensors when
 * custom_cuda is set (mx/mx_ops.py:259-263, mx/elemwise_ops.py:122-124).
 * Arguments as in mxq_quantize_mx / mxq_quantize_elemwise without the packed
 * outputs; all pointers are host pointers; results equal the GPU kernels'.
 * nthreads: OpenMP threads to use, 0 = all (the reference's loop is single-threaded).
 */
int mxq_cpu_quantize_mx(const void* in, void* out, int dtype, int64_t pre, int64_t axis_len, int64_t post,
                        int block, int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                        int flush_fp32_subnorms, int rmode, const void* noise, int nthreads);
int mxq_cpu_quantize_elemwise(const void* in, void* out, int in_dtype, int out_dtype, int64_t n, int bits,
                              int exp_bits, float max_norm, int rmode, int saturate_normals, int allow_denorm,
                              const void* noise, int nthreads);

/*
 * Sum / max over the innermost dimension of an fp32 [rows, inner] matrix into
 * out[rows].  Replace reduce_sum_inner_dim / reduce_max_inner_dim
 * (mx/cpp/funcs.cpp:219-231, mx/cpp/reduce.cu:15-89).  Any inner >= 1 is
 * accepted (the reference requires a multiple of 32).
 */
int mxq_reduce_sum_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream);
int mxq_reduce_max_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream);

/*
 * Fused bfloat16 vector chains.  The reference runs these layers as one
 * elementwise kernel per vector operation, each followed by a rounding to the
 * bfloat format (mx/vector_ops.py:1-130); for bfloat16 CUDA tensors with
 * bfloat = 16 every step computes in fp32 and rounds to nearest-even bfloat16.
 * These entry points run the same chain per element in registers.
 *
 * mxq_silu_bf16: SiLUFunction.forward (mx/activations.py:418-439)
 *   e = exp(-g); a = e + 1; sig = 1 / a; out = g * sig; with `up`: out = out * up
 *   (the simd_mul of a gated feed-forward block, mx/simd_ops.py:189-237).
 *   gate, up, out, sig: n bfloat16 elements, 16-byte aligned; up and sig may be NULL.
 * mxq_rmsnorm_bf16: RMSNormFunction.forward (mx/layernorm.py:113-129)
 *   ms = mean(x*x); rinv = 1/sqrt(ms + eps); x_norm = x * rinv; out = weight * x_norm + bias
 *   over the last dimension of x [rows, hidden]; the row sum is accumulated in
 *   fp32 and rounded to bfloat16 once (like the library reduction the reference
 *   calls, whose summation order is unspecified).  bias, x_norm [rows, hidden]
 *   and rms_inv [rows] may be NULL.  hidden % 8 == 0 needs 16-byte aligned
 *   pointers; other widths take an element-wise path.
 * Large inputs (>= 4 Mi elements) of mxq_silu_bf16 and mxq_softmax_bf16, and every call of
 * mxq_swiglu_quantize_mx, read the sigmoid chain / exp from a table over all 65536 bfloat16 bit
 * patterns that the first such call on a device builds by running the chain itself (one cudaMalloc of
 * 128 KB, one kernel on the default stream, one synchronize; kept until exit).  Make that first
 * call outside stream capture.
 * mxq_softmax_bf16: SoftmaxFunction.forward over the last dimension (mx/softmax.py:18-41)
 *   m = max(x); d = x - m; e = exp(d) (exp2(d) if use_exp2); s = sum(e); out = e / s;
 *   the row sum is accumulated in fp32 and rounded once.  cols % 8 == 0, cols <= 2048
 *   (MXQ_ERR_UNSUPPORTED otherwise), 16-byte aligned pointers.
 */
int mxq_softmax_bf16(const void* x, void* out, int64_t rows, int64_t cols, int use_exp2, void* stream);
int mxq_silu_bf16(const void* gate, const void* up, void* out, void* sig, int64_t n, void* stream);
int mxq_rmsnorm_bf16(const void* x, const void* weight, const void* bias, void* out, void* x_norm,
                     void* rms_inv, int64_t rows, int64_t hidden, float eps, void* stream);

/*
 * SiLU(gate) * up (the chain of mxq_silu_bf16) fused into the MX packing of the
 * product along its last axis: what mxq_silu_bf16 followed by mxq_quantize_mx
 * (codes + scales, no dequantized output) writes, without the bfloat16 product
 * ever reaching memory.  gate, up: bfloat16 [rows, K], K % 32 == 0, block 32;
 * fp element formats with a one-byte container; rmode nearest / floor / even;
 * flags: MXQ_SCALES_GEMM_LAYOUT or 0.  Replaces, for the gated feed-forward block,
 * silu + simd_mul + the quantize_mx_op of the down projection's input
 * (mx/activations.py:418-439, mx/simd_ops.py:189-237, mx/linear.py:75-83).
 */
int mxq_swiglu_quantize_mx(const void* gate, const void* up, void* codes, void* scales, int64_t rows, int64_t K,
                           int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                           int flush_fp32_subnorms, int rmode, int flags, int64_t sf_rows_per_batch, void* stream);

/*
 * Softmax over the last dimension (the chain of mxq_softmax_bf16, exp only)
 * fused into the MX packing of the probabilities along that dimension: what
 * mxq_softmax_bf16 followed by mxq_quantize_mx (codes + scales) writes, with the
 * score matrix read once and the probabilities never re-read.  Replaces, in an
 * attention block, SoftmaxFunction.forward (mx/softmax.py:18-41) and the
 * quantize_mx_op of the left operand of the product that follows
 * (mx/bmm.py:40-59, mx/matmul.py:68-86).
 *   x       bfloat16 [rows, cols], cols % 32 == 0, cols <= 2048
 *   probs   bfloat16 [rows, cols] or NULL (the caller does not need them)
 *   codes, scales, element format, rmode, flags, sf_rows_per_batch
 *           as in mxq_swiglu_quantize_mx (block 32, nearest / floor / even)
 * Reads exp from the table mxq_softmax_bf16 describes (built by the first call
 * on a device: make that call outside stream capture).
 */
int mxq_softmax_quantize_mx(const void* x, void* probs, void* codes, void* scales, int64_t rows, int64_t cols,
                            int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                            int flush_fp32_subnorms, int rmode, int flags, int64_t sf_rows_per_batch, void* stream);

/*
 * Block-scaled MX GEMM on the tensor cores (tcgen05 kind::mxf8f6f4):
 *   C[b] = A[b] (M x K) * B[b]^T (N x K),  b < batch, fp32 accumulation.
 * Takes the place of the library GEMM the reference runs on dequantized
 * operands: F.linear / torch.matmul / torch.bmm in mx/linear.py:86,147,179,
 * mx/matmul.py:86,167,172 and mx/bmm.py:59,116,121, together with the
 * quantize_elemwise_op that follows it (mx/linear.py:88-96).
 *   a_codes [batch, M, K], b_codes [batch, N, K]   element codes from
 *             mxq_quantize_mx (K contiguous)
 *   a_scales, b_scales   E8M0 scales in the MXQ_SCALES_GEMM_LAYOUT layout
 *   a_fmt, b_fmt         code container: 0 = e4m3, 1 = e5m2
 *   c         [batch, M, N], out_dtype MXQ_F32 or MXQ_BF16
 *   out_bfloat_bits, out_round   bfloat rounding of the result (mx_specs
 *             'bfloat' and 'round_output'); 0 or 32 bits, or round -1: none
 *   bias      fp32 [N] or NULL: c = round(round(acc) + bias)
 *   tile_n    0 (automatic), 128 or 256
 * K must be a multiple of 32 (when it is not a multiple of 128, the scale bytes of
 * the missing blocks of the last 128-wide group must be zero, as mxq_quantize_mx
 * leaves them in a zero-initialised buffer); pointers 16-byte aligned.  The first call on a
 * device allocates a 4-byte status word with cudaMalloc (kept until exit); a
 * kernel that gives up on a wait stores MXQ_ERR_DEVICE there, see
 * mxq_device_status.
 */
int mxq_gemm_mx(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int a_fmt, int b_fmt,
                int out_dtype, int out_bfloat_bits, int out_round, const void* bias, int tile_n,
                void* stream);

/* Bytes of a scales buffer in the GEMM layout for a [batch, rows, K] operand. */
int64_t mxq_sf_bytes(int64_t batch, int64_t rows, int64_t K);

/*
 * Scattering GEMM for a row-parallel layer split over several GPUs (no
 * reference counterpart: the reference is single-device).  Same product as
 * mxq_gemm_mx with batch = 1 and no bias, but rows
 * [d * rows_per_dest, (d+1) * rows_per_dest) of the result are stored into
 * dests[d], a [rows_per_dest, N] buffer that may live on another GPU (a peer
 * mapping in this process).  Each 128-row tile leaves through a bulk store as
 * soon as it is finished, so the transfer overlaps the remaining tiles; nothing
 * waits on another GPU inside the kernel.  The caller orders the consumers
 * (a barrier between ranks after the call), then adds the slabs it received
 * with mxq_sum_slabs_f32.  rows_per_dest % 128 == 0, n_dests <= 8,
 * N * element size % 16 == 0, M <= n_dests * rows_per_dest.
 */
int mxq_gemm_mx_scatter(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                        void* const* dests, int n_dests, int64_t rows_per_dest, int64_t M, int64_t N, int64_t K,
                        int a_fmt, int b_fmt, int out_dtype, int out_bfloat_bits, int out_round, int tile_n,
                        void* stream);
/* out[i] = ((slab0[i] + slab1[i]) + slab2[i]) + ...  for n_slabs consecutive fp32 slabs of elems_per_slab. */
int mxq_sum_slabs_f32(const void* slabs, int n_slabs, int64_t elems_per_slab, void* out, void* stream);

/*
 * Forward of an MX linear layer whose weights were packed once:
 *   y[M,N] = round(MX(x)[M,K] * W[N,K]^T (+ bias)),
 * i.e. the activation quantization (mx/linear.py:62-68, block 32 along K) and
 * the product with its output rounding (mx/linear.py:83-96) in one call.
 *   x          [M, K], x_dtype
 *   a_*        element format, rounding, scale width and subnormal flush of
 *              the activation quantization (as in mxq_quantize_mx)
 *   w_codes, w_scales, w_fmt   the weight as mxq_quantize_mx packed it
 *              ([N, K] codes, scales in MXQ_SCALES_GEMM_LAYOUT, container id)
 *   y, y_dtype, out_bfloat_bits, out_round, bias   as in mxq_gemm_mx
 *   workspace  device memory for the packed activations, 256-byte aligned,
 *              at least mxq_linear_workspace_bytes(M, K) bytes; its first
 *              4 bytes are the status word of this call (0, or MXQ_ERR_DEVICE)
 * K must be a multiple of 128.  Allocates nothing.
 */
int mxq_linear_fwd(const void* x, int x_dtype, int64_t M, int64_t K, int a_ebits, int a_mbits,
                   float a_max_norm, int a_round, int scale_bits, int flush_fp32_subnorms,
                   const void* w_codes, const void* w_scales, int64_t N, int w_fmt, void* y, int y_dtype,
                   int out_bfloat_bits, int out_round, const void* bias, void* workspace,
                   int64_t workspace_bytes, void* stream);
int64_t mxq_linear_workspace_bytes(int64_t M, int64_t K);

/*
 * One MX linear layer of a training step as two calls: forward with the weight
 * quantized in the call (the reference does so on every forward,
 * mx/linear.py:40-96), and both gradient products of LinearFunction.backward
 * (mx/linear.py:103-200) at once.  Each call only chains this library's kernels on
 * `stream` (MX packings + block-scaled GEMMs); the packed operands live in the
 * caller's workspace of mxq_linear_train_workspace_bytes(M, K, N) bytes (256-byte
 * aligned; its first 4 bytes are the call's status word: 0 or MXQ_ERR_DEVICE).
 *   x [M, K], w [N, K], grad_out [M, N]: `dtype`, contiguous
 *   mxq_elem_format: element format and MX rounding of one operand (float formats
 *     with a one-byte container; round nearest / floor / even)
 *   forward:  y = round(MX_a(x) MX_w(w)^T (+ bias)), blocks of 32 along K (K % 32 == 0)
 *   backward: grad_w [N, K] = round(MX(go)^T MX(x)), blocks along the M tokens
 *             (go_fmt_gw = a_elem_format_bp_ex, x_fmt_gw = a_elem_format_bp);
 *             grad_x [M, K] = round(MX(go) MX(w)), blocks along N
 *             (go_fmt_gi = a_elem_format_bp_os, w_fmt_gi = w_elem_format_bp);
 *             M % 32 == 0, N % 32 == 0, K % 4 == 0; grad_x or grad_w may be NULL.
 *   out_bfloat_bits and the round_* arguments: as in mxq_gemm_mx.
 */
typedef struct mxq_elem_format {
    int ebits;
    int mbits;
    float max_norm;
    int round;
} mxq_elem_format;
int64_t mxq_linear_train_workspace_bytes(int64_t M, int64_t K, int64_t N);
int mxq_linear_fwd_train(const void* x, const void* w, int dtype, int64_t M, int64_t K, int64_t N,
                         const mxq_elem_format* a_fmt, const mxq_elem_format* w_fmt, int scale_bits,
                         int flush_fp32_subnorms, void* y, int y_dtype, int out_bfloat_bits, int out_round,
                         const void* bias, void* workspace, int64_t workspace_bytes, void* stream);
int mxq_linear_bwd(const void* grad_out, const void* x, const void* w, int dtype, int64_t M, int64_t K, int64_t N,
                   const mxq_elem_format* go_fmt_gw, const mxq_elem_format* x_fmt_gw,
                   const mxq_elem_format* go_fmt_gi, const mxq_elem_format* w_fmt_gi, int scale_bits,
                   int flush_fp32_subnorms, void* grad_x, void* grad_w, int g_dtype, int out_bfloat_bits,
                   int round_grad_input, int round_grad_weight, void* workspace, int64_t workspace_bytes,
                   void* stream);

/*
 * One batched MX product as one call (no single reference counterpart: MatMulFunction.forward,
 * mx/matmul.py:68-86, and BMMFunction.forward, mx/bmm.py:40-59, each make two quantize_mx_op calls
 * and one torch.matmul / torch.bmm): C[i] = op(A[i]) op(B[i]) for i < batch, both operands MX-quantized
 * in blocks of 32 along the contraction axis, fp32 accumulation, the output rounded as mxq_gemm_mx
 * rounds it.  A: [batch, M, K], or [batch, K, M] with a_trans; B: [batch, K, N], or [batch, N, K]
 * with b_trans.  If a_codes is not NULL, A is already packed (codes [batch, M, K] and scales in the
 * GEMM layout, e.g. from mxq_softmax_quantize_mx) and `a` is not read.  K % 32 == 0; a transposed
 * operand needs its row length (M or N) % 4 == 0.  The packed operands live in `workspace`
 * (256-byte aligned, >= mxq_matmul_workspace_bytes(batch, M, K, N)); nothing is allocated.
 */
int64_t mxq_matmul_workspace_bytes(int64_t batch, int64_t M, int64_t K, int64_t N);
int mxq_matmul_fwd(const void* a, const void* b, int dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                   int a_trans, int b_trans, const mxq_elem_format* a_fmt, const mxq_elem_format* b_fmt,
                   int scale_bits, int flush_fp32_subnorms, const void* a_codes, const void* a_scales,
                   void* c, int c_dtype, int out_bfloat_bits, int out_round, const void* bias,
                   void* workspace, int64_t workspace_bytes, void* stream);

/*
 * mxq_linear_fwd for callers that cannot allocate and have no buffer to lend.
 * No counterpart in the reference (which allocates a fresh tensor in every
 * call, mx/cpp/mx.cu:27-28).  Same arguments and result as mxq_linear_fwd
 * without the workspace: the packed activations and the status word live in a
 * fixed array inside the library image, 256 B + 33 MiB of device memory that
 * every GPU loading libmxq.so holds until the process exits.
 *   - Limit: ceil(M/128)*128 * K <= mxq_linear_static_max_elems() (32 Mi, e.g.
 *     8192 x 4096); larger shapes return MXQ_ERR_TOO_LARGE and launch nothing.
 *   - Calls cudaMalloc / cudaFree never; the first call on each device looks up
 *     the array's device address (cudaGetSymbolAddress) and should be made
 *     before any stream capture begins.
 *   - All calls on a device share the array: two calls whose kernels can
 *     overlap on the GPU (different streams) race on it; calls on one stream
 *     are ordered and safe.  The array keeps the last call's contents; each
 *     call re-zeroes the parts it relies on (status word, scale region).
 *   - The array is the CURRENT device's: x, y and the weight must live on the
 *     current device (MXQ_ERR_BAD_ARG otherwise; nothing is launched).
 *   - mxq_linear_static_status() reads the status word of the last call on the
 *     current device: 0, or MXQ_ERR_DEVICE if a kernel gave up on a wait.  It
 *     copies with a blocking cudaMemcpy, which does not wait for work on
 *     non-blocking streams: synchronize the stream the call was made on first.
 */
int mxq_linear_fwd_static(const void* x, int x_dtype, int64_t M, int64_t K, int a_ebits, int a_mbits,
                          float a_max_norm, int a_round, int scale_bits, int flush_fp32_subnorms,
                          const void* w_codes, const void* w_scales, int64_t N, int w_fmt, void* y,
                          int y_dtype, int out_bfloat_bits, int out_round, const void* bias, void* stream);
int64_t mxq_linear_static_max_elems(void);
int mxq_linear_static_status(void);

/* Reads (and optionally clears) the current device's status word: 0, or
 * MXQ_ERR_DEVICE after a kernel timed out on a wait.  The read is a blocking
 * cudaMemcpy, which does not wait for work on non-blocking streams:
 * synchronize the streams the GEMMs ran on first. */
int mxq_device_status(int clear);

#ifdef __cplusplus
}
#endif
#endif /* MXQ_H */
