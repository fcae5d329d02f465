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

const char* mxq_status_string(int status);
int mxq_version(void);

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
 */
int mxq_quantize_mx(const void* in, void* out, void* codes, void* scales, int dtype,
                    int64_t pre, int64_t axis_len, int64_t post, int block,
                    int scale_bits, int elem_ebits, int elem_mbits, float elem_max_norm,
                    int flush_fp32_subnorms, int rmode, const void* noise, int flags,
                    void* stream);

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
 * Sum / max over the innermost dimension of an fp32 [rows, inner] matrix into
 * out[rows].  Replace reduce_sum_inner_dim / reduce_max_inner_dim
 * (mx/cpp/funcs.cpp:219-231, mx/cpp/reduce.cu:15-89).  Any inner >= 1 is
 * accepted (the reference requires a multiple of 32).
 */
int mxq_reduce_sum_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream);
int mxq_reduce_max_inner(const void* in, void* out, int64_t rows, int64_t inner, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXQ_H */
