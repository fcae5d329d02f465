/*
 * ref_shim.cpp -- C entry points around the reference's own C++ quantization
 * code, compiled from the headers where they lie in the reference checkout
 * (mx/cpp/funcs.h, quantize.cuh, shared_exp.cuh, common.cuh); no reference
 * source is copied.  TEST INFRASTRUCTURE ONLY: used to validate the C oracle
 * and as the "reference" CPU baseline of the benchmark.
 *
 * The loops are the reference's: quantize_mx_cpp<T> (mx/cpp/funcs.h:61-100) is
 * called on slabs of the leading dimension from OpenMP threads (the reference
 * itself is single-threaded, mx/cpp/funcs.cpp:23-98); the per-block maximum it
 * needs is computed here the way the Python caller does (mx/mx_ops.py:247).
 */
#include <torch/extension.h>
#include <cstdint>
#include <cmath>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif
#include "funcs.h"

extern "C" {

/* fp32 [pre, axis_len, post]; blocks of `block` along the middle axis,
 * axis_len % block == 0 (the reference reshapes to blocks first,
 * mx/mx_ops.py:95-154). */
int mxref_quantize_mx_f32(const float* in, float* out, int64_t pre, int64_t axis_len,
                          int64_t post, int block, int scale_bits, int ebits, int mbits,
                          float max_norm, int flush, int rmode, int nthreads)
{
    if (block <= 0) block = (int)axis_len;
    if (axis_len % block) return -1;
    const int64_t nblk = axis_len / block;
    const int64_t outer = pre * nblk;            /* each outer slab is [block, post] */
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
    nthreads = 1;
#endif
    #pragma omp parallel num_threads(nthreads)
    {
        std::vector<float> mx((size_t)post);
        #pragma omp for schedule(static)
        for (int64_t o = 0; o < outer; ++o) {
            const float* a = in + o * block * post;
            float* b = out + o * block * post;
            for (int64_t j = 0; j < post; ++j) {
                float m = 0.0f;
                for (int k = 0; k < block; ++k) {
                    const float v = std::fabs(a[k * post + j]);
                    m = (v > m || std::isnan(v)) ? v : m;
                }
                mx[(size_t)j] = m;
            }
            quantize_mx_cpp<float>(a, scale_bits, ebits, mbits, max_norm, mx.data(),
                                   block, 1, (int)post, flush != 0,
                                   static_cast<RoundingMode>(rmode), b);
        }
    }
    return 0;
}

int mxref_quantize_elemwise_f32(const float* in, float* out, int64_t n, int bits, int exp_bits,
                                float max_norm, int rmode, int saturate, int allow_denorm,
                                int nthreads)
{
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
    nthreads = 1;
#endif
    #pragma omp parallel for num_threads(nthreads) schedule(static)
    for (int64_t i = 0; i < n; ++i)
        out[i] = quantize_elemwise(in[i], bits, exp_bits, max_norm,
                                   static_cast<RoundingMode>(rmode), saturate != 0, allow_denorm != 0);
    return 0;
}

float mxref_shared_scale(float absmax, int scale_bits, float max_norm)
{
    return mx_get_shared_scale(get_biased_exponent(absmax), scale_bits, max_norm);
}

int mxref_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
