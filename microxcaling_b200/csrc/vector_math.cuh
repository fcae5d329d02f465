// Per-element pieces of the bfloat16 vector chains: an fp32 operation followed by
// a round-to-nearest-even to bfloat16, as every vector operation of the reference
// behaves on bfloat16 CUDA tensors (mx/vector_ops.py:38-130 with bfloat = 16).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mxq {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// fp32 -> nearest-even bfloat16, as a float
__device__ __forceinline__ float rb(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);   // both already on the bf16 grid
}

// two fp32 values -> packed pair of nearest-even bfloat16 (lo in bits 0..15): one conversion instruction
__device__ __forceinline__ uint32_t rb2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// sigmoid and SiLU of one bfloat16 value q with every intermediate rounded to
// bfloat16: e = exp(-q), a = e + 1, s = 1 / a, y = q * s  (mx/activations.py:428-434)
__device__ __forceinline__ void silu_chain(float q, float& s, float& y) {
    const float e = rb(expf(-q));
    const float a = rb(e + 1.0f);
    s = rb(__frcp_rn(a));                 // correctly rounded, hence equal to 1.0f / a
    y = rb(q * s);
}

// Device table of the sigmoid chain for every bfloat16 bit pattern (64 Ki entries of 2 bytes), built on
// first use on the current device by running silu_chain on each pattern; nullptr on failure.
const uint16_t* sigmoid_table();
// The same for exp rounded to bfloat16 (the numerator of the softmax chain, mx/softmax.py:28-33).
const uint16_t* exp_table();

}  // namespace mxq
