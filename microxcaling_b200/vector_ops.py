"""Non-differentiable vector primitives: a torch op followed by a rounding to
the vector format of mx_specs (bfloat / fp).  Same names and semantics as the
reference's mx/vector_ops.py:38-130."""
import numpy as np
import torch

from .elemwise_ops import quantize_elemwise_op

torch_exp, torch_exp2, torch_sqrt, torch_tanh = torch.exp, torch.exp2, torch.sqrt, torch.tanh
LN_2_EXACT = 0.69314718056
LOG2_E_BF16 = 1.4453125         # log2(e) rounded to bfloat16


def _q(x, mx_specs, round):
    return quantize_elemwise_op(x, mx_specs=mx_specs, round=round)


def fused_bf16_ok(mx_specs, *tensors):
    """True when a chain of vector ops on these tensors is 'fp32 op, round to
    nearest-even bfloat16' at every step, i.e. bfloat16 CUDA tensors whose
    vector format (bfloatX, X >= 16) leaves bfloat16 values untouched; such
    chains have fused kernels in libmxq (mxq_silu_bf16, mxq_rmsnorm_bf16)."""
    sp = mx_specs
    if not sp or sp["fp"] > 0 or sp["bfloat"] < 16 or not sp["bfloat_subnorms"]:
        return False
    if sp["round"] not in ("nearest", "floor", "even") or sp["vec_use_exp2"] or sp["vec_use_recip"]:
        return False
    return all(t is not None and t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


def vec_quantize(input, mx_specs=None, round=None):
    return _q(input, mx_specs, round)


def vec_add(a, b, mx_specs=None, round=None):
    return _q(a + b, mx_specs, round)


def vec_sub(a, b, mx_specs=None, round=None):
    return _q(a - b, mx_specs, round)


def vec_mul(a, b, mx_specs=None, round=None):
    return _q(a * b, mx_specs, round)


def vec_recip(input, mx_specs=None, round=None):
    return _q(1.0 / input, mx_specs, round)


def vec_div(a, b, mx_specs=None, round=None):
    if mx_specs and mx_specs["vec_use_recip"]:
        return vec_mul(a, vec_recip(b, mx_specs=mx_specs, round=round), mx_specs=mx_specs, round=round)
    return _q(a / b, mx_specs, round)


def vec_exp2(input, mx_specs=None, round=None):
    return _q(torch_exp2(input), mx_specs, round)


def vec_exp(input, mx_specs=None, round=None):
    if mx_specs and mx_specs["vec_use_exp2"]:
        return vec_exp2(_q(LOG2_E_BF16 * input, mx_specs, round), mx_specs=mx_specs, round=round)
    return _q(torch_exp(input), mx_specs, round)


def vec_sqrt(input, mx_specs=None, round=None):
    return _q(torch_sqrt(input), mx_specs, round)


def vec_tanh(input, mx_specs=None, round=None):
    return _q(torch_tanh(input), mx_specs, round)


def vec_reduce_sum(input, dim, keepdim=False, mx_specs=None, round=None):
    return _q(input.sum(dim, keepdim=keepdim), mx_specs, round)


def vec_reduce_mean(input, dim, keepdim=False, mx_specs=None, round=None):
    dims = dim if type(dim) is list else [dim]
    denom = np.prod([input.shape[i] for i in dims])
    s = vec_reduce_sum(input, dims, keepdim=keepdim, mx_specs=mx_specs, round=round)
    return vec_div(s, denom, mx_specs=mx_specs, round=round)
