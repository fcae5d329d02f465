"""Differentiable bfloat quantization (reference: mx/quantize.py:14-48): the
forward value and the incoming gradient are both rounded to the vector format."""
import torch

from .elemwise_ops import quantize_elemwise_op
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test


class QuantizeBfloatFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mx_specs, round=None):
        round = mx_specs["round"] if round is None else round
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        ctx.round = round
        return quantize_elemwise_op(x, mx_specs=mx_specs, round=round)

    @staticmethod
    def backward(ctx, grad_output):
        return (quantize_elemwise_op(grad_output, mx_specs=ctx.mx_specs, round=ctx.round), None, None)


def quantize_bfloat(x, mx_specs, round=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return x
    mx_specs = apply_mx_specs(mx_specs)
    return QuantizeBfloatFunction.apply(x, mx_specs, mx_specs["round"] if round is None else round)
