"""MX bmm: drop-in for the reference's mx/bmm.py (BMMFunction :18-135, bmm
:138-145).  Like torch.bmm but with any number of leading dims; both operands
use the activation element format."""
import torch

from ._autograd import call
from ._mxgemm import mx_gemm
from .elemwise_ops import quantize_elemwise_op
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test

torch_bmm = torch.bmm


class BMMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, in1, in2, mx_specs, name):
        bf_in1 = quantize_elemwise_op(in1, mx_specs=mx_specs, round=mx_specs["round_output"])
        bf_in2 = quantize_elemwise_op(in2, mx_specs=mx_specs, round=mx_specs["round_output"])
        if mx_specs["quantize_backprop"]:
            ctx.save_for_backward(bf_in1, bf_in2)
        else:
            ctx.save_for_backward(in1, in2)
        f = mx_specs["a_elem_format"]
        out = mx_gemm(bf_in1, bf_in2, f, f, mx_specs, mx_specs["round_mx_output"], mx_specs["round_mx_output"],
                      mx_specs["round_output"])
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        sp = ctx.mx_specs
        in1, in2 = ctx.saved_tensors
        grad_out = quantize_elemwise_op(grad_out, mx_specs=sp, round=sp["round_grad_input"])
        r_in, r_g = sp["round_mx_input_grad_input"], sp["round_mx_grad_output_grad_input"]
        grad_in1 = mx_gemm(grad_out, in2, sp["a_elem_format_bp_os"], sp["a_elem_format_bp"], sp, r_g, r_in,
                           sp["round_grad_input"], trans2=True)
        grad_in2 = mx_gemm(in1, grad_out, sp["a_elem_format_bp"], sp["a_elem_format_bp_os"], sp, r_in, r_g,
                           sp["round_grad_input"], trans1=True)
        return (grad_in1, grad_in2, None, None)


def bmm(in1, in2, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch_bmm(in1, in2)
    mx_specs = apply_mx_specs(mx_specs)
    return call(BMMFunction, in1, in2, mx_specs, name)
