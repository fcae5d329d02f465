"""MX matmul: drop-in for the reference's mx/matmul.py (MatMulFunction :19-203,
matmul :206-217).  in1 [..., M, K] @ in2 [..., K, N] (or a shared [K, N]), with
`mode_config` choosing the activation / weight element format per operand."""
import numpy as np
import torch

from ._autograd import call
from ._mxgemm import mx_gemm
from .elemwise_ops import quantize_elemwise_op
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test

torch_matmul = torch.matmul
torch_addmm = torch.addmm


class MatMulFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, in1, in2, bias, mx_specs, name, mode_config="aa"):
        assert mode_config in ["aa", "aw", "wa"]
        ctx.mode_config = mode_config
        f1 = mx_specs["a_elem_format" if mode_config[0] == "a" else "w_elem_format"]
        f2 = mx_specs["a_elem_format" if mode_config[1] == "a" else "w_elem_format"]
        bf_in1 = quantize_elemwise_op(in1, mx_specs=mx_specs, round=mx_specs["round_output"])
        bf_in2 = quantize_elemwise_op(in2, mx_specs=mx_specs, round=mx_specs["round_output"])
        bf_bias = None
        ctx.bias_shape = None
        if bias is not None:
            bf_bias = quantize_elemwise_op(bias, mx_specs=mx_specs, round=mx_specs["round_weight"])
            ctx.bias_shape = list(bias.shape)
        if mx_specs["quantize_backprop"]:
            ctx.save_for_backward(bf_in1, bf_in2)
        else:
            ctx.save_for_backward(in1, in2)
        out = mx_gemm(bf_in1, bf_in2, f1, f2, mx_specs, mx_specs["round_mx_output"], mx_specs["round_mx_output"],
                      mx_specs["round_output"], bias=bf_bias)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        sp = ctx.mx_specs
        f1 = sp["a_elem_format_bp" if ctx.mode_config[0] == "a" else "w_elem_format_bp"]
        f2 = sp["a_elem_format_bp" if ctx.mode_config[1] == "a" else "w_elem_format_bp"]
        in1, in2 = ctx.saved_tensors
        grad_out = quantize_elemwise_op(grad_out, mx_specs=sp, round=sp["round_grad_input"])
        r_in = sp["round_mx_input_grad_input"]
        r_g = sp["round_mx_grad_output_grad_input"]
        # grad_in1 [..., M, K] = g [..., M, N] @ in2^T, blocks along N
        grad_in1 = mx_gemm(grad_out, in2, sp["a_elem_format_bp_os"], f2, sp, r_g, r_in, sp["round_grad_input"],
                           trans2=True)
        # grad_in2 [..., K, N] = in1^T @ g, blocks along M
        if in2.dim() == 2 and in1.dim() > 2:
            # shared right operand: the reference lets torch broadcast and autograd sum the
            # per-batch products; it blocks along M inside each batch element
            from .mx_ops import quantize_mx_op
            q1 = quantize_mx_op(in1, sp, elem_format=f1, axes=[-2], round=r_in)
            qg = quantize_mx_op(grad_out, sp, elem_format=sp["a_elem_format_bp_os"], axes=[-2], round=r_g)
            grad_in2 = quantize_elemwise_op(torch_matmul(q1.transpose(-1, -2), qg), mx_specs=sp,
                                            round=sp["round_grad_input"])
            grad_in2 = grad_in2.reshape(-1, *in2.shape).sum(0)
        else:
            grad_in2 = mx_gemm(in1, grad_out, f1, sp["a_elem_format_bp_os"], sp, r_in, r_g, sp["round_grad_input"],
                               trans1=True)
        grad_bias = None
        if ctx.bias_shape is not None:
            inner = grad_out.shape[-1]
            assert np.prod(ctx.bias_shape) == inner
            grad_bias = quantize_elemwise_op(grad_out.reshape(-1, inner).sum(0).reshape(ctx.bias_shape),
                                             mx_specs=sp, round=sp["round_grad_weight"])
        return (grad_in1, grad_in2, grad_bias, None, None, None)


def matmul(in1, in2, bias=None, mx_specs=None, name=None, mode_config="aa"):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch_matmul(in1, in2) if bias is None else torch_addmm(bias, in1, in2)
    mx_specs = apply_mx_specs(mx_specs)
    return call(MatMulFunction, in1, in2, bias, mx_specs, name, mode_config)
