"""Differentiable bfloat-emulated elementwise arithmetic with broadcasting
(reference: mx/simd_ops.py; add :75, sub :111, mul :154, div :204).  Only the
four binary operators are provided here."""
import torch

from ._autograd import call
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import vec_add, vec_div, vec_mul, vec_quantize, vec_sub

torch_sum = torch.sum


def _broadcast_gradient(grad_out, in_shape, mx_specs):
    """Gradient of y = broadcast(x): sum over the broadcast dims, with the
    summand and the sum rounded to the vector format."""
    if list(grad_out.shape) == list(in_shape):
        return grad_out
    assert grad_out.ndim >= len(in_shape)
    reduce_dims = []
    for i in range(grad_out.ndim):
        if i + 1 > len(in_shape):
            reduce_dims.append(-1 - i)
        elif grad_out.shape[-1 - i] != in_shape[-1 - i]:
            if in_shape[-1 - i] != 1:
                raise ValueError("simd gradient shape error: grad_out is %s and input is %s"
                                 % (tuple(grad_out.shape), tuple(in_shape)))
            reduce_dims.append(-1 - i)
    if reduce_dims:
        g = vec_quantize(grad_out, mx_specs=mx_specs)
        g = vec_quantize(torch_sum(g, dim=reduce_dims), mx_specs=mx_specs)
        return g.view(in_shape)
    return grad_out.view(in_shape)


class _Binary(torch.autograd.Function):
    """Shared forward: quantize both inputs, apply `op`, remember shapes."""
    op = None
    save_inputs = False

    @classmethod
    def _fwd(cls, ctx, in1, in2, mx_specs):
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        assert isinstance(in1, torch.Tensor)
        q1 = vec_quantize(in1, mx_specs=mx_specs)
        ctx.in2_const = not isinstance(in2, torch.Tensor)
        if ctx.in2_const:
            q2 = ctx.in2 = in2
            if cls.save_inputs:
                ctx.save_for_backward(q1 if mx_specs["quantize_backprop"] else in1)
        else:
            ctx.in1_shape, ctx.in2_shape = list(in1.shape), list(in2.shape)
            q2 = vec_quantize(in2, mx_specs=mx_specs)
            if cls.save_inputs:
                ctx.save_for_backward(*((q1, q2) if mx_specs["quantize_backprop"] else (in1, in2)))
        return cls.op(q1, q2, mx_specs=mx_specs)


class SIMDAdd(_Binary):
    op = staticmethod(vec_add)

    @staticmethod
    def forward(ctx, in1, in2, mx_specs=None):
        return SIMDAdd._fwd(ctx, in1, in2, mx_specs)

    @staticmethod
    def backward(ctx, g):
        g = vec_quantize(g, mx_specs=ctx.mx_specs)
        if ctx.in2_const:
            return (g, None, None)
        return (_broadcast_gradient(g, ctx.in1_shape, ctx.mx_specs),
                _broadcast_gradient(g, ctx.in2_shape, ctx.mx_specs), None)


class SIMDSub(_Binary):
    op = staticmethod(vec_sub)

    @staticmethod
    def forward(ctx, in1, in2, mx_specs=None):
        return SIMDSub._fwd(ctx, in1, in2, mx_specs)

    @staticmethod
    def backward(ctx, g):
        if ctx.in2_const:
            return (g, None, None)
        ng = vec_quantize(-g, mx_specs=ctx.mx_specs)
        return (_broadcast_gradient(g, ctx.in1_shape, ctx.mx_specs),
                _broadcast_gradient(ng, ctx.in2_shape, ctx.mx_specs), None)


class SIMDMul(_Binary):
    op = staticmethod(vec_mul)
    save_inputs = True

    @staticmethod
    def forward(ctx, in1, in2, mx_specs=None):
        return SIMDMul._fwd(ctx, in1, in2, mx_specs)

    @staticmethod
    def backward(ctx, g):
        sp = ctx.mx_specs
        g = vec_quantize(g, mx_specs=sp)
        if ctx.in2_const:
            return (vec_mul(g, ctx.in2, mx_specs=sp), None, None)
        in1, in2 = ctx.saved_tensors
        return (_broadcast_gradient(vec_mul(g, in2, mx_specs=sp), ctx.in1_shape, sp),
                _broadcast_gradient(vec_mul(g, in1, mx_specs=sp), ctx.in2_shape, sp), None)


class SIMDDiv(_Binary):
    op = staticmethod(vec_div)
    save_inputs = True

    @staticmethod
    def forward(ctx, in1, in2, mx_specs=None):
        return SIMDDiv._fwd(ctx, in1, in2, mx_specs)

    @staticmethod
    def backward(ctx, g):
        sp = ctx.mx_specs
        g = vec_quantize(g, mx_specs=sp)
        if ctx.in2_const:
            return (vec_div(g, ctx.in2, mx_specs=sp), None, None)
        in1, in2 = ctx.saved_tensors
        g1 = vec_div(g, in2, mx_specs=sp)                       # d/dx1 = 1/x2
        g2 = vec_mul(vec_div(-in1, vec_mul(in2, in2, mx_specs=sp), mx_specs=sp), g, mx_specs=sp)
        return (_broadcast_gradient(g1, ctx.in1_shape, sp), _broadcast_gradient(g2, ctx.in2_shape, sp), None)


def _wrap(fn_cls, torch_fn):
    def f(in1, in2, mx_specs=None):
        mx_assert_test(mx_specs)
        if mx_specs is None:
            return torch_fn(in1, in2)
        return call(fn_cls, in1, in2, apply_mx_specs(mx_specs))
    return f


simd_add = _wrap(SIMDAdd, torch.add)
simd_sub = _wrap(SIMDSub, torch.sub)
simd_mul = _wrap(SIMDMul, torch.mul)
simd_div = _wrap(SIMDDiv, torch.div)
