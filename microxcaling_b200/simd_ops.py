"""Differentiable bfloat-emulated elementwise arithmetic with broadcasting
(reference: mx/simd_ops.py; add :75, sub :111, mul :154, div :204), the unary
operators (split :262, square :286, sqrt :311, exp :334, log :355) and the
reductions built on them (sum :382, mean :524, Frobenius norm :543)."""
import numpy as np
import torch

from ._autograd import call
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import vec_add, vec_div, vec_exp, vec_mul, vec_quantize, vec_reduce_sum, vec_sqrt, vec_sub

# stock callables captured before any injection replaces them
torch_sum, torch_mean, torch_log = torch.sum, torch.mean, torch.log


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
    """y = x1 / x2;  dy/dx1 = 1 / x2,  dy/dx2 = -y / x2 (formed from the rounded quotient, which is what the
    forward pass keeps)."""
    op = staticmethod(vec_div)

    @staticmethod
    def forward(ctx, in1, in2, mx_specs=None):
        out = SIMDDiv._fwd(ctx, in1, in2, mx_specs)
        if not ctx.in2_const:
            ctx.save_for_backward(out, vec_quantize(in2, mx_specs=mx_specs) if mx_specs["quantize_backprop"] else in2)
        return out

    @staticmethod
    def backward(ctx, g):
        sp = ctx.mx_specs
        g = vec_quantize(g, mx_specs=sp)
        if ctx.in2_const:
            return (vec_div(g, ctx.in2, mx_specs=sp), None, None)
        out, in2 = ctx.saved_tensors
        g1 = vec_div(g, in2, mx_specs=sp)
        g2 = vec_mul(g, vec_div(-out, in2, mx_specs=sp), mx_specs=sp)
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


class SIMDSplit(torch.autograd.Function):
    """Two copies of x; the gradient is the rounded sum of the two incoming gradients (one of them alone
    when the other branch has none)."""

    @staticmethod
    def forward(ctx, in1, mx_specs=None):
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        ctx.set_materialize_grads(False)
        return in1.clone(), in1.clone()

    @staticmethod
    def backward(ctx, g1, g2):
        if g1 is None or g2 is None:
            return (g2 if g1 is None else g1, None)
        sp = ctx.mx_specs
        return (vec_add(vec_quantize(g1, mx_specs=sp), vec_quantize(g2, mx_specs=sp), mx_specs=sp), None)


class _Unary(torch.autograd.Function):
    """y = f(q(x)), rounded; what the gradient needs is saved by the subclass's `keep`."""

    @classmethod
    def _fwd(cls, ctx, in1, mx_specs):
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        q = vec_quantize(in1, mx_specs=mx_specs)
        out = cls.f(q, mx_specs)
        ctx.save_for_backward(cls.keep(in1, q, out, mx_specs))
        return out


class SIMDSquare(_Unary):
    """y = x^2; dy/dx = 2 x."""
    f = staticmethod(lambda q, sp: vec_quantize(q ** 2, mx_specs=sp))
    keep = staticmethod(lambda x, q, y, sp: q if sp["quantize_backprop"] else x)

    @staticmethod
    def forward(ctx, in1, mx_specs=None):
        return SIMDSquare._fwd(ctx, in1, mx_specs)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        sp = ctx.mx_specs
        return (vec_mul(vec_quantize(g, mx_specs=sp), vec_mul(x, 2, mx_specs=sp), mx_specs=sp), None)


class SIMDSqrt(_Unary):
    """y = sqrt(x); dy/dx = 0.5 / y."""
    f = staticmethod(lambda q, sp: vec_sqrt(q, mx_specs=sp))
    keep = staticmethod(lambda x, q, y, sp: y)

    @staticmethod
    def forward(ctx, in1, mx_specs=None):
        return SIMDSqrt._fwd(ctx, in1, mx_specs)

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        sp = ctx.mx_specs
        return (vec_div(vec_mul(vec_quantize(g, mx_specs=sp), 0.5, mx_specs=sp), y, mx_specs=sp), None)


class SIMDExp(_Unary):
    """y = e^x; dy/dx = y."""
    f = staticmethod(lambda q, sp: vec_exp(q, mx_specs=sp))
    keep = staticmethod(lambda x, q, y, sp: y)

    @staticmethod
    def forward(ctx, in1, mx_specs=None):
        return SIMDExp._fwd(ctx, in1, mx_specs)

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        sp = ctx.mx_specs
        return (vec_mul(vec_quantize(g, mx_specs=sp), y, mx_specs=sp), None)


class SIMDLog(_Unary):
    """y = ln x; dy/dx = 1 / x."""
    f = staticmethod(lambda q, sp: vec_quantize(torch_log(q), mx_specs=sp))
    keep = staticmethod(lambda x, q, y, sp: q if sp["quantize_backprop"] else x)

    @staticmethod
    def forward(ctx, in1, mx_specs=None):
        return SIMDLog._fwd(ctx, in1, mx_specs)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        sp = ctx.mx_specs
        return (vec_div(vec_quantize(g, mx_specs=sp), x, mx_specs=sp), None)


class SIMDReduceSum(torch.autograd.Function):
    """y = sum of q(x) over `dim`, rounded; the gradient is the rounded incoming gradient expanded over the
    summed dimensions (a view: callers must not write into it)."""

    @staticmethod
    def forward(ctx, in1, dim, keepdim=False, mx_specs=None):
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        ctx.dim = [dim] if type(dim) == int else dim
        ctx.keepdim, ctx.input_shape = keepdim, list(in1.shape)
        return vec_reduce_sum(vec_quantize(in1, mx_specs=mx_specs), ctx.dim, keepdim=keepdim, mx_specs=mx_specs)

    @staticmethod
    def backward(ctx, g):
        n = len(ctx.input_shape)
        dims = sorted(d + n if d < 0 else d for d in ctx.dim)
        g = vec_quantize(g, mx_specs=ctx.mx_specs)
        if not ctx.keepdim:
            for d in dims:
                g = g.unsqueeze(d)
        return (g.expand([ctx.input_shape[i] if i in dims else -1 for i in range(n)]), None, None, None)


def simd_split(in1, mx_specs=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return in1, in1
    return SIMDSplit.apply(in1, apply_mx_specs(mx_specs))


def _wrap1(fn_cls, torch_fn):
    def f(in1, mx_specs=None):
        mx_assert_test(mx_specs)
        if mx_specs is None:
            return torch_fn(in1)
        return fn_cls.apply(in1, apply_mx_specs(mx_specs))
    return f


simd_square = _wrap1(SIMDSquare, torch.square)
simd_sqrt = _wrap1(SIMDSqrt, torch.sqrt)
simd_exp = _wrap1(SIMDExp, torch.exp)
simd_log = _wrap1(SIMDLog, torch.log)


def simd_reduce_sum(in1, dim=None, keepdim=False, mx_specs=None):
    mx_assert_test(mx_specs)
    if dim is None:
        dim = list(range(in1.ndim))
    if mx_specs is None:
        return torch_sum(in1, dim, keepdim=keepdim)
    return SIMDReduceSum.apply(in1, dim, keepdim, apply_mx_specs(mx_specs))


def simd_reduce_mean(in1, dim=None, keepdim=False, mx_specs=None):
    """Rounded sum times the reciprocal of the element count (one more rounding)."""
    mx_assert_test(mx_specs)
    if dim is None:
        dim = list(range(in1.ndim))
    if mx_specs is None:
        return torch_mean(in1, dim, keepdim=keepdim)
    sp = apply_mx_specs(mx_specs)
    dim = dim if type(dim) is list else [dim]
    count = np.prod([in1.shape[i] for i in dim])                  # 1.0 for an empty list
    return SIMDMul.apply(SIMDReduceSum.apply(in1, dim, keepdim, sp), 1 / count, sp)


def simd_norm(in1, keepdim=False, mx_specs=None):
    """Frobenius norm sqrt(sum(x^2)) over all dimensions, as torch.linalg.norm(x)."""
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch.linalg.norm(in1, keepdim=keepdim)
    sp = apply_mx_specs(mx_specs)
    sq = SIMDSquare.apply(in1, sp)
    return SIMDSqrt.apply(SIMDReduceSum.apply(sq, list(range(sq.ndim)), keepdim, sp), sp)
