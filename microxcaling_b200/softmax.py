"""bfloat-emulated softmax (reference: mx/softmax.py:18-124): every step of
max-subtract, exp (or exp2), sum and divide is rounded to the vector format."""
import torch
import torch.nn.functional as F

from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import fused_bf16_ok, vec_div, vec_exp, vec_exp2, vec_mul, vec_quantize, vec_reduce_sum, vec_sub

f_softmax = F.softmax
LN_2_BF16 = 0.69140625
_SOFTMAX_FUSED_MAX_COLS = 2048      # row length the one-warp-per-row kernel keeps in registers


class SoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, dim=None, mx_specs=None, name=None):
        dim = dim + input.dim() if dim < 0 else dim
        ctx.dim = dim
        rnd = mx_specs["round"]
        if dim == input.dim() - 1 and fused_bf16_ok(mx_specs, input) and input.shape[-1] % 8 == 0 \
                and 0 < input.shape[-1] <= _SOFTMAX_FUSED_MAX_COLS:
            from . import _backend
            out = _backend.softmax_bf16(input.contiguous(), mx_specs.get("softmax_exp2", False))
        else:
            x = vec_quantize(input, mx_specs=mx_specs)
            x = vec_sub(x, x.max(dim, keepdim=True)[0], mx_specs=mx_specs, round=rnd)
            e = (vec_exp2 if mx_specs.get("softmax_exp2", False) else vec_exp)(x, mx_specs=mx_specs, round=rnd)
            s = vec_reduce_sum(e, dim, keepdim=True, mx_specs=mx_specs, round=rnd)
            out = vec_div(e, s, mx_specs=mx_specs, round=rnd)
        ctx.save_for_backward(out)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (out,) = ctx.saved_tensors
        sp = ctx.mx_specs
        rnd = sp["round"]
        g = vec_quantize(grad_output, mx_specs=sp, round=rnd)
        dot = vec_reduce_sum(vec_mul(g, out, mx_specs=sp, round=rnd), ctx.dim, keepdim=True, mx_specs=sp, round=rnd)
        gi = vec_mul(out, vec_sub(g, dot, mx_specs=sp, round=rnd), mx_specs=sp, round=rnd)
        if sp.get("softmax_exp2", False):
            gi = vec_mul(gi, LN_2_BF16, mx_specs=sp, round=rnd)
        return (gi, None, None, None)


def softmax(input, dim=-1, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_softmax(input, dim=dim)
    return SoftmaxFunction.apply(input, dim, apply_mx_specs(mx_specs), name)


class Softmax(torch.nn.Softmax):
    def __init__(self, dim=None, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(dim)

    def apply_mx_specs(self, mx_specs):
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def forward(self, input):
        if self.mx_none:
            return super().forward(input)
        return SoftmaxFunction.apply(input, self.dim, self.mx_specs, self.name)
