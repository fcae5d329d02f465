"""bfloat-emulated SiLU (reference: mx/activations.py:418-455 and its silu / SiLU
wrappers), and the sigmoid and tanh the LSTM cell is built from
(mx/activations.py:237-297).  The reference's other activations are outside the
scope of this package."""
import torch
import torch.nn.functional as F

from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import fused_bf16_ok, vec_add, vec_exp, vec_mul, vec_quantize, vec_recip, vec_sub, vec_tanh

f_silu = F.silu
torch_sigmoid, torch_tanh = torch.sigmoid, torch.tanh


class SiLUFunction(torch.autograd.Function):
    """y = x * sigmoid(x);  dy/dx = sigmoid(x) + y * (1 - sigmoid(x))."""

    @staticmethod
    def forward(ctx, input, inplace=False, mx_specs=None, name=None):
        sp = mx_specs
        if fused_bf16_ok(sp, input):
            from . import _backend
            if ctx.needs_input_grad[0]:
                out, sig = _backend.silu_bf16(input.contiguous(), None, want_sig=True)
            else:
                out, sig = _backend.silu_bf16(input.contiguous(), None), None
        else:
            q_in = vec_quantize(input, mx_specs=sp)
            sig = vec_recip(vec_add(vec_exp(-q_in, mx_specs=sp), 1.0, mx_specs=sp), mx_specs=sp)
            out = vec_mul(q_in, sig, mx_specs=sp)
        if inplace:
            ctx.mark_dirty(input)
            input.copy_(out)
            out = input
        if sig is not None:
            ctx.save_for_backward(out, sig)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        y, sig = ctx.saved_tensors
        sp = ctx.mx_specs
        g = vec_quantize(grad_output, mx_specs=sp)
        d = vec_add(sig, vec_mul(y, vec_sub(1.0, sig, mx_specs=sp), mx_specs=sp), mx_specs=sp)
        return (vec_mul(d, g, mx_specs=sp), None, None, None)


def silu(input, inplace=False, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_silu(input, inplace=inplace)
    return SiLUFunction.apply(input, inplace, apply_mx_specs(mx_specs), name)


class SiLU(torch.nn.SiLU):
    def __init__(self, inplace=False, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(inplace=inplace)

    def apply_mx_specs(self, mx_specs):
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def forward(self, input):
        if self.mx_none:
            return super().forward(input)
        return SiLUFunction.apply(input, self.inplace, self.mx_specs, self.name)


class SigmoidFunction(torch.autograd.Function):
    """y = 1 / (1 + exp(-x));  dy/dx = y * (1 - y)."""

    @staticmethod
    def forward(ctx, input, mx_specs=None, name=None):
        sp = mx_specs
        q = vec_quantize(input, mx_specs=sp)
        out = vec_recip(vec_add(vec_exp(-q, mx_specs=sp), 1.0, mx_specs=sp), mx_specs=sp)
        ctx.save_for_backward(out)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (y,) = ctx.saved_tensors
        sp = ctx.mx_specs
        g = vec_quantize(grad_output, mx_specs=sp)
        d = vec_mul(y, vec_sub(1, y, mx_specs=sp), mx_specs=sp)
        return (vec_mul(d, g, mx_specs=sp), None, None)


class TanhFunction(torch.autograd.Function):
    """y = tanh(x);  dy/dx = 1 - y * y."""

    @staticmethod
    def forward(ctx, input, mx_specs=None, name=None):
        out = vec_tanh(vec_quantize(input, mx_specs=mx_specs), mx_specs=mx_specs)
        ctx.save_for_backward(out)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (y,) = ctx.saved_tensors
        sp = ctx.mx_specs
        g = vec_quantize(grad_output, mx_specs=sp)
        d = vec_sub(1, vec_mul(y, y, mx_specs=sp), mx_specs=sp)
        return (vec_mul(d, g, mx_specs=sp), None, None)


def sigmoid(input, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch_sigmoid(input)
    return SigmoidFunction.apply(input, apply_mx_specs(mx_specs), name)


def tanh(input, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch_tanh(input)
    return TanhFunction.apply(input, apply_mx_specs(mx_specs), name)
