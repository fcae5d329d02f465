"""bfloat-emulated activations, drop-ins for the reference's mx/activations.py: SiLU (:418-455, fused kernel
for bfloat16 CUDA tensors), sigmoid and tanh (:237-297), ReLU / ReLU6 / LeakyReLU (:300-415) and GELU in its
two sigmoid approximations (:458-560).  Every arithmetic step is followed by a rounding to the vector format of
mx_specs, in the reference's order."""
import torch
import torch.nn.functional as F

from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import fused_bf16_ok, vec_add, vec_exp, vec_mul, vec_quantize, vec_recip, vec_sub, vec_tanh

f_silu, f_relu, f_relu6, f_leaky_relu, f_gelu = F.silu, F.relu, F.relu6, F.leaky_relu, F.gelu
torch_sigmoid, torch_tanh, torch_relu = torch.sigmoid, torch.tanh, torch.relu   # F.relu itself calls torch.relu


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


class _ClampFunction(torch.autograd.Function):
    """ReLU (upper None) or ReLU6 (upper 6): clamp, round; the gradient passes where the OUTPUT lies strictly
    inside the clamp range (mx/activations.py:300-380)."""

    @staticmethod
    def forward(ctx, input, upper, inplace=False, mx_specs=None, name=None):
        clamp = torch_relu if upper is None else f_relu6
        out = vec_quantize(clamp(input), mx_specs=mx_specs)          # a mask needs no rounding of its input
        if inplace:
            ctx.mark_dirty(input)
            input.copy_(out)
            out = input
        mask = out > 0 if upper is None else torch.logical_and(out > 0, out < upper)
        ctx.save_for_backward(mask)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        gi = torch.where(mask, grad_output, torch.zeros([1], dtype=grad_output.dtype, device=grad_output.device))
        return (vec_quantize(gi, mx_specs=ctx.mx_specs), None, None, None, None)


class ReLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, inplace=False, mx_specs=None, name=None):
        return _ClampFunction.forward(ctx, input, None, inplace, mx_specs, name)

    @staticmethod
    def backward(ctx, grad_output):
        return _ClampFunction.backward(ctx, grad_output)[:1] + (None, None, None)


class ReLU6Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, inplace=False, mx_specs=None, name=None):
        return _ClampFunction.forward(ctx, input, 6, inplace, mx_specs, name)

    @staticmethod
    def backward(ctx, grad_output):
        return _ClampFunction.backward(ctx, grad_output)[:1] + (None, None, None)


class LeakyReLUFunction(torch.autograd.Function):
    """x for x > 0, slope * x otherwise; the gradient is dy or slope * dy by the sign of the output
    (mx/activations.py:383-415)."""

    @staticmethod
    def forward(ctx, input, negative_slope=0.01, inplace=False, mx_specs=None, name=None):
        ctx.negative_slope = negative_slope
        out = vec_quantize(f_leaky_relu(vec_quantize(input, mx_specs=mx_specs), negative_slope=negative_slope),
                           mx_specs=mx_specs)
        if inplace:
            ctx.mark_dirty(input)
            input.copy_(out)
            out = input
        ctx.save_for_backward(out > 0)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        sp = ctx.mx_specs
        g = vec_quantize(grad_output, mx_specs=sp)
        return (torch.where(mask, g, vec_mul(g, ctx.negative_slope, mx_specs=sp)), None, None, None, None)


# bfloat16 roundings of the constants of the two sigmoid forms of GELU (Hendrycks & Gimpel):
#   x * sigmoid(1.702 x)   and   x * sigmoid(1.5958 (x + 0.044715 x^3));  0.21406859 = 3 * 0.044715 * 1.5958
_G1, _G3, _GS, _GD = 1.703125, 0.044677734, 1.59375, 0.21386719


class GELUFunction(torch.autograd.Function):
    """y = x * phi, phi = sigmoid(u), u = 1.702 x (first order) or 1.5958 (x + 0.044715 x^3);
    dy/dx = phi + x * phi (1 - phi) u'  (mx/activations.py:458-560)."""

    @staticmethod
    def forward(ctx, input, mx_specs=None, first_order_gelu=False, name=None):
        sp = mx_specs
        ctx.first_order_gelu = first_order_gelu
        x = vec_quantize(input, mx_specs=sp)
        if first_order_gelu:
            u = vec_mul(_G1, x, mx_specs=sp)
        else:
            cube = vec_mul(vec_mul(x, x, mx_specs=sp), x, mx_specs=sp)
            u = vec_mul(_GS, vec_add(vec_mul(_G3, cube, mx_specs=sp), x, mx_specs=sp), mx_specs=sp)
        phi = vec_recip(vec_add(vec_exp(-u, mx_specs=sp), 1., mx_specs=sp), mx_specs=sp)
        ctx.save_for_backward(x if sp["quantize_backprop"] else input, phi)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return vec_mul(x, phi, mx_specs=sp)

    @staticmethod
    def backward(ctx, grad_output):
        x, phi = ctx.saved_tensors
        sp = ctx.mx_specs
        g = vec_quantize(grad_output, mx_specs=sp)
        dphi = vec_mul(phi, vec_sub(1, phi, mx_specs=sp), mx_specs=sp)
        if ctx.first_order_gelu:
            dphi = vec_mul(_G1, dphi, mx_specs=sp)
        else:
            du = vec_add(_GS, vec_mul(_GD, vec_mul(x, x, mx_specs=sp), mx_specs=sp), mx_specs=sp)
            dphi = vec_mul(du, dphi, mx_specs=sp)
        d = vec_add(phi, vec_mul(x, dphi, mx_specs=sp), mx_specs=sp)
        return (vec_mul(d, g, mx_specs=sp), None, None, None)


def relu(input, inplace=False, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_relu(input, inplace=inplace)
    return ReLUFunction.apply(input, inplace, apply_mx_specs(mx_specs), name)


def relu6(input, inplace=False, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_relu6(input, inplace=inplace)
    return ReLU6Function.apply(input, inplace, apply_mx_specs(mx_specs), name)


def leaky_relu(input, negative_slope=0.01, inplace=False, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_leaky_relu(input, negative_slope=negative_slope, inplace=inplace)
    return LeakyReLUFunction.apply(input, negative_slope, inplace, apply_mx_specs(mx_specs), name)


def gelu(input, mx_specs=None, first_order_gelu=False, approximate=None, name=None):
    """`approximate` only mirrors torch's signature: with mx_specs the tanh-equivalent sigmoid form (or the
    first-order one) is always used; without, torch's tanh approximation."""
    mx_assert_test(mx_specs)
    if mx_specs is None and not first_order_gelu:
        try:
            return f_gelu(input, approximate="tanh")
        except TypeError:
            return f_gelu(input)
    return GELUFunction.apply(input, apply_mx_specs(mx_specs), first_order_gelu, name)


class _MxAct:
    """Shared part of the module forms: torch's module when mx_specs is None, else the function above."""

    def _mx_init(self, mx_specs, name, mx_none=None):
        mx_assert_test(mx_specs)
        self.mx_none = (mx_specs is None) if mx_none is None else mx_none
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)

    def apply_mx_specs(self, mx_specs):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix


class Sigmoid(_MxAct, torch.nn.Sigmoid):
    def __init__(self, mx_specs=None, name=None):
        torch.nn.Sigmoid.__init__(self)
        self._mx_init(mx_specs, name)

    def forward(self, input):
        if self.mx_none:
            return torch.nn.Sigmoid.forward(self, input)
        return SigmoidFunction.apply(input, self.mx_specs, self.name)


class Tanh(_MxAct, torch.nn.Tanh):
    def __init__(self, mx_specs=None, name=None):
        torch.nn.Tanh.__init__(self)
        self._mx_init(mx_specs, name)

    def forward(self, input):
        if self.mx_none:
            return torch.nn.Tanh.forward(self, input)
        return TanhFunction.apply(input, self.mx_specs, self.name)


class ReLU(_MxAct, torch.nn.ReLU):
    def __init__(self, inplace=False, mx_specs=None, name=None):
        torch.nn.ReLU.__init__(self, inplace=inplace)
        self._mx_init(mx_specs, name)

    def forward(self, input):
        if self.mx_none:
            return torch.nn.ReLU.forward(self, input)
        return ReLUFunction.apply(input, self.inplace, self.mx_specs, self.name)


class ReLU6(_MxAct, torch.nn.ReLU6):
    def __init__(self, inplace=False, mx_specs=None, name=None):
        torch.nn.ReLU6.__init__(self, inplace=inplace)
        self._mx_init(mx_specs, name)

    def forward(self, input):
        if self.mx_none:
            return torch.nn.ReLU6.forward(self, input)
        return ReLU6Function.apply(input, self.inplace, self.mx_specs, self.name)


class LeakyReLU(_MxAct, torch.nn.LeakyReLU):
    def __init__(self, negative_slope=0.01, inplace=False, mx_specs=None, name=None):
        torch.nn.LeakyReLU.__init__(self, negative_slope=negative_slope, inplace=inplace)
        self._mx_init(mx_specs, name)

    def forward(self, input):
        if self.mx_none:
            return torch.nn.LeakyReLU.forward(self, input)
        return LeakyReLUFunction.apply(input, self.negative_slope, self.inplace, self.mx_specs, self.name)


class GELU(_MxAct, torch.nn.GELU):
    """torch's module (tanh approximation) when mx_specs is None and first_order_gelu is off; `approximate`
    only mirrors torch's signature."""

    def __init__(self, mx_specs=None, first_order_gelu=False, approximate=None, name=None):
        try:
            torch.nn.GELU.__init__(self, approximate="tanh")
        except TypeError:
            torch.nn.GELU.__init__(self)
        self._mx_init(mx_specs, name, mx_none=(mx_specs is None and not first_order_gelu))
        self.first_order_gelu = first_order_gelu

    def forward(self, input):
        if self.mx_none:
            return torch.nn.GELU.forward(self, input)
        return GELUFunction.apply(input, self.mx_specs, self.first_order_gelu, self.name)
