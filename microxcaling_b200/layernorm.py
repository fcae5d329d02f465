"""bfloat-emulated RMSNorm (reference: mx/layernorm.py:98-200, fused kernel for bfloat16 CUDA tensors) and
LayerNorm (mx/layernorm.py:17-96, 203-210)."""
import torch

from ._autograd import call
from .norm_utils import norm_backward_ln, norm_forward
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import (fused_bf16_ok, vec_add, vec_mul, vec_quantize, vec_recip, vec_reduce_mean, vec_reduce_sum,
                         vec_sqrt, vec_sub)


class RMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, mx_specs=None, name=None):
        sp = mx_specs
        if fused_bf16_ok(sp, x, weight, bias) and x.shape[-1] == weight.numel() == bias.numel():
            from . import _backend
            if any(ctx.needs_input_grad[:3]):
                out, x_norm, rms_inv = _backend.rmsnorm_bf16(x.contiguous(), weight.contiguous(), bias.contiguous(),
                                                             eps, want_saved=True)
            else:                                             # inference: nothing is kept for backward
                out = _backend.rmsnorm_bf16(x.contiguous(), weight.contiguous(), bias.contiguous(), eps)
                ctx.mx_specs = get_backwards_mx_specs(sp)
                return out
            bf_w = weight
        else:
            x = vec_quantize(x, mx_specs=sp)
            ms = vec_reduce_mean(vec_mul(x, x, mx_specs=sp), -1, keepdim=True, mx_specs=sp)
            rms_inv = vec_recip(vec_sqrt(vec_add(ms, eps, mx_specs=sp), mx_specs=sp), mx_specs=sp)
            x_norm = vec_mul(x, rms_inv, mx_specs=sp)
            bf_w = vec_quantize(weight, mx_specs=sp)
            bf_b = vec_quantize(bias, mx_specs=sp)
            out = vec_add(vec_mul(bf_w, x_norm, mx_specs=sp), bf_b, mx_specs=sp)
        ctx.save_for_backward(x_norm, rms_inv, bf_w if sp["quantize_backprop"] else weight)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        sp = ctx.mx_specs
        x_norm, rms_inv, weight = ctx.saved_tensors
        lead = list(range(grad_output.dim() - 1))
        g = vec_quantize(grad_output, mx_specs=sp)
        grad_bias = vec_reduce_sum(g, lead, mx_specs=sp)
        grad_weight = vec_reduce_sum(vec_mul(g, x_norm, mx_specs=sp), lead, mx_specs=sp)
        dx1 = vec_mul(vec_mul(g, weight, mx_specs=sp), rms_inv, mx_specs=sp)
        m = vec_reduce_mean(vec_mul(dx1, x_norm, mx_specs=sp), -1, keepdim=True, mx_specs=sp)
        grad_input = vec_sub(dx1, vec_mul(x_norm, m, mx_specs=sp))       # last step unrounded, as in the reference
        return (grad_input, grad_weight, grad_bias, None, None, None)


class RMSNorm(torch.nn.LayerNorm):
    def __init__(self, hidden_size, eps=1e-12, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(normalized_shape=hidden_size, eps=eps)

    def apply_mx_specs(self, mx_specs):
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def forward(self, x):
        return call(RMSNormFunction, x, self.weight, self.bias, self.eps, self.mx_specs, self.name)


torch_layer_norm = torch.nn.functional.layer_norm


class LayerNormFunction(torch.autograd.Function):
    """Normalisation over the last dimension, eps inside the square root; keeps the normalised input and
    (variance + eps) for the gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, mx_specs=None, name=None):
        sp = mx_specs
        bf_w = vec_quantize(weight, mx_specs=sp)
        r = norm_forward(vec_quantize(x, mx_specs=sp), -1, bf_w, vec_quantize(bias, mx_specs=sp), eps, sp)
        ctx.save_for_backward(r.x_norm, r.x_vare, bf_w if sp["quantize_backprop"] else weight)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return r.output

    @staticmethod
    def backward(ctx, grad_output):
        sp = ctx.mx_specs
        x_norm, x_vare, weight = ctx.saved_tensors
        lead = list(range(grad_output.ndim - 1))
        g = vec_quantize(grad_output, mx_specs=sp)
        grad_bias = vec_reduce_sum(g, lead, mx_specs=sp)
        grad_weight = vec_reduce_sum(vec_mul(g, x_norm, mx_specs=sp), lead, mx_specs=sp)
        return (norm_backward_ln(g, -1, weight, x_norm, x_vare, sp), grad_weight, grad_bias, None, None, None)


class LayerNorm(torch.nn.LayerNorm):
    def __init__(self, hidden_size, eps=1e-12, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(normalized_shape=hidden_size, eps=eps)

    def apply_mx_specs(self, mx_specs):
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def forward(self, x):
        if self.mx_none:
            return super().forward(x)
        return LayerNormFunction.apply(x, self.weight, self.bias, self.eps, self.mx_specs, self.name)


def layer_norm(input, normalized_shape, weight, bias, eps=1e-12, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return torch_layer_norm(input, normalized_shape, weight, bias, eps)
    assert normalized_shape == weight.shape
    return LayerNormFunction.apply(input, weight, bias, eps, apply_mx_specs(mx_specs), name)
