"""bfloat-emulated GroupNorm over (N, C, ...) inputs: the channels are split into groups and each group is
normalised over its channels and all spatial positions; drop-in for the reference's mx/groupnorm.py
(autograd function :16-78, function :81-90, module :93-120)."""
import torch
import torch.nn.functional as F

from .norm_utils import norm_backward, norm_forward
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import vec_mul, vec_quantize, vec_reduce_sum

f_group_norm = F.group_norm


class GroupNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, num_groups, weight, bias, eps, mx_specs=None, name=None):
        sp = mx_specs
        ctx.num_groups = num_groups
        x = vec_quantize(x, mx_specs=sp)
        bf_w = vec_quantize(weight, mx_specs=sp)
        r = norm_forward(x, list(range(1, x.ndim)), bf_w, vec_quantize(bias, mx_specs=sp), eps, sp,
                         groups=num_groups, weight_axis=1)
        ctx.save_for_backward(r.x_shift, r.x_norm, r.x_std_inv, bf_w if sp["quantize_backprop"] else weight)
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return r.output

    @staticmethod
    def backward(ctx, grad_output):
        sp = ctx.mx_specs
        x_shift, x_norm, x_std_inv, weight = ctx.saved_tensors
        not_channel = [0] + list(range(2, grad_output.ndim))
        g = vec_quantize(grad_output, mx_specs=sp)
        grad_bias = vec_reduce_sum(g, not_channel, mx_specs=sp)
        grad_weight = vec_reduce_sum(vec_mul(g, x_norm, mx_specs=sp), not_channel, mx_specs=sp)
        grad_input = norm_backward(g, list(range(1, g.ndim)), weight, x_shift, x_std_inv, sp,
                                   groups=ctx.num_groups, weight_axis=1)
        return (grad_input, None, grad_weight, grad_bias, None, None, None)


def group_norm(x, num_groups, weight, bias, eps=1e-5, mx_specs=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_group_norm(x, num_groups, weight=weight, bias=bias, eps=eps)
    return GroupNormFunction.apply(x, num_groups, weight, bias, eps, apply_mx_specs(mx_specs))


class GroupNorm(torch.nn.GroupNorm):
    def __init__(self, num_groups, num_channels, mx_specs=None, name=None, **kwargs):
        super().__init__(num_groups, num_channels, **kwargs)
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)

    def forward(self, input):
        if self.mx_none:
            return super().forward(input)
        return group_norm(input, self.num_groups, self.weight, self.bias, self.eps, self.mx_specs)
