"""bfloat-emulated adaptive average pooling over the last two dimensions of a [B, C, H, W] tensor; drop-in for
the reference's mx/adaptive_avg_pooling.py (function :20-26, module :32-47, autograd function :62-146).

Output cell (i, j) is the mean, rounded to the vector format, of the input window rows
[floor(i H / h), ceil((i + 1) H / h)) x columns [floor(j W / w), ceil((j + 1) W / w)).  The gradient of a cell is
spread evenly over its window (divided by the window's height, then by its width, unrounded) and added, with a
rounding per window, in row-major order of the cells; windows overlap when H is not a multiple of h.  Like the
reference, the result and the input gradient are allocated in torch's default dtype."""
import math

import torch
import torch.nn.functional as F

from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import vec_add, vec_reduce_mean

f_adaptive_avg_pool2d = F.adaptive_avg_pool2d


def _windows(n_out, n_in):
    """[(start, stop)] of the n_out pooling windows along an axis of n_in elements."""
    return [(math.floor(float(i) * float(n_in) / n_out), math.ceil(float(i + 1) * float(n_in) / n_out))
            for i in range(n_out)]


def _output_hw(output_size, H, W):
    if isinstance(output_size, tuple) and len(output_size) == 2:
        return output_size[0] or H, output_size[1] or W          # None keeps the input size
    if isinstance(output_size, int):
        return output_size, output_size
    if output_size is None:
        return H, W
    raise ValueError("expected 1D or 2D output_size (got {}D output_size)".format(len(output_size)))


class AdaptiveAvgPool2dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, output_size, mx_specs=None, name=None):
        B, C, H, W = input.size()
        h, w = _output_hw(output_size, H, W)
        if input.dim() != 4:
            raise ValueError("expected 4D input (got {}D input)".format(input.dim()))
        rows, cols = _windows(h, H), _windows(w, W)
        out = torch.zeros(B, C, h, w, device=input.device)
        for i, (r0, r1) in enumerate(rows):
            for j, (c0, c1) in enumerate(cols):
                out[:, :, i, j] = vec_reduce_mean(input[:, :, r0:r1, c0:c1], [2, 3], keepdim=False, mx_specs=mx_specs)
        ctx.geometry = (B, C, H, W, rows, cols, input.device)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        B, C, H, W, rows, cols, device = ctx.geometry
        gi = torch.zeros(B, C, H, W, device=device)
        for i, (r0, r1) in enumerate(rows):
            for j, (c0, c1) in enumerate(cols):
                share = (grad_output[:, :, i, j] / (r1 - r0) / (c1 - c0))[:, :, None, None]
                gi[:, :, r0:r1, c0:c1] = vec_add(gi[:, :, r0:r1, c0:c1], share.expand(B, C, r1 - r0, c1 - c0),
                                                 mx_specs=ctx.mx_specs)
        return (gi, None, None, None)


def adaptive_avg_pool2d(input, output_size, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_adaptive_avg_pool2d(input, output_size)
    return AdaptiveAvgPool2dFunction.apply(input, output_size, apply_mx_specs(mx_specs), name)


class AdaptiveAvgPool2d(torch.nn.Module):
    def __init__(self, output_size, mx_specs=None, name=None):
        super().__init__()
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.output_size = output_size
        self.mx_specs = apply_mx_specs(mx_specs)
        self.name = name

    def forward(self, inputs):
        if self.mx_none:
            return f_adaptive_avg_pool2d(inputs, self.output_size)
        return AdaptiveAvgPool2dFunction.apply(inputs, self.output_size, self.mx_specs, self.name)
