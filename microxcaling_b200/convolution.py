"""MX convolutions: drop-in for the reference's mx/convolution.py (ConvFunction :107-300,
conv1d/2d/3d :303-389, Conv1d/2d/3d :392-end) and mx/transpose_convolution.py
(ConvTranspose2dFunction :17-212, ConvTranspose2d).

The convolution itself stays torch's (cuDNN); what this package contributes is the
quantization around it, which on CUDA tensors runs the sm_100a MX kernels:

  forward      input and weight MX-quantized along in_channels (axis 1 of both; for the
               transposed convolution the weight is [in, out/groups, ...], axis 0), output
               rounded to the vector format
  grad_weight  input and grad_output MX-quantized along the batch axis
  grad_input   weight along out_channels, grad_output along its channel axis
"""
import torch
import torch.nn.functional as F
from torch.nn import grad as nn_grad

from .elemwise_ops import quantize_elemwise_op
from .mx_ops import quantize_mx_op
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test

_FWD = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}
_GRAD_IN = {1: nn_grad.conv1d_input, 2: nn_grad.conv2d_input, 3: nn_grad.conv3d_input}
_GRAD_W = {1: nn_grad.conv1d_weight, 2: nn_grad.conv2d_weight, 3: nn_grad.conv3d_weight}
f_conv_transpose2d = F.conv_transpose2d
f_conv2d = F.conv2d


def conv_weight(input, weight_shape, grad_output, stride=1, padding=0, dilation=1, groups=1):
    """Gradient of an N-d convolution with respect to its weight (torch.nn.grad.convNd_weight)."""
    nd = input.ndim - 2
    if nd not in _GRAD_W:
        raise ValueError("conv_weight does not work with input with ndim=%d" % input.ndim)
    return _GRAD_W[nd](input, weight_shape, grad_output, stride=stride, padding=padding, dilation=dilation,
                       groups=groups)


def _q(x, sp, key):
    return quantize_elemwise_op(x, mx_specs=sp, round=sp[key])


class ConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, mx_specs=None, name=None):
        nd = input.ndim - 2
        assert nd in (1, 2, 3)
        assert input.shape[1] % groups == 0
        sp = mx_specs
        ctx.geom = dict(stride=stride, padding=padding, dilation=dilation, groups=groups)
        ctx.has_bias, ctx.nd, ctx.name = bias is not None, nd, name
        x, w = _q(input, sp, "round_output"), _q(weight, sp, "round_weight")
        b = _q(bias, sp, "round_weight") if bias is not None else None
        ctx.save_for_backward(*((x, w) if sp["quantize_backprop"] else (input, weight)))
        qx = quantize_mx_op(x, sp, elem_format=sp["a_elem_format"], axes=[1])
        qw = quantize_mx_op(w, sp, elem_format=sp["w_elem_format"], axes=[1])
        out = _q(_FWD[nd](qx, qw, b, stride, padding, dilation, groups), sp, "round_output")
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.shape[1] % ctx.geom["groups"] == 0
        input, weight = ctx.saved_tensors
        sp = ctx.mx_specs
        g = _q(grad_output, sp, "round_grad_input")
        af, wf = sp["a_elem_format"], sp["w_elem_format"]
        # grad_weight: reduction over the batch axis
        gw = conv_weight(quantize_mx_op(input, sp, elem_format=af, axes=[0]), weight.shape,
                         quantize_mx_op(g, sp, elem_format=af, axes=[0]), **ctx.geom)
        gw = _q(gw, sp, "round_grad_weight")
        # grad_input: reduction over out_channels
        gi = _GRAD_IN[ctx.nd](input.shape, quantize_mx_op(weight, sp, elem_format=wf, axes=[0]),
                              quantize_mx_op(g, sp, elem_format=af, axes=[1]), **ctx.geom)
        gi = _q(gi, sp, "round_grad_input")
        gb = None
        if ctx.has_bias:
            gb = _q(g.sum([0] + list(range(2, g.ndim))), sp, "round_grad_weight")
        return (gi, gw, gb, None, None, None, None, None, None)


def _conv_fn(nd):
    stock = _FWD[nd]

    def conv(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        if mx_specs is None:
            return stock(input, weight, bias=bias, stride=stride, padding=padding, dilation=dilation, groups=groups)
        return ConvFunction.apply(input, weight, bias, stride, padding, dilation, groups, apply_mx_specs(mx_specs), name)
    conv.__name__ = "conv%dd" % nd
    return conv


conv1d, conv2d, conv3d = _conv_fn(1), _conv_fn(2), _conv_fn(3)


def _conv_module(base, fn):
    class Conv(base):
        def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                     bias=True, mx_specs=None, name=None):
            mx_assert_test(mx_specs)
            self.mx_none = mx_specs is None
            self.name = name
            self.mx_specs = apply_mx_specs(mx_specs)
            super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias)

        def apply_mx_specs(self, mx_specs):
            mx_assert_test(mx_specs)
            self.mx_none = mx_specs is None
            self.mx_specs = apply_mx_specs(mx_specs)

        def append_name(self, postfix):
            self.name += postfix

        def forward(self, inputs):
            if self.mx_none:
                return super().forward(inputs)
            return fn(inputs, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups,
                      mx_specs=self.mx_specs, name=self.name)
    Conv.__name__ = Conv.__qualname__ = base.__name__
    return Conv


Conv1d = _conv_module(torch.nn.Conv1d, conv1d)
Conv2d = _conv_module(torch.nn.Conv2d, conv2d)
Conv3d = _conv_module(torch.nn.Conv3d, conv3d)


class ConvTranspose2dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1,
                mx_specs=None, name=None):
        assert input.shape[1] % groups == 0
        sp = mx_specs
        ctx.geom = dict(stride=stride, padding=padding, dilation=dilation, groups=groups)
        ctx.has_bias, ctx.name = bias is not None, name
        x, w = _q(input, sp, "round_output"), _q(weight, sp, "round_weight")
        b = _q(bias, sp, "round_weight") if bias is not None else None
        ctx.save_for_backward(*((x, w) if sp["quantize_backprop"] else (input, weight)))
        qx = quantize_mx_op(x, sp, elem_format=sp["a_elem_format"], axes=[1])
        qw = quantize_mx_op(w, sp, elem_format=sp["w_elem_format"], axes=[0])       # weight is [in, out/groups, kH, kW]
        out = _q(f_conv_transpose2d(qx, qw, b, stride, padding, output_padding, groups, dilation), sp, "round_output")
        ctx.mx_specs = get_backwards_mx_specs(sp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.shape[1] % ctx.geom["groups"] == 0
        input, weight = ctx.saved_tensors
        sp = ctx.mx_specs
        g = _q(grad_output, sp, "round_grad_input")
        af, wf = sp["a_elem_format"], sp["w_elem_format"]
        # the transposed convolution is the input-gradient of a convolution from its output to its input
        gw = conv_weight(quantize_mx_op(g, sp, elem_format=af, axes=[0]), weight.shape,
                         quantize_mx_op(input, sp, elem_format=af, axes=[0]), **ctx.geom)
        gw = _q(gw, sp, "round_grad_weight")
        gi = f_conv2d(quantize_mx_op(g, sp, elem_format=af, axes=[1]), quantize_mx_op(weight, sp, elem_format=wf, axes=[1]),
                      bias=None, **ctx.geom)
        gi = _q(gi, sp, "round_grad_input")
        gb = _q(g.sum(dim=(3, 2, 0)), sp, "round_grad_weight") if ctx.has_bias else None
        return (gi, gw, gb, None, None, None, None, None, None, None)


def conv_transpose2d(input, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1,
                     mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_conv_transpose2d(input, weight, bias, stride, padding, output_padding, groups, dilation)
    return ConvTranspose2dFunction.apply(input, weight, bias, stride, padding, output_padding, groups, dilation,
                                         apply_mx_specs(mx_specs), name)


class ConvTranspose2d(torch.nn.ConvTranspose2d):
    """Argument order of the reference's module (dilation before groups); zero padding mode."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, dilation=1,
                 groups=1, bias=True, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=padding,
                         output_padding=output_padding, groups=groups, bias=bias, dilation=dilation)

    def apply_mx_specs(self, mx_specs):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def forward(self, inputs, output_size=None):
        if self.mx_none:
            return super().forward(inputs, output_size)
        output_padding = self._output_padding(inputs, output_size, self.stride, self.padding, self.kernel_size, 2,
                                              self.dilation)
        return conv_transpose2d(inputs, self.weight, self.bias, self.stride, self.padding, output_padding,
                                self.groups, self.dilation, mx_specs=self.mx_specs, name=self.name)
