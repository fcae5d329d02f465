"""Process-wide injection of the MX operators into the torch namespaces
(reference: mx/mx_mapping.py:26-122), with the reference's full function and
module tables.  Every mapped function and module takes `mx_specs`; the injected
wrappers supply it."""
from contextlib import contextmanager

import torch

from .activations import (GELU, LeakyReLU, ReLU, ReLU6, Sigmoid, SiLU, Tanh, gelu, leaky_relu, relu, relu6, sigmoid, silu,
                          tanh)
from .adaptive_avg_pooling import AdaptiveAvgPool2d, adaptive_avg_pool2d
from .batchnorm import BatchNorm1d, BatchNorm2d, BatchNorm3d, batch_norm
from .bmm import bmm
from .convolution import Conv1d, Conv2d, Conv3d, ConvTranspose2d, conv1d, conv2d, conv3d
from .groupnorm import GroupNorm, group_norm
from .layernorm import LayerNorm, layer_norm
from .linear import Linear, linear
from .matmul import MatMulFunction, matmul
from .rnn import LSTM
from .simd_ops import (simd_add, simd_div, simd_exp, simd_log, simd_mul, simd_norm, simd_reduce_mean, simd_reduce_sum,
                       simd_square, simd_sub)
from .softmax import Softmax, softmax
from .specs import apply_mx_specs

DEBUG = False
torch_addmm = torch.addmm


def tracer_decorator(func, mx_specs):
    def wrapper(*args, **kwargs):
        dtype = kwargs.pop("dtype", None)
        if DEBUG:
            print(func.__name__, mx_specs)
        res = func(*args, mx_specs=mx_specs, **kwargs)
        return res if dtype is None else res.to(dtype)
    return wrapper


def addmm_mx(bias, in1, in2, mx_specs=None, name=None):
    if mx_specs is None:
        return torch_addmm(bias, in1, in2)
    return MatMulFunction.apply(in1, in2, bias, apply_mx_specs(mx_specs), name)


MODULE_MAPPING = {
    "AdaptiveAvgPool2d": AdaptiveAvgPool2d, "BatchNorm1d": BatchNorm1d, "BatchNorm2d": BatchNorm2d,
    "BatchNorm3d": BatchNorm3d, "Conv1d": Conv1d, "Conv2d": Conv2d, "Conv3d": Conv3d,
    "ConvTranspose2d": ConvTranspose2d, "GELU": GELU, "GroupNorm": GroupNorm, "LSTM": LSTM, "LayerNorm": LayerNorm,
    "LeakyReLU": LeakyReLU, "Linear": Linear, "ReLU": ReLU, "ReLU6": ReLU6, "SiLU": SiLU, "Sigmoid": Sigmoid,
    "Softmax": Softmax, "Tanh": Tanh,
}
FUNCTION_MAPPING = {
    "adaptive_avg_pool2d": adaptive_avg_pool2d, "batch_norm": batch_norm, "conv1d": conv1d, "conv2d": conv2d,
    "conv3d": conv3d, "gelu": gelu, "group_norm": group_norm, "layer_norm": layer_norm, "leaky_relu": leaky_relu,
    "linear": linear, "relu": relu, "relu6": relu6, "sigmoid": sigmoid, "silu": silu, "softmax": softmax,
    "tanh": tanh,
    "add": simd_add, "sub": simd_sub, "mul": simd_mul, "div": simd_div, "exp": simd_exp, "log": simd_log,
    "sum": simd_reduce_sum, "mean": simd_reduce_mean, "norm": simd_norm, "square": simd_square,
    "matmul": matmul, "mm": matmul, "addmm": addmm_mx, "bmm": bmm,
}


def inject_pyt_ops(mx_specs):
    """Replace torch.<fn>, torch.nn.functional.<fn> and torch.nn.<Module> with
    the MX versions bound to `mx_specs`.  The MX operators captured the stock
    torch callables at import time, so there is no recursion."""
    def bind_module(cls):
        def __init__(self, *args, **kwargs):
            cls.__init__(self, *args, mx_specs=mx_specs, **kwargs)
        return type(f"{cls.__name__}_inj", (cls,), {"__init__": __init__})

    for k, v in FUNCTION_MAPPING.items():
        if k in torch.__dict__:
            torch.__dict__[k] = tracer_decorator(v, mx_specs)
        if k in torch.nn.functional.__dict__:
            torch.nn.functional.__dict__[k] = tracer_decorator(v, mx_specs)
    for k, v in MODULE_MAPPING.items():
        torch.nn.__dict__[k] = bind_module(v)


# The stock callables, captured when this module is imported (before any injection).
_STOCK = {"torch": {k: torch.__dict__[k] for k in FUNCTION_MAPPING if k in torch.__dict__},
          "functional": {k: torch.nn.functional.__dict__[k] for k in FUNCTION_MAPPING
                         if k in torch.nn.functional.__dict__},
          "nn": {k: torch.nn.__dict__[k] for k in MODULE_MAPPING}}


def restore_pyt_ops():
    """Undo inject_pyt_ops: put the stock torch callables and modules back (the reference has no
    counterpart; its injection lasts for the life of the process)."""
    torch.__dict__.update(_STOCK["torch"])
    torch.nn.functional.__dict__.update(_STOCK["functional"])
    torch.nn.__dict__.update(_STOCK["nn"])


@contextmanager
def injected(mx_specs):
    """`with injected(specs):` = inject_pyt_ops(specs) for the duration of the block."""
    inject_pyt_ops(mx_specs)
    try:
        yield
    finally:
        restore_pyt_ops()
