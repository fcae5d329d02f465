"""Context manager kept for API compatibility with the reference's
mx/matmul_precision.py:38-53.  There it switches torch's fp32 matmul to bf16
inputs when both element formats fit bf16 exactly.  Here products of FP formats
with block size 32 run on the block-scaled tensor cores and never consult this
flag; the remaining products (fixed-point formats, other block sizes) follow the
reference's construction, a torch GEMM on fake-quantized values inside this
manager.  The global torch settings are restored on exit, also on exceptions."""
from contextlib import contextmanager

import torch

from .formats import ElemFormat

_NARROW = (ElemFormat.int4, ElemFormat.int2, ElemFormat.fp6_e3m2, ElemFormat.fp6_e2m3, ElemFormat.fp4)


def get_elem_format(inp):
    if inp is None:
        return "Unknown"
    return ElemFormat.from_str(inp) if type(inp) is str else inp


@contextmanager
def set_matmul_precision(a, b, a_elem_format, b_elem_format, force_bf16=False):
    fa, fb = get_elem_format(a_elem_format), get_elem_format(b_elem_format)
    prev = torch.get_float32_matmul_precision()
    prev_red = torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction
    try:
        if a.is_cuda and b.is_cuda and torch.cuda.is_bf16_supported() and \
                ((fa in _NARROW and fb in _NARROW) or force_bf16):
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
            torch.set_float32_matmul_precision("medium")
        yield
    finally:
        torch.set_float32_matmul_precision(prev)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = prev_red
