"""Shared GEMM plumbing of mx.linear / mx.matmul / mx.bmm.

`mx_gemm` computes op1(in1) @ op2(in2) with each operand MX-quantized along
its contraction axis and the result rounded to the vector format of mx_specs.
On CUDA tensors with FP element formats and block size 32 it runs as
quantize-to-packed-operand kernels plus the tcgen05 block-scaled GEMM; every
other case (CPU tensors, fixed-point formats, odd block sizes, contraction
length not a multiple of 32) follows the reference's construction: fake-quantize
both operands, multiply with torch, round the result
(mx/linear.py:62-96, mx/matmul.py:68-96, mx/bmm.py:40-62).
"""
import torch

from .elemwise_ops import quantize_elemwise_op
from .formats import ElemFormat, _get_format_params
from .matmul_precision import set_matmul_precision
from .mx_ops import quantize_mx_op
from .packed import PackedMX, packed_note

_MODE = {"nearest": 0, "floor": 1, "even": 2}
_torch_matmul = torch.matmul


def _fmt(f):
    if f is None:
        return None
    return ElemFormat.from_str(f) if isinstance(f, str) else f


def _fast_ok(in1, in2, f1, f2, specs, K, r1, r2, out_round):
    if not (in1.is_cuda and in2.is_cuda) or f1 is None or f2 is None:
        return False
    if in1.dtype != in2.dtype or in1.dtype not in (torch.bfloat16, torch.float32, torch.float16):
        return False
    if specs["block_size"] != 32 or K % 32 != 0 or specs["shared_exp_method"] != "max":
        return False
    if specs["fp"] > 0 or (0 < specs["bfloat"] < 10):
        return False
    for f in (f1, f2):
        ebits, mbits, _, _, _ = _get_format_params(f)
        if ebits == 0 or mbits > 5:          # fixed point and wide formats have no fp8 container
            return False
    return r1 in _MODE and r2 in _MODE and out_round in _MODE


_CFMT = {}


def _cfmt(fmt, rnd):
    """struct mxq_elem_format of an element format (one-byte float container) and an MX rounding mode."""
    key = (fmt, rnd)
    c = _CFMT.get(key)
    if c is None:
        from . import _backend as be
        ebits, mbits, _, max_norm, _ = _get_format_params(fmt)
        c = _CFMT[key] = be.ElemFormatC(ebits, mbits, max_norm, _MODE[rnd])
    return c


def _pack(x, fmt, specs, rnd, contraction_last):
    """x [..., R, K] (contraction_last) or [..., K, R] -> PackedMX with batch = the leading dimensions."""
    return PackedMX.quantize(x, fmt, specs, round=rnd, contraction_last=contraction_last)


def mx_gemm(in1, in2, fmt1, fmt2, specs, round1, round2, out_round, bias=None, trans1=False, trans2=False,
            in1_packed=None, in2_packed=None):
    """op1(in1) @ op2(in2), op(x) = x^T of the last two dims when trans is set.

    in1: [..., M, K] (or [..., K, M] with trans1); in2: [..., K, N] (or [..., N, K] with trans2),
    in2 may have fewer leading dims than in1 (a shared 2-D matrix).  `bias` is an
    already-quantized vector added after the first output rounding.  `in1_packed` /
    `in2_packed`: a PackedMX holding the operand already quantized with (fmt, round) along the
    contraction axis (a frozen layer weight, or probabilities packed by the fused softmax);
    the tensor argument then only supplies shape, dtype and device."""
    fmt1, fmt2 = _fmt(fmt1), _fmt(fmt2)
    M, K = (in1.shape[-1], in1.shape[-2]) if trans1 else (in1.shape[-2], in1.shape[-1])
    N, K2 = (in2.shape[-2], in2.shape[-1]) if trans2 else (in2.shape[-1], in2.shape[-2])
    assert K == K2, "contraction sizes differ"
    lead1, lead2 = in1.shape[:-2], in2.shape[:-2]
    shared_b = len(lead2) == 0 and len(lead1) > 0
    fast = _fast_ok(in1, in2, fmt1, fmt2, specs, K, round1, round2, out_round) and in1.numel() > 0 and in2.numel() > 0
    if fast and not shared_b and tuple(lead1) != tuple(lead2):
        fast = False                          # general broadcasting: reference construction
    if fast and shared_b and trans1:
        fast = False
    if fast:
        from . import _backend as be
        if shared_b:
            batch, rows = 1, in1.numel() // K       # leading dims of in1 fold into M
        else:
            batch, rows = (in1.numel() // (M * K)), M
        a = in1_packed
        if a is None and not trans1:
            # probabilities packed by the fused softmax carry their packing along
            a = packed_note(in1, fmt1, round1, specs)
            if a is not None and shared_b and a.rows % 128 != 0:
                a = None                        # scale chunks were laid out per batch element
        bits = specs["bfloat"] if specs["bfloat"] >= 10 else 0
        if in2_packed is None and (a is not None or not trans1 or M % 4 == 0) and (trans2 or N % 4 == 0):
            # both packings and the GEMM as one library call (a third of the host time of three calls)
            if a is not None and (a.batch * a.rows != batch * rows or a.K != K):
                raise ValueError("packed operand does not match the product's shape")
            out = be.matmul_fwd(None if a is not None else in1.contiguous(), in2.contiguous(), batch, rows, K, N,
                                trans1, trans2, _cfmt(fmt1, round1), _cfmt(fmt2, round2), specs["scale_bits"] or 8,
                                specs["mx_flush_fp32_subnorms"],
                                in1.dtype if in1.dtype != torch.float16 else torch.float32, bits, _MODE[out_round],
                                bias=None if bias is None else bias.reshape(-1),
                                a_packed=None if a is None else (a.codes, a.scales))
            if in1.dtype == torch.float16:
                out = out.to(torch.float16)
            return out.reshape(*lead1, M, N)
        if a is None:
            # with a shared right operand the scales are laid out for all rows in one batch element
            a = _pack(in1.reshape(-1, K) if shared_b else in1, fmt1, specs, round1, not trans1)
        b = in2_packed if in2_packed is not None else _pack(in2, fmt2, specs, round2, trans2)
        if a.batch * a.rows != batch * rows or a.K != K or b.rows != N or b.K != K or b.batch != batch:
            raise ValueError("packed operand does not match the product's shape")
        out = be.gemm_mx(a.codes, a.scales, b.codes, b.scales, batch, rows, N, K, a.container, b.container,
                         out_dtype=in1.dtype if in1.dtype != torch.float16 else torch.float32,
                         bfloat_bits=bits, round_mode=_MODE[out_round],
                         bias=None if bias is None else bias.reshape(-1))
        if in1.dtype == torch.float16:
            out = out.to(torch.float16)
        return out.reshape(*lead1, M, N)
    if in1_packed is not None or in2_packed is not None:
        raise ValueError("a packed operand needs the tensor-core path (CUDA tensors, FP formats, block size 32)")

    # reference construction
    q1 = quantize_mx_op(in1, specs, elem_format=fmt1, axes=[-2 if trans1 else -1], round=round1)
    q2 = quantize_mx_op(in2, specs, elem_format=fmt2, axes=[-1 if trans2 else -2], round=round2)
    if q2.dtype != q1.dtype:
        q2 = q2.to(q1.dtype)
    a = q1.transpose(-1, -2) if trans1 else q1
    b = q2.transpose(-1, -2) if trans2 else q2
    with set_matmul_precision(a, b, fmt1, fmt2):
        out = _torch_matmul(a, b)
    out = quantize_elemwise_op(out, mx_specs=specs, round=out_round)
    if bias is not None:
        out = quantize_elemwise_op(out + bias, mx_specs=specs, round=out_round)
    return out
