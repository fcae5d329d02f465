"""Elementwise (bfloatX / fpX / eXmY) quantization.

Drop-in for the reference's mx/elemwise_ops.py: `quantize_elemwise_op` (:233)
and the internal `_quantize_elemwise_core` (:82), `_quantize_elemwise` (:173),
`_quantize_bfloat` (:191), `_quantize_fp` (:209).

CUDA tensors always run the sm_100a kernel behind the C ABI (there is no eager
path for them); CPU tensors use the library's host quantizer when `custom_cuda`
is set (the chunked GPU pipeline when they are pinned) and an exact float64
formulation in torch ops otherwise.
"""
import torch

from .formats import RoundingMode, _get_format_params, _get_max_norm, _get_min_norm

_MODE = {"nearest": 0, "floor": 1, "even": 2, "dither": 3}


def _emin(exp_bits):
    return 0 if exp_bits == 0 else 2 - (1 << (exp_bits - 1))


def _round_host(A, bits, exp_bits, max_norm, round, saturate_normals, allow_denorm, noise=None):
    """Exact CPU formulation: in float64 the value divided by its grid spacing
    is exact, so floor/round on it are the mathematically correct roundings."""
    x = A.detach().to(torch.float64)
    a = x.abs()
    P = bits - 1
    emin = _emin(exp_bits)
    finite = torch.isfinite(x)
    a0 = torch.where(finite, a, torch.zeros_like(a))
    _, e = torch.frexp(a0)                           # a0 = m * 2^e, m in [0.5, 1)
    ue = (e - 1).clamp(min=-127)
    qe = torch.clamp(ue, min=emin) - (P - 1)
    y = torch.ldexp(a0, -qe)
    if round == "nearest":
        r = torch.floor(y + 0.5)
    elif round == "floor":
        r = torch.floor(y)
    elif round == "even":
        r = torch.round(y)
    elif round == "dither":
        n = noise if noise is not None else torch.rand_like(A, dtype=torch.float32)
        r = torch.floor((y.to(torch.float32) + n.to(torch.float32))).to(torch.float64)
    else:
        raise Exception("Unrecognized round method %s" % (round))
    out = torch.ldexp(r, qe)
    if exp_bits != 0 and not allow_denorm:
        out = torch.where(a0 < _get_min_norm(exp_bits), torch.zeros_like(out), out)
    if saturate_normals or exp_bits == 0:
        out = out.clamp(max=max_norm)
    else:
        out = torch.where(out > max_norm, torch.full_like(out, float("inf")), out)
    out = torch.where(x < 0, -out, out)
    out = torch.where(finite, out, x)                # Inf and NaN pass through
    return out.to(A.dtype)


def _quantize_elemwise_core(A, bits, exp_bits, max_norm, round="nearest", saturate_normals=False,
                            allow_denorm=True, custom_cuda=False, noise=None):
    """Round every element of A to `bits` (sign + significand incl. implicit one)
    and `exp_bits` exponent bits (0 = fixed point); magnitudes above max_norm
    saturate (ints, or saturate_normals) or become Inf."""
    if A.is_sparse:
        if A.layout != torch.sparse_coo:
            raise NotImplementedError("Only COO layout sparse tensors are currently supported.")
        sp = A.coalesce()
        vals = _quantize_elemwise_core(sp.values().clone(), bits, exp_bits, max_norm, round,
                                       saturate_normals, allow_denorm, custom_cuda, noise)
        return torch.sparse_coo_tensor(sp.indices(), vals, sp.size(), dtype=sp.dtype, device=sp.device)
    if round not in _MODE:
        raise Exception("Unrecognized round method %s" % (round))
    if A.is_cuda:
        from . import _backend
        if round == "dither" and noise is None:
            noise = torch.rand_like(A, dtype=torch.float32)
        return _backend.quantize_elemwise(A.contiguous(), bits, exp_bits, max_norm, _MODE[round],
                                          saturate_normals, allow_denorm,
                                          noise.contiguous() if noise is not None else None)
    if custom_cuda and round != "dither" and bits <= 24 and A.is_pinned() and A.is_contiguous() \
            and torch.cuda.is_available():
        from . import _backend
        return _backend.quantize_elemwise_host(A, bits, exp_bits, max_norm, _MODE[round], saturate_normals, allow_denorm)
    if custom_cuda and bits <= 24 and A.dtype in (torch.float32, torch.float16, torch.bfloat16) and \
            (round != "dither" or noise is not None):
        # CPU tensor with custom_cuda: the library's host quantizer (the reference calls its C++ loop here,
        # mx/elemwise_ops.py:122-124)
        from . import _backend
        return _backend.cpu_quantize_elemwise(A, bits, exp_bits, max_norm, _MODE[round], saturate_normals,
                                              allow_denorm, noise)
    return _round_host(A, bits, exp_bits, max_norm, round, saturate_normals, allow_denorm, noise)


def _quantize_elemwise(A, elem_format, round="nearest", custom_cuda=False, saturate_normals=False,
                       allow_denorm=True):
    if elem_format is None:
        return A
    ebits, mbits, _, max_norm, _ = _get_format_params(elem_format)
    return _quantize_elemwise_core(A, mbits, ebits, max_norm, round=round, allow_denorm=allow_denorm,
                                   saturate_normals=saturate_normals, custom_cuda=custom_cuda)


def _quantize_bfloat(A, bfloat, round="nearest", custom_cuda=False, allow_denorm=True):
    """bfloatX: 1 sign, 8 exponent, X-9 mantissa bits; X in {0, 32} is a no-op."""
    if bfloat == 0 or bfloat == 32:
        return A
    return _quantize_elemwise_core(A, bits=bfloat - 7, exp_bits=8, max_norm=_get_max_norm(8, bfloat - 7),
                                   round=round, allow_denorm=allow_denorm, custom_cuda=custom_cuda)


def _quantize_fp(A, exp_bits=None, mantissa_bits=None, round="nearest", custom_cuda=False, allow_denorm=True):
    """IEEE-style fpX with Inf/NaN and subnormals like fp16."""
    if exp_bits is None or mantissa_bits is None:
        return A
    return _quantize_elemwise_core(A, bits=mantissa_bits + 2, exp_bits=exp_bits,
                                   max_norm=_get_max_norm(exp_bits, mantissa_bits + 2), round=round,
                                   allow_denorm=allow_denorm, custom_cuda=custom_cuda)


def quantize_elemwise_op(A, mx_specs, round=None):
    """Quantize A to the vector format of mx_specs ('bfloat' or 'fp')."""
    if mx_specs is None:
        return A
    if round is None:
        round = mx_specs["round"]
    if mx_specs["bfloat"] == 16 and round == "even" and mx_specs["bfloat_subnorms"] == True \
            and torch.cuda.is_available() and torch.cuda.is_bf16_supported():  # noqa: E712
        # the dtype changes to bfloat16 here, as in the reference
        if A.dtype == torch.bfloat16:
            return A
        if A.is_cuda and A.dtype == torch.float32:
            from . import _backend
            return _backend.quantize_elemwise(A.contiguous(), 9, 8, _get_max_norm(8, 9), 2, False, True,
                                              out_dtype=torch.bfloat16)
        if not A.is_cuda and A.dtype == torch.float32 and mx_specs["custom_cuda"] and A.layout == torch.strided \
                and A.is_pinned() and A.is_contiguous():
            # pinned host tensor with custom_cuda: rounded on the GPU, chunked, result in pinned memory
            from . import _backend
            return _backend.quantize_elemwise_host(A, 9, 8, _get_max_norm(8, 9), 2, False, True,
                                                   out_dtype=torch.bfloat16)
        return A.to(torch.bfloat16)
    if mx_specs["bfloat"] > 0 and mx_specs["fp"] > 0:
        raise ValueError("Cannot set both [bfloat] and [fp] in mx_specs.")
    if A.dtype == torch.bfloat16 and A.is_cuda and 16 <= mx_specs["bfloat"] and mx_specs["bfloat_subnorms"] \
            and round in ("nearest", "floor", "even"):
        return A        # every bfloat16 value is on the bfloatX grid (X >= 16): nothing to round
    if mx_specs["bfloat"] > 9:
        return _quantize_bfloat(A, bfloat=mx_specs["bfloat"], round=round, custom_cuda=mx_specs["custom_cuda"],
                                allow_denorm=mx_specs["bfloat_subnorms"])
    if mx_specs["bfloat"] > 0:
        raise ValueError("Cannot set [bfloat] <= 9 in mx_specs.")
    if mx_specs["fp"] > 6:
        return _quantize_fp(A, exp_bits=5, mantissa_bits=mx_specs["fp"] - 6, round=round,
                            custom_cuda=mx_specs["custom_cuda"], allow_denorm=mx_specs["bfloat_subnorms"])
    if mx_specs["fp"] > 0:
        raise ValueError("Cannot set [fp] <= 6 in mx_specs.")
    return A
