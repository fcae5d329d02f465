"""MX block quantization.

Drop-in for the reference's mx/mx_ops.py: `quantize_mx_op` (:301) and the
internal `_quantize_mx` (:173), with the block helpers `_shared_exponents`
(:49), `_reshape_to_blocks` (:95) and `_undo_reshape_to_blocks` (:157).

CUDA tensors with one shared axis go to the sm_100a kernels through the C ABI
whatever `custom_cuda` says (a single launch).  Several shared axes (the
reference's mx_ops.py:228-296 handles them with torch ops on the tensor's
device) run the exact torch formulation `_host_mx` on the tensor's device.
CPU tensors use the library's host quantizer when `custom_cuda` is set (the
reference calls its C++ loop there, mx_ops.py:259-263), the chunked GPU
pipeline when they are pinned, and the torch formulation otherwise.
"""
import torch

from .formats import ElemFormat, _get_format_params
from .specs import mx_assert_test

_MODE = {"nearest": 0, "floor": 1, "even": 2, "dither": 3}


def _host_mx(A, scale_bits, ebits, mbits, max_norm, axes, block_size, round, flush, noise=None):
    """Exact torch formulation for CPU tensors, any number of shared axes."""
    from .elemwise_ops import _round_host
    if A.is_cuda and round == "dither" and noise is None:
        noise = torch.rand_like(A, dtype=torch.float32)
    x = A.detach().to(torch.float64)
    nd = x.dim()
    axes = sorted(a % nd for a in axes)
    # view each shared axis as (blocks, block), zero-padding a ragged tail
    shape, pads = [], []
    for d in range(nd):
        n = x.shape[d]
        if d in axes:
            b = block_size if 0 < block_size < n else n
            nb = (n + b - 1) // b if n else 0
            pads.append(nb * b - n)
            shape += [nb, b]
        else:
            pads.append(0)
            shape.append(n)
    if any(pads):
        pad = []
        for p in reversed(pads):
            pad += [0, p]
        x = torch.nn.functional.pad(x, pad)
    xb = x.reshape(shape)
    red, k = [], 0
    for d in range(nd):
        if d in axes:
            red.append(k + 1)
            k += 2
        else:
            k += 1
    a = xb.abs()
    amax = torch.amax(torch.where(torch.isnan(a), torch.full_like(a, float("inf")), a), dim=red, keepdim=True)
    amax32 = amax.to(torch.float32)
    E = (amax32.view(torch.int32) >> 23) & 0xFF                  # biased exponent of the maximum
    _, emax_elem = torch.frexp(torch.tensor(float(max_norm)))
    emax_elem = int(emax_elem) - 1
    smax = (1 << (scale_bits - 1)) - 1
    nan_blk = E == 255
    Es = E - emax_elem
    nan_blk = nan_blk | ((Es - 127) > smax)
    Es = torch.where((Es - 127) < -smax, torch.full_like(Es, 127 - smax), Es)
    dead = (E == 0) if flush else torch.zeros_like(nan_blk)
    se = (Es - 127).to(torch.int32)
    v = torch.ldexp(xb, (-se).expand_as(xb))
    v = torch.where(dead.expand_as(v), torch.zeros_like(v), v)
    v = torch.where(torch.isfinite(v), v, torch.zeros_like(v))
    nz = None
    if noise is not None:
        nz = noise.to(torch.float32)
        if any(pads):
            nz = torch.nn.functional.pad(nz, pad)
        nz = nz.reshape(shape)
    q = _round_host(v, mbits, ebits, max_norm, round, True, True, nz)
    y = torch.ldexp(q, se.expand_as(q))
    y = torch.where(nan_blk.expand_as(y), torch.full_like(y, float("nan")), y)
    y = y.reshape(x.shape)
    if any(pads):
        y = y[tuple(slice(0, n) for n in A.shape)]
    return y.to(A.dtype)


def _quantize_mx(A, scale_bits, elem_format, shared_exp_method="max", axes=None, block_size=0,
                 round="nearest", flush_fp32_subnorms=False, custom_cuda=False, noise=None):
    """MX fake-quantization: blocks of `block_size` elements along each axis of
    `axes` share a power-of-two scale of `scale_bits` bits."""
    if elem_format is None:
        return A
    assert scale_bits > 0
    if axes is None:
        raise Exception("axes required in order to determine which dimension to apply block size to")
    axes = [axes] if type(axes) == int else list(axes)
    axes = [x + A.ndim if x < 0 else x for x in axes]
    if shared_exp_method == "none":
        # an exponent for each value (mx_ops.py:70-71): blocks of one element
        block_size, axes = 1, [A.ndim - 1] if A.ndim else [0]
    elif shared_exp_method != "max":
        raise Exception("Unrecognized shared exponent selection method %s" % (shared_exp_method))
    if round not in _MODE:
        raise Exception("Unrecognized round method %s" % (round))
    ebits, mbits, _, max_norm, _ = _get_format_params(elem_format)
    if A.is_cuda and len(axes) != 1:
        if A.numel() == 0:
            return A.clone()
        return _host_mx(A, scale_bits, ebits, mbits, max_norm, axes, block_size, round, flush_fp32_subnorms, noise)
    if A.is_cuda:
        from . import _backend
        if round == "dither" and noise is None:
            noise = torch.rand_like(A, dtype=torch.float32)
        return _backend.quantize_mx(A.contiguous(), scale_bits, ebits, mbits, max_norm, block_size, axes[0],
                                    flush_fp32_subnorms, _MODE[round],
                                    noise.contiguous() if noise is not None else None)
    if A.numel() == 0:
        return A.clone()
    if custom_cuda and len(axes) == 1 and round != "dither" and A.is_pinned() and A.is_contiguous() \
            and torch.cuda.is_available():
        # a pinned host tensor with custom_cuda: quantize on the GPU, chunked, result back in pinned memory
        from . import _backend
        return _backend.quantize_mx_host(A, scale_bits, ebits, mbits, max_norm, block_size, axes[0],
                                         flush_fp32_subnorms, _MODE[round])
    if custom_cuda and len(axes) == 1 and A.dtype in (torch.float32, torch.float16, torch.bfloat16) and \
            (round != "dither" or noise is not None):
        from . import _backend
        return _backend.cpu_quantize_mx(A, scale_bits, ebits, mbits, max_norm, block_size, axes[0],
                                        flush_fp32_subnorms, _MODE[round], noise)
    return _host_mx(A, scale_bits, ebits, mbits, max_norm, axes, block_size, round, flush_fp32_subnorms, noise)


def _reshape_to_blocks(A, axes, block_size):
    """Split every axis of `axes` into (blocks, block_size); a ragged tail is zero-padded.

    Same contract as the reference's helper (mx_ops.py:95-154): returns the
    blocked view, the positions of the `blocks` dimensions in it (the block
    dimension follows each), the shape with the inserted unit dimensions before
    padding, and that shape after padding."""
    if axes is None:
        raise Exception("axes required in order to determine which dimension to apply block size to")
    if block_size == 0:
        raise Exception("block_size == 0 in _reshape_to_blocks")
    nd = A.ndim
    split = sorted(a % nd for a in axes)
    # every split axis gains a unit dimension right after it
    new_axes = [a + i for i, a in enumerate(split)]
    unit_shape, k = [], 0
    for d in range(nd):
        unit_shape.append(A.shape[d])
        if d in split:
            unit_shape.append(1)
    orig_shape = torch.Size(unit_shape)
    padded = list(unit_shape)
    pad_per_dim = [0] * len(unit_shape)
    for ax in new_axes:
        rem = padded[ax] % block_size
        if rem:
            pad_per_dim[ax] = block_size - rem
            padded[ax] += block_size - rem
    A = A.reshape(unit_shape)
    if any(pad_per_dim):
        flat = []
        for p in reversed(pad_per_dim):          # F.pad lists the last dimension first
            flat += [0, p]
        A = torch.nn.functional.pad(A, flat, mode="constant")
    padded_shape = torch.Size(padded)
    blocked = list(padded)
    for ax in new_axes:
        n = blocked[ax]
        # an axis shorter than a block is one block of its own length
        blocked[ax], blocked[ax + 1] = (n // block_size, block_size) if n >= block_size else (1, n)
    return A.reshape(blocked), new_axes, orig_shape, padded_shape


def _undo_reshape_to_blocks(A, padded_shape, orig_shape, axes):
    """Inverse of _reshape_to_blocks (reference: mx_ops.py:157-170)."""
    A = A.reshape(tuple(padded_shape))
    if tuple(padded_shape) != tuple(orig_shape):
        A = A[tuple(slice(0, n) for n in orig_shape)]
    return A.reshape([n for i, n in enumerate(orig_shape) if i - 1 not in axes])


def _shared_exponents(A, method="max", axes=None, ebits=0):
    """floor(log2(.)) of the block maxima (or of every |value| with method 'none'), read from the
    exponent bits instead of computed with a logarithm; zero maps to -126 like the reference's
    FP32_MIN_NORMAL substitution (mx_ops.py:49-92).  With ebits > 0 the result is restricted to
    +-(2^(ebits-1) - 1): larger becomes NaN, smaller is clamped."""
    if method == "max":
        if axes is None:
            m = torch.max(torch.abs(A))
        else:
            m = A
            for axis in axes:
                m, _ = torch.max(torch.abs(m), dim=axis, keepdim=True)
    elif method == "none":
        m = torch.abs(A)
    else:
        raise Exception("Unrecognized shared exponent selection method %s" % (method))
    m32 = m.to(torch.float32)
    _, e = torch.frexp(torch.where(m32 == 0, torch.full_like(m32, 2.0 ** -126), m32))
    shared_exp = (e - 1).to(m.dtype if m.dtype.is_floating_point else torch.float32)
    shared_exp = torch.where(torch.isfinite(m32), shared_exp, m32.to(shared_exp.dtype))   # Inf / NaN pass through
    if ebits > 0:
        emax = 2 ** (ebits - 1) - 1
        shared_exp = shared_exp.clone()
        shared_exp[shared_exp > emax] = float("NaN")
        shared_exp[shared_exp < -emax] = -emax
    return shared_exp


def quantize_mx_op(A, mx_specs: dict, elem_format=None, block_size=None, axes=None, round="nearest",
                   expand_and_reshape=False):
    """Quantize A to the MX format `elem_format` along `axes` per mx_specs."""
    mx_assert_test(mx_specs)
    if elem_format is None:
        return A
    if type(elem_format) is str:
        elem_format = ElemFormat.from_str(elem_format)
    if block_size is None:
        block_size = mx_specs["block_size"]
    scale_bits = 8 if mx_specs["scale_bits"] == 0 else mx_specs["scale_bits"]
    return _quantize_mx(A, scale_bits, elem_format, block_size=block_size, axes=axes, round=round,
                        shared_exp_method=mx_specs["shared_exp_method"],
                        flush_fp32_subnorms=mx_specs["mx_flush_fp32_subnorms"],
                        custom_cuda=mx_specs["custom_cuda"])
