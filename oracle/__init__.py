"""CPU checkers for the quantization path (test infrastructure only).

Nothing in ``microxcaling_b200`` imports this package.  It is used by the
tests, by the smoke test and by the benchmark's CPU-baseline leg.

``oracle.lib()``  -> ctypes handle of the C restatement (mxq_oracle.c)
``oracle.ref()``  -> ctypes handle of the reference's own C++ math compiled in
                     place (``_ref/libmxq_ref.so``), or None when it was never
                     built on this machine.
The numpy helpers below wrap both with the same argument order.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = False

F32, F16, BF16 = 0, 1, 2
ROUND = {"nearest": 0, "floor": 1, "even": 2}

# (ebits, mbits incl. sign and implicit one, max_norm): mx/formats.py:61-125
FORMATS = {
    "int8": (0, 8, 1.984375), "int4": (0, 4, 1.75), "int2": (0, 2, 1.0),
    "fp8_e5m2": (5, 4, 57344.0), "fp8_e4m3": (4, 5, 448.0),
    "fp6_e3m2": (3, 4, 28.0), "fp6_e2m3": (2, 5, 7.5),
    "fp4_e2m1": (2, 3, 6.0), "fp4": (2, 3, 6.0),
    "fp16": (5, 12, 65504.0), "float16": (5, 12, 65504.0),
    "bf16": (8, 9, 3.3895313892515355e38), "bfloat16": (8, 9, 3.3895313892515355e38),
}


def build(force=False):
    """Compile the checkers with the Makefile beside this file."""
    so = os.path.join(_HERE, "libmxq_oracle.so")
    if force or not os.path.exists(so) or \
            os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "mxq_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "libmxq_oracle.so"],
                              stdout=subprocess.DEVNULL)
    ref_src = os.environ.get("MXQ_REFERENCE_DIR", "")
    if not ref_src:
        # the conventional place of the reference checkout beside this repository's parent
        cand = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
        ref_src = cand if os.path.isfile(os.path.join(cand, "mx", "cpp", "funcs.h")) else ""
    if ref_src:
        subprocess.call(["make", "-C", _HERE, "ref", "REF=" + ref_src], stdout=subprocess.DEVNULL,
                        stderr=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libmxq_oracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        i64, i32, f32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
        L.mxo_quantize_mx.argtypes = [vp, vp, vp, vp, i32, i64, i64, i64, i32, i32, i32, i32,
                                      f32, i32, i32, i32]
        L.mxo_quantize_elemwise.argtypes = [vp, vp, i32, i32, i64, i32, i32, f32, i32, i32, i32, i32]
        L.mxo_reduce_sum_inner.argtypes = [vp, vp, i64, i64, i32]
        L.mxo_reduce_max_inner.argtypes = [vp, vp, i64, i64, i32]
        L.mxo_gemm_nt.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i32]
        L.mxo_round_elem.argtypes = [f32, i32, i32, f32, i32, i32, i32]
        L.mxo_round_elem.restype = f32
        L.mxo_scale_exp.argtypes = [f32, i32, f32, vp]
        L.mxo_decode_elem.argtypes = [ctypes.c_uint8, i32, i32, i32]
        L.mxo_decode_elem.restype = f32
        _LIB = L
    return _LIB


def ref():
    global _REF
    if _REF is False:
        so = os.path.join(_HERE, "_ref", "libmxq_ref.so")
        if os.path.exists(so):
            R = ctypes.CDLL(so)
            i64, i32, f32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
            R.mxref_quantize_mx_f32.argtypes = [vp, vp, i64, i64, i64, i32, i32, i32, i32, f32,
                                                i32, i32, i32]
            R.mxref_quantize_elemwise_f32.argtypes = [vp, vp, i64, i32, i32, f32, i32, i32, i32, i32]
            R.mxref_shared_scale.argtypes = [f32, i32, f32]
            R.mxref_shared_scale.restype = f32
            _REF = R
        else:
            _REF = None
    return _REF


def _dtype_code(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    if a.dtype == np.uint16:        # bf16 bit patterns
        return BF16
    raise TypeError(a.dtype)


def _split(shape, axis):
    axis = axis % len(shape)
    pre = int(np.prod(shape[:axis], dtype=np.int64))
    post = int(np.prod(shape[axis + 1:], dtype=np.int64))
    return pre, int(shape[axis]), post


def quantize_mx(x, fmt, axis=-1, block=32, scale_bits=8, round="nearest", flush=False,
                want_packed=False, nthreads=0):
    """Fake-quantize numpy array ``x`` (float32, float16, or uint16 holding bf16
    bits).  Returns the dequantized array; with ``want_packed`` also the element
    codes (uint8, x's shape) and E8M0 scale bytes ([pre, nblocks, post])."""
    ebits, mbits, mn = FORMATS[fmt] if isinstance(fmt, str) else fmt
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    if x.size == 0:
        return (out, None, None) if want_packed else out
    pre, n, post = _split(x.shape, axis)
    blk = block if block > 0 else n
    nblk = (n + blk - 1) // blk
    codes = np.empty(x.shape, np.uint8) if want_packed else None
    scales = np.empty((pre, nblk, post), np.uint8) if want_packed else None
    rc = lib().mxo_quantize_mx(x.ctypes.data, out.ctypes.data,
                               codes.ctypes.data if want_packed else None,
                               scales.ctypes.data if want_packed else None,
                               _dtype_code(x), pre, n, post, blk, scale_bits, ebits, mbits, mn,
                               int(flush), ROUND[round] if isinstance(round, str) else round,
                               nthreads)
    assert rc == 0
    return (out, codes, scales) if want_packed else out


def quantize_elemwise(x, bits, exp_bits, max_norm, round="nearest", saturate=False,
                      allow_denorm=True, out_dtype=None, nthreads=0):
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, out_dtype or x.dtype)
    if x.size:
        lib().mxo_quantize_elemwise(x.ctypes.data, out.ctypes.data, _dtype_code(x),
                                    _dtype_code(out), x.size, bits, exp_bits, max_norm,
                                    ROUND[round] if isinstance(round, str) else round,
                                    int(saturate), int(allow_denorm), nthreads)
    return out


def reduce_inner(x, op):
    x = np.ascontiguousarray(x, np.float32)
    rows, inner = int(np.prod(x.shape[:-1], dtype=np.int64)), x.shape[-1]
    out = np.empty(x.shape[:-1], np.float32)
    fn = lib().mxo_reduce_sum_inner if op == "sum" else lib().mxo_reduce_max_inner
    fn(x.ctypes.data, out.ctypes.data, rows, inner, 0)
    return out


def gemm_nt(a, b, want_abs=False):
    """a [batch, M, K] @ b[batch, N, K]^T in double accumulation."""
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    if a.ndim == 2:
        a, b = a[None], b[None]
    B, M, K = a.shape
    N = b.shape[1]
    c = np.empty((B, M, N), np.float64)
    ca = np.empty((B, M, N), np.float64) if want_abs else None
    lib().mxo_gemm_nt(a.ctypes.data, b.ctypes.data, c.ctypes.data,
                      ca.ctypes.data if want_abs else None, B, M, N, K, 0)
    return (c, ca) if want_abs else c


def ref_quantize_mx_f32(x, fmt, axis=-1, block=32, scale_bits=8, round="nearest", flush=False,
                        nthreads=0):
    """The reference's own C++ loop (needs ``_ref/libmxq_ref.so``)."""
    ebits, mbits, mn = FORMATS[fmt] if isinstance(fmt, str) else fmt
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    pre, n, post = _split(x.shape, axis)
    rc = ref().mxref_quantize_mx_f32(x.ctypes.data, out.ctypes.data, pre, n, post,
                                     block if block > 0 else n, scale_bits, ebits, mbits, mn,
                                     int(flush), ROUND[round], nthreads)
    assert rc == 0
    return out


def ref_quantize_elemwise_f32(x, bits, exp_bits, max_norm, round="nearest", saturate=False,
                              allow_denorm=True, nthreads=0):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    ref().mxref_quantize_elemwise_f32(x.ctypes.data, out.ctypes.data, x.size, bits, exp_bits,
                                      max_norm, ROUND[round], int(saturate), int(allow_denorm),
                                      nthreads)
    return out


def same_values(a, b):
    """The reference's comparator (mx/tests/common_lib.py:91-134) at tol 0 with
    Inf/NaN masks compared: numeric equality, NaN==NaN, -0==+0.  Accepts float
    arrays or uint16 bf16 bit patterns."""
    def f(v):
        if v.dtype == np.uint16:
            return (v.astype(np.uint32) << 16).view(np.float32)
        return v.astype(np.float32)
    a, b = f(np.asarray(a)), f(np.asarray(b))
    if a.shape != b.shape:
        return False
    na, nb = np.isnan(a), np.isnan(b)
    if not np.array_equal(na, nb):
        return False
    return bool(np.all((a == b) | na))
