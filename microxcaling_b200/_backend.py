"""ctypes binding of libmxq.so: the only way the Python layer reaches the GPU.

Takes the place of the reference's mx/custom_extensions.py (a
torch.utils.cpp_extension JIT build).  The library is prebuilt in-tree by
``python -m microxcaling_b200.build``; there is no CPU or eager fallback for CUDA
tensors: if the library is missing, loading raises.

``funcs`` keeps the seven names the reference's pybind module exports
(mx/cpp/funcs.cpp:234-242) so reference-style callers keep working.
"""
import contextlib
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmxq.so")
_lib = None

F32, F16, BF16 = 0, 1, 2
_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
ROUND_DITHER = 3
CODES_TRANSPOSED = 1
SCALES_GEMM_LAYOUT = 2


class MxqError(RuntimeError):
    pass


class ElemFormatC(ctypes.Structure):
    """struct mxq_elem_format of include/mxq.h"""
    _fields_ = [("ebits", ctypes.c_int), ("mbits", ctypes.c_int), ("max_norm", ctypes.c_float), ("round", ctypes.c_int)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise MxqError("libmxq.so not built: run `python -m microxcaling_b200.build` "
                           "(needs nvcc with sm_100a support)")
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
        L.mxq_status_string.restype = ctypes.c_char_p
        L.mxq_status_string.argtypes = [i32]
        L.mxq_quantize_mx.argtypes = [vp, vp, vp, vp, i32, i64, i64, i64, i32, i32, i32, i32, f32,
                                      i32, i32, vp, i32, i64, vp]
        L.mxq_gemm_mx.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, i32, i32, vp, i32, vp]
        L.mxq_sf_bytes.argtypes = [i64, i64, i64]
        L.mxq_sf_bytes.restype = i64
        L.mxq_device_status.argtypes = [i32]
        L.mxq_quantize_mx_host.argtypes = [vp, vp, i32, i64, i64, i64, i32, i32, i32, i32, f32, i32, i32, vp, i64, vp]
        L.mxq_quantize_elemwise_host.argtypes = [vp, vp, i32, i32, i64, i32, i32, f32, i32, i32, i32, vp, i64, vp]
        L.mxq_host_workspace_bytes.restype = i64
        L.mxq_linear_fwd.argtypes = [vp, i32, i64, i64, i32, i32, f32, i32, i32, i32, vp, vp, i64, i32, vp, i32,
                                     i32, i32, vp, vp, i64, vp]
        L.mxq_linear_workspace_bytes.argtypes = [i64, i64]
        L.mxq_linear_workspace_bytes.restype = i64
        L.mxq_quantize_elemwise.argtypes = [vp, vp, i32, i32, i64, i32, i32, f32, i32, i32, i32, vp, vp]
        L.mxq_reduce_sum_inner.argtypes = [vp, vp, i64, i64, vp]
        L.mxq_reduce_max_inner.argtypes = [vp, vp, i64, i64, vp]
        L.mxq_silu_bf16.argtypes = [vp, vp, vp, vp, i64, vp]
        L.mxq_softmax_bf16.argtypes = [vp, vp, i64, i64, i32, vp]
        L.mxq_swiglu_quantize_mx.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, i32, f32, i32, i32, i32, i64, vp]
        L.mxq_softmax_quantize_mx.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, i32, f32, i32, i32, i32, i64, vp]
        L.mxq_gemm_mx_scatter.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, i64, i64, i64, i32, i32, i32,
                                          i32, i32, i32, vp]
        L.mxq_sum_slabs_f32.argtypes = [vp, i32, i64, vp, vp]
        L.mxq_rmsnorm_bf16.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, f32, vp]
        fp = ctypes.POINTER(ElemFormatC)
        L.mxq_linear_train_workspace_bytes.argtypes = [i64, i64, i64]
        L.mxq_linear_train_workspace_bytes.restype = i64
        L.mxq_linear_fwd_train.argtypes = [vp, vp, i32, i64, i64, i64, fp, fp, i32, i32, vp, i32, i32, i32, vp, vp, i64, vp]
        L.mxq_linear_bwd.argtypes = [vp, vp, vp, i32, i64, i64, i64, fp, fp, fp, fp, i32, i32, vp, vp, i32, i32, i32, i32,
                                     vp, i64, vp]
        L.mxq_matmul_workspace_bytes.argtypes = [i64, i64, i64, i64]
        L.mxq_matmul_workspace_bytes.restype = i64
        L.mxq_matmul_fwd.argtypes = [vp, vp, i32, i64, i64, i64, i64, i32, i32, fp, fp, i32, i32, vp, vp, vp, i32, i32, i32,
                                     vp, vp, i64, vp]
        L.mxq_gemm_sm_budget.argtypes = [i32]
        L.mxq_cpu_quantize_mx.argtypes = [vp, vp, i32, i64, i64, i64, i32, i32, i32, i32, f32, i32, i32, vp, i32]
        L.mxq_cpu_quantize_elemwise.argtypes = [vp, vp, i32, i32, i64, i32, i32, f32, i32, i32, i32, vp, i32]
        _lib = L
    return _lib


def check(status):
    if status != 0:
        raise MxqError("libmxq: %s (status %d)" % (lib().mxq_status_string(status).decode(), status))


def _stream(t):
    """Raw handle of torch's current stream on t's device (an int; ctypes converts it)."""
    idx = t.device.index
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device() if idx is None else idx)


class _device_of:
    """Makes t's device current around a library call; free when it already is."""
    __slots__ = ("idx", "guard")

    def __init__(self, dev):
        idx = dev.index
        self.idx = None if idx is None or idx == torch.cuda.current_device() else idx
        self.guard = None

    def __enter__(self):
        if self.idx is not None:
            self.guard = torch.cuda.device(self.idx)
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def _require_cuda(t, name="tensor"):
    if not t.is_cuda:
        raise MxqError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise MxqError("%s must be contiguous" % name)
    if t.dtype not in _DT:
        raise MxqError("Tensor dtype not supported: %s" % t.dtype)


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def _split(shape, axis):
    pre = 1
    for s in shape[:axis]:
        pre *= s
    post = 1
    for s in shape[axis + 1:]:
        post *= s
    return pre, shape[axis], post


def quantize_mx(A, scale_bits, ebits, mbits, max_norm, block, axis, flush=False, rmode=0,
                noise=None, want_dq=True, want_codes=False, transposed=False, gemm_layout=False,
                rows_per_batch=0):
    """MX-quantize CUDA tensor A in blocks of `block` along `axis`.

    Returns the dequantized tensor (A's dtype), or with want_codes a tuple
    (dq or None, codes uint8, scales uint8).  Codes/scales layouts are those of
    mxq_quantize_mx in include/mxq.h."""
    _require_cuda(A, "A")
    axis = axis % A.dim() if A.dim() else 0
    shape = list(A.shape)
    pre, n, post = _split(shape, axis)
    blk = int(block) if block and block > 0 else n
    blk = min(blk, n) if n > 0 else 1
    nblk = (n + blk - 1) // blk if n else 0
    out = torch.empty_like(A) if want_dq else None
    codes = scales = None
    if want_codes:
        if transposed:
            codes = torch.empty(shape[:axis] + shape[axis + 1:] + [nblk * blk], dtype=torch.uint8, device=A.device)
        else:
            codes = torch.empty(shape, dtype=torch.uint8, device=A.device)
        if gemm_layout:
            # [batch, rows, K] operand: 512-byte chunks per 128 rows x 128 K; padding bytes are defined as
            # zero (they exist only when rows or K is not a multiple of 128)
            if transposed:
                nb, rows = pre, post
            else:
                rows = rows_per_batch if rows_per_batch else pre
                nb = pre // rows if rows else 0
            kpad = nblk * blk
            nbytes = nb * ((rows + 127) // 128) * ((kpad + 127) // 128) * 512
            alloc = torch.empty if rows % 128 == 0 and kpad % 128 == 0 else torch.zeros
            scales = alloc(nbytes, dtype=torch.uint8, device=A.device)
        elif transposed:
            scales = torch.empty(shape[:axis] + shape[axis + 1:] + [nblk], dtype=torch.uint8, device=A.device)
        else:
            scales = torch.empty(shape[:axis] + [nblk] + shape[axis + 1:], dtype=torch.uint8, device=A.device)
    if noise is not None:
        _require_cuda(noise, "noise")
        assert noise.dtype == torch.float32 and noise.shape == A.shape
    with _device_of(A.device):
        check(lib().mxq_quantize_mx(_ptr(A), _ptr(out), _ptr(codes), _ptr(scales), _DT[A.dtype],
                                    pre, n, post, blk, int(scale_bits), int(ebits), int(mbits),
                                    float(max_norm), int(bool(flush)), int(rmode), _ptr(noise),
                                    (CODES_TRANSPOSED if transposed else 0) | (SCALES_GEMM_LAYOUT if gemm_layout else 0),
                                    int(rows_per_batch), _stream(A)))
    if want_codes:
        return out, codes, scales
    return out


def quantize_elemwise(A, bits, exp_bits, max_norm, rmode=0, saturate_normals=False,
                      allow_denorm=True, noise=None, out_dtype=None):
    _require_cuda(A, "A")
    out = torch.empty_like(A) if out_dtype in (None, A.dtype) else \
        torch.empty(A.shape, dtype=out_dtype, device=A.device)
    if bits > 24:
        raise MxqError("quantize_elemwise with bits > 24 leads to negative shifts")
    if noise is not None:
        _require_cuda(noise, "noise")
    with _device_of(A.device):
        check(lib().mxq_quantize_elemwise(_ptr(A), _ptr(out), _DT[A.dtype], _DT[out.dtype], A.numel(),
                                          int(bits), int(exp_bits), float(max_norm), int(rmode),
                                          int(bool(saturate_normals)), int(bool(allow_denorm)),
                                          _ptr(noise), _stream(A)))
    return out


_host_ws = {}


def _host_workspace(device):
    ws = _host_ws.get(device.index)
    if ws is None:
        ws = torch.empty(lib().mxq_host_workspace_bytes(), dtype=torch.uint8, device=device)
        _host_ws[device.index] = ws
    return ws


def quantize_mx_host(A, scale_bits, ebits, mbits, max_norm, block, axis, flush=False, rmode=0, out=None,
                     device=None):
    """MX-quantize a pinned HOST tensor on the GPU, result in pinned host memory (chunked, copies
    overlapped with the kernel).  Returns after the result is complete."""
    if A.is_cuda or not A.is_contiguous() or A.dtype not in _DT:
        raise MxqError("quantize_mx_host needs a contiguous CPU tensor of a supported dtype")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty(A.shape, dtype=A.dtype, pin_memory=True)      # torch's caching host allocator
    axis = axis % A.dim() if A.dim() else 0
    pre, n, post = _split(list(A.shape), axis)
    if A.numel():
        with torch.cuda.device(device):
            ws = _host_workspace(device)
            st = torch.cuda.current_stream(device)
            check(lib().mxq_quantize_mx_host(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(out.data_ptr()), _DT[A.dtype],
                                             pre, n, post, int(block) if block and block > 0 else n, int(scale_bits),
                                             int(ebits), int(mbits), float(max_norm), int(bool(flush)), int(rmode),
                                             _ptr(ws), ws.numel(), ctypes.c_void_p(st.cuda_stream)))
            st.synchronize()
    return out


def quantize_elemwise_host(A, bits, exp_bits, max_norm, rmode=0, saturate_normals=False, allow_denorm=True,
                           out=None, out_dtype=None, device=None):
    """Elementwise rounding of a pinned HOST tensor on the GPU; see quantize_mx_host."""
    if A.is_cuda or not A.is_contiguous() or A.dtype not in _DT:
        raise MxqError("quantize_elemwise_host needs a contiguous CPU tensor of a supported dtype")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty(A.shape, dtype=out_dtype or A.dtype, pin_memory=True)
    if A.numel():
        with torch.cuda.device(device):
            ws = _host_workspace(device)
            st = torch.cuda.current_stream(device)
            check(lib().mxq_quantize_elemwise_host(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                   _DT[A.dtype], _DT[out.dtype], A.numel(), int(bits), int(exp_bits),
                                                   float(max_norm), int(rmode), int(bool(saturate_normals)),
                                                   int(bool(allow_denorm)), _ptr(ws), ws.numel(),
                                                   ctypes.c_void_p(st.cuda_stream)))
            st.synchronize()
    return out


def _require_cpu(t, name="tensor"):
    if t.is_cuda or t.layout != torch.strided:
        raise MxqError("%s must be a dense CPU tensor" % name)
    if t.dtype not in _DT:
        raise MxqError("Tensor dtype not supported: %s" % t.dtype)


def cpu_quantize_mx(A, scale_bits, ebits, mbits, max_norm, block, axis, flush=False, rmode=0, noise=None,
                    nthreads=0):
    """MX-quantize a CPU tensor on the host cores (mxq_cpu_quantize_mx); same results as the GPU kernels."""
    _require_cpu(A, "A")
    A = A.contiguous()
    out = torch.empty_like(A)
    if A.numel() == 0:
        return out
    axis = axis % A.dim()
    pre, n, post = _split(list(A.shape), axis)
    if noise is not None:
        noise = noise.to(torch.float32).contiguous()
        assert noise.shape == A.shape and not noise.is_cuda
    check(lib().mxq_cpu_quantize_mx(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(out.data_ptr()), _DT[A.dtype],
                                    pre, n, post, int(block) if block and block > 0 else n, int(scale_bits),
                                    int(ebits), int(mbits), float(max_norm), int(bool(flush)), int(rmode),
                                    ctypes.c_void_p(noise.data_ptr()) if noise is not None else None, int(nthreads)))
    return out


def cpu_quantize_elemwise(A, bits, exp_bits, max_norm, rmode=0, saturate_normals=False, allow_denorm=True,
                          noise=None, out_dtype=None, nthreads=0):
    """Elementwise rounding of a CPU tensor on the host cores (mxq_cpu_quantize_elemwise)."""
    _require_cpu(A, "A")
    if bits > 24:
        raise MxqError("quantize_elemwise with bits > 24 leads to negative shifts")
    A = A.contiguous()
    out = torch.empty_like(A) if out_dtype in (None, A.dtype) else torch.empty(A.shape, dtype=out_dtype)
    if A.numel() == 0:
        return out
    if noise is not None:
        noise = noise.to(torch.float32).contiguous()
        assert noise.shape == A.shape and not noise.is_cuda
    check(lib().mxq_cpu_quantize_elemwise(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                          _DT[A.dtype], _DT[out.dtype], A.numel(), int(bits), int(exp_bits),
                                          float(max_norm), int(rmode), int(bool(saturate_normals)),
                                          int(bool(allow_denorm)),
                                          ctypes.c_void_p(noise.data_ptr()) if noise is not None else None,
                                          int(nthreads)))
    return out


def gemm_mx(a_codes, a_scales, b_codes, b_scales, batch, M, N, K, a_fmt=0, b_fmt=0,
            out_dtype=torch.bfloat16, bfloat_bits=16, round_mode=0, bias=None, tile_n=0, out=None):
    """C[b] = A[b] @ B[b]^T on the block-scaled tensor cores; see mxq_gemm_mx."""
    for t in (a_codes, b_codes, a_scales, b_scales):
        if not t.is_cuda or not t.is_contiguous() or t.dtype != torch.uint8:
            raise MxqError("GEMM operands must be contiguous uint8 CUDA tensors")
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a_codes.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    with _device_of(a_codes.device):
        check(lib().mxq_gemm_mx(_ptr(a_codes), _ptr(a_scales), _ptr(b_codes), _ptr(b_scales), _ptr(out),
                                batch, M, N, K, a_fmt, b_fmt, _DT[out.dtype], int(bfloat_bits), int(round_mode),
                                _ptr(bias), int(tile_n), _stream(a_codes)))
    return out


def gemm_mx_scatter(a_codes, a_scales, b_codes, b_scales, dest_ptrs, rows_per_dest, M, N, K, a_fmt=0, b_fmt=0,
                    out_dtype=torch.float32, bfloat_bits=0, round_mode=-1, tile_n=0):
    """A @ B^T with rows [d*rows_per_dest, (d+1)*rows_per_dest) stored into the buffer at dest_ptrs[d]
    (device pointers, possibly peer mappings); see mxq_gemm_mx_scatter."""
    for t in (a_codes, b_codes, a_scales, b_scales):
        if not t.is_cuda or not t.is_contiguous() or t.dtype != torch.uint8:
            raise MxqError("GEMM operands must be contiguous uint8 CUDA tensors")
    arr = (ctypes.c_void_p * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
    with _device_of(a_codes.device):
        check(lib().mxq_gemm_mx_scatter(_ptr(a_codes), _ptr(a_scales), _ptr(b_codes), _ptr(b_scales), arr,
                                        len(dest_ptrs), int(rows_per_dest), M, N, K, a_fmt, b_fmt, _DT[out_dtype],
                                        int(bfloat_bits), int(round_mode), int(tile_n), _stream(a_codes)))


def peer_alloc(device, nbytes):
    """(device pointer, 64-byte handle) of a fresh buffer other processes can map; see mxq_peer_alloc."""
    L = lib()
    ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    L.mxq_peer_alloc.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    with _device_of(device):
        check(L.mxq_peer_alloc(int(nbytes), ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_open(device, handle):
    """Map another process's buffer for kernels of `device`; see mxq_peer_open."""
    L = lib()
    ptr = ctypes.c_void_p()
    L.mxq_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    with _device_of(device):
        check(L.mxq_peer_open(handle, ctypes.byref(ptr)))
    return ptr.value


def peer_close(ptr):
    lib().mxq_peer_close.argtypes = [ctypes.c_void_p]
    return lib().mxq_peer_close(ptr)


def peer_free(ptr):
    lib().mxq_peer_free.argtypes = [ctypes.c_void_p]
    return lib().mxq_peer_free(ptr)


def sum_slabs(slabs, n_slabs=None, shape=None, device=None):
    """Sum of n fp32 slabs, added in order; see mxq_sum_slabs_f32.  `slabs` is a contiguous
    float32 CUDA tensor [n, ...] or a raw device pointer (then n_slabs, shape and device are required)."""
    if isinstance(slabs, int):
        ptr = slabs
    else:
        if not (slabs.is_cuda and slabs.is_contiguous() and slabs.dtype == torch.float32):
            raise MxqError("slabs must be a contiguous float32 CUDA tensor")
        ptr, n_slabs, shape, device = _ptr(slabs), slabs.shape[0], tuple(slabs.shape[1:]), slabs.device
    out = torch.empty(shape, dtype=torch.float32, device=device)
    with _device_of(out.device):
        check(lib().mxq_sum_slabs_f32(ptr, int(n_slabs), out.numel(), _ptr(out), _stream(out)))
    return out


def linear_fwd(x, w_codes, w_scales, w_fmt, a_ebits, a_mbits, a_max_norm, a_round=0, scale_bits=8, flush=False,
               out_dtype=None, bfloat_bits=16, out_round=0, bias=None, workspace=None):
    """y = round(MX(x) @ W^T (+ bias)) with pre-packed W; see mxq_linear_fwd.  Returns (y, workspace)."""
    _require_cuda(x, "x")
    M, K = x.shape
    N = w_codes.shape[0]
    need = lib().mxq_linear_workspace_bytes(M, K)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    y = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    with _device_of(x.device):
        check(lib().mxq_linear_fwd(_ptr(x), _DT[x.dtype], M, K, int(a_ebits), int(a_mbits), float(a_max_norm),
                                   int(a_round), int(scale_bits), int(bool(flush)), _ptr(w_codes), _ptr(w_scales),
                                   N, int(w_fmt), _ptr(y), _DT[y.dtype], int(bfloat_bits), int(out_round),
                                   _ptr(bias), _ptr(workspace), workspace.numel(), _stream(x)))
    return y, workspace


def linear_fwd_train(x, w, a_fmt, w_fmt, scale_bits, flush, out_dtype, bfloat_bits, out_round, bias=None):
    """y = round(MX(x) MX(w)^T (+ bias)) with both operands quantized in the call; see mxq_linear_fwd_train.
    x [M, K], w [N, K] contiguous CUDA tensors of one dtype; a_fmt / w_fmt: ElemFormatC."""
    M, K = x.shape
    N = w.shape[0]
    L = lib()
    ws = torch.empty(L.mxq_linear_train_workspace_bytes(M, K, N), dtype=torch.uint8, device=x.device)
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    with _device_of(x.device):
        check(L.mxq_linear_fwd_train(_ptr(x), _ptr(w), _DT[x.dtype], M, K, N, ctypes.byref(a_fmt), ctypes.byref(w_fmt),
                                     int(scale_bits), int(bool(flush)), _ptr(y), _DT[y.dtype], int(bfloat_bits),
                                     int(out_round), _ptr(bias), _ptr(ws), ws.numel(), _stream(x)))
    return y


def matmul_fwd(a, b, batch, M, K, N, a_trans, b_trans, a_fmt, b_fmt, scale_bits, flush, out_dtype, bfloat_bits,
               out_round, bias=None, a_packed=None):
    """C [batch, M, N] = op(a) op(b) with both operands MX-quantized in the call; see mxq_matmul_fwd.
    a_packed: (codes, scales) of an already packed left operand (a is then only a shape donor)."""
    L = lib()
    ws = torch.empty(L.mxq_matmul_workspace_bytes(batch, M, K, N), dtype=torch.uint8, device=b.device)
    c = torch.empty((batch, M, N), dtype=out_dtype, device=b.device)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    ac, as_ = a_packed if a_packed is not None else (None, None)
    with _device_of(b.device):
        check(L.mxq_matmul_fwd(None if a_packed is not None else _ptr(a), _ptr(b), _DT[b.dtype], batch, M, K, N,
                               int(bool(a_trans)), int(bool(b_trans)), ctypes.byref(a_fmt), ctypes.byref(b_fmt),
                               int(scale_bits), int(bool(flush)), _ptr(ac), _ptr(as_), _ptr(c), _DT[c.dtype],
                               int(bfloat_bits), int(out_round), _ptr(bias), _ptr(ws), ws.numel(), _stream(b)))
    return c


def linear_bwd(go, x, w, go_fmt_gw, x_fmt_gw, go_fmt_gi, w_fmt_gi, scale_bits, flush, out_dtype, bfloat_bits,
               round_grad_input, round_grad_weight, want_gx=True, want_gw=True):
    """(grad_x [M, K] or None, grad_w [N, K] or None) of an MX linear layer; see mxq_linear_bwd."""
    M, N = go.shape
    K = x.shape[1]
    L = lib()
    ws = torch.empty(L.mxq_linear_train_workspace_bytes(M, K, N), dtype=torch.uint8, device=go.device)
    gx = torch.empty((M, K), dtype=out_dtype, device=go.device) if want_gx else None
    gw = torch.empty((N, K), dtype=out_dtype, device=go.device) if want_gw else None
    with _device_of(go.device):
        check(L.mxq_linear_bwd(_ptr(go), _ptr(x), _ptr(w), _DT[go.dtype], M, K, N, ctypes.byref(go_fmt_gw),
                               ctypes.byref(x_fmt_gw), ctypes.byref(go_fmt_gi), ctypes.byref(w_fmt_gi), int(scale_bits),
                               int(bool(flush)), _ptr(gx), _ptr(gw), _DT[out_dtype], int(bfloat_bits),
                               int(round_grad_input), int(round_grad_weight), _ptr(ws), ws.numel(), _stream(go)))
    return gx, gw


def _require_bf16(t, name):
    if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.bfloat16):
        raise MxqError("%s must be a contiguous bfloat16 CUDA tensor" % name)


def silu_bf16(gate, up=None, want_sig=False):
    """Fused bfloat16 SiLU chain (times `up` if given); see mxq_silu_bf16.  Returns out or (out, sig)."""
    _require_bf16(gate, "gate")
    if up is not None:
        _require_bf16(up, "up")
        if up.shape != gate.shape:
            raise MxqError("gate and up must have the same shape")
    out = torch.empty_like(gate)
    sig = torch.empty_like(gate) if want_sig else None
    with _device_of(gate.device):
        check(lib().mxq_silu_bf16(_ptr(gate), _ptr(up), _ptr(out), _ptr(sig), gate.numel(), _stream(gate)))
    return (out, sig) if want_sig else out


def swiglu_quantize_mx(gate, up, scale_bits, ebits, mbits, max_norm, flush=False, rmode=0, gemm_layout=True):
    """Packed MX operand (codes uint8 [rows, K], scales uint8) of SiLU(gate) * up; see mxq_swiglu_quantize_mx."""
    _require_bf16(gate, "gate")
    _require_bf16(up, "up")
    if gate.dim() != 2 or up.shape != gate.shape:
        raise MxqError("gate and up must be [rows, K] tensors of the same shape")
    rows, K = gate.shape
    codes = torch.empty((rows, K), dtype=torch.uint8, device=gate.device)
    if gemm_layout:
        alloc = torch.empty if rows % 128 == 0 and K % 128 == 0 else torch.zeros
        scales = alloc(((rows + 127) // 128) * ((K + 127) // 128) * 512, dtype=torch.uint8, device=gate.device)
    else:
        scales = torch.empty((rows, K // 32), dtype=torch.uint8, device=gate.device)
    with _device_of(gate.device):
        check(lib().mxq_swiglu_quantize_mx(_ptr(gate), _ptr(up), _ptr(codes), _ptr(scales), rows, K, int(scale_bits),
                                           int(ebits), int(mbits), float(max_norm), int(bool(flush)), int(rmode),
                                           SCALES_GEMM_LAYOUT if gemm_layout else 0, rows, _stream(gate)))
    return codes, scales


SOFTMAX_MAX_COLS = 2048


def softmax_bf16(x, use_exp2=False):
    """Fused bfloat16 softmax over the last dimension; see mxq_softmax_bf16."""
    _require_bf16(x, "x")
    cols = x.shape[-1]
    out = torch.empty_like(x)
    with _device_of(x.device):
        check(lib().mxq_softmax_bf16(_ptr(x), _ptr(out), x.numel() // cols if cols else 0, cols, int(bool(use_exp2)),
                                     _stream(x)))
    return out


def softmax_quantize_mx(x, scale_bits, ebits, mbits, max_norm, flush=False, rmode=0, rows_per_batch=0,
                        want_probs=True):
    """Softmax over the last dimension of bfloat16 x fused with the MX packing of the probabilities;
    see mxq_softmax_quantize_mx.  Returns (probs or None, codes uint8 like x, scales uint8 in the GEMM layout)."""
    _require_bf16(x, "x")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    rpb = rows_per_batch or rows
    probs = torch.empty_like(x) if want_probs else None
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    nb = rows // rpb if rpb else 0
    alloc = torch.empty if rpb % 128 == 0 and cols % 128 == 0 else torch.zeros
    scales = alloc(nb * ((rpb + 127) // 128) * ((cols + 127) // 128) * 512, dtype=torch.uint8, device=x.device)
    with _device_of(x.device):
        check(lib().mxq_softmax_quantize_mx(_ptr(x), _ptr(probs), _ptr(codes), _ptr(scales), rows, cols, int(scale_bits),
                                            int(ebits), int(mbits), float(max_norm), int(bool(flush)), int(rmode),
                                            SCALES_GEMM_LAYOUT, int(rpb), _stream(x)))
    return probs, codes, scales


def rmsnorm_bf16(x, weight, bias, eps, want_saved=False):
    """Fused bfloat16 RMSNorm over the last dimension; see mxq_rmsnorm_bf16.
    Returns out or (out, x_norm, rms_inv)."""
    _require_bf16(x, "x")
    _require_bf16(weight, "weight")
    if bias is not None:
        _require_bf16(bias, "bias")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    out = torch.empty_like(x)
    xn = torch.empty_like(x) if want_saved else None
    ri = torch.empty(x.shape[:-1] + (1,), dtype=x.dtype, device=x.device) if want_saved else None
    with _device_of(x.device):
        check(lib().mxq_rmsnorm_bf16(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(xn), _ptr(ri), rows, hidden,
                                     float(eps), _stream(x)))
    return (out, xn, ri) if want_saved else out


def launch_count(what):
    """Launches made by this process: 0 = block-scaled GEMMs, 1 = MX quantizations; see mxq_launch_count."""
    L = lib()
    L.mxq_launch_count.restype = ctypes.c_int64
    L.mxq_launch_count.argtypes = [ctypes.c_int]
    return int(L.mxq_launch_count(int(what)))


@contextlib.contextmanager
def gemm_sm_budget(sms):
    """Within the block the persistent GEMM kernels occupy at most `sms` SMs (0 = all), which leaves a
    collective running beside them CTAs to run on; see mxq_gemm_sm_budget."""
    prev = lib().mxq_gemm_sm_budget(int(sms))
    try:
        yield
    finally:
        lib().mxq_gemm_sm_budget(int(prev))


def device_status(clear=True):
    """Synchronous read of the device status word (0 = no kernel gave up on a wait)."""
    return lib().mxq_device_status(1 if clear else 0)


def _reduce(A, fn):
    _require_cuda(A, "A")
    if A.dtype != torch.float32:
        raise MxqError("reduce over the inner dim supports float32 only")
    inner = A.shape[-1]
    rows = A.numel() // inner if inner else 0
    out = torch.empty(A.shape[:-1], dtype=A.dtype, device=A.device)
    with _device_of(A.device):
        check(fn(_ptr(A), _ptr(out), rows, inner, _stream(A)))
    return out


class _Funcs:
    """The reference extension's exported names on top of the C ABI."""

    @staticmethod
    def quantize_mx_by_tile_func_cuda(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm,
                                      tile_size, axis, flush_fp32_subnorms=False, rmode=0):
        if axis >= A.dim():
            raise MxqError("quantize_mx_by_tile axis exceeds input dimensions")
        return quantize_mx(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm, tile_size, axis,
                           flush_fp32_subnorms, int(rmode))

    @staticmethod
    def quantize_mx_func_cuda(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm, max_values,
                              axis, flush_fp32_subnorms=False, rmode=0):
        # the whole `axis` is one block; its maximum is recomputed in-kernel
        if axis >= A.dim():
            raise MxqError("quantize_mx_func_cuda axis exceeds input dimensions")
        return quantize_mx(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm, 0, axis,
                           flush_fp32_subnorms, int(rmode))

    @staticmethod
    def quantize_elemwise_func_cuda(A, bits, exp_bits, max_norm, rmode=0, saturate_normals=False,
                                    allow_denorm=True):
        return quantize_elemwise(A, bits, exp_bits, max_norm, int(rmode), saturate_normals, allow_denorm)

    @staticmethod
    def quantize_mx_func_cpp(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm, max_values, axis,
                             flush_fp32_subnorms=False, rmode=0):
        # the whole `axis` is one block (the caller reshaped to blocks); its maximum is recomputed
        if not 1 <= A.dim() <= 5:
            raise MxqError("quantize_mx_func_cpp needs a tensor of 1 to 5 dimensions")
        if axis >= A.dim():
            raise MxqError("quantize_mx_func_cpp axis exceeds input dimensions")
        return cpu_quantize_mx(A, scale_bits, elem_ebits, elem_mbits, elem_max_norm, 0, axis, flush_fp32_subnorms,
                               int(rmode))

    @staticmethod
    def quantize_elemwise_func_cpp(A, bits, exp_bits, max_norm, rmode=0, saturate_normals=False,
                                   allow_denorm=True):
        return cpu_quantize_elemwise(A, bits, exp_bits, max_norm, int(rmode), saturate_normals, allow_denorm)

    @staticmethod
    def reduce_sum_inner_dim(A):
        return _reduce(A, lib().mxq_reduce_sum_inner)

    @staticmethod
    def reduce_max_inner_dim(A):
        return _reduce(A, lib().mxq_reduce_max_inner)


funcs = _Funcs()
