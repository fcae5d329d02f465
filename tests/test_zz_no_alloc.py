"""mxq_linear_fwd_static: the linear-layer forward for callers that may not
allocate device memory (a server that handed all of it to its own pools, a
loop that cannot take cudaMalloc's device-wide stall) and have no workspace to
pass.  Its scratch is a fixed array inside libmxq.so.

Called here straight through the C ABI, twice in a row, and compared bit for
bit with mxq_linear_fwd (same kernels, caller-provided workspace).  The second
call uses a smaller, ragged shape so that it runs over the first call's left-
over scratch contents.  This file is collected last on purpose."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
E4M3 = (4, 5, 448.0)
E2M1 = (2, 3, 6.0)


def _lib():
    L = ctypes.CDLL(os.path.join(ROOT, "microxcaling_b200", "libmxq.so"))
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    L.mxq_quantize_mx.argtypes = [vp, vp, vp, vp, i32, i64, i64, i64, i32, i32, i32, i32, f32, i32, i32, vp, i32, i64, vp]
    lin = [vp, i32, i64, i64, i32, i32, f32, i32, i32, i32, vp, vp, i64, i32, vp, i32, i32, i32, vp]
    L.mxq_linear_fwd.argtypes = lin + [vp, i64, vp]
    L.mxq_linear_fwd_static.argtypes = lin + [vp]
    L.mxq_linear_workspace_bytes.argtypes = [i64, i64]
    L.mxq_linear_workspace_bytes.restype = i64
    L.mxq_sf_bytes.argtypes = [i64, i64, i64]
    L.mxq_sf_bytes.restype = i64
    L.mxq_linear_static_max_elems.restype = i64
    return L


def _pack_weight(L, w, st):
    N, K = w.shape
    codes = torch.empty(N, K, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(L.mxq_sf_bytes(1, N, K), dtype=torch.uint8, device="cuda")
    rc = L.mxq_quantize_mx(w.data_ptr(), None, codes.data_ptr(), scales.data_ptr(), 2, N, K, 1, 32, 8,
                           E2M1[0], E2M1[1], E2M1[2], 0, 0, None, 2, N, st)
    assert rc == 0
    return codes, scales


def _run_pair(L, M, K, N, seed, with_bias):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).to(torch.bfloat16).float().cuda() if with_bias else None
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    wc, ws = _pack_weight(L, w, st)
    common = [x.data_ptr(), 2, M, K, E4M3[0], E4M3[1], E4M3[2], 0, 8, 0, wc.data_ptr(), ws.data_ptr(), N, 0]
    tail = [2, 16, 0, bias.data_ptr() if with_bias else None]
    y_ws = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    y_st = torch.ones(M, N, dtype=torch.bfloat16, device="cuda")
    need = L.mxq_linear_workspace_bytes(M, K)
    wsp = torch.empty(need, dtype=torch.uint8, device="cuda")
    assert L.mxq_linear_fwd(*common, y_ws.data_ptr(), *tail, wsp.data_ptr(), need, st) == 0
    assert L.mxq_linear_fwd_static(*common, y_st.data_ptr(), *tail, st) == 0
    torch.cuda.synchronize()
    assert L.mxq_linear_static_status() == 0
    assert int(wsp[:4].view(torch.int32).item()) == 0
    assert torch.isfinite(y_ws.float()).all()
    assert torch.equal(y_st.view(torch.int16), y_ws.view(torch.int16)), (M, K, N)


def test_static_scratch_matches_workspace_entry_point_twice():
    L = _lib()
    _run_pair(L, 512, 1024, 384, seed=1, with_bias=True)
    _run_pair(L, 200, 256, 136, seed=2, with_bias=False)      # smaller and ragged: runs over stale scratch


def test_static_scratch_rejects_oversize_and_bad_shapes():
    L = _lib()
    lim = L.mxq_linear_static_max_elems()
    assert lim == 32 << 20
    dummy = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    args = lambda M, K: [p, 2, M, K, 4, 5, 448.0, 0, 8, 0, p, p, 128, 0, p, 2, 16, 0, None, None]
    assert L.mxq_linear_fwd_static(*args(8192 + 128, 4096)) == -5        # MXQ_ERR_TOO_LARGE, nothing launched
    assert L.mxq_linear_fwd_static(*args(1 << 30, 1 << 20)) == -5
    assert L.mxq_linear_fwd_static(*args(128, 100)) == -2                # K not a multiple of 128
    torch.cuda.synchronize()


def test_static_entry_point_allocates_nothing_and_runs_at_its_limit():
    """What the entry point is for: device memory in use does not move across a call once the first call
    on the device has looked the array up.  The call is made at exactly the documented limit
    (ceil(M/128)*128 * K == 32 Mi), where the scratch layout ends at the end of the fixed array, and its
    result is compared with the workspace entry point."""
    L = _lib()
    M, K, N = 8192, 4096, 128
    assert M * K == L.mxq_linear_static_max_elems()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16).cuda()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    wc, ws = _pack_weight(L, w, st)
    common = [x.data_ptr(), 2, M, K, E4M3[0], E4M3[1], E4M3[2], 0, 8, 0, wc.data_ptr(), ws.data_ptr(), N, 0]
    tail = [2, 16, 0, None]
    y_ws = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    y_st = torch.ones(M, N, dtype=torch.bfloat16, device="cuda")
    need = L.mxq_linear_workspace_bytes(M, K)
    wsp = torch.empty(need, dtype=torch.uint8, device="cuda")
    assert L.mxq_linear_fwd(*common, y_ws.data_ptr(), *tail, wsp.data_ptr(), need, st) == 0
    assert L.mxq_linear_fwd_static(*common, y_st.data_ptr(), *tail, st) == 0       # warm-up (first-call set-up)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    y_st.fill_(1.0)
    assert L.mxq_linear_fwd_static(*common, y_st.data_ptr(), *tail, st) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)              # no cudaMalloc, no torch allocation behind the call
    assert L.mxq_linear_static_status() == 0
    assert torch.equal(y_st.view(torch.int16), y_ws.view(torch.int16))
