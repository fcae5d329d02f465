"""CPU tests of host-side logic that needs no GPU: sharding bounds, the packed-weight
bookkeeping of mx.Linear, the condition under which the fused bfloat16 vector kernels
may replace a chain of vector operations, and the scale-slab slicing of the pipelined
down projection."""
import gc

import pytest
import torch

from microxcaling_b200 import _mxgemm
from microxcaling_b200.specs import finalize_mx_specs
from microxcaling_b200.tp import shard_bounds
from microxcaling_b200.vector_ops import fused_bf16_ok


def test_shard_bounds():
    assert shard_bounds(28672, 3, 8, multiple=128) == (3 * 3584, 4 * 3584)
    assert shard_bounds(16384, 0, 1) == (0, 16384)
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 3)
    with pytest.raises(ValueError):
        shard_bounds(28672, 0, 16, multiple=1024)


class _FakeCuda:
    """Stands in for a CUDA tensor in the cache key."""
    is_cuda = True
    dtype = torch.bfloat16
    shape = (8, 8)


def test_packed_weight_cache_bookkeeping(monkeypatch):
    calls = []
    monkeypatch.setattr(_mxgemm, "_pack", lambda x, fmt, sp, rnd, cl: (calls.append(fmt), ("packed", len(calls)))[1])
    sp = {"scale_bits": 8, "mx_flush_fp32_subnorms": False, "bfloat": 16, "fp": 0, "round_weight": "nearest"}
    w = torch.randn(8, 8)
    a = _mxgemm._pack_cached(w, _FakeCuda(), "fp8_e4m3", sp, "nearest", True)
    assert _mxgemm._pack_cached(w, _FakeCuda(), "fp8_e4m3", sp, "nearest", True) is a and len(calls) == 1
    _mxgemm._pack_cached(w, _FakeCuda(), "fp4_e2m1", sp, "nearest", True)            # other format: packed again
    assert len(calls) == 2
    with torch.no_grad():
        w.add_(1.0)                                                                   # in-place update bumps the version
    _mxgemm._pack_cached(w, _FakeCuda(), "fp4_e2m1", sp, "nearest", True)
    assert len(calls) == 3
    _mxgemm._pack_cached(None, _FakeCuda(), "fp4_e2m1", sp, "nearest", True)          # no source tensor: never cached
    assert len(calls) == 4
    n = len(_mxgemm._PACK_CACHE)
    del w
    gc.collect()
    assert len(_mxgemm._PACK_CACHE) == n - 1                                          # entry dropped with the tensor


def test_fused_vector_kernels_only_for_identity_rounding_of_bf16_cuda_tensors():
    sp = finalize_mx_specs({"bfloat": 16})
    cpu = torch.zeros(4, dtype=torch.bfloat16)
    assert not fused_bf16_ok(sp, cpu)                       # CPU tensor
    assert not fused_bf16_ok(None, cpu)
    fake = type("T", (), {"is_cuda": True, "dtype": torch.bfloat16})()
    assert fused_bf16_ok(sp, fake)
    assert not fused_bf16_ok(sp, fake, None)                # a missing operand (e.g. no bias)
    assert not fused_bf16_ok(sp, type("T", (), {"is_cuda": True, "dtype": torch.float32})())
    for bad in ({"bfloat": 12}, {"bfloat": 0, "fp": 16}, {"bfloat": 16, "vec_use_exp2": True},
                {"bfloat": 16, "vec_use_recip": True}, {"bfloat": 16, "bfloat_subnorms": False},
                {"bfloat": 16, "round": "dither"}):
        assert not fused_bf16_ok(finalize_mx_specs(bad), fake), bad


def test_scale_slab_slicing_matches_the_chunk_layout():
    """Rows [c*slab, (c+1)*slab) of a packed [H, K] operand own a contiguous run of 512-byte scale chunks."""
    H, K, n_slabs = 1024, 384, 4
    kchunks = (K + 127) // 128
    flat = torch.arange((H // 128) * kchunks * 512)
    slab = H // n_slabs
    for c in range(n_slabs):
        lo, hi = (c * slab // 128) * kchunks * 512, ((c + 1) * slab // 128) * kchunks * 512
        piece = flat[lo:hi]
        # chunk index of (row r, k block kb) = (r // 128) * kchunks + kb // 4
        first_chunk = (c * slab // 128) * kchunks
        assert piece[0] == first_chunk * 512 and piece.numel() == (slab // 128) * kchunks * 512
