"""CPU tests of host-side logic that needs no GPU: sharding bounds, the packed-weight
bookkeeping of mx.Linear, the condition under which the fused bfloat16 vector kernels
may replace a chain of vector operations, and the scale-slab slicing of the pipelined
down projection."""
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


def test_packed_operand_file_roundtrip(tmp_path):
    """The on-disk layout of a packed MX operand: header fields, sizes, and a save/load round trip."""
    from microxcaling_b200.packed import PackedMX
    g = torch.Generator().manual_seed(3)
    batch, rows, K = 2, 130, 96
    codes = torch.randint(0, 256, (batch, rows, K), dtype=torch.uint8, generator=g)
    scales = torch.randint(100, 140, (PackedMX.scales_bytes(batch, rows, K),), dtype=torch.uint8, generator=g)
    p = PackedMX(codes, scales, 0, 4, 5, 8, batch, rows, K)
    path = str(tmp_path / "w.mxq")
    p.save(path)
    raw = open(path, "rb").read()
    assert raw[:4] == b"MXQP" and len(raw) == 128 + codes.numel() + scales.numel()
    q = PackedMX.load(path)
    assert (q.batch, q.rows, q.K, q.container, q.ebits, q.mbits, q.scale_bits) == (batch, rows, K, 0, 4, 5, 8)
    assert torch.equal(q.codes, codes) and torch.equal(q.scales, scales)
    # the scale of (b, r, k) sits at the documented byte of the chunk layout
    sr = q.scale_bytes_rowmajor()
    b_, r, k = 1, 129, 2
    off = ((b_ * 2 + r // 128) * 1 + k // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + k % 4
    assert int(sr[b_, r, k]) == int(scales[off])
    # decoding: code 0x38 is 1.0 in e4m3, scale byte 128 doubles it
    one = PackedMX(torch.full((1, 1, 32), 0x38, dtype=torch.uint8), torch.full((512,), 128, dtype=torch.uint8),
                   0, 4, 5, 8, 1, 1, 32)
    assert torch.equal(one.dequantize(), torch.full((1, 1, 32), 2.0))
    open(path, "wb").write(raw[:200])
    with pytest.raises(ValueError):
        PackedMX.load(path)


def test_linear_keeps_a_packed_weight_only_when_asked(monkeypatch):
    """mx.Linear re-quantizes its weight in every call, as the reference does, unless
    prequantize_weights() froze it; the frozen packed operand follows the parameter's version."""
    import microxcaling_b200 as mx
    from microxcaling_b200 import linear as L
    sp = finalize_mx_specs({"w_elem_format": "fp8_e4m3", "a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16,
                            "round": "even"})
    lin = mx.Linear(64, 32, bias=False, mx_specs=sp)
    assert lin.packed_weight() is None                      # CPU weight: no tensor-core path, nothing kept
    packs = []
    monkeypatch.setattr(_mxgemm, "_fast_ok", lambda *a, **k: True)
    monkeypatch.setattr(_mxgemm, "_pack", lambda x, fmt, sp_, rnd, cl: (packs.append(x._version), ("packed", len(packs)))[1])
    fake_w = torch.nn.Parameter(torch.randn(32, 64))
    monkeypatch.setattr(type(fake_w), "is_cuda", property(lambda self: True), raising=False)
    lin.weight = fake_w
    a = lin.packed_weight()
    assert lin.packed_weight() is a and len(packs) == 1     # same storage, same version: kept
    with torch.no_grad():
        lin.weight.add_(1.0)
    assert lin.packed_weight() is not a and len(packs) == 2  # the version counter moved: packed again


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
