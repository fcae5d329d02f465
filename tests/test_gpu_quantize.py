"""GPU parity of the quantization kernels, called through the C ABI
(microxcaling_b200._backend -> libmxq.so), against the CPU oracle and the
fixtures recorded from the reference.  Bit-exact work: tolerance zero, with the
reference's own notion of equality (numeric equality, NaN == NaN, -0 == +0)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import all_encodings, sha, bf16_bits, bf16_vals, dequant_packed

pytestmark = pytest.mark.gpu

FMTS = ["fp8_e4m3", "fp8_e5m2", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8", "int4", "int2"]
ROUNDS = {"nearest": 0, "floor": 1, "even": 2}


@pytest.fixture(scope="module")
def be():
    from microxcaling_b200 import _backend
    _backend.lib()
    return _backend


def gpu_mx(be, x, fmt, axis=-1, block=32, scale_bits=8, round="nearest", flush=False, **kw):
    eb, mb, mn = oracle.FORMATS[fmt]
    t = torch.as_tensor(x).cuda()
    return be.quantize_mx(t, scale_bits, eb, mb, mn, block, axis, flush, ROUNDS[round], **kw)


def to_np(t):
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.float().cpu().numpy()


def test_recorded_reference_calls(be, golden_recorded):
    meta, z = golden_recorded
    bad = []
    for i, rec in enumerate(meta):
        if "recipe" in rec:
            e, m, inf = rec["recipe"]
            x = all_encodings(e, m, bool(inf)).reshape(rec["shape"])
        else:
            x = z["x%d" % i]
        p = rec["params"]
        if x.ndim == 0:
            continue
        if rec["kind"] == "mx":
            y = to_np(gpu_mx(be, x, p["fmt"], p["axis"], p["block"], p["scale_bits"], p["round"], p["flush"]))
        else:
            y = to_np(be.quantize_elemwise(torch.as_tensor(x).cuda(), p["bits"], p["exp_bits"], p["max_norm"],
                                           ROUNDS[p["round"]], p["saturate"], p["allow_denorm"]))
        ok = (sha(y) == rec["sha"]) if "sha" in rec else oracle.same_values(y, z["y%d" % i])
        if not ok:
            bad.append((i, rec["kind"], p))
    assert not bad, (len(bad), bad[:5])


def test_seeded_sweep(be, golden_sweep):
    meta, z = golden_sweep
    bad = []
    for rec in meta:
        x = z["in_" + rec["in"]]
        if rec["kind"] == "mx":
            y = to_np(gpu_mx(be, x, rec["fmt"], rec["axis"], rec["block"], rec["scale_bits"], rec["round"], rec["flush"]))
        else:
            if rec["spec"] == "bfloat":
                bits, eb = rec["val"] - 7, 8
                mn = 2.0 ** 127 * (2 ** (bits - 1) - 1) / 2 ** (bits - 2)
            else:
                bits, eb = rec["val"] - 4, 5
                mn = 2.0 ** 15 * (2 ** (bits - 1) - 1) / 2 ** (bits - 2)
            y = to_np(be.quantize_elemwise(torch.as_tensor(x).cuda(), bits, eb, mn, ROUNDS[rec["round"]],
                                           False, rec["subnorms"]))
        if sha(y) != rec["sha"]:
            bad.append(rec)
    assert not bad, (len(bad), bad[:5])


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("round", list(ROUNDS))
def test_mx_all_bf16_patterns(be, fmt, round):
    """Every bf16 bit pattern (NaN/Inf rows included) in blocks of 8, 32 and 64
    along the last axis and of 32 along axis 0, scale widths 8 and 5."""
    u = np.arange(1 << 16, dtype=np.uint32) << 16
    rng = np.random.default_rng(1)
    x = rng.permutation(u).view(np.float32).reshape(256, 256)
    for sb in (8, 5):
        for axis, block in ((-1, 8), (-1, 32), (-1, 64), (0, 32), (0, 16)):
            for flush in (False, True):
                want = oracle.quantize_mx(x, fmt, axis=axis, block=block, scale_bits=sb, round=round, flush=flush)
                got = to_np(gpu_mx(be, x, fmt, axis, block, sb, round, flush))
                assert oracle.same_values(got, want), (fmt, round, sb, axis, block, flush)
                got = to_np(gpu_mx(be, torch.as_tensor(x).to(torch.bfloat16), fmt, axis, block, sb, round, flush))
                assert oracle.same_values(got, want), (fmt, round, sb, axis, block, flush, "bf16 tensor")


def _anchored_bf16_blocks():
    """Blocks of 32 bf16 values: one anchor that fixes the block maximum, then 31
    values from every (sign, mantissa) pattern at an exponent 0..17 binades below
    it -- every tie and near-tie of the normal and subnormal range of each format."""
    rows = []
    for e0 in (60, 127, 190):
        for anchor_m in (0x00, 0x7f):
            anchor = (e0 << 7) | anchor_m
            for k in range(0, 18):
                pats = np.array([(s << 15) | ((e0 - k) << 7) | m for s in (0, 1) for m in range(128)], dtype=np.uint32)
                pats = np.concatenate([pats, np.zeros((-len(pats)) % 31, dtype=np.uint32)]).reshape(-1, 31)
                blk = np.concatenate([np.full((pats.shape[0], 1), anchor, dtype=np.uint32), pats], axis=1)
                rows.append(blk)
    return (np.concatenate(rows, axis=0) << 16).view(np.float32)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("round", list(ROUNDS))
def test_mx_bf16_ties_at_every_relative_exponent(be, fmt, round):
    x = _anchored_bf16_blocks()                       # [n_blocks, 32]
    want = oracle.quantize_mx(x, fmt, axis=-1, block=32, scale_bits=8, round=round)
    n = x.shape[0] // 8 * 8
    xt = np.ascontiguousarray(x[:n].T)                # blocks along axis 0, 8-aligned columns
    for dt in (torch.bfloat16, torch.float32):        # the values are bf16 patterns: both casts are exact
        got = to_np(gpu_mx(be, torch.as_tensor(x).to(dt), fmt, -1, 32, 8, round, False))
        assert oracle.same_values(got, want), (fmt, round, dt, "last axis")
        got = to_np(gpu_mx(be, torch.as_tensor(xt).to(dt), fmt, 0, 32, 8, round, False))
        assert oracle.same_values(got, np.ascontiguousarray(want[:n].T)), (fmt, round, dt, "axis 0")


@pytest.mark.parametrize("fmt", ["fp8_e4m3", "fp8_e5m2", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1"])
@pytest.mark.parametrize("round", list(ROUNDS))
def test_mx_codes_only_ties_at_every_relative_exponent(be, fmt, round):
    """The packing-only kernels (no dequantized output: element rounding by the hardware conversions
    where the format has one) on the same tie walk, blocks along the last axis and along axis 0 with
    transposed codes; the packed operand, decoded, must equal the oracle's values bit for bit."""
    eb, mb, mn = oracle.FORMATS[fmt]
    x = _anchored_bf16_blocks()
    want = oracle.quantize_mx(x, fmt, axis=-1, block=32, scale_bits=8, round=round)
    xb = torch.as_tensor(x).to(torch.bfloat16).cuda()
    _, codes, scales = be.quantize_mx(xb, 8, eb, mb, mn, 32, 1, False, ROUNDS[round], want_dq=False, want_codes=True)
    got = dequant_packed(codes.cpu().numpy(), scales.cpu().numpy(), 32, 1, eb, mb)
    assert oracle.same_values(got, want), (fmt, round, "last axis")
    n = x.shape[0] // 8 * 8
    xt = torch.as_tensor(np.ascontiguousarray(x[:n].T)).to(torch.bfloat16).cuda()[None]     # [1, 32, n]
    _, codes, scales = be.quantize_mx(xt, 8, eb, mb, mn, 32, 1, False, ROUNDS[round], want_dq=False, want_codes=True,
                                      transposed=True)
    got = dequant_packed(codes.cpu().numpy()[0], scales.cpu().numpy()[0], 32, 1, eb, mb)   # [n, 32], [n, 1]
    assert oracle.same_values(got, want[:n]), (fmt, round, "axis 0, transposed codes")


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("axis", [0, 1, 2])
def test_mx_dtypes_and_axes(be, dtype, axis):
    rng = np.random.default_rng(2)
    x = (rng.standard_t(3, (4, 96, 160)) * np.where(rng.random((4, 96, 160)) < 1e-3, 1e3, 1.0)).astype(np.float32)
    if dtype == "bf16":
        t = torch.as_tensor(x).to(torch.bfloat16)
        xin = bf16_bits(t.float().numpy())
    elif dtype == "f16":
        t = torch.as_tensor(x).to(torch.float16)
        xin = t.numpy()
    else:
        t = torch.as_tensor(x)
        xin = x
    for fmt in FMTS:
        for rnd in ROUNDS:
            eb, mb, mn = oracle.FORMATS[fmt]
            got = be.quantize_mx(t.cuda(), 8, eb, mb, mn, 32, axis, False, ROUNDS[rnd])
            assert got.dtype == t.dtype
            want = oracle.quantize_mx(xin, fmt, axis=axis, round=rnd)
            if dtype == "bf16":
                want = bf16_vals(want)
            assert oracle.same_values(to_np(got), want.astype(np.float32)), (dtype, axis, fmt, rnd)


@pytest.mark.parametrize("shape,axis,block", [((7, 33), 1, 32), ((33, 7), 0, 32), ((5, 9), 1, 9), ((1,), 0, 32),
                                              ((3, 1, 5), 1, 32), ((2, 40, 6), 1, 16), ((64, 100), 1, 10),
                                              ((130, 24), 0, 64), ((4, 4096), 1, 0), ((257, 8), 0, 0)])
def test_mx_ragged_and_odd_shapes(be, shape, axis, block):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(shape).astype(np.float32) * 3
    for fmt in ("fp8_e4m3", "fp4_e2m1", "int8"):
        for rnd in ROUNDS:
            want = oracle.quantize_mx(x, fmt, axis=axis, block=block, round=rnd)
            got = to_np(gpu_mx(be, x, fmt, axis, block, 8, rnd))
            assert oracle.same_values(got, want), (shape, axis, block, fmt, rnd)


def test_mx_empty(be):
    x = torch.empty(0, device="cuda")
    y = be.quantize_mx(x, 8, 4, 5, 448.0, 32, 0)
    assert y.numel() == 0
    y = be.quantize_elemwise(x, 9, 8, 3.38e38)
    assert y.numel() == 0


@pytest.mark.parametrize("fmt", ["fp8_e4m3", "fp8_e5m2", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8"])
@pytest.mark.parametrize("case", ["last", "strided", "strided_T", "generic", "generic_T", "codes_only"])
def test_mx_packed_operand(be, fmt, case):
    """codes (fp8 container) x 2^(scale-127) must equal the dequantized output,
    in the plain and in the transposed (blocked axis innermost) layout."""
    rng = np.random.default_rng(4)
    eb, mb, mn = oracle.FORMATS[fmt]
    if case in ("last", "codes_only"):
        shape, axis, block, tr = (1, 48, 256), 2, 32, False
    elif case.startswith("strided"):
        shape, axis, block, tr = (3, 96, 64), 1, 32, case.endswith("_T")
    else:
        shape, axis, block, tr = (3, 50, 7), 1, 32, case.endswith("_T")
    x = (rng.standard_t(3, shape) * 2).astype(np.float32)
    x.reshape(-1)[5] = np.nan
    xb = torch.as_tensor(x).to(torch.bfloat16)
    dq, codes, scales = be.quantize_mx(xb.cuda(), 8, eb, mb, mn, block, axis, want_dq=(case != "codes_only"),
                                       want_codes=True, transposed=tr)
    want = bf16_vals(oracle.quantize_mx(bf16_bits(xb.float().numpy()), fmt, axis=axis, block=block))
    if dq is not None:
        assert oracle.same_values(dq.float().cpu().numpy(), want)
    codes, scales = codes.cpu().numpy(), scales.cpu().numpy()
    n = shape[axis]
    nblk = (n + block - 1) // block
    if tr:
        assert codes.shape == (shape[0], shape[2], nblk * block) and scales.shape == (shape[0], shape[2], nblk)
        assert not codes[..., n:].any()
        codes = np.moveaxis(codes, -1, 1)[:, :n]
        scales = np.moveaxis(scales, -1, 1)
    else:
        assert codes.shape == shape and scales.shape == shape[:axis] + (nblk,) + shape[axis + 1:]
    got = dequant_packed(codes, scales, block, axis, eb, mb)
    assert oracle.same_values(got, want), (fmt, case)


@pytest.mark.parametrize("in_dt,out_dt", [("f32", "f32"), ("bf16", "bf16"), ("f16", "f16"), ("f32", "bf16")])
def test_elemwise_formats(be, in_dt, out_dt):
    TD = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
    u = (np.arange(1 << 16, dtype=np.uint32) << 16).view(np.float32)
    rng = np.random.default_rng(6)
    r = (rng.standard_normal(50001) * np.exp2(rng.integers(-150, 128, 50001).astype(np.float64))).astype(np.float32)
    x = np.concatenate([u, r])
    t = torch.as_tensor(x).to(TD[in_dt])
    xin = t.float().numpy()
    for bits, eb, mn in ((9, 8, 3.3895313892515355e38), (5, 8, 2.0 ** 127 * 1.75), (3, 8, 2.0 ** 127),
                         (12, 5, 65504.0), (6, 5, 61440.0), (4, 5, 57344.0), (5, 4, 448.0), (8, 0, 1.984375),
                         (24, 8, 3.4028234663852886e38)):
        for rnd in ROUNDS:
            for sat in (False, True):
                for den in (True, False):
                    got = be.quantize_elemwise(t.cuda(), bits, eb, mn, ROUNDS[rnd], sat, den, out_dtype=TD[out_dt])
                    assert got.dtype == TD[out_dt]
                    want = oracle.quantize_elemwise(xin, bits, eb, mn, rnd, sat, den)
                    want = torch.as_tensor(want).to(TD[out_dt]).float().numpy()
                    assert oracle.same_values(got.float().cpu().numpy(), want), (bits, eb, rnd, sat, den)


def test_bfloat16_even_equals_torch_cast(be):
    """mx/tests/test_quantize_elemwise.py:111-125: bfloat16 'even' == x.to(bfloat16)."""
    x = torch.as_tensor(all_encodings(8, 9))
    y = be.quantize_elemwise(x.cuda(), 9, 8, 3.3895313892515355e38, 2, False, True, out_dtype=torch.bfloat16)
    t = x.to(torch.bfloat16)
    fin = torch.isfinite(t.float())
    assert torch.equal(y.cpu()[fin], t[fin])


@pytest.mark.parametrize("S,H", [(5, 32), (35, 32), (7, 512), (3, 1024), (15, 2048), (11, 4096), (3, 33), (2, 5000)])
def test_reduce_inner(be, S, H):
    """mx/tests/test_reduce.py:17-46 (tolerance 1e-6 relative to the RMS)."""
    rng = np.random.default_rng(8)
    m = rng.standard_normal((64, S, H)).astype(np.float32)
    t = torch.as_tensor(m).cuda()
    s = be.funcs.reduce_sum_inner_dim(t).cpu().numpy()
    mx = be.funcs.reduce_max_inner_dim(t).cpu().numpy()
    ws, wm = oracle.reduce_inner(m, "sum"), oracle.reduce_inner(m, "max")
    assert np.array_equal(mx, wm)
    tol = 1e-6 + 1e-6 * np.sqrt(np.mean(ws.astype(np.float64) ** 2))
    assert np.max(np.abs(s - ws)) <= tol * 4
    neg = -np.abs(m)          # the reference's atomic path returns 0 here for H > 1024
    assert np.array_equal(be.funcs.reduce_max_inner_dim(torch.as_tensor(neg).cuda()).cpu().numpy(), neg.max(-1))


def test_config1_full_size(be):
    """fp32 [4096,4096] N(0,1), fp8_e4m3, block 32 along the last axis, nearest."""
    torch.manual_seed(0)
    x = torch.randn(4096, 4096)
    got = gpu_mx(be, x.numpy(), "fp8_e4m3").cpu().numpy()
    want = oracle.quantize_mx(x.numpy(), "fp8_e4m3")
    assert oracle.same_values(got, want)


def test_config2_full_size_properties(be):
    """bf16 [8192,8192] Student-t(3) with outliers: a [1024,8192] slab against the
    oracle for each format/axis, and idempotence + slab-independence at full size."""
    g = torch.Generator().manual_seed(0)
    t = torch.distributions.StudentT(3.0).sample((8192, 8192))
    mask = torch.rand(8192, 8192, generator=g) < 1e-3
    x = torch.where(mask, t * 1e3, t).to(torch.bfloat16).cuda()
    slab = bf16_bits(x[:1024].float().cpu().numpy())
    for fmt in ("fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8"):
        eb, mb, mn = oracle.FORMATS[fmt]
        for axis in (0, 1):
            y = be.quantize_mx(x, 8, eb, mb, mn, 32, axis)
            want = bf16_vals(oracle.quantize_mx(slab, fmt, axis=axis))
            assert oracle.same_values(y[:1024].float().cpu().numpy(), want), (fmt, axis)
            y2 = be.quantize_mx(y, 8, eb, mb, mn, 32, axis)
            assert torch.equal(y2.view(torch.int16), y.view(torch.int16)), ("idempotence", fmt, axis)
    # elementwise bfloat16 round-even of an fp32 copy is the bf16 tensor itself
    y = be.quantize_elemwise(x.float(), 9, 8, 3.3895313892515355e38, 2, False, True, out_dtype=torch.bfloat16)
    assert torch.equal(y.view(torch.int16), x.view(torch.int16))


@pytest.mark.parametrize("shape,axis", [((1024, 4096), 0), ((1024, 4096), 1), ((3, 700, 96), 1), ((5, 64, 33), 2),
                                        ((40000,), 0), ((4100, 1000), 0), ((8192, 4096), 0), ((6000, 4096), 1)])
def test_host_buffer_pipeline(be, shape, axis):
    """mxq_quantize_mx_host / mxq_quantize_elemwise_host (chunked, copies overlapped) == device entry points,
    also through quantize_mx_op on a pinned host tensor with custom_cuda."""
    from microxcaling_b200.mx_ops import quantize_mx_op
    from microxcaling_b200.specs import finalize_mx_specs
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(shape, generator=g) * 3).to(torch.bfloat16)
    hx = x.pin_memory()
    eb, mb, mn = oracle.FORMATS["fp6_e2m3"]
    want = be.quantize_mx(x.cuda(), 8, eb, mb, mn, 32, axis).cpu()
    got = be.quantize_mx_host(hx, 8, eb, mb, mn, 32, axis)
    assert not got.is_cuda and torch.equal(got.view(torch.int16), want.view(torch.int16))
    sp = finalize_mx_specs({"a_elem_format": "fp6_e2m3", "block_size": 32, "custom_cuda": True})
    got2 = quantize_mx_op(hx, sp, elem_format="fp6_e2m3", axes=[axis])
    assert not got2.is_cuda and torch.equal(got2.view(torch.int16), want.view(torch.int16))
    xf = x.float().pin_memory()
    e_want = be.quantize_elemwise(xf.cuda(), 5, 8, 2.0 ** 127 * 1.875, 2).cpu()
    e_got = be.quantize_elemwise_host(xf, 5, 8, 2.0 ** 127 * 1.875, 2)
    assert torch.equal(e_got, e_want)


def test_dither_with_caller_noise(be):
    """round='dither' = floor(|x| / quantum + noise) (mx/elemwise_ops.py:57-59, PyTorch-only in the
    reference, which draws the noise itself).  With the noise tensor supplied by the caller the GPU kernels
    (MX along both axes, fp32 / bf16 storage, and the elementwise kernel) must equal the torch formulation
    for CPU tensors and the library's host quantizer, value for value."""
    from microxcaling_b200.mx_ops import _quantize_mx
    from microxcaling_b200.elemwise_ops import _quantize_elemwise_core
    torch.manual_seed(11)
    x = torch.randn(96, 160) * torch.exp2(torch.randint(-6, 6, (96, 160)).float())
    n = torch.rand(96, 160)
    for dt in (torch.float32, torch.bfloat16):
        xd = x.to(dt)
        for fmt in ("fp8_e4m3", "fp6_e2m3", "fp4_e2m1", "int8"):
            for axis in (0, 1):
                want = _quantize_mx(xd, 8, fmt, axes=[axis], block_size=32, round="dither", noise=n)
                twin = _quantize_mx(xd, 8, fmt, axes=[axis], block_size=32, round="dither", noise=n, custom_cuda=True)
                got = _quantize_mx(xd.cuda(), 8, fmt, axes=[axis], block_size=32, round="dither", noise=n.cuda())
                assert oracle.same_values(to_np(got), to_np(want)), (dt, fmt, axis)
                assert oracle.same_values(to_np(twin), to_np(want)), (dt, fmt, axis, "host quantizer")
                # dither never moves a value by more than one quantum from its floor
                lo = _quantize_mx(xd, 8, fmt, axes=[axis], block_size=32, round="floor")
                assert bool((want.float().abs() >= lo.float().abs()).all())
        for bits, eb, mn in ((5, 8, 2.0 ** 127 * 1.75), (7, 5, 57344.0), (8, 0, 1.984375)):
            want = _quantize_elemwise_core(xd, bits, eb, mn, "dither", noise=n)
            got = _quantize_elemwise_core(xd.cuda(), bits, eb, mn, "dither", noise=n.cuda())
            assert oracle.same_values(to_np(got), to_np(want)), (dt, bits, eb)
    # two different noise tensors give different results; the same one is reproducible
    a = _quantize_mx(x.cuda(), 8, "fp4_e2m1", axes=[1], block_size=32, round="dither", noise=n.cuda())
    b = _quantize_mx(x.cuda(), 8, "fp4_e2m1", axes=[1], block_size=32, round="dither", noise=torch.rand(96, 160).cuda())
    assert not torch.equal(a, b)
    assert torch.equal(a, _quantize_mx(x.cuda(), 8, "fp4_e2m1", axes=[1], block_size=32, round="dither", noise=n.cuda()))
