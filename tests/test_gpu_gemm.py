"""GPU parity of the block-scaled MX GEMM (tcgen05 kind::mxf8f6f4), through the
C ABI, against the oracle's double-accumulated product of the dequantized
operands.

Tolerance (fp32 accumulation order only): before output rounding
    |c - ref| <= 2^-22 * sum_k |a_k * b_k|
(observed worst case on these inputs: 0.9 * 2^-24 of that sum); after bfloat16
output rounding the result may differ from round(ref) by at most one bf16 ulp,
and only where ref sits within the accumulation error of a rounding boundary."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
ROUNDS = {"nearest": 0, "floor": 1, "even": 2}


@pytest.fixture(scope="module")
def be():
    from microxcaling_b200 import _backend
    _backend.lib()
    return _backend


def quant_operand(be, X, fmt, rows_per_batch):
    eb, mb, mn = oracle.FORMATS[fmt]
    dq, codes, scales = be.quantize_mx(X, 8, eb, mb, mn, 32, X.dim() - 1, want_codes=True, gemm_layout=True,
                                       rows_per_batch=rows_per_batch)
    return dq, codes, scales, (1 if eb == 5 else 0)


def run_case(be, batch, M, N, K, fa, fb, tile_n=0, out_dtype=torch.float32, bf_bits=0, rnd="nearest", bias=False,
             seed=0):
    g = torch.Generator().manual_seed(seed)
    A = (torch.randn(batch * M, K, generator=g) * 2).to(torch.bfloat16).cuda()
    B = (torch.randn(batch * N, K, generator=g) * 0.5).to(torch.bfloat16).cuda()
    dqa, ca, sa, ka = quant_operand(be, A, fa, M)
    dqb, cb, sb, kb = quant_operand(be, B, fb, N)
    bias_t = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16).float().cuda() if bias else None
    C = be.gemm_mx(ca, sa, cb, sb, batch, M, N, K, ka, kb, out_dtype, bf_bits, ROUNDS[rnd], bias_t, tile_n)
    torch.cuda.synchronize()
    assert be.device_status() == 0
    ref, refabs = oracle.gemm_nt(dqa.float().cpu().numpy().reshape(batch, M, K),
                                 dqb.float().cpu().numpy().reshape(batch, N, K), want_abs=True)
    return C.float().cpu().numpy().astype(np.float64), ref, refabs, (bias_t.cpu().numpy() if bias else None)


@pytest.mark.parametrize("shape", [(1, 128, 128, 128), (1, 128, 128, 512), (1, 256, 384, 256), (3, 256, 128, 384),
                                   (1, 200, 136, 256), (1, 200, 100, 256), (2, 384, 512, 256), (1, 2304, 512, 256),
                                   (1, 1024, 1024, 4096)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_raw_accumulator(be, shape, tile_n):
    batch, M, N, K = shape
    got, ref, refabs, _ = run_case(be, batch, M, N, K, "fp8_e4m3", "fp8_e4m3", tile_n)
    assert np.all(np.abs(got - ref) <= 2.0 ** -22 * refabs + 1e-30)


@pytest.mark.parametrize("K", [32, 96, 160, 416, 1056])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_contraction_not_multiple_of_128(be, K, tile_n):
    """K only has to be whole 32-element blocks: the last, short K group is zero-filled by the tiled loads."""
    got, ref, refabs, _ = run_case(be, 1, 384, 256, K, "fp8_e4m3", "fp6_e3m2", tile_n, seed=K)
    assert np.all(np.abs(got - ref) <= 2.0 ** -22 * refabs + 1e-30)
    got, ref, refabs, _ = run_case(be, 2, 200, 136, K, "fp8_e5m2", "fp4_e2m1", 0, seed=K + 1)
    assert np.all(np.abs(got - ref) <= 2.0 ** -22 * refabs + 1e-30)


@pytest.mark.parametrize("fa,fb", [("fp8_e4m3", "fp8_e5m2"), ("fp8_e5m2", "fp8_e5m2"), ("fp8_e4m3", "fp4_e2m1"),
                                   ("fp6_e3m2", "fp6_e3m2"), ("fp6_e2m3", "fp4_e2m1"), ("fp4_e2m1", "fp4_e2m1")])
def test_gemm_format_pairs(be, fa, fb):
    got, ref, refabs, _ = run_case(be, 2, 256, 256, 512, fa, fb)
    assert np.all(np.abs(got - ref) <= 2.0 ** -22 * refabs + 1e-30)


def _bf_round(x, bits, mode):
    import oracle as o
    mn = 2.0 ** 127 * (2 ** (bits - 8) - 1) / 2 ** (bits - 9)
    return o.quantize_elemwise(x.astype(np.float32), bits - 7, 8, mn, mode).astype(np.float64)


@pytest.mark.parametrize("rnd", ["nearest", "floor", "even"])
@pytest.mark.parametrize("out_dtype,bits", [(torch.bfloat16, 16), (torch.float32, 16), (torch.float32, 12),
                                            (torch.bfloat16, 0)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_output_rounding(be, rnd, out_dtype, bits, bias):
    got, ref, refabs, b = run_case(be, 1, 256, 384, 512, "fp8_e4m3", "fp8_e4m3", 0, out_dtype, bits, rnd, bias, seed=3)
    tol = 2.0 ** -22 * refabs
    eff_bits = bits if bits else (16 if out_dtype == torch.bfloat16 else 0)
    mode = rnd if bits else "even"          # no bfloat rounding requested: only the bf16 storage cast (RNE)
    if eff_bits:
        bb = b[None, None, :] if b is not None else None

        def model(x):
            if bits == 0:                   # only the storage cast, applied once after the bias add
                return _bf_round(x + bb if bb is not None else x, eff_bits, mode)
            y = _bf_round(x, eff_bits, mode)
            return _bf_round(y + bb, eff_bits, mode) if bb is not None else y
        lo, hi, mid = model(ref - tol), model(ref + tol), model(ref)
        assert np.all((got >= np.minimum(lo, hi)) & (got <= np.maximum(lo, hi)))
        # and almost everywhere it is exactly the rounding of the reference value
        assert np.mean(got == mid) > 0.995
    else:
        assert np.all(np.abs(got - ref - (b[None, None, :] if b is not None else 0)) <= tol + 1e-6)


def test_gemm_nan_block_and_zero_rows(be):
    A = torch.randn(128, 256).to(torch.bfloat16)
    A[5, 40] = float("nan")
    A[7] = 0
    B = torch.randn(128, 256).to(torch.bfloat16)
    dqa, ca, sa, _ = quant_operand(be, A.cuda(), "fp8_e4m3", 128)
    dqb, cb, sb, _ = quant_operand(be, B.cuda(), "fp8_e4m3", 128)
    C = be.gemm_mx(ca, sa, cb, sb, 1, 128, 128, 256, 0, 0, torch.float32, 0, 0, None, 0)[0].cpu().numpy()
    assert np.isnan(C[5]).all() and not np.isnan(np.delete(C, 5, axis=0)).any()
    assert (C[7] == 0).all()


def test_gemm_rejects_bad_arguments(be):
    z = torch.zeros(128 * 128, dtype=torch.uint8, device="cuda")
    with pytest.raises(be.MxqError):
        be.gemm_mx(z, z, z, z, 1, 128, 128, 80)           # K not a multiple of 32
    with pytest.raises(be.MxqError):
        be.gemm_mx(z, z, z, z, 1, 128, 128, 128, a_fmt=3)


def test_gemm_transposed_operand_layout(be):
    """The backward GEMMs contract over the row axis of their inputs: quantize
    along axis -2 with transposed codes and multiply.  grad_w = g^T x."""
    gen = torch.Generator().manual_seed(5)
    Mtok, N, K = 512, 256, 384
    G = torch.randn(Mtok, N, generator=gen).to(torch.bfloat16).cuda()
    X = torch.randn(Mtok, K, generator=gen).to(torch.bfloat16).cuda()
    eb, mb, mn = oracle.FORMATS["fp8_e5m2"]
    dqg, cg, sg = be.quantize_mx(G, 8, eb, mb, mn, 32, 0, want_codes=True, transposed=True, gemm_layout=True)
    dqx, cx, sx = be.quantize_mx(X, 8, eb, mb, mn, 32, 0, want_codes=True, transposed=True, gemm_layout=True)
    assert cg.shape == (N, Mtok) and cx.shape == (K, Mtok)
    C = be.gemm_mx(cg, sg, cx, sx, 1, N, K, Mtok, 1, 1, torch.float32, 0, 0, None, 0)[0].cpu().numpy().astype(np.float64)
    ref, refabs = oracle.gemm_nt(dqg.float().cpu().numpy().T.copy(), dqx.float().cpu().numpy().T.copy(), want_abs=True)
    assert np.all(np.abs(C - ref[0]) <= 2.0 ** -22 * refabs[0] + 1e-30)


def test_linear_fwd_composite_equals_two_calls(be):
    """mxq_linear_fwd (quantize into a workspace + GEMM) == mxq_quantize_mx followed by mxq_gemm_mx."""
    gen = torch.Generator().manual_seed(9)
    for (M, K, N) in ((256, 512, 384), (200, 256, 136)):
        x = torch.randn(M, K, generator=gen).to(torch.bfloat16).cuda()
        w = (torch.randn(N, K, generator=gen) * 0.1).to(torch.bfloat16).cuda()
        bias = torch.randn(N, generator=gen).to(torch.bfloat16).float().cuda()
        ea, ma, na = oracle.FORMATS["fp8_e4m3"]
        ew, mw, nw = oracle.FORMATS["fp4_e2m1"]
        _, wc, ws = be.quantize_mx(w, 8, ew, mw, nw, 32, 1, want_dq=False, want_codes=True, gemm_layout=True)
        _, xc, xs = be.quantize_mx(x, 8, ea, ma, na, 32, 1, want_dq=False, want_codes=True, gemm_layout=True)
        want = be.gemm_mx(xc, xs, wc, ws, 1, M, N, K, 0, 0, torch.bfloat16, 16, 0, bias)[0]
        got, wsp = be.linear_fwd(x, wc, ws, 0, ea, ma, na, bias=bias)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        assert int(wsp[:4].view(torch.int32).item()) == 0


@pytest.mark.parametrize("n_dests,rows_per_dest,M", [(2, 256, 512), (4, 128, 512), (3, 256, 700), (1, 384, 384)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_scatter_equals_plain_gemm(be, n_dests, rows_per_dest, M, tile_n):
    """The scattering GEMM stores rows [d*R, (d+1)*R) into destination d: same values, bit for bit, as the
    plain GEMM (here all destinations are buffers on the same GPU); rows past M are left untouched."""
    N, K = 384, 256
    g = torch.Generator().manual_seed(11)
    A = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16).cuda()
    B = (torch.randn(N, K, generator=g) * 0.5).to(torch.bfloat16).cuda()
    _, ca, sa, ka = quant_operand(be, A, "fp8_e4m3", M)
    _, cb, sb, kb = quant_operand(be, B, "fp4_e2m1", N)
    want = be.gemm_mx(ca, sa, cb, sb, 1, M, N, K, ka, kb, torch.float32, 0, -1, None, tile_n)[0]
    dests = [torch.full((rows_per_dest, N), -7.0, dtype=torch.float32, device="cuda") for _ in range(n_dests)]
    be.gemm_mx_scatter(ca, sa, cb, sb, [d.data_ptr() for d in dests], rows_per_dest, M, N, K, ka, kb, tile_n=tile_n)
    torch.cuda.synchronize()
    assert be.device_status() == 0
    got = torch.cat(dests, 0)
    assert torch.equal(got[:M], want)
    assert bool((got[M:] == -7.0).all())


def test_gemm_scatter_rejects_bad_arguments(be):
    u8 = torch.zeros(128 * 128, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(512, dtype=torch.uint8, device="cuda")
    d = torch.zeros(128, 128, dtype=torch.float32, device="cuda")
    with pytest.raises(be.MxqError):          # rows per destination not a multiple of 128
        be.gemm_mx_scatter(u8, sf, u8, sf, [d.data_ptr()], 100, 128, 128, 128)
    with pytest.raises(be.MxqError):          # more rows than the destinations hold
        be.gemm_mx_scatter(u8, sf, u8, sf, [d.data_ptr()], 128, 256, 128, 128)
    with pytest.raises(be.MxqError):          # too many destinations
        be.gemm_mx_scatter(u8, sf, u8, sf, [d.data_ptr()] * 9, 128, 128, 128, 128)


def test_sum_slabs_adds_in_order(be):
    torch.manual_seed(2)
    s = (torch.randn(5, 300, 64, device="cuda") * torch.tensor([1e8, 1.0, -1e8, 3.0, 1e-3], device="cuda").view(5, 1, 1))
    want = s[0]
    for k in range(1, 5):
        want = want + s[k]
    assert torch.equal(be.sum_slabs(s.contiguous()), want)


def _sampled_gemm_check(be, M, N, K, fa, fb, n_rows=24, n_cols=512, seed=0):
    """Full-size GEMM (whatever tile engine the library picks for it) checked on a random sample of output
    rows x columns against the double-accumulated product of the dequantized operands."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = (torch.randn(M, K, generator=g, device="cuda") * 1.5).to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, device="cuda") * K ** -0.5).to(torch.bfloat16)
    dqa, ca, sa, ka = quant_operand(be, A, fa, M)
    dqb, cb, sb, kb = quant_operand(be, B, fb, N)
    C = be.gemm_mx(ca, sa, cb, sb, 1, M, N, K, ka, kb, torch.float32, 0, -1)[0]
    torch.cuda.synchronize()
    assert be.device_status() == 0
    rs = np.random.default_rng(seed)
    rows = np.sort(rs.choice(M, n_rows, replace=False))
    cols = np.sort(rs.choice(N, n_cols, replace=False))
    a = dqa[torch.as_tensor(rows, device="cuda")].float().cpu().numpy()[None]
    b = dqb[torch.as_tensor(cols, device="cuda")].float().cpu().numpy()[None]
    ref, refabs = oracle.gemm_nt(a, b, want_abs=True)
    got = C[torch.as_tensor(rows, device="cuda")][:, torch.as_tensor(cols, device="cuda")].cpu().numpy().astype(np.float64)
    assert np.all(np.abs(got - ref[0]) <= 2.0 ** -22 * refabs[0] + 1e-30)


def test_config3_gemm_full_size_sampled(be):
    """Config 3: 8192 tokens x 4096 -> 4096, MXFP8 operands (forward product)."""
    _sampled_gemm_check(be, 8192, 4096, 4096, "fp8_e4m3", "fp8_e4m3")


def test_config5_gemm_full_size_sampled(be):
    """Config 5 gate/up projection: 16384 tokens x 8192 -> 28672, fp8_e4m3 activations x fp4_e2m1 weights."""
    _sampled_gemm_check(be, 16384, 28672, 8192, "fp8_e4m3", "fp4_e2m1", n_rows=16, n_cols=384, seed=1)


def test_gemm_sm_budget_leaves_results_unchanged(be):
    """A smaller SM budget only changes how many persistent CTAs walk the tiles: the output bits stay, for the
    CTA-pair engine (4096 x 4096 x 2048) and the single-CTA one (512 x 384 x 256); the setter hands back
    the previous value and the block form restores it."""
    for M, N, K in ((4096, 4096, 2048), (512, 384, 256)):
        g = torch.Generator().manual_seed(M)
        A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        B = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
        _, ca, sa, ka = quant_operand(be, A, "fp8_e4m3", M)
        _, cb, sb, kb = quant_operand(be, B, "fp8_e4m3", N)
        run = lambda: be.gemm_mx(ca, sa, cb, sb, 1, M, N, K, ka, kb, torch.bfloat16, 16, 0, None, 0)
        full = run()
        assert be.lib().mxq_gemm_sm_budget(-1) == 0
        for sms in (116, 7, 1):
            with be.gemm_sm_budget(sms):
                assert be.lib().mxq_gemm_sm_budget(-1) == sms
                part = run()
            assert be.lib().mxq_gemm_sm_budget(-1) == 0
            assert torch.equal(full, part), (M, N, K, sms)
    torch.cuda.synchronize()
    assert be.device_status() == 0


@pytest.mark.parametrize("batch,M,K,N", [(1, 256, 128, 256), (3, 200, 96, 136), (2, 384, 256, 64), (4, 128, 2048, 128)])
@pytest.mark.parametrize("a_trans,b_trans", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_fwd_equals_the_three_calls(be, batch, M, K, N, a_trans, b_trans):
    """mxq_matmul_fwd (both packings and the GEMM chained inside the library) gives the bits of
    mxq_quantize_mx x 2 + mxq_gemm_mx, for every operand layout, ragged row counts, and with the left
    operand handed over already packed."""
    from microxcaling_b200._mxgemm import _cfmt
    from microxcaling_b200.formats import ElemFormat
    g = torch.Generator().manual_seed(batch * 1000 + M + N)
    a = (torch.randn((batch, K, M) if a_trans else (batch, M, K), generator=g) * 2).to(torch.bfloat16).cuda()
    b = torch.randn((batch, N, K) if b_trans else (batch, K, N), generator=g).to(torch.bfloat16).cuda()
    fa, fb = ElemFormat.fp6_e3m2, ElemFormat.fp8_e5m2
    ea, ma, na = oracle.FORMATS["fp6_e3m2"]
    eb, mb, nb = oracle.FORMATS["fp8_e5m2"]
    if a_trans:
        _, ca, sa = be.quantize_mx(a, 8, ea, ma, na, 32, 1, want_dq=False, want_codes=True, transposed=True, gemm_layout=True)
    else:
        _, ca, sa = be.quantize_mx(a.reshape(-1, K), 8, ea, ma, na, 32, 1, want_dq=False, want_codes=True,
                                   gemm_layout=True, rows_per_batch=M)
    if b_trans:
        _, cb, sb = be.quantize_mx(b.reshape(-1, K), 8, eb, mb, nb, 32, 1, False, 2, want_dq=False, want_codes=True,
                                   gemm_layout=True, rows_per_batch=N)
    else:
        _, cb, sb = be.quantize_mx(b, 8, eb, mb, nb, 32, 1, False, 2, want_dq=False, want_codes=True, transposed=True,
                                   gemm_layout=True)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16).float().cuda()
    want = be.gemm_mx(ca, sa, cb, sb, batch, M, N, K, 0, 1, torch.bfloat16, 16, 0, bias, 0)
    got = be.matmul_fwd(a, b, batch, M, K, N, a_trans, b_trans, _cfmt(fa, "nearest"), _cfmt(fb, "even"), 8, False,
                        torch.bfloat16, 16, 0, bias=bias)
    assert torch.equal(got, want)
    got2 = be.matmul_fwd(None, b, batch, M, K, N, False, b_trans, _cfmt(fa, "nearest"), _cfmt(fb, "even"), 8, False,
                         torch.bfloat16, 16, 0, bias=bias, a_packed=(ca, sa))
    assert torch.equal(got2, want)
    torch.cuda.synchronize()
    assert be.device_status() == 0
