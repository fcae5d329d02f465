"""GPU parity of the fused bfloat16 vector chains (mxq_silu_bf16,
mxq_rmsnorm_bf16) against the same layers composed from single vector
operations, i.e. the way the reference runs them (one torch kernel per
operation, every result rounded to bfloat16), on the same device.

SiLU is a pure elementwise chain: every output must be equal.  RMSNorm contains
one row sum whose fp32 accumulation order is unspecified in the composed path
(a library reduction); when the fp32 sums differ in their last bits the
bfloat16 mean can land on the neighbouring value, which moves a whole row by at
most one bfloat16 ulp per later rounding step.  The test therefore demands that
almost all rows are identical and that the rest stay within two ulps."""
import numpy as np
import pytest
import torch

import microxcaling_b200 as mx
from microxcaling_b200 import vector_ops
from microxcaling_b200.specs import finalize_mx_specs

pytestmark = pytest.mark.gpu

SP = finalize_mx_specs({"bfloat": 16})


def composed(monkeypatch, fn):
    """Run fn with the fused kernels switched off."""
    with monkeypatch.context() as m:
        import importlib
        for name in ("activations", "layernorm", "softmax", "tp"):
            mod = importlib.import_module("microxcaling_b200." + name)
            m.setattr(mod, "fused_bf16_ok", lambda *a, **k: False)
        return fn()


def same(a, b):
    a, b = a.float(), b.float()
    return bool(((a == b) | (a.isnan() & b.isnan())).all())


def all_bf16_patterns():
    bits = torch.arange(1 << 16, dtype=torch.int32)
    return (bits << 16).view(torch.float32).to(torch.bfloat16).cuda()


def test_fused_path_is_taken(monkeypatch):
    from microxcaling_b200 import _backend
    calls = []
    real = _backend.silu_bf16
    monkeypatch.setattr(_backend, "silu_bf16", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    mx.silu(torch.randn(64, 64, device="cuda", dtype=torch.bfloat16), mx_specs=SP)
    assert calls


@pytest.mark.parametrize("n", [1 << 16, 8191, 5])
def test_silu_every_pattern(monkeypatch, n):
    x = all_bf16_patterns()[:n].clone()
    got = mx.silu(x, mx_specs=SP)
    want = composed(monkeypatch, lambda: mx.silu(x, mx_specs=SP))
    assert same(got, want)


def test_silu_large_tensor_uses_the_table_and_matches(monkeypatch):
    """>= 4 Mi elements take the table-driven kernel: same bits as the composed chain, every pattern included."""
    torch.manual_seed(9)
    x = torch.cat([all_bf16_patterns(), (torch.randn((1 << 22) + 4096, device="cuda") * 3).to(torch.bfloat16)])
    x = x[: (x.numel() // 8) * 8].contiguous()
    up = (torch.randn(x.numel(), device="cuda") * 2).to(torch.bfloat16)
    from microxcaling_b200 import _backend
    got, sig = _backend.silu_bf16(x, None, want_sig=True)
    want = composed(monkeypatch, lambda: mx.silu(x, mx_specs=SP))
    assert same(got, want)
    got2 = _backend.silu_bf16(x, up)
    want2 = composed(monkeypatch, lambda: mx.simd_mul(mx.silu(x, mx_specs=SP), up, mx_specs=SP))
    assert same(got2, want2)
    small_sig = _backend.silu_bf16(x[:4096].contiguous(), None, want_sig=True)[1]
    assert same(sig[:4096], small_sig)


def test_silu_backward_uses_saved_sigmoid(monkeypatch):
    torch.manual_seed(0)
    x = (torch.randn(300, 257, device="cuda") * 4).to(torch.bfloat16)
    g = torch.randn(300, 257, device="cuda").to(torch.bfloat16)
    xa = x.clone().requires_grad_()
    mx.silu(xa, mx_specs=SP).backward(g)
    xb = x.clone().requires_grad_()
    composed(monkeypatch, lambda: mx.silu(xb, mx_specs=SP).backward(g))
    assert same(xa.grad, xb.grad)


def test_silu_times_up(monkeypatch):
    from microxcaling_b200 import _backend
    torch.manual_seed(1)
    gate = all_bf16_patterns().reshape(256, 256)
    up = (torch.randn(256, 256, device="cuda") * 3).to(torch.bfloat16)
    got = _backend.silu_bf16(gate, up)
    want = composed(monkeypatch, lambda: mx.simd_mul(mx.silu(gate, mx_specs=SP), up, mx_specs=SP))
    assert same(got, want)


@pytest.mark.parametrize("rows,hidden", [(64, 8192), (37, 96), (5, 1000), (3, 33), (1, 8), (200, 4096)])
def test_rmsnorm(monkeypatch, rows, hidden):
    torch.manual_seed(rows * 7 + hidden)
    x = (torch.randn(rows, hidden, device="cuda") * 2.5).to(torch.bfloat16)
    norm = mx.RMSNorm(hidden, eps=1e-5, mx_specs=SP).cuda().to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(torch.randn(hidden) * 0.5 + 1)
        norm.bias.copy_(torch.randn(hidden) * 0.1)
    got = norm(x).float()
    want = composed(monkeypatch, lambda: norm(x)).float()
    row_equal = (got == want).all(dim=1)
    assert float(row_equal.float().mean()) >= 0.98, float(row_equal.float().mean())
    ulp = want.abs().clamp_min(1e-30) * 2.0 ** -7
    assert bool(((got - want).abs() <= 2 * ulp).all())


@pytest.mark.parametrize("shape", [(4, 64, 2048), (300, 8), (33, 1000), (7, 3, 136)])
@pytest.mark.parametrize("exp2", [False, True])
def test_softmax(monkeypatch, shape, exp2):
    """One row sum of unspecified order, as in RMSNorm: almost all rows identical, the rest within 2 ulp."""
    sp = finalize_mx_specs({"bfloat": 16, "softmax_exp2": exp2})
    torch.manual_seed(sum(shape))
    x = (torch.randn(*shape, device="cuda") * 3).to(torch.bfloat16)
    x.view(-1, shape[-1])[0, :3] = float("-inf")
    got = mx.softmax(x, dim=-1, mx_specs=sp).float().view(-1, shape[-1])
    want = composed(monkeypatch, lambda: mx.softmax(x, dim=-1, mx_specs=sp)).float().view(-1, shape[-1])
    row_equal = (got == want).all(dim=1)
    assert float(row_equal.float().mean()) >= 0.95, float(row_equal.float().mean())
    ulp = want.abs().clamp_min(1e-30) * 2.0 ** -7
    assert bool(((got - want).abs() <= 2 * ulp).all())


def test_softmax_large_input_uses_the_table_and_matches(monkeypatch):
    """>= 4 Mi elements: exp from the table and e * (1/s) instead of e / s; same rows as the composed chain."""
    torch.manual_seed(21)
    x = (torch.randn(4096, 1024, device="cuda") * 4).to(torch.bfloat16)
    x[5, :100] = -120.0                                   # exp underflows into the subnormals and to zero
    x[6, 0] = 80.0
    got = mx.softmax(x, dim=-1, mx_specs=SP).float()
    want = composed(monkeypatch, lambda: mx.softmax(x, dim=-1, mx_specs=SP)).float()
    row_equal = (got == want).all(dim=1)
    assert float(row_equal.float().mean()) >= 0.95, float(row_equal.float().mean())
    ulp = want.abs().clamp_min(1e-38) * 2.0 ** -7
    assert bool(((got - want).abs() <= 2 * ulp + 1e-38).all())


def test_reciprocal_multiply_rounds_like_division_for_bf16_operands():
    """The identity the softmax kernel relies on: for bfloat16 e in (0, 1] and s in [1, 2048],
    bf16(e * fl(1/s)) == bf16(e / s) whenever the quotient is a normal bfloat16 number."""
    e = all_bf16_patterns()
    e = e[(e > 0) & (e <= 1) & (e.float() >= 1e-30)].float()
    s = all_bf16_patterns()
    s = s[(s >= 1) & (s <= 2048)].float()
    for chunk in s.split(64):
        q_div = (e[:, None] / chunk[None, :]).to(torch.bfloat16)
        q_mul = (e[:, None] * (1.0 / chunk)[None, :]).to(torch.bfloat16)
        assert torch.equal(q_div, q_mul)


def test_softmax_nan_row_and_wide_rows_fall_back(monkeypatch):
    x = torch.randn(4, 64, device="cuda").to(torch.bfloat16)
    x[1, 5] = float("nan")
    got = mx.softmax(x, dim=-1, mx_specs=SP).float()
    want = composed(monkeypatch, lambda: mx.softmax(x, dim=-1, mx_specs=SP)).float()
    assert bool(got[1].isnan().all()) and bool(want[1].isnan().all())
    assert same(got[[0, 2, 3]], want[[0, 2, 3]]) or bool(((got - want)[[0, 2, 3]].abs() <= want[[0, 2, 3]].abs() * 2.0 ** -6).all())
    wide = torch.randn(2, 4096, device="cuda").to(torch.bfloat16)          # longer than the fused kernel takes
    assert same(mx.softmax(wide, dim=-1, mx_specs=SP), composed(monkeypatch, lambda: mx.softmax(wide, dim=-1, mx_specs=SP)))
    other = torch.randn(16, 8, 24, device="cuda").to(torch.bfloat16)       # not the last dimension
    assert same(mx.softmax(other, dim=1, mx_specs=SP), composed(monkeypatch, lambda: mx.softmax(other, dim=1, mx_specs=SP)))


def test_rmsnorm_backward_matches_composed(monkeypatch):
    torch.manual_seed(5)
    x = torch.randn(48, 512, device="cuda").to(torch.bfloat16)
    g = torch.randn(48, 512, device="cuda").to(torch.bfloat16)
    norm = mx.RMSNorm(512, eps=1e-5, mx_specs=SP).cuda().to(torch.bfloat16)

    def run():
        xa = x.clone().requires_grad_()
        norm.zero_grad()
        norm(xa).backward(g)
        return xa.grad.float(), norm.weight.grad.float()
    gx, gw = run()
    cx, cw = composed(monkeypatch, run)
    # identical saved x_norm / rms_inv on (almost) every row -> identical gradients there
    assert float((gx == cx).all(dim=1).float().mean()) >= 0.95
    assert torch.allclose(gw, cw, rtol=2 ** -6, atol=1e-3)


def test_ffn_block_fused_equals_composed(monkeypatch):
    from microxcaling_b200.tp import TensorParallelFFN
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32,
                            "bfloat": 16})
    torch.manual_seed(3)
    ffn = TensorParallelFFN(256, 512, sp, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        for w in (ffn.w_gate, ffn.w_up, ffn.w_down):
            w.copy_(torch.randn(w.shape, device="cuda") * w.shape[1] ** -0.5)
    x = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    got = ffn(x).float()
    want = composed(monkeypatch, lambda: ffn(x)).float()
    row_equal = (got == want).all(dim=1)
    assert float(row_equal.float().mean()) >= 0.95


@pytest.mark.parametrize("fmt", ["fp8_e4m3", "fp8_e5m2", "fp6_e3m2", "fp4_e2m1"])
@pytest.mark.parametrize("rnd", [0, 1, 2])
@pytest.mark.parametrize("gemm_layout", [False, True])
def test_swiglu_quantize_equals_two_steps(fmt, rnd, gemm_layout):
    """SiLU x up fused into the MX packing == mxq_silu_bf16 followed by mxq_quantize_mx, byte for byte;
    the input walks every bf16 pattern (NaN / Inf / huge / tiny blocks take the slow path)."""
    import oracle
    from microxcaling_b200 import _backend as be
    eb, mb, mn = oracle.FORMATS[fmt]
    torch.manual_seed(4)
    gate = all_bf16_patterns().reshape(256, 256)
    up = (torch.randn(256, 256, device="cuda") * 3).to(torch.bfloat16)
    up[7, :40] = 0
    gate2 = torch.cat([gate, (torch.randn(128, 256, device="cuda") * 2).to(torch.bfloat16)])
    up2 = torch.cat([up, (torch.randn(128, 256, device="cuda")).to(torch.bfloat16)])
    act = be.silu_bf16(gate2, up2)
    _, c_want, s_want = be.quantize_mx(act, 8, eb, mb, mn, 32, 1, False, rnd, want_dq=False, want_codes=True,
                                       gemm_layout=gemm_layout, rows_per_batch=gate2.shape[0] if gemm_layout else 0)
    c_got, s_got = be.swiglu_quantize_mx(gate2, up2, 8, eb, mb, mn, False, rnd, gemm_layout=gemm_layout)
    assert torch.equal(c_got, c_want)
    assert torch.equal(s_got.view(-1), s_want.view(-1))


@pytest.mark.parametrize("fmt", ["fp6_e3m2", "fp8_e4m3", "fp8_e5m2", "fp4_e2m1"])
@pytest.mark.parametrize("rnd", [0, 1, 2])
def test_softmax_quantize_equals_two_steps(fmt, rnd):
    """mxq_softmax_quantize_mx = mxq_softmax_bf16 followed by mxq_quantize_mx (codes + scales in the GEMM
    layout): probabilities, code bytes and scale bytes all equal, for rows with ordinary logits, with a
    dominant logit (probabilities spanning the whole bfloat16 range, zeros included), -inf entries and a
    NaN row; with and without the probabilities being written."""
    import oracle
    from microxcaling_b200 import _backend as be
    eb, mb, mn = oracle.FORMATS[fmt]
    torch.manual_seed(1)
    x = torch.randn(3, 160, 2048, device="cuda") * 1.5
    x[0, 1, ::7] += 40.0
    x[0, 2, 5] = 90.0
    x[1, 3, 100:400] = float("-inf")
    x[2, 4, 17] = float("nan")
    x[2, 5, :] = -1e30
    x = x.to(torch.bfloat16)
    for cols in (2048, 96):
        xs = x[..., :cols].contiguous()
        p, codes, scales = be.softmax_quantize_mx(xs, 8, eb, mb, mn, False, rnd, rows_per_batch=xs.shape[-2])
        p2 = be.softmax_bf16(xs)
        _, c2, s2 = be.quantize_mx(p2.reshape(-1, cols), 8, eb, mb, mn, 32, 1, False, rnd, want_dq=False,
                                   want_codes=True, gemm_layout=True, rows_per_batch=xs.shape[-2])
        assert same(p, p2), (fmt, rnd, cols)
        assert torch.equal(codes.reshape(-1, cols), c2), (fmt, rnd, cols)
        assert torch.equal(scales, s2), (fmt, rnd, cols)
        none, c3, s3 = be.softmax_quantize_mx(xs, 8, eb, mb, mn, False, rnd, rows_per_batch=xs.shape[-2], want_probs=False)
        assert none is None and torch.equal(c3, codes) and torch.equal(s3, scales)


def test_softmax_hands_its_packing_to_the_next_product():
    """mx.softmax on batched score matrices writes the MX packing of the probabilities in the same pass and
    mx.bmm picks it up: only the right operand is quantized by the product, the result equals the unfused
    sequence, and a changed probability tensor is packed again."""
    from microxcaling_b200 import _backend
    sp = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "block_size": 32, "scale_bits": 8, "bfloat": 16,
                            "custom_cuda": True})
    torch.manual_seed(0)
    s = (torch.randn(8, 512, 1024, device="cuda") * 2).to(torch.bfloat16)
    v = torch.randn(8, 1024, 64, device="cuda").to(torch.bfloat16)
    packs = lambda: _backend.launch_count(1)                     # MX quantizations launched inside the library
    with torch.no_grad():
        p = mx.softmax(s, dim=-1, mx_specs=sp)
        assert getattr(p, "_mx_packed", None) is not None
        n0 = packs()
        o = mx.bmm(p, v, mx_specs=sp)
        assert packs() - n0 == 1                                 # V only
        p_plain = _backend.softmax_bf16(s)
        assert same(p, p_plain)
        n0 = packs()
        o_plain = mx.bmm(p_plain, v, mx_specs=sp)
        assert packs() - n0 == 2
        assert torch.equal(o, o_plain)
        p.mul_(0.5)                                              # the note no longer describes the tensor
        n0 = packs()
        o_half = mx.bmm(p, v, mx_specs=sp)
        assert packs() - n0 == 2
        assert torch.equal(o_half, mx.bmm(p_plain * 0.5, v, mx_specs=sp))
    # with autograd the backward pass still sees the probabilities
    s2 = s.clone().requires_grad_()
    p2 = mx.softmax(s2, dim=-1, mx_specs=sp)
    mx.bmm(p2, v, mx_specs=sp).sum().backward()
    assert s2.grad is not None and torch.isfinite(s2.grad.float()).all()
