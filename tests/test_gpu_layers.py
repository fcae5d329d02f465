"""GPU tests of the layer API: mx.linear / matmul / bmm forward and backward on
CUDA tensors (packed operands + tcgen05 block-scaled GEMM with fused output
rounding) against outputs recorded from the reference on the same seeded
inputs (fp32 containers of bf16 values).

Tolerance.  The GEMM accumulates in fp32 in a different order than the
reference's library GEMM, and the result is then rounded to bfloat16, so an
output can land on the neighbouring bf16 value when the exact sum sits within
accumulation error of a rounding boundary: at most one bf16 ulp (2^-8 relative
for the half-away mode... 2^-7 of the value), on a small fraction of elements;
everything else must be equal."""
import numpy as np
import pytest
import torch

import microxcaling_b200 as mx
from microxcaling_b200.specs import finalize_mx_specs

pytestmark = pytest.mark.gpu


def close_bf16(got, ref, name, min_exact=0.97):
    a = got.detach().float().cpu().numpy().astype(np.float64)
    b = ref.astype(np.float64)
    assert a.shape == b.shape, name
    ulp = np.maximum(np.abs(b), 1e-30) * 2.0 ** -7
    ok = np.abs(a - b) <= ulp
    worst = np.unravel_index(np.argmax(np.abs(a - b) / ulp), a.shape)
    assert ok.all(), (name, np.abs(a - b).max(), int((~ok).sum()), "worst at", worst, float(a[worst]), float(b[worst]))
    exact = float((a == b).mean())
    assert exact >= min_exact, (name, exact)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_match_reference(golden_layers, dtype):
    meta, z = golden_layers
    dev = "cuda"
    for m in meta:
        if m["op"] == "vec":
            continue
        sp = finalize_mx_specs(dict(m["specs"], custom_cuda=True))
        t = m["tag"]
        go = torch.tensor(z[t + "_go"]).to(dev, dtype)
        if m["op"] == "linear":
            x = torch.tensor(z[t + "_x"]).to(dev, dtype).requires_grad_()
            w = torch.tensor(z[t + "_w"]).to(dev, dtype).requires_grad_()
            b = torch.tensor(z[t + "_b"]).to(dev, dtype).requires_grad_() if m["bias"] else None
            y = mx.linear(x, w, b, mx_specs=sp)
            if sp["round"] != "even":      # bfloat16 + 'even' casts to torch.bfloat16, as the reference does
                assert y.dtype == dtype, t
            y.backward(go)
            close_bf16(y, z[t + "_y"], t + ".y")
            close_bf16(x.grad, z[t + "_gx"], t + ".gx")
            close_bf16(w.grad, z[t + "_gw"], t + ".gw")
            if m["bias"]:
                close_bf16(b.grad, z[t + "_gb"], t + ".gb", min_exact=0.9)
        else:
            a = torch.tensor(z[t + "_a"]).to(dev, dtype).requires_grad_()
            b = torch.tensor(z[t + "_b"]).to(dev, dtype).requires_grad_()
            y = (mx.bmm if m["op"] == "bmm" else mx.matmul)(a, b, mx_specs=sp)
            y.backward(go)
            close_bf16(y, z[t + "_y"], t + ".y")
            close_bf16(a.grad, z[t + "_ga"], t + ".ga")
            close_bf16(b.grad, z[t + "_gb"], t + ".gb")


def test_fast_path_is_taken(monkeypatch):
    """FP8/FP6/FP4 formats with block 32 and K % 128 == 0 must reach the tensor-core GEMM."""
    from microxcaling_b200 import _backend
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32,
                            "bfloat": 16, "custom_cuda": True})
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    lin = mx.Linear(512, 384, bias=True, mx_specs=sp).cuda().to(torch.bfloat16)
    g0, q0 = _backend.launch_count(0), _backend.launch_count(1)
    y = lin(x)
    y.backward(torch.randn_like(y))
    assert _backend.launch_count(0) - g0 == 3   # forward, grad_weight, grad_input on the tensor cores
    assert _backend.launch_count(1) - q0 == 6   # two MX packings per product
    assert _backend.device_status() == 0


def test_vector_layers_on_gpu(golden_layers):
    """softmax / SiLU / RMSNorm / simd_mul on CUDA: same chains of torch op + bfloat
    rounding kernel; exp, reciprocal and sqrt differ between the CPU and CUDA
    math libraries by an ulp of fp32, which after bfloat16 rounding shows up as
    at most one bf16 ulp on a small fraction of elements."""
    meta, z = golden_layers
    for m in meta:
        if m["op"] != "vec":
            continue
        sp = finalize_mx_specs(dict(m["specs"], custom_cuda=True))
        t = m["tag"]
        go = torch.tensor(z[t + "_sm_go"]).cuda()
        x = torch.tensor(z[t + "_sm_x"]).cuda().requires_grad_()
        y = mx.softmax(x, dim=-1, mx_specs=sp)
        y.backward(go)
        close_bf16(y, z[t + "_sm_y"], t + ".softmax", 0.9)
        x = torch.tensor(z[t + "_silu_x"]).cuda().requires_grad_()
        y = mx.silu(x, mx_specs=sp)
        y.backward(go)
        close_bf16(y, z[t + "_silu_y"], t + ".silu", 0.9)
        x = torch.tensor(z[t + "_rms_x"]).cuda().requires_grad_()
        norm = mx.RMSNorm(96, eps=1e-5, mx_specs=sp).cuda()
        with torch.no_grad():
            norm.weight.copy_(torch.tensor(z[t + "_rms_w"]))
            norm.bias.copy_(torch.tensor(z[t + "_rms_b"]))
        y = norm(x)
        close_bf16(y, z[t + "_rms_y"], t + ".rmsnorm", 0.9)
        a = torch.tensor(z[t + "_mul_a"]).cuda().requires_grad_()
        b = torch.tensor(z[t + "_mul_b"]).cuda().requires_grad_()
        y = mx.simd_mul(a, b, mx_specs=sp)
        y.backward(go)
        assert np.array_equal(y.detach().float().cpu().numpy(), z[t + "_mul_y"])
        assert np.array_equal(a.grad.float().cpu().numpy(), z[t + "_mul_ga"])


def test_attention_shaped_bmm_softmax_bmm():
    """Config-4 shape at reduced head count: Q K^T -> softmax -> P V with fp6_e3m2 operands."""
    torch.manual_seed(0)
    H, S, D = 2, 256, 128
    q, k, v = [(torch.randn(H, S, D) * 128 ** -0.25).to(torch.bfloat16) for _ in range(3)]
    outs = {}
    for dev in ("cpu", "cuda"):
        sp = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "block_size": 32, "bfloat": 16, "custom_cuda": dev == "cuda"})
        Q, K, V = q.float().to(dev), k.float().to(dev), v.float().to(dev)
        s = mx.bmm(Q, K.transpose(-1, -2).contiguous(), mx_specs=sp)
        outs[dev] = (s, V, sp)
    close_bf16(outs["cuda"][0], outs["cpu"][0].numpy(), "scores")
    # second product on identical probabilities, so only the GEMM differs
    p = mx.softmax(outs["cpu"][0], dim=-1, mx_specs=outs["cpu"][2])
    o_cpu = mx.bmm(p, outs["cpu"][1], mx_specs=outs["cpu"][2])
    o_gpu = mx.bmm(p.cuda(), outs["cuda"][1], mx_specs=outs["cuda"][2])
    close_bf16(o_gpu, o_cpu.numpy(), "out")


def test_weight_is_requantized_every_call_unless_frozen(monkeypatch, tmp_path):
    """Like the reference, mx.Linear quantizes its weight in every forward call, so an in-place update
    through `.data` (which moves neither the pointer nor the version counter) is seen at once.  After
    prequantize_weights() the packed weight is kept and reused; it can be saved and loaded."""
    from microxcaling_b200 import _backend
    from microxcaling_b200.packed import PackedMX
    sp = finalize_mx_specs({"w_elem_format": "fp8_e4m3", "a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16,
                            "round": "even"})
    lin = mx.Linear(256, 128, bias=False, mx_specs=sp).cuda().to(torch.bfloat16)
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    packs = lambda: _backend.launch_count(1)
    with torch.no_grad():
        y1 = lin(x)
        lin.weight.data.mul_(2.0)                   # invisible to data_ptr / _version
        n = packs()
        y2 = lin(x)
        assert packs() - n == 2                     # activations and weight packed again
        assert torch.equal(y2.float(), 2.0 * y1.float())
        lin.eval()
        lin.prequantize_weights()
        y3 = lin(x)
        n = packs()
        y4 = lin(x)
        assert packs() - n == 1                     # only the activations
        assert torch.equal(y3, y4) and torch.equal(y3, y2)
        lin.weight.mul_(0.5)                        # a tracked in-place update: the packed weight follows
        n = packs()
        y5 = lin(x)
        assert packs() - n == 2 and torch.equal(y5, y1)
        # file round trip of the packed weight, used in place of the tensor
        pw = lin.packed_weight()
        path = str(tmp_path / "w.mxq")
        pw.save(path)
        back = PackedMX.load(path, device="cuda")
        assert torch.equal(back.codes, pw.codes) and torch.equal(back.scales, pw.scales)
        y6 = mx.linear(x, lin.weight, None, mx_specs=sp, prequantized_weights=True, packed_weight=back)
        assert torch.equal(y6, y5)
        # and its decoded values are the fake-quantized weight
        from microxcaling_b200.mx_ops import quantize_mx_op
        wq = quantize_mx_op(lin.weight.detach(), sp, elem_format="fp8_e4m3", axes=[-1], round=sp["round_mx_output"])
        assert torch.equal(back.dequantize(torch.float32)[0], wq.float())


def test_linear_with_odd_feature_count_takes_the_tensor_core_path(monkeypatch):
    """in_features = 96 (whole 32-blocks, not a multiple of 128): packed GEMM, same result as the
    reference construction (fake-quantized operands, torch GEMM, rounding) up to accumulation order."""
    from microxcaling_b200 import _backend, _mxgemm
    sp = finalize_mx_specs({"w_elem_format": "fp8_e4m3", "a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16})
    torch.manual_seed(0)
    lin = mx.Linear(96, 160, bias=False, mx_specs=sp).cuda().to(torch.bfloat16)
    x = torch.randn(200, 96, device="cuda", dtype=torch.bfloat16)
    g0 = _backend.launch_count(0)
    with torch.no_grad():
        got = lin(x)
    assert _backend.launch_count(0) - g0 == 1
    import importlib
    linear_mod = importlib.import_module("microxcaling_b200.linear")
    monkeypatch.setattr(_mxgemm, "_fast_ok", lambda *a, **k: False)
    monkeypatch.setattr(linear_mod, "_one_call_ok", lambda *a, **k: False)
    with torch.no_grad():
        want = lin(x)
    assert _backend.launch_count(0) - g0 == 1
    close_bf16(got, want.float().cpu().numpy(), "linear K=96")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_variants_match_reference(golden_layers2, dtype):
    """mode_config aw / wa, matmul bias, addmm, quantize_backprop=False and per-tensor rounding modes on CUDA
    tensors against outputs recorded from the reference.  With quantize_backprop=False the backward products
    are plain (unquantized) torch GEMMs: compared in fp32 with a relative tolerance, only for fp32 tensors."""
    from test_host_layers import _run_layers2_case
    meta, z = golden_layers2
    for m in meta:
        if m["op"] in ("ffn", "lstm"):
            continue
        nobp = m["specs"].get("quantize_backprop") is False
        for name, (got, want) in _run_layers2_case(m, z, "cuda", dtype).items():
            tag = m["tag"] + "." + name
            if nobp and name != "y":
                if dtype == torch.float32:
                    a = got.detach().float().cpu().numpy()
                    assert np.allclose(a, want, rtol=1e-4, atol=1e-4 * np.abs(want).max()), tag
                continue
            if m["tag"] == "mm_bias_3d_shared" and name == "gb" and dtype == torch.bfloat16:
                # gradient of a right operand shared by the batch: autograd sums the per-batch products in the
                # tensor's dtype, so bfloat16 storage rounds that sum once more than the fp32 containers do
                # (and a per-batch product that lands on the neighbouring bfloat16 value moves the sum by an ulp
                # of that product, not of the sum)
                a = got.detach().float().cpu().numpy().astype(np.float64)
                assert (np.abs(a - want) <= np.abs(want) * 2.0 ** -7 + np.abs(want).max() * 2.0 ** -6).all(), tag
                continue
            if m["op"].startswith("conv"):
                # the convolution itself is the vendor library's (Winograd / TF32 / bfloat16 algorithms whose error
                # is relative to the size of the summands, not of the sum): bound relative to the tensor's values
                a = got.detach().float().cpu().numpy().astype(np.float64)
                rms = np.sqrt((want.astype(np.float64) ** 2).mean())
                assert (np.abs(a - want) <= 2.0 ** -6 * (np.abs(want) + rms)).all(), (tag, float(np.abs(a - want).max()), rms)
                assert float((a == want).mean()) >= (0.3 if dtype == torch.bfloat16 else 0.5), (tag, float((a == want).mean()))
                continue
            bias_grad = name in ("gbias", "gb") and got.dim() == 1
            if bias_grad and dtype == torch.bfloat16 and m["specs"].get("round_grad_weight") == "floor":
                # the bias gradient is a torch sum: on bfloat16 storage torch rounds it to nearest-even before the
                # 'floor' rounding step sees it (nothing left to round), on fp32 containers the fp32 sum is
                # rounded toward zero: half of the values sit one ulp apart
                close_bf16(got, want, tag, min_exact=0.3)
                continue
            close_bf16(got, want, tag, min_exact=0.9 if bias_grad else 0.97)


def test_mx_quantization_over_two_axes_on_cuda(golden_sweep):
    """Several shared axes on a CUDA tensor (the reference handles them with torch ops on the tensor's
    device, mx/mx_ops.py:228-296): equals the host formulation; and shared_exp_method='none'."""
    from microxcaling_b200.mx_ops import _quantize_mx
    torch.manual_seed(3)
    x = torch.randn(6, 40, 24) * 3
    for axes, bs in (([0, 2], 4), ([-1, -2], 8), ([1, 2], 32)):
        for fmt in ("fp8_e4m3", "int8", "fp4_e2m1"):
            for rnd in ("nearest", "even"):
                want = _quantize_mx(x, 8, fmt, axes=axes, block_size=bs, round=rnd)
                got = _quantize_mx(x.cuda(), 8, fmt, axes=axes, block_size=bs, round=rnd)
                assert got.is_cuda and torch.equal(got.cpu(), want), (axes, bs, fmt, rnd)
    want = _quantize_mx(x, 8, "fp6_e2m3", shared_exp_method="none", axes=[-1], block_size=32)
    got = _quantize_mx(x.cuda(), 8, "fp6_e2m3", shared_exp_method="none", axes=[-1], block_size=32)
    assert torch.equal(got.cpu(), want)
    xb = x.to(torch.bfloat16)
    got = _quantize_mx(xb.cuda(), 8, "fp8_e4m3", axes=[0, 1], block_size=2)
    assert got.dtype == torch.bfloat16 and torch.equal(got.cpu(), _quantize_mx(xb, 8, "fp8_e4m3", axes=[0, 1], block_size=2))


def test_lstm_matches_reference_on_gpu(golden_layers2):
    """Two-layer bidirectional MX LSTM on CUDA (fp32 tensors: the fixture's arithmetic; every product on the
    tensor cores).  Differences of one bfloat16 ulp in a product travel through the recurrence, so the bound
    is relative to the size of the values of the same tensor, not per element."""
    from test_host_layers import run_lstm_case
    from microxcaling_b200 import _backend
    meta, z = golden_layers2
    m = [r for r in meta if r["op"] == "lstm"][0]
    g0 = _backend.launch_count(0)
    res = run_lstm_case(m, z, "cuda", torch.float32)
    # per direction and layer: 1 input + 5 hidden products forward, two gradient products each backward,
    # less the gradient with respect to the initial hidden state (not needed) of each direction and layer
    assert _backend.launch_count(0) - g0 == 3 * (4 + 4 * 5) - 4
    for name, (got, want) in res.items():
        a, b = got.detach().float().cpu().numpy().astype(np.float64), want.astype(np.float64)
        scale = np.sqrt((b ** 2).mean())
        assert (np.abs(a - b) <= 2.0 ** -5 * (np.abs(b) + scale)).all(), (name, float(np.abs(a - b).max()), scale)
        assert float((a == b).mean()) >= 0.5, (name, float((a == b).mean()))


def test_activations_simd_and_norm_layers_on_gpu():
    """The vector-op layers recorded in layers3.npz (activations, simd operators, LayerNorm, GroupNorm,
    BatchNorm, adaptive average pooling) on fp32 CUDA tensors with custom_cuda: the same chains with the
    roundings done by the library's elementwise kernel.  CUDA's exp / tanh / sqrt / division and its reduction
    order differ from the host's in the last fp32 bit, which moves a value only when it sits on a rounding
    boundary: at least 97 % of every tensor must be identical and nothing may differ by more than one vector-format
    step at the scale of the tensor."""
    import os
    import sys
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    if here not in sys.path:
        sys.path.insert(0, here)
    import vector_cases as vc
    z = np.load(os.path.join(here, "layers3.npz"))

    class OnGpu:
        """`mx` with modules moved to the GPU after construction."""
        def __getattr__(self, name):
            obj = getattr(mx, name)
            if isinstance(obj, type) and issubclass(obj, torch.nn.Module):
                return lambda *a, **k: obj(*a, **k).cuda()
            return obj

    checked = 0
    for case in vc.CASES:
        tensors = {k.split("/", 1)[1]: torch.tensor(z[k]).cuda() for k in z.files
                   if k.startswith(case + "/") and k.count("/") == 1}
        for sname in ("bf16", "bf16_even"):
            sp = finalize_mx_specs(dict(vc.SPECS[sname], custom_cuda=True), early_exit=False)
            got = vc.run_case(OnGpu(), case, tensors, sp)
            for name, g in got.items():
                want = z["%s/%s/%s" % (case, sname, name)].astype(np.float64)
                a = g.detach().float().cpu().numpy().astype(np.float64)
                assert a.shape == want.shape, (case, sname, name)
                step = 2.0 ** -7 * max(np.abs(want).max(), 1e-30)
                assert np.abs(a - want).max() <= step, (case, sname, name, np.abs(a - want).max(), step)
                assert (a == want).mean() >= 0.97, (case, sname, name, (a == want).mean())
                checked += 1
    assert checked > 120
