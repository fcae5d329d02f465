"""CPU tests of the layer API (linear / matmul / bmm, softmax, RMSNorm, SiLU,
simd ops, injection) against outputs recorded from the reference on the same
seeded inputs.  On CPU tensors the layers follow the reference's construction
with torch's own GEMM, so forward values and gradients must match exactly."""
import numpy as np
import pytest
import torch

import microxcaling_b200 as mx
from microxcaling_b200.specs import finalize_mx_specs


def _same(t, ref):
    a = t.detach().numpy()
    return np.array_equal(a, ref, equal_nan=True)


def test_linear_matmul_bmm_match_reference(golden_layers):
    meta, z = golden_layers
    for m in meta:
        if m["op"] == "vec":
            continue
        sp = finalize_mx_specs(dict(m["specs"], custom_cuda=False))
        t = m["tag"]
        go = torch.tensor(z[t + "_go"])
        if m["op"] == "linear":
            x = torch.tensor(z[t + "_x"], requires_grad=True)
            w = torch.tensor(z[t + "_w"], requires_grad=True)
            b = torch.tensor(z[t + "_b"], requires_grad=True) if m["bias"] else None
            y = mx.linear(x, w, b, mx_specs=sp)
            y.backward(go)
            assert _same(y, z[t + "_y"]) and _same(x.grad, z[t + "_gx"]) and _same(w.grad, z[t + "_gw"]), t
            if m["bias"]:
                assert _same(b.grad, z[t + "_gb"]), t
        else:
            a = torch.tensor(z[t + "_a"], requires_grad=True)
            b = torch.tensor(z[t + "_b"], requires_grad=True)
            y = (mx.bmm if m["op"] == "bmm" else mx.matmul)(a, b, mx_specs=sp)
            y.backward(go)
            assert _same(y, z[t + "_y"]) and _same(a.grad, z[t + "_ga"]) and _same(b.grad, z[t + "_gb"]), t


def test_vector_layers_match_reference(golden_layers):
    meta, z = golden_layers
    seen = 0
    for m in meta:
        if m["op"] != "vec":
            continue
        seen += 1
        sp = finalize_mx_specs(dict(m["specs"], custom_cuda=False))
        t = m["tag"]
        go = torch.tensor(z[t + "_sm_go"])
        x = torch.tensor(z[t + "_sm_x"], requires_grad=True)
        y = mx.softmax(x, dim=-1, mx_specs=sp)
        y.backward(go)
        assert _same(y, z[t + "_sm_y"]) and _same(x.grad, z[t + "_sm_gx"]), t
        x = torch.tensor(z[t + "_silu_x"], requires_grad=True)
        y = mx.silu(x, mx_specs=sp)
        y.backward(go)
        assert _same(y, z[t + "_silu_y"]) and _same(x.grad, z[t + "_silu_gx"]), t
        x = torch.tensor(z[t + "_rms_x"], requires_grad=True)
        norm = mx.RMSNorm(96, eps=1e-5, mx_specs=sp)
        with torch.no_grad():
            norm.weight.copy_(torch.tensor(z[t + "_rms_w"]))
            norm.bias.copy_(torch.tensor(z[t + "_rms_b"]))
        y = norm(x)
        y.backward(go)
        assert _same(y, z[t + "_rms_y"]) and _same(x.grad, z[t + "_rms_gx"]), t
        assert _same(norm.weight.grad, z[t + "_rms_gw"]) and _same(norm.bias.grad, z[t + "_rms_gb"]), t
        a = torch.tensor(z[t + "_mul_a"], requires_grad=True)
        b = torch.tensor(z[t + "_mul_b"], requires_grad=True)
        y = mx.simd_mul(a, b, mx_specs=sp)
        y.backward(go)
        assert _same(y, z[t + "_mul_y"]) and _same(a.grad, z[t + "_mul_ga"]) and _same(b.grad, z[t + "_mul_gb"]), t
    assert seen == 2


def test_mx_specs_none_is_stock_torch():
    # mx/tests/test_mxfp_none.py: with mx_specs=None every op is the torch op
    torch.manual_seed(0)
    x, w, b = torch.randn(5, 16), torch.randn(8, 16), torch.randn(8)
    assert torch.equal(mx.linear(x, w, b, mx_specs=None), torch.nn.functional.linear(x, w, b))
    assert torch.equal(mx.matmul(x, w.t(), mx_specs=None), torch.matmul(x, w.t()))
    assert torch.equal(mx.bmm(x[None], w.t()[None], mx_specs=None), torch.bmm(x[None], w.t()[None]))
    assert torch.equal(mx.softmax(x, -1, mx_specs=None), torch.softmax(x, -1))
    assert torch.equal(mx.silu(x, mx_specs=None), torch.nn.functional.silu(x))
    lin = mx.Linear(16, 8, mx_specs=None)
    assert torch.equal(lin(x), torch.nn.functional.linear(x, lin.weight, lin.bias))
    assert mx.quantize_bfloat(x, None) is x


def test_quantization_disabled_matches_torch():
    # mx/tests/test_linear.py:64-95: bfloat=0 and no element formats -> plain GEMM
    torch.manual_seed(1)
    sp = finalize_mx_specs({}, early_exit=False)
    x = torch.randn(6, 32, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    lin = mx.Linear(32, 12, mx_specs=sp)
    ref = torch.nn.Linear(32, 12)
    ref.load_state_dict(lin.state_dict())
    y, y2 = lin(x), ref(x2)
    y.sum().backward()
    y2.sum().backward()
    assert torch.allclose(y, y2, atol=1e-6) and torch.allclose(x.grad, x2.grad, atol=1e-6)
    assert torch.allclose(lin.weight.grad, ref.weight.grad, atol=1e-6)


def test_inject_pyt_ops_and_restore():
    from microxcaling_b200 import mx_mapping
    saved = {k: torch.__dict__.get(k) for k in mx_mapping.FUNCTION_MAPPING}
    saved_f = {k: torch.nn.functional.__dict__.get(k) for k in mx_mapping.FUNCTION_MAPPING}
    saved_m = {k: torch.nn.__dict__.get(k) for k in mx_mapping.MODULE_MAPPING}
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16})
    try:
        mx_mapping.inject_pyt_ops(sp)
        torch.manual_seed(2)
        lin = torch.nn.Linear(64, 32, bias=False)
        assert isinstance(lin, mx.Linear) and lin.mx_specs["w_elem_format"] == "fp4_e2m1"
        x = torch.randn(4, 64)
        y = lin(x)
        y_direct = mx.linear(x, lin.weight, None, mx_specs=sp)
        assert torch.equal(y, y_direct)
        assert not torch.equal(y, saved_f["linear"](x, lin.weight))
        z = torch.mul(torch.nn.functional.silu(y), y)
        assert torch.equal(z, mx.simd_mul(mx.silu(y, mx_specs=sp), y, mx_specs=sp))
        assert torch.matmul(x, lin.weight.t(), dtype=torch.float64).dtype == torch.float64
    finally:
        for k, v in saved.items():
            if v is not None:
                torch.__dict__[k] = v
        for k, v in saved_f.items():
            if v is not None:
                torch.nn.functional.__dict__[k] = v
        for k, v in saved_m.items():
            torch.nn.__dict__[k] = v
    assert torch.nn.Linear is saved_m["Linear"]


def test_gradcheck_no_quantization():
    # mx/tests/test_gradcheck.py:44-63: float64 gradcheck with default (no-quant) specs
    sp = finalize_mx_specs({}, early_exit=False)
    x = torch.randn(3, 8, dtype=torch.float64, requires_grad=True)
    w = torch.randn(5, 8, dtype=torch.float64, requires_grad=True)
    b = torch.randn(5, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, c, d: mx.linear(a, c, d, mx_specs=sp), (x, w, b))
    a = torch.randn(2, 3, 4, dtype=torch.float64, requires_grad=True)
    c = torch.randn(2, 4, 5, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda u, v: mx.bmm(u, v, mx_specs=sp), (a, c))
    assert torch.autograd.gradcheck(lambda u, v: mx.matmul(u, v, mx_specs=sp), (a, c))


def _run_layers2_case(m, z, dev, dtype):
    """Runs one recorded case of layers2.npz; returns {name: (got tensor, recorded array)}."""
    from microxcaling_b200 import mx_mapping
    sp = finalize_mx_specs(dict(m["specs"], custom_cuda=(dev != "cpu")))
    t = m["tag"]
    ld = lambda k, grad=True: torch.tensor(z[t + "_" + k]).to(dev, dtype).requires_grad_(grad)
    go = ld("go", False)
    out = {}
    if m["op"] in ("matmul", "addmm"):
        a, b = ld("a"), ld("b")
        bias = ld("bias") if m["bias"] else None
        if m["op"] == "addmm":
            y = mx_mapping.addmm_mx(bias, a, b, mx_specs=sp)
        else:
            y = mx.matmul(a, b, bias=bias, mx_specs=sp, mode_config=m["mode_config"])
        y.backward(go)
        out = {"y": (y, z[t + "_y"]), "ga": (a.grad, z[t + "_ga"]), "gb": (b.grad, z[t + "_gb"])}
        if bias is not None:
            out["gbias"] = (bias.grad, z[t + "_gbias"])
    elif m["op"] == "bmm":
        a, b = ld("a"), ld("b")
        y = mx.bmm(a, b, mx_specs=sp)
        y.backward(go)
        out = {"y": (y, z[t + "_y"]), "ga": (a.grad, z[t + "_ga"]), "gb": (b.grad, z[t + "_gb"])}
    elif m["op"] in ("conv1d", "conv2d", "conv3d", "convT2d"):
        x, w = ld("x"), ld("w")
        b = ld("b") if m["bias"] else None
        fn = {"conv1d": mx.conv1d, "conv2d": mx.conv2d, "conv3d": mx.conv3d, "convT2d": mx.conv_transpose2d}[m["op"]]
        y = fn(x, w, b, mx_specs=sp, **m["geom"])
        y.backward(go)
        out = {"y": (y, z[t + "_y"]), "gx": (x.grad, z[t + "_gx"]), "gw": (w.grad, z[t + "_gw"])}
        if b is not None:
            out["gb"] = (b.grad, z[t + "_gb"])
    elif m["op"] == "linear":
        x, w = ld("x"), ld("w")
        b = ld("b") if m["bias"] else None
        y = mx.linear(x, w, b, mx_specs=sp)
        y.backward(go)
        out = {"y": (y, z[t + "_y"]), "gx": (x.grad, z[t + "_gx"]), "gw": (w.grad, z[t + "_gw"])}
        if b is not None:
            out["gb"] = (b.grad, z[t + "_gb"])
    return out


def test_layer_variants_match_reference(golden_layers2):
    """mode_config aw / wa, matmul bias, addmm, quantize_backprop=False, per-tensor rounding modes and the
    convolutions: on CPU tensors the layers follow the reference's construction, so values must match exactly."""
    meta, z = golden_layers2
    assert {m["tag"] for m in meta} >= {"mm_aw", "mm_wa", "mm_bias", "addmm", "lin_nobp", "bmm_nobp", "lin_rounds",
                                        "mm_rounds", "conv2d", "conv1d_groups", "conv3d", "convT2d"}
    for m in meta:
        if m["op"] in ("ffn", "lstm"):
            continue
        for name, (got, want) in _run_layers2_case(m, z, "cpu", torch.float32).items():
            assert _same(got, want), (m["tag"], name)


def run_lstm_case(m, z, dev, dtype):
    sp = finalize_mx_specs(dict(m["specs"], custom_cuda=(dev != "cpu")))
    lstm = mx.LSTM(m["input_size"], m["hidden_size"], num_layers=m["num_layers"], bidirectional=m["bidirectional"],
                   mx_specs=sp)
    lstm.load_state_dict({k[len("lstm_p_"):]: torch.tensor(z[k]) for k in z.files if k.startswith("lstm_p_")})
    lstm = lstm.to(dev).to(dtype)
    x = torch.tensor(z["lstm_x"]).to(dev, dtype).requires_grad_()
    out, (hn, cn) = lstm(x)
    out.backward(torch.tensor(z["lstm_go"]).to(dev, dtype))
    return {"out": (out, z["lstm_out"]), "hn": (hn, z["lstm_hn"]), "cn": (cn, z["lstm_cn"]), "gx": (x.grad, z["lstm_gx"]),
            "g_weight_hh_l0": (lstm.weight_hh_l0.grad, z["lstm_g_weight_hh_l0"]),
            "g_weight_ih_l1_reverse": (lstm.weight_ih_l1_reverse.grad, z["lstm_g_weight_ih_l1_reverse"])}


def test_lstm_matches_reference(golden_layers2):
    """Two-layer bidirectional MX LSTM, forward and backward, against the reference's (CPU: exact)."""
    meta, z = golden_layers2
    m = [r for r in meta if r["op"] == "lstm"][0]
    for name, (got, want) in run_lstm_case(m, z, "cpu", torch.float32).items():
        assert _same(got, want), name
    lstm = mx.LSTM(8, 8, mx_specs=finalize_mx_specs(dict(m["specs"])))
    with pytest.raises(ValueError):
        lstm(torch.nn.utils.rnn.pack_sequence([torch.zeros(3, 8), torch.zeros(2, 8)]))


def test_ffn_via_inject_pyt_ops_matches_reference_on_cpu(golden_layers2):
    """The gated feed-forward block built from stock torch modules after inject_pyt_ops equals the
    block the reference builds the same way (CPU tensors: exact)."""
    import torch.nn.functional as F
    from microxcaling_b200 import mx_mapping
    meta, z = golden_layers2
    m = [r for r in meta if r["op"] == "ffn"][0]
    sp = finalize_mx_specs(dict(m["specs"], custom_cuda=False))
    H, I = m["hidden"], m["inter"]
    t = lambda k: torch.tensor(z["ffn_" + k])
    norm = mx.RMSNorm(H, eps=1e-5, mx_specs=sp)
    with mx_mapping.injected(sp):
        gate, up, down = torch.nn.Linear(H, I, bias=False), torch.nn.Linear(H, I, bias=False), torch.nn.Linear(I, H, bias=False)
        assert isinstance(gate, mx.Linear)
        with torch.no_grad():
            norm.weight.copy_(t("norm_w")); norm.bias.copy_(t("norm_b"))
            gate.weight.copy_(t("wg")); up.weight.copy_(t("wu")); down.weight.copy_(t("wd"))
            h = norm(t("x"))
            g_, u_ = gate(h), up(h)
            act = torch.mul(F.silu(g_), u_)
            y = down(act)
    assert torch.nn.Linear is not type(gate) and not issubclass(torch.nn.Linear, mx.Linear)   # restored
    for name, got in (("h", h), ("gate", g_), ("up", u_), ("act", act), ("y", y)):
        assert _same(got, z["ffn_" + name]), name


def _layers3():
    import os
    import sys
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    if here not in sys.path:
        sys.path.insert(0, here)
    import vector_cases as vc
    return vc, np.load(os.path.join(here, "layers3.npz"))


def test_activations_simd_and_norm_layers_match_reference():
    """Activations (ReLU, ReLU6, LeakyReLU, both GELU forms, sigmoid, tanh, SiLU), the unary and reduction simd
    operators, LayerNorm, GroupNorm, BatchNorm (training with its running statistics, evaluation) and adaptive
    average pooling: outputs, every gradient and the updated statistics equal the values recorded from the
    reference (mx/activations.py, mx/simd_ops.py, mx/norm_utils.py, mx/layernorm.py, mx/groupnorm.py,
    mx/batchnorm.py, mx/adaptive_avg_pooling.py) under three vector formats, exactly (CPU tensors)."""
    vc, z = _layers3()
    n = 0
    for case in vc.CASES:
        tensors = {k.split("/", 1)[1]: torch.tensor(z[k]) for k in z.files if k.startswith(case + "/") and k.count("/") == 1}
        for sname, sdict in vc.SPECS.items():
            sp = finalize_mx_specs(dict(sdict, custom_cuda=False), early_exit=False)
            got = vc.run_case(mx, case, tensors, sp)
            want = {k.rsplit("/", 1)[1]: z[k] for k in z.files if k.startswith("%s/%s/" % (case, sname))}
            assert set(got) == set(want), (case, sname)
            for name, g in got.items():
                assert _same(g, want[name]), (case, sname, name)
                n += 1
    assert n > 200


def test_full_injection_tables_and_restore():
    """inject_pyt_ops maps the reference's whole function and module tables (mx/mx_mapping.py:68-122); after
    restore_pyt_ops the stock callables are back."""
    import torch.nn.functional as F
    from microxcaling_b200 import mx_mapping
    assert len(mx_mapping.FUNCTION_MAPPING) == 30 and len(mx_mapping.MODULE_MAPPING) == 20
    stock = (torch.sum, torch.exp, F.relu, F.layer_norm, torch.nn.LayerNorm, torch.nn.ReLU)
    sp = finalize_mx_specs({"bfloat": 16, "custom_cuda": False}, early_exit=False)
    x = torch.randn(4, 8)
    with mx_mapping.injected(sp):
        assert torch.sum is not stock[0] and issubclass(torch.nn.LayerNorm, mx.LayerNorm)
        y = F.relu(torch.exp(x))
        s = torch.sum(y, 1)
        ln = torch.nn.LayerNorm(8)(x)
    assert (torch.sum, torch.exp, F.relu, F.layer_norm, torch.nn.LayerNorm, torch.nn.ReLU) == stock
    assert _same(y, mx.relu(mx.simd_exp(x, mx_specs=sp), mx_specs=sp).numpy())
    assert _same(s, mx.simd_reduce_sum(y, 1, mx_specs=sp).numpy())
    assert _same(ln, mx.LayerNorm(8, mx_specs=sp)(x).detach().numpy())                 # the MX module's own default eps (1e-12)
