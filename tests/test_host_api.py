"""CPU-side tests: the drop-in Python API (specs, formats, dispatch) and the
exact host formulation used for CPU tensors, against the recorded reference
outputs; and that the C-ABI library loads and exports what include/mxq.h
declares (no compute calls here)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import oracle
from helpers import all_encodings, sha
from microxcaling_b200 import specs as S
from microxcaling_b200.formats import ElemFormat, RoundingMode, _get_format_params
from microxcaling_b200.mx_ops import _quantize_mx, quantize_mx_op
from microxcaling_b200.elemwise_ops import _quantize_elemwise_core, _quantize_bfloat, quantize_elemwise_op

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_abi_exports_match_header():
    hdr = open(os.path.join(ROOT, "include", "mxq.h")).read()
    names = set(re.findall(r"\b(mxq_[a-z0-9_]+)\s*\(", hdr))
    assert {"mxq_quantize_mx", "mxq_quantize_elemwise", "mxq_reduce_sum_inner", "mxq_reduce_max_inner",
            "mxq_status_string", "mxq_version"} <= names
    lib = ctypes.CDLL(os.path.join(ROOT, "microxcaling_b200", "libmxq.so"))
    for n in names:
        assert hasattr(lib, n), n
    lib.mxq_status_string.restype = ctypes.c_char_p
    assert lib.mxq_status_string(0) == b"ok"
    assert lib.mxq_version() >= 1


def test_format_table():
    # mx/tests/test_formats.py:12-95
    expect = {"int8": (0, 8, 0, 1.984375, 0), "int4": (0, 4, 0, 1.75, 0), "int2": (0, 2, 0, 1.0, 0),
              "fp8_e5m2": (5, 4, 15, 57344.0, 2 ** -14), "fp8_e4m3": (4, 5, 8, 448.0, 2 ** -6),
              "fp6_e3m2": (3, 4, 4, 28.0, 2 ** -2), "fp6_e2m3": (2, 5, 2, 7.5, 1.0),
              "fp4_e2m1": (2, 3, 2, 6.0, 1.0), "fp4": (2, 3, 2, 6.0, 1.0),
              "float16": (5, 12, 15, 65504.0, 2 ** -14), "bfloat16": (8, 9, 127, 3.3895313892515355e38, 2 ** -126)}
    for k, v in expect.items():
        assert _get_format_params(k) == v, k
        assert _get_format_params(ElemFormat.from_str(k)) == v
    assert RoundingMode["nearest"] == 0 and RoundingMode["floor"] == 1 and RoundingMode["even"] == 2
    assert RoundingMode.string_enums() == ["nearest", "floor", "even"]
    with pytest.raises(Exception):
        ElemFormat.from_str("fp5_e2m2")


def test_finalize_specs():
    # mx/tests/test_finalize_mxfp.py:17-43 and mx/specs.py:279-326
    assert S.finalize_mx_specs({}) is None
    assert S.finalize_mx_specs({"block_size": 32, "round": "even"}) is None
    sp = S.finalize_mx_specs({}, early_exit=False)
    assert sp["bfloat"] == 0 and sp["round_output"] == "nearest"
    sp = S.finalize_mx_specs({"w_elem_format": "fp8_e4m3", "a_elem_format": "fp6_e3m2", "a_elem_format_bp_os": "int8",
                              "round": "even", "round_grad_input": "floor", "round_mx_output": None,
                              "block_size": 32, "bfloat": 16})
    assert sp["w_elem_format_bp"] == "fp8_e4m3" and sp["a_elem_format_bp"] == "fp6_e3m2"
    assert sp["a_elem_format_bp_ex"] == "fp6_e3m2" and sp["a_elem_format_bp_os"] == "int8"
    assert sp["round_output"] == "even" and sp["round_weight"] == "even" and sp["round_mx_output"] == "even"
    assert sp["round_mx_weight_grad_input"] == "floor" and sp["round_mx_input_grad_weight"] == "floor"
    with pytest.raises(KeyError):
        S.apply_mx_specs({"not_a_key": 1})
    with pytest.raises(AssertionError):
        S.MxSpecs({"not_a_key": 1})
    b = S.get_backwards_mx_specs(S.MxSpecs({"a_elem_format": "int8", "bfloat": 16, "quantize_backprop": False,
                                            "block_size": 32}))
    assert b["a_elem_format"] is None and b["bfloat"] == 0 and b["block_size"] == 0
    b = S.get_backwards_mx_specs(S.MxSpecs({"a_elem_format": "int8", "bfloat": 16}))
    assert b["a_elem_format"] == "int8" and b["bfloat"] == 16


def test_argparse_roundtrip():
    import argparse
    p = S.add_mx_args(argparse.ArgumentParser())
    assert S.get_mx_specs(p.parse_args([])) is None
    sp = S.get_mx_specs(p.parse_args(["--a_elem_format", "fp4_e2m1", "--block_size", "32", "--no_quantize_backprop",
                                      "--bfloat", "16"]))
    assert sp["a_elem_format"] == "fp4_e2m1" and sp["block_size"] == 32 and sp["quantize_backprop"] is False
    assert sp["bfloat_subnorms"] is True and sp["custom_cuda"] is False
    sp = S.get_mx_specs(p.parse_args(["--skip_early_exit"]))
    assert sp is not None and sp["bfloat"] == 0


def test_host_formulation_matches_recorded_reference(golden_recorded):
    meta, z = golden_recorded
    bad = []
    for i, rec in enumerate(meta):
        if "recipe" in rec:
            e, m, inf = rec["recipe"]
            x = all_encodings(e, m, bool(inf)).reshape(rec["shape"])
            if i % 7:                      # the large sweeps are sampled to keep this suite short
                continue
        else:
            x = z["x%d" % i]
        if x.ndim == 0:
            continue
        p = rec["params"]
        t = torch.as_tensor(x)
        if rec["kind"] == "mx":
            y = _quantize_mx(t, p["scale_bits"], p["fmt"], axes=[p["axis"]], block_size=p["block"],
                             round=p["round"], flush_fp32_subnorms=p["flush"]).numpy()
        else:
            y = _quantize_elemwise_core(t, p["bits"], p["exp_bits"], p["max_norm"], p["round"], p["saturate"],
                                        p["allow_denorm"]).numpy()
        ok = (sha(y) == rec["sha"]) if "sha" in rec else oracle.same_values(y, z["y%d" % i])
        if not ok:
            bad.append((i, p))
    assert not bad, bad[:5]


def test_op_level_dispatch():
    x = torch.randn(8, 64)
    sp = S.finalize_mx_specs({"a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16})
    assert quantize_mx_op(x, sp, elem_format=None, axes=[-1]) is x
    assert quantize_elemwise_op(x, None) is x
    y = quantize_mx_op(x, sp, elem_format="fp8_e4m3", axes=[-1])
    assert oracle.same_values(y.numpy(), oracle.quantize_mx(x.numpy(), "fp8_e4m3"))
    y0 = quantize_mx_op(x, sp, elem_format="fp8_e4m3", axes=[0], block_size=0)
    assert oracle.same_values(y0.numpy(), oracle.quantize_mx(x.numpy(), "fp8_e4m3", axis=0, block=0))
    sp5 = S.finalize_mx_specs({"a_elem_format": "int4", "block_size": 16, "scale_bits": 5})
    y5 = quantize_mx_op(x * 1e6, sp5, elem_format="int4", axes=[1], round="even")
    assert oracle.same_values(y5.numpy(), oracle.quantize_mx((x * 1e6).numpy(), "int4", block=16, scale_bits=5,
                                                             round="even"))
    z = quantize_elemwise_op(x, sp, round="nearest")
    assert oracle.same_values(z.numpy(), oracle.quantize_elemwise(x.numpy(), 9, 8, 3.3895313892515355e38))
    assert _quantize_bfloat(x, 0) is x and _quantize_bfloat(x, 32) is x
    for bad in ({"bfloat": 16, "fp": 16}, {"bfloat": 8}, {"fp": 5}):
        with pytest.raises(ValueError):
            quantize_elemwise_op(x, S.MxSpecs(bad))
    # two shared axes (host path only): equals the oracle applied on 2-D tiles
    y2 = _quantize_mx(torch.ones(4, 4), 8, "int8", axes=[0, 1], block_size=2)
    assert torch.equal(y2, torch.ones(4, 4))


def test_dither_is_reproducible_with_given_noise():
    torch.manual_seed(3)
    x = torch.randn(16, 64)
    n = torch.rand(16, 64)
    a = _quantize_mx(x, 8, "fp6_e2m3", axes=[-1], block_size=32, round="dither", noise=n)
    b = _quantize_mx(x, 8, "fp6_e2m3", axes=[-1], block_size=32, round="dither", noise=n)
    lo = _quantize_mx(x, 8, "fp6_e2m3", axes=[-1], block_size=32, round="floor")
    assert torch.equal(a, b)
    q = (a - lo).abs()
    assert (q >= 0).all() and ((a.abs() >= lo.abs()) | (a == lo)).all()


def test_cpu_twins_match_recorded_reference(golden_recorded):
    """mxq_cpu_quantize_mx / mxq_cpu_quantize_elemwise (the host C++ quantizers behind
    funcs.quantize_mx_func_cpp / quantize_elemwise_func_cpp) against every call recorded from the
    reference's own CPU test-suite."""
    from microxcaling_b200 import _backend as be
    meta, z = golden_recorded
    bad = []
    for i, rec in enumerate(meta):
        if "recipe" in rec:
            e, m, inf = rec["recipe"]
            x = all_encodings(e, m, bool(inf)).reshape(rec["shape"])
        else:
            x = z["x%d" % i]
        if x.ndim == 0:
            continue
        p = rec["params"]
        t = torch.as_tensor(x)
        if rec["kind"] == "mx":
            eb, mb, mn = oracle.FORMATS[p["fmt"]]
            y = be.cpu_quantize_mx(t, p["scale_bits"], eb, mb, mn, p["block"], p["axis"], p["flush"],
                                   oracle.ROUND[p["round"]]).numpy()
        else:
            y = be.cpu_quantize_elemwise(t, p["bits"], p["exp_bits"], p["max_norm"], oracle.ROUND[p["round"]],
                                         p["saturate"], p["allow_denorm"]).numpy()
        ok = (sha(y) == rec["sha"]) if "sha" in rec else oracle.same_values(y, z["y%d" % i])
        if not ok:
            bad.append((i, rec["kind"], p))
    assert not bad, bad[:5]


def test_cpu_twins_storage_types_and_legacy_names():
    """fp16 / bf16 host tensors, the dispatch of custom_cuda=True on CPU tensors, the seven legacy names."""
    from microxcaling_b200 import _backend as be
    torch.manual_seed(1)
    x = torch.randn(33, 96) * torch.exp2(torch.randint(-20, 20, (33, 96)).float())
    for dt in (torch.float16, torch.bfloat16):
        xd = x.to(dt)
        for fmt in ("fp8_e4m3", "fp4_e2m1", "int8"):
            eb, mb, mn = oracle.FORMATS[fmt]
            for axis in (0, 1):
                y = be.cpu_quantize_mx(xd, 8, eb, mb, mn, 32, axis)
                want = oracle.quantize_mx(xd.float().numpy(), fmt, axis=axis)
                assert y.dtype == dt
                assert oracle.same_values(y.float().numpy(), torch.as_tensor(want).to(dt).float().numpy()), (dt, fmt, axis)
        y = be.cpu_quantize_elemwise(xd, 5, 8, 2.0 ** 127 * 1.75, 2)
        want = oracle.quantize_elemwise(xd.float().numpy(), 5, 8, 2.0 ** 127 * 1.75, "even")
        assert oracle.same_values(y.float().numpy(), torch.as_tensor(want).to(dt).float().numpy())
    # fp32 in, bf16 out, round-even = torch's cast
    y = be.cpu_quantize_elemwise(x, 9, 8, 3.3895313892515355e38, 2, out_dtype=torch.bfloat16)
    assert torch.equal(y, x.to(torch.bfloat16))
    # custom_cuda=True on an ordinary CPU tensor reaches the host quantizer and equals the torch formulation
    a = _quantize_mx(x, 8, "fp6_e3m2", axes=[0], block_size=32, custom_cuda=True)
    b = _quantize_mx(x, 8, "fp6_e3m2", axes=[0], block_size=32, custom_cuda=False)
    assert oracle.same_values(a.numpy(), b.numpy())
    a = _quantize_elemwise_core(x, 7, 5, 57344.0, "nearest", custom_cuda=True)
    b = _quantize_elemwise_core(x, 7, 5, 57344.0, "nearest", custom_cuda=False)
    assert oracle.same_values(a.numpy(), b.numpy())
    # the reference's call pattern: blocks reshaped onto their own axis, that whole axis shared
    xb = x[:32].reshape(1, 32, 96)
    mv = xb.abs().max(dim=1, keepdim=True).values
    y = be.funcs.quantize_mx_func_cpp(xb, 8, 4, 5, 448.0, mv, 1, False, 0)
    assert oracle.same_values(y.reshape(32, 96).numpy(), oracle.quantize_mx(x[:32].numpy(), "fp8_e4m3", axis=0))
    y = be.funcs.quantize_elemwise_func_cpp(x, 9, 8, 3.3895313892515355e38, 0, False, True)
    assert oracle.same_values(y.numpy(), oracle.quantize_elemwise(x.numpy(), 9, 8, 3.3895313892515355e38))
    with pytest.raises(be.MxqError):
        be.funcs.quantize_mx_func_cpp(torch.zeros(1, 1, 1, 1, 1, 2), 8, 4, 5, 448.0, None, 1)
    # dither with a caller noise tensor: host quantizer == torch formulation
    n = torch.rand_like(x)
    a = _quantize_mx(x, 8, "fp6_e2m3", axes=[-1], block_size=32, round="dither", noise=n, custom_cuda=True)
    b = _quantize_mx(x, 8, "fp6_e2m3", axes=[-1], block_size=32, round="dither", noise=n, custom_cuda=False)
    assert oracle.same_values(a.numpy(), b.numpy())


def test_shared_exp_method_none_and_block_helpers():
    """shared_exp_method='none' (an exponent per value) = blocks of one element; the block
    helpers keep the reference's contract (mx/mx_ops.py:49-170)."""
    from microxcaling_b200.mx_ops import _reshape_to_blocks, _undo_reshape_to_blocks, _shared_exponents
    torch.manual_seed(2)
    x = torch.randn(6, 40)
    y = _quantize_mx(x, 8, "fp4_e2m1", shared_exp_method="none", axes=[-1], block_size=32)
    assert oracle.same_values(y.numpy(), oracle.quantize_mx(x.numpy(), "fp4_e2m1", axis=1, block=1))
    with pytest.raises(Exception):
        _quantize_mx(x, 8, "fp4_e2m1", shared_exp_method="mean", axes=[-1], block_size=32)
    b, axes, orig, padded = _reshape_to_blocks(x, [-1], 32)
    assert tuple(b.shape) == (6, 2, 32) and axes == [1] and tuple(orig) == (6, 40, 1) and tuple(padded) == (6, 64, 1)
    assert torch.equal(_undo_reshape_to_blocks(b, padded, orig, axes), x)
    e = _shared_exponents(b, "max", [2])
    assert tuple(e.shape) == (6, 2, 1)
    assert torch.equal(e[:, 0, 0], torch.floor(torch.log2(x[:, :32].abs().max(dim=1).values)))
    assert float(_shared_exponents(torch.zeros(4), "max", [0])) == -126.0


def test_derived_specs_are_reused_only_while_unchanged():
    """apply_mx_specs / get_backwards_mx_specs (mx/specs.py:212-276, 193-209) run on every layer call;
    what they derive from an MxSpecs object is reused until that object, or the derived one, changes."""
    from microxcaling_b200.specs import MxSpecs, apply_mx_specs, finalize_mx_specs, get_backwards_mx_specs
    sp = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "w_elem_format": "fp4_e2m1", "block_size": 32, "bfloat": 16})
    a = apply_mx_specs(sp)
    assert a is apply_mx_specs(sp) and dict(a) == dict(sp)
    assert get_backwards_mx_specs(a) is get_backwards_mx_specs(a)
    sp["round"] = "even"                                     # the source changed: derived again
    b = apply_mx_specs(sp)
    assert b is not a and b["round"] == "even" and a["round"] == "nearest"
    b["bfloat"] = 12                                         # a caller changed the derived object: not handed out again
    c = apply_mx_specs(sp)
    assert c is not b and c["bfloat"] == 16
    off = c.copy()
    off["quantize_backprop"] = False
    bw = get_backwards_mx_specs(off)
    assert bw["a_elem_format"] is None and bw["block_size"] == 0 and off["a_elem_format"] == "fp6_e3m2"
    assert isinstance(off, MxSpecs) and len(off) == len(sp)
    assert apply_mx_specs({"bfloat": 16})["bfloat"] == 16    # plain dicts still work
    with pytest.raises(KeyError):
        apply_mx_specs({"no_such_key": 1})


def test_forward_without_autograd_equals_function_apply():
    """Layers called where nothing can need a gradient run their forward directly; values are those of
    Function.apply, and a parameter that requires a gradient still gets one."""
    import microxcaling_b200 as mx
    from microxcaling_b200.specs import finalize_mx_specs
    sp = finalize_mx_specs({"a_elem_format": "fp8_e4m3", "w_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16})
    torch.manual_seed(3)
    x, w = torch.randn(16, 64), torch.randn(24, 64)
    with torch.no_grad():
        y0 = mx.linear(x, w, mx_specs=sp)
    y1 = mx.linear(x, w, mx_specs=sp)                        # grad mode on, nothing requires grad
    wg = w.clone().requires_grad_()
    y2 = mx.linear(x, wg, mx_specs=sp)
    assert not y0.requires_grad and not y1.requires_grad and y2.requires_grad
    assert torch.equal(y0, y1) and torch.equal(y0, y2.detach())
    y2.sum().backward()
    assert wg.grad is not None and wg.grad.shape == w.shape
    a, b = torch.randn(2, 8, 64), torch.randn(2, 64, 8)
    with torch.no_grad():
        assert torch.equal(mx.bmm(a, b, mx_specs=sp), mx.bmm(a, b.clone().requires_grad_(), mx_specs=sp))
