"""Pins the CPU oracle: it must reproduce (a) every call the reference's own
test-suite makes on its pure-PyTorch path, which the reference asserts equal to
its known-answer vectors, (b) a seeded sweep recorded from the reference, and
(c) the reference's C++ math compiled in place, where that library exists."""
import numpy as np
import pytest

import oracle
from helpers import all_encodings, sha, bf16_bits, bf16_vals


def _input(rec, z, i):
    if "recipe" in rec:
        e, m, inf = rec["recipe"]
        return all_encodings(e, m, bool(inf)).reshape(rec["shape"])
    return z["x%d" % i]


def test_recorded_reference_calls(golden_recorded):
    meta, z = golden_recorded
    assert len(meta) > 500
    bad = []
    for i, rec in enumerate(meta):
        x = _input(rec, z, i)
        p = rec["params"]
        if rec["kind"] == "mx":
            if x.ndim == 0:
                continue
            y = oracle.quantize_mx(x, p["fmt"], axis=p["axis"], block=p["block"],
                                   scale_bits=p["scale_bits"], round=p["round"], flush=p["flush"])
        else:
            y = oracle.quantize_elemwise(x, p["bits"], p["exp_bits"], p["max_norm"], round=p["round"],
                                         saturate=p["saturate"], allow_denorm=p["allow_denorm"])
        ok = (sha(y) == rec["sha"]) if "sha" in rec else oracle.same_values(y, z["y%d" % i])
        if not ok:
            bad.append((i, rec["kind"], p))
    assert not bad, bad[:5]


def test_seeded_sweep(golden_sweep):
    meta, z = golden_sweep
    bad = []
    for rec in meta:
        x = z["in_" + rec["in"]]
        if rec["kind"] == "mx":
            y = oracle.quantize_mx(x, rec["fmt"], axis=rec["axis"], block=rec["block"],
                                   scale_bits=rec["scale_bits"], round=rec["round"], flush=rec["flush"])
        else:
            if rec["spec"] == "bfloat":
                bits, eb = rec["val"] - 7, 8
                mn = 2.0 ** 127 * (2 ** (bits - 1) - 1) / 2 ** (bits - 2)
            else:
                bits, eb = rec["val"] - 4, 5
                mn = 2.0 ** 15 * (2 ** (bits - 1) - 1) / 2 ** (bits - 2)
            y = oracle.quantize_elemwise(x, bits, eb, mn, round=rec["round"], allow_denorm=rec["subnorms"])
        if sha(y) != rec["sha"]:
            bad.append(rec)
    assert not bad, (len(bad), bad[:5])


def test_bf16_storage_equals_fp32_container(golden_sweep):
    """bf16 storage in, bf16 storage out must equal the fp32-container result
    (the native reference converts to fp32 first, mx/cpp/mx.cuh:72)."""
    _, z = golden_sweep
    x = z["in_studentt_outliers_96x128_bf16vals"]
    for fmt in ("fp8_e4m3", "fp6_e2m3", "fp4_e2m1", "int8"):
        for axis in (0, 1):
            y32 = oracle.quantize_mx(x, fmt, axis=axis)
            y16 = oracle.quantize_mx(bf16_bits(x), fmt, axis=axis)
            assert oracle.same_values(bf16_vals(y16), y32)


@pytest.mark.skipif(oracle.ref() is None, reason="compiled reference not built here")
def test_against_compiled_reference():
    x = all_encodings(8, 9)
    for fmt in ("fp8_e5m2", "fp8_e4m3", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8", "int4"):
        for rnd in ("nearest", "floor", "even"):
            for sb in (8, 5):
                for blk in (8, 32, 64):
                    a = oracle.quantize_mx(x, fmt, block=blk, scale_bits=sb, round=rnd)
                    b = oracle.ref_quantize_mx_f32(x, fmt, block=blk, scale_bits=sb, round=rnd)
                    assert oracle.same_values(a, b), (fmt, rnd, sb, blk)
    rng = np.random.default_rng(5)
    r = (rng.standard_normal(1 << 16) * np.exp2(rng.integers(-40, 40, 1 << 16))).astype(np.float32)
    for bits, eb, mn in ((9, 8, 3.3895313892515355e38), (5, 8, 2.0 ** 127 * 1.75), (12, 5, 65504.0),
                         (4, 5, 57344.0), (5, 4, 448.0), (8, 0, 1.984375)):
        for rnd in ("nearest", "floor", "even"):
            for sat in (False, True):
                for den in (False, True):
                    for xin in (x, r):
                        a = oracle.quantize_elemwise(xin, bits, eb, mn, rnd, sat, den)
                        b = oracle.ref_quantize_elemwise_f32(xin, bits, eb, mn, rnd, sat, den)
                        assert oracle.same_values(a, b), (bits, eb, rnd, sat, den)


def test_format_table():
    """(ebits, mbits, max_norm) of every element format: mx/tests/test_formats.py:12-95."""
    expect = {"int8": (0, 8, 1.984375), "int4": (0, 4, 1.75), "int2": (0, 2, 1.0),
              "fp8_e5m2": (5, 4, 57344.0), "fp8_e4m3": (4, 5, 448.0), "fp6_e3m2": (3, 4, 28.0),
              "fp6_e2m3": (2, 5, 7.5), "fp4_e2m1": (2, 3, 6.0), "fp16": (5, 12, 65504.0)}
    for k, v in expect.items():
        assert oracle.FORMATS[k] == v


def test_packed_roundtrip():
    """codes + E8M0 scales decode back to the dequantized output."""
    rng = np.random.default_rng(7)
    x = (rng.standard_t(3, (64, 96)) * 3).astype(np.float32)
    L = oracle.lib()
    for fmt in ("fp8_e4m3", "fp8_e5m2", "fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8"):
        eb, mb, _ = oracle.FORMATS[fmt]
        for axis in (0, 1):
            y, codes, scales = oracle.quantize_mx(x, fmt, axis=axis, want_packed=True)
            pre, n, post = oracle._split(x.shape, axis)
            c3 = codes.reshape(pre, n, post)
            y3 = y.reshape(pre, n, post)
            for (i, k, j) in [(0, 0, 0), (pre - 1, n - 1, post - 1), (0, n // 2, post // 2), (0, 33, 0)]:
                d = L.mxo_decode_elem(int(c3[i, k, j]), eb, mb, int(scales[i, k // 32, j]))
                assert d == y3[i, k, j], (fmt, axis, i, k, j)
