"""MX configuration dictionary (`MxSpecs`) and its helpers.

Drop-in for the reference's mx/specs.py: same keys, defaults, derivation rules
and function names (MxSpecs :61, get_backwards_mx_specs :193, apply_mx_specs
:212, add_mx_args :234, finalize_mx_specs :279, get_mx_specs :329,
mx_assert_test :351).  The option table is one declarative list here.
"""
import argparse
import collections
import json
import os
import traceback

import torch

# MX_ASSERT=True makes `mx_specs is None` an error in every user-facing op
_ASSERT_MODE = os.environ.get("MX_ASSERT", "False")

_FMT_HELP = "MX elem format, one of {fp8_e5m2, fp8_e4m3, fp6_e3m2, fp6_e2m3, fp4_e2m1, int8, int4}"
# (key, default, help)
_OPTIONS = [
    ("scale_bits", 0, "Bits (sign + magnitude) to use for shared exponent/scale"),
    ("w_elem_format", None, "Weight " + _FMT_HELP),
    ("a_elem_format", None, "Activation " + _FMT_HELP),
    ("w_elem_format_bp", None, "Backpass weight " + _FMT_HELP),
    ("a_elem_format_bp", None, "Backpass stashed activation " + _FMT_HELP),
    ("a_elem_format_bp_ex", None, "Backpass act (grad) " + _FMT_HELP),
    ("a_elem_format_bp_os", None, "Backpass act (grad) " + _FMT_HELP),
    ("mx_flush_fp32_subnorms", False, "MX quantization flushes blocks with subnormal shared scale to zero"),
    ("shared_exp_method", "max", "Shared exponent calculation method. Options: max, none"),
    ("block_size", 0, "mx shared exponent block size"),
    ("bfloat", 0, "BfloatX format (8exp + sign + mantissa). Only one of bfloat or fp can be used"),
    ("fp", 0, "fpX format (5exp + sign + mantissa). Only one of bfloat or fp can be used"),
    ("bfloat_subnorms", True, "Bfloat/FP supports subnorms"),
    ("quantize_backprop", True, "Enable mx/bfloat quantization on backward pass"),
    ("round", "nearest", "Global rounding mode. Choices: nearest, floor"),
    ("round_m", "nearest", "ADAM optimizer m and v rounding mode"),
    ("round_weight", "nearest", "Weight bfloat rounding mode (W in WAGE)"),
    ("round_output", "nearest", "Activation bfloat rounding mode (A in WAGE)"),
    ("round_grad_weight", "nearest", "Weight update rounding mode (G in WAGE)"),
    ("round_grad_input", "nearest", "Error gradient rounding mode (E in WAGE)"),
    ("round_mx_output", "nearest", "Forward pass mx rounding mode"),
    ("round_mx_input_grad_input", "nearest", ""),
    ("round_mx_weight_grad_input", "nearest", ""),
    ("round_mx_grad_output_grad_input", "nearest", ""),
    ("round_mx_input_grad_weight", "nearest", ""),
    ("round_mx_grad_output_grad_weight", "nearest", ""),
    ("softmax_exp2", False, "Softmax uses 2^x instead of e^x"),
    ("vec_use_exp2", False, "Use 2^x to compute e^x"),
    ("vec_use_recip", False, "Use 1/x to compute division"),
    ("custom_cuda", False, "Enable custom CUDA kernels for quantization"),
]
_DEFAULTS = {k: d for k, d, _ in _OPTIONS}
_HELP = {k: h for k, _, h in _OPTIONS}

# key -> key it inherits from when unset (applied in this order)
_INHERIT = [
    ("w_elem_format_bp", "w_elem_format"), ("a_elem_format_bp", "a_elem_format"),
    ("a_elem_format_bp_os", "a_elem_format"), ("a_elem_format_bp_ex", "a_elem_format"),
    ("round_m", "round"), ("round_output", "round"), ("round_grad_weight", "round"),
    ("round_grad_input", "round"), ("round_weight", "round"), ("round_mx_output", "round"),
    ("round_mx_input_grad_input", "round_grad_input"),
    ("round_mx_weight_grad_input", "round_grad_input"),
    ("round_mx_grad_output_grad_input", "round_grad_input"),
    ("round_mx_input_grad_weight", "round_grad_input"),
    ("round_mx_grad_output_grad_weight", "round_grad_input"),
]
_QUANT_KEYS = ("w_elem_format", "a_elem_format", "w_elem_format_bp", "a_elem_format_bp",
               "a_elem_format_bp_os", "a_elem_format_bp_ex", "bfloat", "fp")


class MxSpecs(collections.UserDict):
    """Dictionary of quantization parameters; unknown keys are rejected.  Every change bumps `_version`,
    which lets apply_mx_specs / get_backwards_mx_specs reuse what they derived from an unchanged object
    (the layers call them on every forward)."""

    def __init__(self, *args, **kwargs):
        self._version = 0
        self._derived = {}
        super().__init__(*args, **kwargs)
        self.help_strings = dict(_HELP)
        for k, d in _DEFAULTS.items():
            self.data.setdefault(k, d)
        for k in self.data:
            assert k in _DEFAULTS, k

    def __setitem__(self, key, value):
        self._version += 1
        self.data[key] = value

    def __delitem__(self, key):
        self._version += 1
        del self.data[key]

    def copy(self):
        c = MxSpecs.__new__(MxSpecs)
        c._version, c._derived = 0, {}
        c.data = dict(self.data)
        c.help_strings = self.help_strings
        return c

    def _cached(self, what, make):
        """make() derived from this object, remembered while neither this object nor the result changes."""
        hit = self._derived.get(what)
        if hit is not None and hit[0] == self._version and hit[2] == hit[1]._version:
            return hit[1]
        out = make()
        self._derived[what] = (self._version, out, out._version)
        return out

    def safe_json(self, indent=None):
        return json.dumps(self.data, indent=indent,
                          default=lambda o: f"<<non-serializable: {type(o).__qualname__}>>")

    def __str__(self):
        return self.safe_json(indent=4)


def get_default_mx_specs():
    """Specs with every quantization switched off."""
    return MxSpecs()


def get_backwards_mx_specs(specs):
    """Copy of `specs` for the backward pass: all quantization off when
    quantize_backprop is False."""
    if isinstance(specs, MxSpecs):
        return specs._cached("backward", lambda: _backwards(specs))
    return _backwards(specs)


def _backwards(specs):
    b = specs.copy()
    if b["quantize_backprop"] == False:  # noqa: E712 (0 counts as False, as in the reference)
        for k in _QUANT_KEYS:
            b[k] = None if k.endswith("format") or "elem_format" in k else 0
        b["block_size"] = 0
    return b


def apply_mx_specs(mx_specs, default_mx_specs=None):
    """Overlay the non-None entries of mx_specs on the defaults -> MxSpecs."""
    if not default_mx_specs and isinstance(mx_specs, MxSpecs):
        return mx_specs._cached("applied", lambda: _overlay(mx_specs, get_default_mx_specs()))
    if not default_mx_specs:
        default_mx_specs = get_default_mx_specs()
    if not mx_specs:
        return default_mx_specs
    return _overlay(mx_specs, default_mx_specs)


def _overlay(mx_specs, default_mx_specs):
    for k in mx_specs:
        if mx_specs[k] != None:  # noqa: E711
            if k not in default_mx_specs:
                raise KeyError(f"Unknown key '{k}' passed to mx specs")
            default_mx_specs[k] = mx_specs[k]
    return default_mx_specs


def add_mx_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """One command-line option per spec: strings/ints default to None, False
    bools become --key, True bools become --no_key."""
    group = parser.add_argument_group("mx", "MX specs")
    group.add_argument("--mx_dir", type=str, default=None, help="Path to mx library")
    for k, v, h in _OPTIONS:
        h = h or "No help string"
        if "elem_format" in k:
            group.add_argument("--" + k, type=str, default=v, help=h)
        elif v is False:
            group.add_argument("--" + k, action="store_true", help=h)
        elif v is True:
            group.add_argument("--no_" + k, action="store_true", help=h)
        else:
            group.add_argument("--" + k, type=type(v), default=None, help=h)
    group.add_argument("--skip_early_exit", action="store_true", default=False,
                       help="Don't early exit if no quantization is specified")
    return parser


def finalize_mx_specs(specs, early_exit=True):
    """Fill dependent keys from their base keys; returns None when nothing is
    quantized (unless early_exit is False)."""
    if early_exit and not any(specs.get(k, 0) for k in _QUANT_KEYS):
        return None
    if specs.get("custom_cuda"):
        assert torch.cuda.is_available(), "'custom_cuda' is only supported on CUDA devices."
    for dst, src in _INHERIT:
        if (dst not in specs or specs[dst] is None) and src in specs:
            specs[dst] = specs[src]
    return apply_mx_specs(specs, get_default_mx_specs())


def get_mx_specs(parsed_args: argparse.Namespace):
    """Specs from the output of a parser built with add_mx_args."""
    parsed = {}
    for k, v, _ in _OPTIONS:
        if v is True:
            if hasattr(parsed_args, "no_" + k):
                parsed[k] = not getattr(parsed_args, "no_" + k)
        elif hasattr(parsed_args, k):
            parsed[k] = getattr(parsed_args, k)
    early_exit = not getattr(parsed_args, "skip_early_exit", False)
    return finalize_mx_specs(parsed, early_exit=early_exit)


def mx_assert_test(mx_specs):
    if _ASSERT_MODE == "True" and mx_specs is None:
        stack = traceback.extract_stack()
        f1, f2 = stack[-2], stack[-3]
        raise ValueError("MX assert test failed!\n"
                         f"mx_specs is None in function {f1.name}\n"
                         f"Called from {f2.filename}, line {f2.lineno}\n  {f2.line}")
