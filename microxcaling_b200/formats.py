"""Element formats and rounding modes of the MX path.

Same names and values as the reference's mx/formats.py (RoundingMode :12-19,
ElemFormat :22-44, _get_format_params :61-125); the parameter table is computed
from a declarative description of each format instead of an if-chain.
"""
from enum import Enum, IntEnum

FP32_EXPONENT_BIAS = 127
FP32_MIN_NORMAL = 2.0 ** (-FP32_EXPONENT_BIAS + 1)


class RoundingMode(IntEnum):
    nearest = 0     # ties away from zero
    floor = 1       # toward zero
    even = 2        # ties to even

    @staticmethod
    def string_enums():
        return [m.name for m in RoundingMode]


class ElemFormat(Enum):
    int8 = 1
    int4 = 2
    int2 = 3
    fp8_e5m2 = 4
    fp8_e4m3 = 5
    fp6_e3m2 = 6
    fp6_e2m3 = 7
    fp4 = 8
    fp4_e2m1 = 8
    float16 = 9
    fp16 = 9
    bfloat16 = 10
    bf16 = 10

    @staticmethod
    def from_str(s):
        assert s is not None, "String elem_format == None"
        s = s.lower()
        if hasattr(ElemFormat, s):
            return getattr(ElemFormat, s)
        raise Exception("Undefined elem format", s)


def _get_min_norm(ebits):
    """Smallest normal magnitude of a float format with `ebits` exponent bits."""
    return 0 if ebits == 0 else 2.0 ** (2 - 2 ** (ebits - 1))


def _get_max_norm(ebits, mbits):
    """Largest normal magnitude of a float format whose top exponent is
    reserved for Inf/NaN (mbits counts sign and implicit one)."""
    assert ebits >= 5, "invalid for floats that don't define NaN"
    emax = 2 ** (ebits - 1) - 1
    return 2.0 ** emax * float(2 ** (mbits - 1) - 1) / 2 ** (mbits - 2)


# name -> (ebits, mbits incl. sign and implicit one, top exponent usable for normals?)
_LAYOUT = {
    ElemFormat.int8: (0, 8, None), ElemFormat.int4: (0, 4, None), ElemFormat.int2: (0, 2, None),
    ElemFormat.fp8_e5m2: (5, 4, False), ElemFormat.fp8_e4m3: (4, 5, True),
    ElemFormat.fp6_e3m2: (3, 4, True), ElemFormat.fp6_e2m3: (2, 5, True),
    ElemFormat.fp4: (2, 3, True), ElemFormat.float16: (5, 12, False),
    ElemFormat.bfloat16: (8, 9, False),
}
_FORMAT_CACHE = {}


def _get_format_params(fmt):
    """-> (ebits, mbits, emax, max_norm, min_norm) for an ElemFormat or its name."""
    if type(fmt) is str:
        fmt = ElemFormat.from_str(fmt)
    hit = _FORMAT_CACHE.get(fmt)
    if hit is not None:
        return hit
    if fmt not in _LAYOUT:
        raise Exception("Unknown element format %s" % fmt)
    ebits, mbits, top_is_normal = _LAYOUT[fmt]
    if ebits == 0:
        emax = 0
    else:
        emax = 2 ** (ebits - 1) - (0 if top_is_normal else 1)
    if fmt == ElemFormat.fp8_e4m3:
        max_norm = 2 ** emax * 1.75          # S.1111.111 is NaN, so 448 not 480
    else:
        max_norm = 2 ** emax * float(2 ** (mbits - 1) - 1) / 2 ** (mbits - 2)
    out = (ebits, mbits, emax, max_norm, _get_min_norm(ebits))
    _FORMAT_CACHE[fmt] = out
    return out
