"""Shared helpers of the test-suite (input recipes and the canonical hash the
fixtures use)."""
import hashlib

import numpy as np


def canon_bytes(a):
    a = np.ascontiguousarray(a, np.float32).copy()
    nan = np.isnan(a)
    a[a == 0] = 0.0
    u = a.view(np.uint32)
    u[nan] = 0x7FC00000
    return u.tobytes()


def sha(a):
    return hashlib.sha256(canon_bytes(a)).hexdigest()


def all_encodings(e, m, encodes_infs=True):
    """Every value of an eXmY format, positives then negatives (zeros where the
    top exponent would encode Inf/NaN)."""
    n = 1 << (e + m)
    idx = np.arange(n)
    with np.errstate(over="ignore"):
        if e > 0:
            ef = idx >> m
            mant = (idx & ((1 << m) - 1)) / float(1 << m)
            bias = (1 << (e - 1)) - 1
            val = np.where(ef == 0, np.ldexp(mant, 1 - bias), np.ldexp(1.0 + mant, ef - bias))
            if encodes_infs:
                val = np.where(ef == (1 << e) - 1, 0.0, val)
            if e == 4 and m == 3:
                val = np.where(idx == n - 1, 0.0, val)
        else:
            val = idx / float(1 << (m - 1))
        return np.concatenate([val, -val]).astype(np.float32)


def bf16_bits(x):
    """float32 array (bf16-representable values) -> uint16 bit patterns."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_vals(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


def decode_container(codes, ebits, mbits):
    """Element codes as libmxq writes them -> float64 values (before scaling):
    e5m2 container for ebits == 5, e4m3 container for other float formats,
    two's complement with (mbits-2) fraction bits for fixed point."""
    c = codes.astype(np.int64)
    if ebits == 0:
        v = c & ((1 << mbits) - 1)
        v = np.where(v >= (1 << (mbits - 1)), v - (1 << mbits), v)
        return v / float(1 << (mbits - 2))
    E, M = (5, 2) if ebits == 5 else (4, 3)
    bias = (1 << (E - 1)) - 1
    s = np.where((c >> (E + M)) & 1, -1.0, 1.0)
    ef = (c >> M) & ((1 << E) - 1)
    m = c & ((1 << M) - 1)
    mag = np.where(ef == 0, np.ldexp(m.astype(np.float64), 1 - bias - M),
                   np.ldexp((m | (1 << M)).astype(np.float64), ef - bias - M))
    return s * mag


def dequant_packed(codes, scales, block, axis, ebits, mbits):
    """codes [.., n, ..] and E8M0 scales [.., nblk, ..] -> float32 values (NaN
    where the scale byte is 255)."""
    v = decode_container(codes, ebits, mbits)
    n = codes.shape[axis]
    se = np.repeat(scales.astype(np.int64), block, axis=axis)
    se = np.take(se, np.arange(n), axis=axis)
    out = np.ldexp(v, (se - 127).astype(np.int64))
    out = np.where(se == 255, np.nan, out)
    return out.astype(np.float32)
