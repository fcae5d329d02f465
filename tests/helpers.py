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
