"""Packed MX operands: element codes + E8M0 block scales, as the block-scaled
GEMM reads them, with a file format.

The reference never stores an MX tensor: it keeps fake-quantized fp32 / bf16
values and re-quantizes a layer's weight on every forward call
(mx/linear.py:40-47, 62-83); `Linear.prequantize_weights` (mx/linear.py:246-274)
only rounds the weights to bfloat16 once.  Here a quantized operand can be kept,
handed to `mx_gemm` in place of the tensor it was made from, and written to disk.

File layout (little endian), version 1:

    offset  size  field
    0       4     magic "MXQP"
    4       4     version (1)
    8       4     container: 0 = fp8 e4m3 codes, 1 = fp8 e5m2 codes
    12      4     elem_ebits      16  4  elem_mbits (sign + significand incl. implicit one)
    20      4     block size (32) 24  4  scale_bits
    28      4     reserved (0)
    32      8     batch           40  8  rows          48  8  K (contraction length, multiple of 32)
    56      8     codes_bytes  = batch * rows * K
    64      8     scales_bytes = batch * ceil(rows/128) * ceil(K/128) * 512
    72      56    reserved (0), header is 128 bytes
    128     codes_bytes   one code byte per element, [batch, rows, K], K contiguous
    ...     scales_bytes  E8M0 bytes in 512-byte chunks per (128 rows x 128 K):
                          byte ((b*ceil(rows/128) + r/128)*ceil(K/128) + k/4)*512
                               + (r%32)*16 + ((r%128)/32)*4 + k%4 for row r, 32-block k
"""
import struct

import torch

from .formats import _get_format_params

_MAGIC = b"MXQP"
_HEADER = 128
_MODE = {"nearest": 0, "floor": 1, "even": 2}


class PackedMX:
    """An MX-quantized [batch, rows, K] operand, blocks of 32 along K."""

    __slots__ = ("codes", "scales", "container", "ebits", "mbits", "scale_bits", "batch", "rows", "K")

    def __init__(self, codes, scales, container, ebits, mbits, scale_bits, batch, rows, K):
        self.codes, self.scales = codes, scales
        self.container, self.ebits, self.mbits, self.scale_bits = int(container), int(ebits), int(mbits), int(scale_bits)
        self.batch, self.rows, self.K = int(batch), int(rows), int(K)

    @property
    def device(self):
        return self.codes.device

    def to(self, device):
        return PackedMX(self.codes.to(device), self.scales.to(device), self.container, self.ebits, self.mbits,
                        self.scale_bits, self.batch, self.rows, self.K)

    @staticmethod
    def scales_bytes(batch, rows, K):
        return batch * ((rows + 127) // 128) * ((K + 127) // 128) * 512

    # ------------------------------------------------------------------ quantize
    @classmethod
    def quantize(cls, x, elem_format, mx_specs=None, round="nearest", contraction_last=True, scale_bits=None,
                 flush=None):
        """MX-quantize CUDA tensor x ([..., rows, K], or [..., K, rows] with contraction_last=False) in
        blocks of 32 along K into a packed operand; leading dimensions become the batch."""
        from . import _backend as be
        ebits, mbits, _, max_norm, _ = _get_format_params(elem_format)
        if ebits == 0 or mbits > 5:
            raise ValueError("format %s has no one-byte float container" % (elem_format,))
        if scale_bits is None:
            scale_bits = (mx_specs["scale_bits"] if mx_specs is not None else 0) or 8
        if flush is None:
            flush = bool(mx_specs["mx_flush_fp32_subnorms"]) if mx_specs is not None else False
        x = x.contiguous()
        if x.shape[-1 if contraction_last else -2] % 32:
            raise ValueError("contraction length must be a multiple of 32")
        if contraction_last:
            R, K = x.shape[-2], x.shape[-1]
            _, codes, scales = be.quantize_mx(x.reshape(-1, K), scale_bits, ebits, mbits, max_norm, 32, 1, flush,
                                              _MODE[round], want_dq=False, want_codes=True, gemm_layout=True,
                                              rows_per_batch=R)
        else:
            K, R = x.shape[-2], x.shape[-1]
            _, codes, scales = be.quantize_mx(x.reshape(-1, K, R), scale_bits, ebits, mbits, max_norm, 32, 1, flush,
                                              _MODE[round], want_dq=False, want_codes=True, transposed=True,
                                              gemm_layout=True)
        batch = x.numel() // (R * K) if R * K else 0
        return cls(codes.reshape(batch, R, -1), scales, 1 if ebits == 5 else 0, ebits, mbits, scale_bits, batch, R, K)

    # ------------------------------------------------------------------ values
    def dequantize(self, dtype=torch.float32):
        """The fake-quantized values [batch, rows, K] this operand stands for (torch ops, any device)."""
        c = self.codes.reshape(self.batch, self.rows, self.K).to(torch.int32)
        E, M = (5, 2) if self.container == 1 else (4, 3)
        bias = (1 << (E - 1)) - 1
        sign = torch.where(((c >> (E + M)) & 1) == 1, -1.0, 1.0).to(torch.float64)
        ef = (c >> M) & ((1 << E) - 1)
        m = c & ((1 << M) - 1)
        mag = torch.where(ef == 0, torch.ldexp(m.to(torch.float64), torch.full_like(ef, 1 - bias - M)),
                          torch.ldexp((m | (1 << M)).to(torch.float64), ef - bias - M))
        s = self.scale_bytes_rowmajor().to(torch.int32)                      # [batch, rows, K/32]
        se = s.repeat_interleave(32, dim=-1)[..., :self.K]
        v = torch.ldexp(sign * mag, se - 127)
        v = torch.where(se == 255, torch.full_like(v, float("nan")), v)
        return v.to(dtype)

    def scale_bytes_rowmajor(self):
        """E8M0 bytes as a plain [batch, rows, K/32] tensor (gathered out of the chunk layout)."""
        nb = self.K // 32
        dev = self.scales.device
        r = torch.arange(self.rows, device=dev).view(1, -1, 1)
        k = torch.arange(nb, device=dev).view(1, 1, -1)
        b = torch.arange(self.batch, device=dev).view(-1, 1, 1)
        r128, kb4 = (self.rows + 127) // 128, (nb + 3) // 4
        idx = ((b * r128 + r // 128) * kb4 + k // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + k % 4
        return self.scales.view(-1)[idx.reshape(-1)].reshape(self.batch, self.rows, nb)

    # ------------------------------------------------------------------ file format
    def save(self, path):
        codes = self.codes.detach().contiguous().cpu().reshape(-1)
        scales = self.scales.detach().contiguous().cpu().reshape(-1)
        want_c, want_s = self.batch * self.rows * self.K, self.scales_bytes(self.batch, self.rows, self.K)
        if codes.numel() != want_c or scales.numel() != want_s:
            raise ValueError("operand buffers do not have the documented sizes")
        hdr = _MAGIC + struct.pack("<7i5q", 1, self.container, self.ebits, self.mbits, 32, self.scale_bits, 0,
                                   self.batch, self.rows, self.K, want_c, want_s)
        hdr += b"\0" * (_HEADER - len(hdr))
        with open(path, "wb") as f:
            f.write(hdr)
            f.write(codes.numpy().tobytes())
            f.write(scales.numpy().tobytes())

    @classmethod
    def load(cls, path, device="cpu"):
        with open(path, "rb") as f:
            hdr = f.read(_HEADER)
            if len(hdr) != _HEADER or hdr[:4] != _MAGIC:
                raise ValueError("%s is not a packed MX operand file" % path)
            version, container, ebits, mbits, block, scale_bits, _r, batch, rows, K, nc, ns = \
                struct.unpack("<7i5q", hdr[4:4 + 28 + 40])
            if version != 1 or block != 32 or container not in (0, 1):
                raise ValueError("unsupported packed MX file (version %d, block %d)" % (version, block))
            if nc != batch * rows * K or ns != cls.scales_bytes(batch, rows, K):
                raise ValueError("packed MX file header is inconsistent")
            body = f.read(nc + ns)
            if len(body) != nc + ns:
                raise ValueError("packed MX file is truncated")
        buf = torch.frombuffer(bytearray(body), dtype=torch.uint8)
        codes = buf[:nc].reshape(batch, rows, K).to(device)
        scales = buf[nc:].clone().to(device)
        return cls(codes, scales, container, ebits, mbits, scale_bits, batch, rows, K)


# ---------------------------------------------------------------------------------------------
# A tensor can carry the packed form of its own values: the fused softmax writes the probabilities
# and their MX packing in one pass, and the product that consumes the probabilities picks the
# packing up instead of quantizing them again.  The note is only honoured while the tensor is
# unchanged (same storage pointer, same version counter) and for the same format and rounding.
# ---------------------------------------------------------------------------------------------
def _note_key(t, fmt, round, specs):
    return (t.data_ptr(), t._version, tuple(t.shape), str(fmt), round, specs["scale_bits"] or 8,
            bool(specs["mx_flush_fp32_subnorms"]))


def attach_packed(t, packed, fmt, round, specs):
    """Remember on tensor `t` that `packed` is MX(t) along its last axis with (fmt, round)."""
    t._mx_packed = (_note_key(t, fmt, round, specs), packed)
    return t


def packed_note(t, fmt, round, specs):
    """The PackedMX attached to `t` for (fmt, round), if `t` still holds the values it was made from."""
    note = getattr(t, "_mx_packed", None)
    if note is None or note[0] != _note_key(t, fmt, round, specs):
        return None
    return note[1]
