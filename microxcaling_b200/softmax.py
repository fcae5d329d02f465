"""bfloat-emulated softmax (reference: mx/softmax.py:18-124): every step of
max-subtract, exp (or exp2), sum and divide is rounded to the vector format."""
import torch
import torch.nn.functional as F

from ._autograd import call
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test
from .vector_ops import fused_bf16_ok, vec_div, vec_exp, vec_exp2, vec_mul, vec_quantize, vec_reduce_sum, vec_sub

f_softmax = F.softmax
LN_2_BF16 = 0.69140625
_SOFTMAX_FUSED_MAX_COLS = 2048      # row length the one-warp-per-row kernel keeps in registers


def _packable_for_matmul(input, mx_specs):
    """Batched score matrices whose probabilities will be the left operand of an MX product
    (a_elem_format with a one-byte container, block 32 along the softmax axis): worth writing the
    packed operand in the same pass.  Large inputs only (the fused kernel loads a 128 KB table per SM)."""
    from ._mxgemm import _fmt
    from .formats import _get_format_params
    f = mx_specs["a_elem_format"]
    if f is None or input.dim() < 3 or input.shape[-1] % 32 != 0 or input.shape[-2] < 32:
        return None
    if mx_specs["block_size"] != 32 or mx_specs["shared_exp_method"] != "max" or mx_specs.get("softmax_exp2", False):
        return None
    if mx_specs["round_mx_output"] not in ("nearest", "floor", "even") or input.numel() < (1 << 22):
        return None
    ebits, mbits, _, max_norm, _ = _get_format_params(_fmt(f))
    if ebits == 0 or mbits > 5:
        return None
    return ebits, mbits, max_norm


class SoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, dim=None, mx_specs=None, name=None):
        dim = dim + input.dim() if dim < 0 else dim
        ctx.dim = dim
        rnd = mx_specs["round"]
        if dim == input.dim() - 1 and fused_bf16_ok(mx_specs, input) and input.shape[-1] % 8 == 0 \
                and 0 < input.shape[-1] <= _SOFTMAX_FUSED_MAX_COLS:
            from . import _backend
            pk = _packable_for_matmul(input, mx_specs)
            if pk is not None:
                # probabilities and their MX packing (the left operand of the product that follows) in one pass
                from ._mxgemm import _MODE, _fmt
                from .packed import PackedMX, attach_packed
                x = input.contiguous()
                R, K = x.shape[-2], x.shape[-1]
                sb = mx_specs["scale_bits"] or 8
                out, codes, scales = _backend.softmax_quantize_mx(x, sb, pk[0], pk[1], pk[2],
                                                                  mx_specs["mx_flush_fp32_subnorms"],
                                                                  _MODE[mx_specs["round_mx_output"]], rows_per_batch=R)
                batch = x.numel() // (R * K)
                ctx.packed = (PackedMX(codes.reshape(batch, R, K), scales, 1 if pk[0] == 5 else 0, pk[0], pk[1], sb,
                                       batch, R, K), _fmt(mx_specs["a_elem_format"]), mx_specs["round_mx_output"])
            else:
                out = _backend.softmax_bf16(input.contiguous(), mx_specs.get("softmax_exp2", False))
        else:
            x = vec_quantize(input, mx_specs=mx_specs)
            x = vec_sub(x, x.max(dim, keepdim=True)[0], mx_specs=mx_specs, round=rnd)
            e = (vec_exp2 if mx_specs.get("softmax_exp2", False) else vec_exp)(x, mx_specs=mx_specs, round=rnd)
            s = vec_reduce_sum(e, dim, keepdim=True, mx_specs=mx_specs, round=rnd)
            out = vec_div(e, s, mx_specs=mx_specs, round=rnd)
        ctx.save_for_backward(out)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        if getattr(ctx, "packed", None) is not None:
            _PENDING.append((out, ctx.packed, mx_specs))
            ctx.packed = None
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (out,) = ctx.saved_tensors
        sp = ctx.mx_specs
        rnd = sp["round"]
        g = vec_quantize(grad_output, mx_specs=sp, round=rnd)
        dot = vec_reduce_sum(vec_mul(g, out, mx_specs=sp, round=rnd), ctx.dim, keepdim=True, mx_specs=sp, round=rnd)
        gi = vec_mul(out, vec_sub(g, dot, mx_specs=sp, round=rnd), mx_specs=sp, round=rnd)
        if sp.get("softmax_exp2", False):
            gi = vec_mul(gi, LN_2_BF16, mx_specs=sp, round=rnd)
        return (gi, None, None, None)


# forward() cannot decorate the tensor autograd hands back to the caller; it leaves the packing here and
# _apply attaches it to that tensor
_PENDING = []


def _apply(input, dim, mx_specs, name):
    del _PENDING[:]
    out = call(SoftmaxFunction, input, dim, mx_specs, name)
    if _PENDING:
        from .packed import attach_packed
        made, (packed, fmt, rnd), sp = _PENDING.pop()
        if made.data_ptr() == out.data_ptr():
            attach_packed(out, packed, fmt, rnd, sp)
    return out


def softmax(input, dim=-1, mx_specs=None, name=None):
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_softmax(input, dim=dim)
    return _apply(input, dim, apply_mx_specs(mx_specs), name)


class Softmax(torch.nn.Softmax):
    def __init__(self, dim=None, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(dim)

    def apply_mx_specs(self, mx_specs):
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def forward(self, input):
        if self.mx_none:
            return super().forward(input)
        return _apply(input, self.dim, self.mx_specs, self.name)
