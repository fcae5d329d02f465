"""MX Linear: drop-in for the reference's mx/linear.py (LinearFunction :19-200,
linear :203, Linear :221-291).

Forward  y = Q(Q(MX(x) MX(w)^T) + b): operands MX-quantized along in_features.
Backward grad_w = MX(g)^T MX(x) with both blocked along the token axis,
         grad_x = MX(g) MX(w) with both blocked along out_features.
Each product runs through `_mxgemm.mx_gemm` (packed operands + block-scaled
tensor-core GEMM with the output rounding fused, where the formats allow it).
"""
import torch
import torch.nn.functional as F

from ._autograd import call
from ._mxgemm import mx_gemm
from .elemwise_ops import quantize_elemwise_op
from .specs import apply_mx_specs, get_backwards_mx_specs, mx_assert_test

f_linear = F.linear
torch_matmul = torch.matmul
_MODE = {"nearest": 0, "floor": 1, "even": 2}


def _cfmt(fmt, rnd):
    """ElemFormatC of an element format name and MX rounding mode, or None when the format has no
    one-byte float container or the mode is not a kernel mode."""
    from . import _backend
    from ._mxgemm import _fmt
    from .formats import _get_format_params
    if fmt is None or rnd not in _MODE:
        return None
    ebits, mbits, _, max_norm, _ = _get_format_params(_fmt(fmt))
    if ebits == 0 or mbits > 5:
        return None
    return _backend.ElemFormatC(ebits, mbits, max_norm, _MODE[rnd])


def _one_call_ok(a, b, sp, out_round):
    """Both tensors CUDA, contiguous-izable, same kernel dtype; block 32, max-exponent scales, bfloat output."""
    if not (a.is_cuda and b.is_cuda) or a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float32):
        return False
    if sp["block_size"] != 32 or sp["shared_exp_method"] != "max" or sp["fp"] > 0 or 0 < sp["bfloat"] < 10:
        return False
    return out_round in _MODE and a.numel() > 0 and b.numel() > 0


class LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias=None, mx_specs=None, prequantized_weights=False, name=None,
                packed_weight=None):
        bf_in = quantize_elemwise_op(input, mx_specs=mx_specs, round=mx_specs["round_output"])
        if prequantized_weights:
            assert weight.dtype == torch.bfloat16
            bf_weight = weight
        else:
            bf_weight = quantize_elemwise_op(weight, mx_specs=mx_specs, round=mx_specs["round_weight"])
        ctx.has_bias = bias is not None
        bf_bias = None
        if bias is not None:
            if prequantized_weights:
                assert bias.dtype == torch.bfloat16
                bf_bias = bias
            else:
                bf_bias = quantize_elemwise_op(bias, mx_specs=mx_specs, round=mx_specs["round_weight"])
        if mx_specs["quantize_backprop"]:
            ctx.save_for_backward(bf_in, bf_weight)
        else:
            ctx.save_for_backward(input, weight)
        if bf_weight.dtype != bf_in.dtype:
            bf_weight = bf_weight.to(bf_in.dtype)
        K = bf_in.shape[-1]
        fa = _cfmt(mx_specs["a_elem_format"], mx_specs["round_mx_output"])
        fw = _cfmt(mx_specs["w_elem_format"], mx_specs["round_mx_output"])
        if packed_weight is None and fa is not None and fw is not None and K % 32 == 0 and bf_in.dim() >= 2 and \
                _one_call_ok(bf_in, bf_weight, mx_specs, mx_specs["round_output"]):
            # quantize both operands and multiply in one library call
            from . import _backend
            y = _backend.linear_fwd_train(bf_in.reshape(-1, K).contiguous(), bf_weight.contiguous(), fa, fw,
                                          mx_specs["scale_bits"] or 8, mx_specs["mx_flush_fp32_subnorms"], bf_in.dtype,
                                          mx_specs["bfloat"] if mx_specs["bfloat"] >= 10 else 0,
                                          _MODE[mx_specs["round_output"]], bf_bias)
            ctx.mx_specs = get_backwards_mx_specs(mx_specs)
            ctx.prequantized_weights = prequantized_weights
            ctx.name = name
            return y.reshape(*bf_in.shape[:-1], weight.shape[0])
        output = mx_gemm(bf_in, bf_weight, mx_specs["a_elem_format"], mx_specs["w_elem_format"], mx_specs,
                         mx_specs["round_mx_output"], mx_specs["round_mx_output"], mx_specs["round_output"],
                         bias=bf_bias, trans2=True, in2_packed=packed_weight)
        ctx.mx_specs = get_backwards_mx_specs(mx_specs)
        ctx.prequantized_weights = prequantized_weights
        ctx.name = name
        return output

    @staticmethod
    def backward(ctx, grad_output):
        assert ctx.prequantized_weights is False, "Cannot use prequantized weights when training!"
        input, weight = ctx.saved_tensors
        sp = ctx.mx_specs
        out_dim, in_dim = weight.shape
        grad_output = quantize_elemwise_op(grad_output, mx_specs=sp, round=sp["round_grad_input"])

        # both gradient products in one library call where the formats and shapes allow it
        flat_ok = input.dim() == 2 or (input.dim() > 2 and sp["block_size"] and input.shape[-2] % sp["block_size"] == 0)
        M = grad_output.numel() // out_dim if out_dim else 0
        f_gw = (_cfmt(sp["a_elem_format_bp_ex"], sp["round_mx_grad_output_grad_weight"]),
                _cfmt(sp["a_elem_format_bp"], sp["round_mx_input_grad_weight"]))
        f_gi = (_cfmt(sp["a_elem_format_bp_os"], sp["round_mx_grad_output_grad_input"]),
                _cfmt(sp["w_elem_format_bp"], sp["round_mx_weight_grad_input"]))
        if flat_ok and None not in f_gw and None not in f_gi and M % 32 == 0 and out_dim % 32 == 0 and in_dim % 4 == 0 \
                and sp["round_grad_input"] in _MODE and sp["round_grad_weight"] in _MODE \
                and _one_call_ok(grad_output, input, sp, sp["round_grad_input"]) and weight.is_cuda:
            from . import _backend
            w = weight if weight.dtype == grad_output.dtype else weight.to(grad_output.dtype)
            gx, gw = _backend.linear_bwd(grad_output.reshape(M, out_dim).contiguous(), input.reshape(M, in_dim).contiguous(),
                                         w.contiguous(), f_gw[0], f_gw[1], f_gi[0], f_gi[1], sp["scale_bits"] or 8,
                                         sp["mx_flush_fp32_subnorms"], grad_output.dtype,
                                         sp["bfloat"] if sp["bfloat"] >= 10 else 0, _MODE[sp["round_grad_input"]],
                                         _MODE[sp["round_grad_weight"]], want_gx=ctx.needs_input_grad[0],
                                         want_gw=ctx.needs_input_grad[1])
            grad_bias = None
            if ctx.has_bias:
                grad_bias = quantize_elemwise_op(grad_output.reshape(-1, out_dim).sum(0), mx_specs=sp,
                                                 round=sp["round_grad_weight"])
            return (gx.reshape(input.shape) if gx is not None else None, gw, grad_bias, None, None, None, None)

        # grad_weight [out, in] = g^T x, blocks along the token axis.  A 3-D input
        # blocks along its own sequence axis; that equals blocking the flattened
        # token axis only when the sequence length is a multiple of the block.
        if input.dim() > 2 and sp["block_size"] and input.shape[-2] % sp["block_size"] == 0:
            g2, x2 = grad_output.reshape(-1, out_dim), input.reshape(-1, in_dim)
        elif input.dim() <= 2:
            g2, x2 = grad_output, input
        else:
            g2 = x2 = None
        if g2 is not None:
            grad_weight = mx_gemm(g2, x2, sp["a_elem_format_bp_ex"], sp["a_elem_format_bp"], sp,
                                  sp["round_mx_grad_output_grad_weight"], sp["round_mx_input_grad_weight"],
                                  sp["round_grad_weight"], trans1=True)
        else:
            from .mx_ops import quantize_mx_op
            qg = quantize_mx_op(grad_output, sp, elem_format=sp["a_elem_format_bp_ex"], axes=[-2],
                                round=sp["round_mx_grad_output_grad_weight"]).reshape(-1, out_dim)
            qx = quantize_mx_op(input, sp, elem_format=sp["a_elem_format_bp"], axes=[-2],
                                round=sp["round_mx_input_grad_weight"]).reshape(-1, in_dim)
            grad_weight = quantize_elemwise_op(torch_matmul(qg.transpose(0, 1), qx), mx_specs=sp,
                                               round=sp["round_grad_weight"])

        # grad_input [..., in] = g w, blocks along out_features
        grad_input = mx_gemm(grad_output, weight.to(grad_output.dtype), sp["a_elem_format_bp_os"],
                             sp["w_elem_format_bp"], sp, sp["round_mx_grad_output_grad_input"],
                             sp["round_mx_weight_grad_input"], sp["round_grad_input"])

        grad_bias = None
        if ctx.has_bias:
            grad_bias = quantize_elemwise_op(grad_output.reshape(-1, out_dim).sum(0), mx_specs=sp,
                                             round=sp["round_grad_weight"])
        return (grad_input, grad_weight, grad_bias, None, None, None, None)


def linear(input, weight, bias=None, mx_specs=None, prequantized_weights=False, name=None, packed_weight=None):
    """`packed_weight`: a PackedMX of `weight` (w_elem_format, round_mx_output, blocks along in_features) made
    once by the caller; the weight is then not quantized again in this call (inference only)."""
    mx_assert_test(mx_specs)
    if mx_specs is None:
        return f_linear(input, weight, bias=bias)
    mx_specs = apply_mx_specs(mx_specs)
    return call(LinearFunction, input, weight, bias, mx_specs, prequantized_weights, name, packed_weight)


class Linear(torch.nn.Linear):
    def __init__(self, in_features, out_features, bias=True, mx_specs=None, name=None):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.name = name
        self.prequantized_weights = False
        self._packed = None                      # (key, PackedMX) of the frozen weight, see prequantize_weights
        self.mx_specs = apply_mx_specs(mx_specs)
        super().__init__(in_features, out_features, bias)

    def apply_mx_specs(self, mx_specs):
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)

    def append_name(self, postfix):
        self.name += postfix

    def packed_weight(self):
        """The weight as a packed MX operand (w_elem_format, blocks of 32 along in_features), made on
        first use after prequantize_weights() and kept while the parameter is the same storage at the
        same version.  Writes that bypass the version counter (`weight.data.mul_()`) are not seen:
        call prequantize_weights() again after such an update.  None when the tensor-core path does
        not apply (CPU weights, fixed-point formats, block size other than 32)."""
        from ._mxgemm import _fast_ok, _fmt, _pack
        sp, w = self.mx_specs, self.weight
        if not (w.is_cuda and _fast_ok(w, w, _fmt(sp["w_elem_format"]), _fmt(sp["w_elem_format"]), sp,
                                       self.in_features, sp["round_mx_output"], sp["round_mx_output"],
                                       sp["round_output"])):
            return None
        key = (w.data_ptr(), w._version, w.dtype, str(sp["w_elem_format"]), sp["round_mx_output"], sp["scale_bits"])
        if self._packed is None or self._packed[0] != key:
            self._packed = (key, _pack(w.detach(), _fmt(sp["w_elem_format"]), sp, sp["round_mx_output"], True))
        return self._packed[1]

    def prequantize_weights(self):
        """Store weight and bias as bfloat16 once (inference only); the forward pass then also keeps
        the MX-packed weight instead of quantizing it in every call."""
        if self.mx_none:
            return
        assert self.mx_specs["round"] == "even", "Bfloat round should be 'even' for prequantizing weights."
        assert torch.cuda.is_bf16_supported(), "Current device does not support bfloat16"
        assert self.mx_specs["bfloat_subnorms"] is True, \
            "Bfloat_subnorms should be set to True for prequantizing weights."
        assert self.mx_specs["bfloat"] == 16, "Only Bfloat16 is supported for prequantizing weights."
        with torch.no_grad():
            self.weight.data = quantize_elemwise_op(self.weight.data, mx_specs=self.mx_specs,
                                                    round=self.mx_specs["round_weight"]).to(torch.bfloat16)
            if self.bias is not None:
                self.bias.data = quantize_elemwise_op(self.bias.data, mx_specs=self.mx_specs,
                                                      round=self.mx_specs["round_weight"]).to(torch.bfloat16)
        self.prequantized_weights = True
        self._packed = None

    def forward(self, inputs):
        if self.mx_none:
            return super().forward(inputs)
        if self.prequantized_weights:
            assert self.training is False, "Cannot use prequantized weights when training!"
        packed = self.packed_weight() if self.prequantized_weights and inputs.is_cuda else None
        return linear(input=inputs, weight=self.weight, bias=self.bias, mx_specs=self.mx_specs,
                      prequantized_weights=self.prequantized_weights, name=self.name, packed_weight=packed)
