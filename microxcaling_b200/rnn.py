"""MX LSTM: drop-in for the reference's mx/rnn.py (LSTM :17-380) for Tensor inputs.

Every product of the recurrence is an `mx.linear` (the input projection of a whole sequence is one call,
the hidden projection one call per time step), i.e. MX-quantized operands and, on CUDA tensors, the
block-scaled tensor-core GEMM; the gate arithmetic is the bfloat-emulated sigmoid / tanh / simd_mul /
simd_add chain of the reference's cell (mx/rnn.py:85-123).  Supported: several layers, both directions,
dropout between layers, biases.  Like the reference: batch_first=False and proj_size=0 only.
PackedSequence inputs are not supported here.
"""
import torch
from torch.nn.utils.rnn import PackedSequence

from .activations import sigmoid, tanh
from .linear import linear
from .simd_ops import simd_add, simd_mul
from .specs import apply_mx_specs, mx_assert_test


class LSTM(torch.nn.LSTM):
    def __init__(self, *args, mx_specs=None, name="", **kwargs):
        super().__init__(*args, **kwargs)
        assert self.batch_first is False
        assert self.proj_size == 0
        mx_assert_test(mx_specs)
        self.mx_none = mx_specs is None
        self.mx_specs = apply_mx_specs(mx_specs)
        self.name = name
        self.dropout_layer = torch.nn.Dropout(p=self.dropout)

    def _params(self, layer, reverse):
        sfx = "_l%d%s" % (layer, "_reverse" if reverse else "")
        return (getattr(self, "weight_ih" + sfx), getattr(self, "weight_hh" + sfx),
                getattr(self, "bias_ih" + sfx, None), getattr(self, "bias_hh" + sfx, None))

    def _cell(self, xw, h, c, w_hh, b_hh):
        """One time step: xw is the pre-projected input [1, N, 4H]; gate order i, f, g, o."""
        sp = self.mx_specs
        gates = simd_add(xw, linear(h, w_hh, bias=b_hh, mx_specs=sp, name=self.name + ".HiddenLinear"), mx_specs=sp)
        gi, gf, gg, go = gates.chunk(4, dim=-1)
        i, f, g, o = sigmoid(gi, mx_specs=sp), sigmoid(gf, mx_specs=sp), tanh(gg, mx_specs=sp), sigmoid(go, mx_specs=sp)
        c = simd_add(simd_mul(f, c, mx_specs=sp), simd_mul(i, g, mx_specs=sp), mx_specs=sp)
        h = simd_mul(o, tanh(c, mx_specs=sp), mx_specs=sp)
        return h, c

    def _run_direction(self, seq, h, c, layer, reverse):
        w_ih, w_hh, b_ih, b_hh = self._params(layer, reverse)
        # input projection of all time steps at once: [L, N, 4H]
        xw = linear(seq, w_ih, bias=b_ih, mx_specs=self.mx_specs,
                    name=self.name + (".InputReverseLinear" if reverse else ".InputLinear"))
        L = seq.shape[0]
        outs = [None] * L
        for t in (range(L - 1, -1, -1) if reverse else range(L)):
            h, c = self._cell(xw[t:t + 1], h, c, w_hh, b_hh)
            outs[t] = h
        return torch.cat(outs, dim=0), h, c

    def forward(self, input, hx=None):
        if self.mx_none:
            return super().forward(input, hx)
        if isinstance(input, PackedSequence):
            raise ValueError("this MX LSTM does not support PackedSequence inputs")
        D = 2 if self.bidirectional else 1
        N = input.size(1)
        if hx is None:
            zeros = torch.zeros(self.num_layers * D, N, self.hidden_size, dtype=input.dtype, device=input.device)
            hx = (zeros, zeros.clone())
        self.check_forward_args(input, hx, None)
        hs, cs = hx
        seq = input
        final_h, final_c = [], []
        for layer in range(self.num_layers):
            outs = []
            for d in range(D):
                k = D * layer + d
                o, h, c = self._run_direction(seq, hs[k:k + 1], cs[k:k + 1], layer, reverse=(d == 1))
                outs.append(o)
                final_h.append(h)
                final_c.append(c)
            seq = outs[0] if D == 1 else torch.cat(outs, dim=-1)
            if layer < self.num_layers - 1:
                seq = self.dropout_layer(seq)
        return seq, (torch.cat(final_h, dim=0), torch.cat(final_c, dim=0))
