"""Regenerates tests/golden/layers2.npz from the reference implementation:

    python tests/golden/make_golden_layers2.py --ref <checkout of microsoft/microxcaling>

Cases (CPU, custom_cuda=False, fp32 containers of bf16-representable values), each forward + backward:

  matmul with mode_config 'aw' and 'wa' (mx/matmul.py:33-43), matmul with a bias and addmm through
  mx_mapping.addmm_mx (mx/matmul.py:92-96, mx/mx_mapping.py:60-65), linear / bmm with
  quantize_backprop=False (mx/specs.py:193-209), linear / matmul with per-tensor rounding modes
  (mx/specs.py:102-113), and a gated feed-forward block (RMSNorm -> gate/up -> SiLU(gate) * up -> down)
  built from stock torch.nn.Linear / F.silu / torch.mul after the reference's inject_pyt_ops
  (mx/mx_mapping.py:41-57), at a reduced width, with the tensors between its stages.

The injection replaces names in the torch namespace for the rest of the process, so that case runs last.
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of microsoft/microxcaling")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    sys.dont_write_bytecode = True
    import torch
    import mx
    from mx import mx_mapping
    from mx.specs import finalize_mx_specs

    g = torch.Generator().manual_seed(4321)
    lay, meta = {}, []

    def bf(x):
        return x.to(torch.bfloat16).float()

    def rec(tag, **arrs):
        for k, v in arrs.items():
            lay[tag + "_" + k] = v.detach().numpy() if isinstance(v, torch.Tensor) else v

    base = {"block_size": 32, "scale_bits": 8, "bfloat": 16}
    s_mixed = dict(base, w_elem_format="fp4_e2m1", a_elem_format="fp8_e4m3")
    s_fp8 = dict(base, w_elem_format="fp8_e4m3", a_elem_format="fp8_e4m3", w_elem_format_bp="fp8_e5m2",
                 a_elem_format_bp="fp8_e5m2", a_elem_format_bp_ex="fp8_e5m2", a_elem_format_bp_os="fp8_e5m2")

    def run_matmul(tag, specs, lead, M, K, N, mode_config="aa", bias=False, addmm=False, shared_b=False):
        sp = finalize_mx_specs(dict(specs, custom_cuda=False))
        a = bf(torch.randn(*lead, M, K, generator=g)).requires_grad_()
        b = bf(torch.randn(*(() if shared_b else lead), K, N, generator=g) * K ** -0.5).requires_grad_()
        bi = bf(torch.randn(N, generator=g) * 0.1).requires_grad_() if (bias or addmm) else None
        go = bf(torch.randn(*lead, M, N, generator=g))
        if addmm:
            y = mx_mapping.addmm_mx(bi, a, b, mx_specs=sp)
        else:
            y = mx.matmul(a, b, bias=bi, mx_specs=sp, mode_config=mode_config)
        y.backward(go)
        rec(tag, a=a, b=b, go=go, y=y, ga=a.grad, gb=b.grad)
        if bi is not None:
            rec(tag, bias=bi, gbias=bi.grad)
        meta.append({"op": "addmm" if addmm else "matmul", "tag": tag, "specs": specs, "mode_config": mode_config,
                     "bias": bi is not None})

    def run_linear(tag, specs, M, K, N, bias):
        sp = finalize_mx_specs(dict(specs, custom_cuda=False))
        x = bf(torch.randn(M, K, generator=g)).requires_grad_()
        w = bf((torch.rand(N, K, generator=g) * 2 - 1) / K ** 0.5).requires_grad_()
        b = bf(torch.randn(N, generator=g) * 0.1).requires_grad_() if bias else None
        go = bf(torch.randn(M, N, generator=g))
        y = mx.linear(x, w, b, mx_specs=sp)
        y.backward(go)
        rec(tag, x=x, w=w, go=go, y=y, gx=x.grad, gw=w.grad)
        if bias:
            rec(tag, b=b, gb=b.grad)
        meta.append({"op": "linear", "tag": tag, "specs": specs, "bias": bias})

    def run_bmm(tag, specs, B, M, K, N):
        sp = finalize_mx_specs(dict(specs, custom_cuda=False))
        a = bf(torch.randn(B, M, K, generator=g)).requires_grad_()
        b = bf(torch.randn(B, K, N, generator=g) * K ** -0.5).requires_grad_()
        go = bf(torch.randn(B, M, N, generator=g))
        y = mx.bmm(a, b, mx_specs=sp)
        y.backward(go)
        rec(tag, a=a, b=b, go=go, y=y, ga=a.grad, gb=b.grad)
        meta.append({"op": "bmm", "tag": tag, "specs": specs})

    run_matmul("mm_aw", s_mixed, (), 96, 128, 64, mode_config="aw")
    run_matmul("mm_wa", s_mixed, (2,), 64, 96, 128, mode_config="wa")
    run_matmul("mm_bias", s_fp8, (), 64, 128, 96, bias=True)
    run_matmul("mm_bias_3d_shared", s_mixed, (3,), 32, 64, 96, mode_config="aw", bias=True, shared_b=True)
    run_matmul("addmm", s_fp8, (), 128, 64, 32, addmm=True)
    run_linear("lin_nobp", dict(s_mixed, quantize_backprop=False), 96, 128, 64, True)
    run_bmm("bmm_nobp", dict(base, a_elem_format="fp6_e3m2", quantize_backprop=False), 2, 64, 96, 32)
    s_round = dict(s_fp8, round="even", round_output="floor", round_mx_output="even", round_grad_input="nearest",
                   round_grad_weight="floor", round_mx_grad_output_grad_weight="floor",
                   round_mx_input_grad_weight="even", round_mx_grad_output_grad_input="nearest",
                   round_mx_weight_grad_input="floor", round_weight="nearest")
    run_linear("lin_rounds", s_round, 128, 96, 64, True)
    s_round2 = dict(s_mixed, round="floor", round_output="even", round_mx_output="floor",
                    round_mx_input_grad_input="even", round_mx_grad_output_grad_input="floor",
                    round_grad_input="even")
    run_matmul("mm_rounds", s_round2, (2,), 64, 64, 96)

    # ---- convolutions (quantize_mx_op along channel / batch axes around torch's convolution) ----
    def run_conv(tag, specs, kind, xshape, wshape, bias, **geom):
        sp = finalize_mx_specs(dict(specs, custom_cuda=False))
        x = bf(torch.randn(*xshape, generator=g)).requires_grad_()
        w = bf(torch.randn(*wshape, generator=g) * 0.2).requires_grad_()
        nb = wshape[0] if kind != "convT2d" else wshape[1] * geom.get("groups", 1)
        b = bf(torch.randn(nb, generator=g) * 0.1).requires_grad_() if bias else None
        if kind == "convT2d":
            from mx.transpose_convolution import ConvTranspose2dFunction
            from mx.specs import apply_mx_specs
            y = ConvTranspose2dFunction.apply(x, w, b, geom.get("stride", 1), geom.get("padding", 0),
                                              geom.get("output_padding", 0), geom.get("groups", 1),
                                              geom.get("dilation", 1), apply_mx_specs(sp), None)
        else:
            y = {"conv1d": mx.conv1d, "conv2d": mx.conv2d, "conv3d": mx.conv3d}[kind](x, w, b, mx_specs=sp, **geom)
        go = bf(torch.randn(*y.shape, generator=g))
        y.backward(go)
        rec(tag, x=x, w=w, go=go, y=y, gx=x.grad, gw=w.grad)
        if bias:
            rec(tag, b=b, gb=b.grad)
        meta.append({"op": kind, "tag": tag, "specs": specs, "bias": bias, "geom": geom})

    run_conv("conv2d", s_fp8, "conv2d", (32, 64, 6, 6), (48, 64, 3, 3), True, stride=1, padding=1)
    run_conv("conv1d_groups", s_mixed, "conv1d", (32, 64, 9), (32, 32, 3), False, stride=2, padding=1, groups=2)
    run_conv("conv3d", dict(base, w_elem_format="fp6_e3m2", a_elem_format="fp6_e3m2"), "conv3d", (32, 32, 3, 4, 4),
             (16, 32, 2, 2, 2), True)
    run_conv("convT2d", s_fp8, "convT2d", (32, 32, 5, 5), (32, 24, 3, 3), True, stride=2, padding=1)

    # ---- LSTM: two layers, both directions (mx.linear products + bfloat-emulated gate arithmetic) ----
    specs = dict(s_fp8)
    sp = finalize_mx_specs(dict(specs, custom_cuda=False))
    torch.manual_seed(77)
    lstm = mx.LSTM(32, 64, num_layers=2, bidirectional=True, mx_specs=sp)
    with torch.no_grad():
        for prm in lstm.parameters():
            prm.copy_(bf(prm))
    x = bf(torch.randn(5, 32, 32, generator=g)).requires_grad_()
    out, (hn, cn) = lstm(x)
    go = bf(torch.randn(*out.shape, generator=g))
    out.backward(go)
    rec("lstm", x=x, go=go, out=out, hn=hn, cn=cn, gx=x.grad)
    for k, v in lstm.state_dict().items():
        rec("lstm", **{"p_" + k: v})
    rec("lstm", g_weight_hh_l0=lstm.weight_hh_l0.grad, g_weight_ih_l1_reverse=lstm.weight_ih_l1_reverse.grad)
    meta.append({"op": "lstm", "tag": "lstm", "specs": specs, "input_size": 32, "hidden_size": 64, "num_layers": 2,
                 "bidirectional": True})

    # ---- gated feed-forward block through the reference's injection (last: it rewires torch for good) ----
    import torch.nn.functional as F
    specs = dict(s_mixed)
    sp = finalize_mx_specs(dict(specs, custom_cuda=False))
    H, I, T = 256, 768, 128
    norm = mx.RMSNorm(H, eps=1e-5, mx_specs=sp)
    mx_mapping.inject_pyt_ops(sp)
    gate, up, down = (torch.nn.Linear(H, I, bias=False), torch.nn.Linear(H, I, bias=False),
                      torch.nn.Linear(I, H, bias=False))
    assert type(gate).__name__ == "Linear_inj"
    with torch.no_grad():
        for lin in (gate, up, down):
            lin.weight.copy_(bf((torch.rand(lin.weight.shape, generator=g) * 2 - 1) * lin.weight.shape[1] ** -0.5))
        norm.weight.copy_(bf(torch.rand(H, generator=g) + 0.5))
        norm.bias.copy_(bf(torch.randn(H, generator=g) * 0.1))
        x = bf(torch.randn(T, H, generator=g))
        h = norm(x)
        gt, ut = gate(h), up(h)
        act = torch.mul(F.silu(gt), ut)
        y = down(act)
    rec("ffn", x=x, norm_w=norm.weight, norm_b=norm.bias, wg=gate.weight, wu=up.weight, wd=down.weight, h=h,
        gate=gt, up=ut, act=act, y=y)
    meta.append({"op": "ffn", "tag": "ffn", "specs": specs, "hidden": H, "inter": I, "tokens": T})

    np.savez_compressed(os.path.join(HERE, "layers2.npz"),
                        meta=np.frombuffer(json.dumps(meta).encode(), np.uint8), **lay)
    print("layers2 cases:", len(meta), "bytes:", os.path.getsize(os.path.join(HERE, "layers2.npz")))


if __name__ == "__main__":
    main()
