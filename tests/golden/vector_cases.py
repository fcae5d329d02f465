"""The vector-op layer cases of layers3.npz, shared by the script that records them from the reference
(make_golden_layers3.py) and the tests that replay them on this package: `run_case(mx, case, tensors, specs)`
calls the same public names on whichever `mx` module it is given and returns every output and gradient."""
import torch

SPECS = {
    "bf16": {"bfloat": 16},
    "bf16_even": {"bfloat": 16, "round": "even"},
    "bf12_nobp": {"bfloat": 12, "quantize_backprop": False},
}

# tag -> (op, input shapes, keyword arguments)
CASES = {
    "relu": ("relu", [(6, 40)], {}),
    "relu6": ("relu6", [(6, 40)], {}),
    "leaky_relu": ("leaky_relu", [(6, 40)], {"negative_slope": 0.4}),
    "gelu_tanh": ("gelu", [(6, 40)], {"first_order_gelu": False}),
    "gelu_first": ("gelu", [(6, 40)], {"first_order_gelu": True}),
    "sigmoid": ("sigmoid", [(6, 40)], {}),
    "tanh": ("tanh", [(6, 40)], {}),
    "silu": ("silu", [(6, 40)], {}),
    "square": ("simd_square", [(5, 33)], {}),
    "sqrt": ("simd_sqrt", [(5, 33)], {"positive": True}),
    "exp": ("simd_exp", [(5, 33)], {}),
    "log": ("simd_log", [(5, 33)], {"positive": True}),
    "sum": ("simd_reduce_sum", [(4, 6, 10)], {"dim": [0, 2], "keepdim": False}),
    "mean": ("simd_reduce_mean", [(4, 6, 10)], {"dim": [1], "keepdim": True}),
    "norm": ("simd_norm", [(4, 6, 10)], {}),
    "split": ("simd_split", [(5, 33)], {}),
    "div_bcast": ("simd_div", [(4, 6, 10), (6, 1)], {"positive2": True}),
    "mul_const": ("simd_mul", [(5, 33)], {"const": 0.3}),
    "layer_norm": ("LayerNorm", [(3, 7, 48)], {"eps": 1e-5}),
    "group_norm": ("GroupNorm", [(3, 8, 5, 6)], {"groups": 4, "eps": 1e-5}),
    "batch_norm_train": ("BatchNorm2d", [(4, 6, 5, 5)], {"train": True}),
    "batch_norm_eval": ("BatchNorm2d", [(4, 6, 5, 5)], {"train": False}),
    "batch_norm_1d": ("BatchNorm1d", [(9, 6)], {"train": True}),
    "adaptive_pool": ("adaptive_avg_pool2d", [(2, 3, 7, 9)], {"output_size": (3, 4)}),
    "adaptive_pool_sq": ("adaptive_avg_pool2d", [(2, 3, 8, 8)], {"output_size": 2}),
}


def make_inputs(case, gen):
    """Seeded fp32 inputs holding bfloat16-representable values (+ parameters for the module cases)."""
    op, shapes, kw = CASES[case]
    bf = lambda t: t.to(torch.bfloat16).float()
    t = {}
    for i, s in enumerate(shapes):
        x = torch.randn(*s, generator=gen) * 2
        if kw.get("positive") or (i == 1 and kw.get("positive2")):
            x = x.abs() + 0.25
        t["in%d" % i] = bf(x)
    C = {"LayerNorm": shapes[0][-1], "GroupNorm": shapes[0][1], "BatchNorm2d": shapes[0][1], "BatchNorm1d": shapes[0][1]}.get(op)
    if C is not None:
        t["weight"] = bf(torch.rand(C, generator=gen) + 0.5)
        t["bias"] = bf(torch.randn(C, generator=gen) * 0.2)
        if op.startswith("BatchNorm"):
            t["running_mean"] = bf(torch.randn(C, generator=gen) * 0.1)
            t["running_var"] = bf(torch.rand(C, generator=gen) + 0.5)
    return t


def run_case(mx, case, t, specs):
    """-> {name: tensor}: outputs, input gradients, parameter gradients, updated running statistics."""
    op, shapes, kw = CASES[case]
    ins = [t["in%d" % i].clone().requires_grad_() for i in range(len(shapes))]
    res = {}
    if op in ("LayerNorm", "GroupNorm", "BatchNorm2d", "BatchNorm1d"):
        if op == "LayerNorm":
            m = mx.LayerNorm(shapes[0][-1], eps=kw["eps"], mx_specs=specs)
        elif op == "GroupNorm":
            m = mx.GroupNorm(kw["groups"], shapes[0][1], eps=kw["eps"], mx_specs=specs)
        else:
            m = getattr(mx, op)(shapes[0][1], mx_specs=specs)
            with torch.no_grad():
                m.running_mean.copy_(t["running_mean"])
                m.running_var.copy_(t["running_var"])
            m.train(kw["train"])
        with torch.no_grad():
            m.weight.copy_(t["weight"])
            m.bias.copy_(t["bias"])
        y = m(ins[0])
        outs = [y]
    else:
        fn = getattr(mx, op)
        args = {k: v for k, v in kw.items() if k not in ("positive", "positive2", "const")}
        if "const" in kw:
            y = fn(ins[0], kw["const"], mx_specs=specs)
        elif op == "adaptive_avg_pool2d":
            y = fn(ins[0], args.pop("output_size"), mx_specs=specs)
        else:
            y = fn(*ins, mx_specs=specs, **args)
        outs = list(y) if isinstance(y, tuple) else [y]
        m = None
    # a fixed, seeded upstream gradient per output: weights that depend on position only
    loss = 0
    for k, o in enumerate(outs):
        res["out%d" % k] = o.detach().clone()
        w = torch.linspace(-1.0, 1.5, o.numel()).reshape(o.shape).to(torch.bfloat16).float().to(o.device) * (k + 1)
        loss = loss + (o * w).sum()
    loss.backward()
    for i, x in enumerate(ins):
        res["grad_in%d" % i] = x.grad.detach().clone()
    if m is not None:
        res["grad_weight"], res["grad_bias"] = m.weight.grad.detach().clone(), m.bias.grad.detach().clone()
        if op.startswith("BatchNorm"):
            res["running_mean_after"], res["running_var_after"] = m.running_mean.detach().clone(), m.running_var.detach().clone()
    return res
