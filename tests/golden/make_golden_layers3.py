"""Regenerates tests/golden/layers3.npz from the reference implementation:

    python tests/golden/make_golden_layers3.py --ref <checkout of microsoft/microxcaling>

Every case of vector_cases.CASES (activations, the unary / reduction simd operators, LayerNorm, GroupNorm,
BatchNorm in training and evaluation, adaptive average pooling) under every spec of vector_cases.SPECS, on CPU
with custom_cuda=False: seeded inputs, outputs, all gradients and the updated running statistics.
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of microsoft/microxcaling")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    sys.path.insert(0, HERE)
    sys.dont_write_bytecode = True
    import torch
    import mx
    from mx.specs import finalize_mx_specs
    import vector_cases as vc

    out = {}
    gen = torch.Generator().manual_seed(777)
    for case in vc.CASES:
        tensors = vc.make_inputs(case, gen)
        for k, v in tensors.items():
            out["%s/%s" % (case, k)] = v.numpy()
        for sname, sdict in vc.SPECS.items():
            sp = finalize_mx_specs(dict(sdict, custom_cuda=False), early_exit=False)
            for k, v in vc.run_case(mx, case, tensors, sp).items():
                out["%s/%s/%s" % (case, sname, k)] = v.numpy()
    path = os.path.join(HERE, "layers3.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
