"""Runs the reference's own test files against this package:

    python tests/golden/run_reference_tests.py --ref <checkout of microsoft/microxcaling> [pytest args]

A temporary directory gets a package named `mx` that re-exports microxcaling_b200 (and registers its
submodules as mx.<name>), a link to the checkout's mx/tests (nothing is copied) and a conftest that turns
torch.cuda.synchronize into a no-op on a host without a GPU; pytest then runs there.  Without a GPU pass
`-k "not cuda"`: the cases that remain and still fail are the ones that allocate CUDA tensors, call
torch.cuda.* or ask for custom_cuda=True (the reference fails the same ones on such a host).
"""
import argparse
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

ALIAS = '''import importlib, pkgutil, sys
import microxcaling_b200 as _p
from microxcaling_b200 import *  # noqa
for m in pkgutil.iter_modules(_p.__path__):
    if m.name.startswith("_") and m.name != "_backend":
        continue
    try:
        sys.modules["mx." + m.name] = importlib.import_module("microxcaling_b200." + m.name)
    except Exception as e:
        print("alias skipped", m.name, e)
'''
CONFTEST = '''import torch
if not torch.cuda.is_available():
    torch.cuda.synchronize = lambda *a, **k: None
'''


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of microsoft/microxcaling")
    args, rest = ap.parse_known_args()
    tests = os.path.join(os.path.abspath(args.ref), "mx", "tests")
    if not os.path.isdir(tests):
        sys.exit("no mx/tests under " + args.ref)
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "mx"))
        with open(os.path.join(tmp, "mx", "__init__.py"), "w") as f:
            f.write(ALIAS)
        with open(os.path.join(tmp, "conftest.py"), "w") as f:
            f.write(CONFTEST)
        os.symlink(tests, os.path.join(tmp, "mx", "tests"))
        env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, tmp, os.environ.get("PYTHONPATH", "")]),
                   PYTHONDONTWRITEBYTECODE="1")
        cmd = [sys.executable, "-m", "pytest", "-p", "no:cacheprovider", "-q", "--no-header", "mx/tests"] + rest
        sys.exit(subprocess.call(cmd, cwd=tmp, env=env))


if __name__ == "__main__":
    main()
