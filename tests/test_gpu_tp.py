"""Tensor-parallel MX FFN on two real GPUs (NCCL + the scattering GEMM over peer
memory) against the unsharded block.  Needs a box with at least two GPUs that can
reach each other; skipped otherwise.  Tolerance: the sharded down-projection adds
per-rank fp32 partial sums, so after the bfloat16 rounding an output may land on
the neighbouring value (<= 1 bf16 ulp, on < 3 % of elements)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tp_ffn_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(here, "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
