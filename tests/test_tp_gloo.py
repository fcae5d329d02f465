"""Multi-process (gloo, CPU) tests of the sharding host logic: the tensor-
parallel FFN over 2 ranks must reproduce the single-process block, and sharded
quantization must equal quantizing the whole tensor."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPECS = {"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32, "scale_bits": 8, "bfloat": 16}
H, I, T = 256, 512, 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _weights():
    g = torch.Generator().manual_seed(11)
    bf = lambda t: t.to(torch.bfloat16).float()
    return (bf(torch.randn(I, H, generator=g) / H ** 0.5), bf(torch.randn(I, H, generator=g) / H ** 0.5),
            bf(torch.randn(H, I, generator=g) / I ** 0.5), bf(torch.rand(H, generator=g) + 0.5),
            bf(torch.randn(T, H, generator=g)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from microxcaling_b200.specs import finalize_mx_specs
        from microxcaling_b200.tp import TensorParallelFFN, shard_bounds
        from microxcaling_b200.mx_ops import quantize_mx_op
        sp = finalize_mx_specs(dict(SPECS))
        wg, wu, wd, nw, x = _weights()
        ffn = TensorParallelFFN(H, I, sp, dtype=torch.float32)
        ffn.load_full(wg, wu, wd, nw)
        lo, hi = shard_bounds(T, rank, world, 128)
        y = ffn(x[lo:hi])
        # row-sharded quantization needs no exchange: each rank's rows are independent along the last axis
        qs = quantize_mx_op(x[lo:hi], sp, elem_format="fp8_e4m3", axes=[-1])
        q.put((rank, y, qs))
        # the ranks disagree on whether the scattering GEMM may be used (one rank's environment forbids
        # it): the choice is made collectively, so every rank must end up on the same branch
        from microxcaling_b200 import tp as tpmod
        tpmod._local_scatter_eligible = lambda device, world_: rank == 0
        ffn._scatter = None
        q.put((rank, "scatter=%s" % ffn._use_scatter(torch.device("cpu")), None))
        # mismatched shard sizes must be refused before any collective is entered
        try:
            ffn(x[lo:hi - 1])
            q.put((rank, "no error", None))
        except ValueError:
            q.put((rank, "refused", None))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_tp_ffn_two_ranks_matches_single_process():
    sys.path.insert(0, ROOT)
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.tp import TensorParallelFFN
    from microxcaling_b200.mx_ops import quantize_mx_op
    sp = finalize_mx_specs(dict(SPECS))
    wg, wu, wd, nw, x = _weights()
    ref = TensorParallelFFN(H, I, sp, dtype=torch.float32)
    ref.load_full(wg, wu, wd, nw)
    y_ref = ref(x)
    q_ref = quantize_mx_op(x, sp, elem_format="fp8_e4m3", axes=[-1])

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(6)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    outs = {r: (y, qs) for r, y, qs in got if isinstance(y, torch.Tensor)}
    flags = sorted(v for _, v, _ in got if isinstance(v, str))
    assert flags == ["refused", "refused", "scatter=False", "scatter=False"]
    y = torch.cat([outs[0][0], outs[1][0]])
    qs = torch.cat([outs[0][1], outs[1][1]])
    assert torch.equal(qs, q_ref)                       # sharded quantization == whole-tensor quantization
    # the down projection sums two partial products: same values up to fp32 summation order, then one
    # bfloat16 rounding -> at most one bf16 ulp apart on a small fraction of elements
    d = (y - y_ref).abs()
    assert (d <= y_ref.abs() * 2.0 ** -7 + 1e-30).all()
    assert (y == y_ref).float().mean() > 0.97


def test_shard_bounds():
    from microxcaling_b200.tp import shard_bounds
    assert shard_bounds(28672, 3, 8, 128) == (3 * 3584, 4 * 3584)
    assert shard_bounds(8192, 0, 1) == (0, 8192)
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 3)
    with pytest.raises(ValueError):
        shard_bounds(512, 0, 8, 128)
