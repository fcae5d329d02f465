"""Worker of tests/test_gpu_tp.py: one rank of a tensor-parallel MX FFN on real GPUs (NCCL).
Launched with torch.distributed.run; rank 0 prints 'TP_OK' when every check passed."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.tp import TensorParallelFFN
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32, "bfloat": 16})
    H, I, T = 256, 128 * world * 2, 128 * world * 3
    g = torch.Generator().manual_seed(0)
    wg, wu = torch.randn(I, H, generator=g) * H ** -0.5, torch.randn(I, H, generator=g) * H ** -0.5
    wd = torch.randn(H, I, generator=g) * I ** -0.5
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dev = torch.device("cuda")
    outs = {}
    for fused in ("1", "0", "pipe"):
        # "1": scattering GEMM; "0": NCCL reduce-scatter; "pipe": NCCL with the forward cut into three token chunks
        os.environ["MXQ_TP_FUSED_SCATTER"] = "1" if fused == "1" else "0"
        os.environ["MXQ_TP_TOKEN_CHUNKS"] = "3" if fused == "pipe" else "1"
        ffn = TensorParallelFFN(H, I, sp, device=dev, dtype=torch.bfloat16)
        ffn.load_full(wg.to(dev), wu.to(dev), wd.to(dev))
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        for _ in range(3):                     # repeated calls reuse the receive buffers
            y = ffn(x[lo:hi].to(dev))
        if fused == "1":
            assert ffn._slabs is not None, "peer access expected on this box"
        full = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(full, y)
        outs[fused] = torch.cat(full, 0).float()
        ffn.release_peer_buffers()
    # the unsharded block, on a one-rank group of this process
    os.environ["MXQ_TP_FUSED_SCATTER"] = "0"
    os.environ["MXQ_TP_TOKEN_CHUNKS"] = "1"
    solo_groups = [dist.new_group([r]) for r in range(world)]
    one = TensorParallelFFN(H, I, sp, group=solo_groups[rank], device=dev, dtype=torch.bfloat16)
    one.load_full(wg.to(dev), wu.to(dev), wd.to(dev))
    ref = one(x.to(dev)).float()
    if rank == 0:
        for k in ("1", "0", "pipe"):
            diff = (outs[k] - ref).abs()
            ulp = ref.abs().clamp_min(1e-30) * 2.0 ** -7
            assert bool((diff <= ulp).all()), (k, float(diff.max()))
            assert float((outs[k] == ref).float().mean()) >= 0.97, k
        from microxcaling_b200 import _backend
        assert _backend.device_status() == 0
        assert torch.equal(outs["pipe"], outs["0"]), "token chunks must not change the NCCL path's sums"
        print("TP_OK world=%d fused_vs_nccl_equal=%.4f" % (world, float((outs["1"] == outs["0"]).float().mean())))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
