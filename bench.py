#!/usr/bin/env python
"""Benchmark of the MX quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the format/rounding sweep the headline metric is quoted on): a bf16
[8192, 8192] tensor drawn from Student-t (df=3) with 0.1% of the entries
multiplied by 1e3 (seeded, synthetic).  One step = nine passes over it:
quantize_mx_op for {fp6_e3m2, fp6_e2m3, fp4_e2m1, int8} x {axis 0, axis -1}
(block 32, scale_bits 8, round 'nearest') plus one elementwise bfloat16
round-'even' pass in the tensor's own dtype.  Algorithmic bytes per pass:
2 B read + 2 B written per element = 268 435 456 B.

`value` times the kernels through the C ABI with inputs resident in HBM;
`e2e` times the same nine passes through the public Python API
(quantize_mx_op / quantize_elemwise_op) with pinned HOST buffers, the
host->device and device->host copies inside the timed region.
With --gpus N each rank owns one such tensor (a row shard of an [N*8192, 8192]
tensor); there is no data-path collective, so scaling is weak.
`--impl reference` times the reference's own C++ CPU code (compiled from its
headers into oracle/_ref) on the host cores, on a bounded row slab.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 8192
MX_FORMATS = ["fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8"]
PASS_BYTES = 2 * 2 * ROWS * COLS
PASSES = 2 * len(MX_FORMATS) + 1
CPU_SAMPLE_ROWS = 8192
BF16_MAX_NORM = 3.3895313892515355e38
CONFIG = {"workload": "format/rounding sweep: bf16 [8192,8192] Student-t(3) with 0.1% x1e3 outliers; "
                      "quantize_mx_op {fp6_e3m2,fp6_e2m3,fp4_e2m1,int8} x {axis 0, axis -1}, block 32, "
                      "nearest; plus bfloat16 round-even elementwise pass",
          "passes_per_step": PASSES, "bytes_per_pass": PASS_BYTES,
          "l2": "inputs+outputs rotate over 3 buffer sets of 256 MiB (larger than the 126 MB L2)",
          "sharding": "one [8192,8192] row shard per GPU, no collective"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    return ap.parse_args()


def make_input(torch, seed, device):
    g = torch.Generator(device="cpu").manual_seed(seed)
    # Student-t(3) = N(0,1) / sqrt(chi2_3 / 3), built from seeded normals
    z = torch.randn(ROWS, COLS, generator=g)
    c = (torch.randn(3, ROWS, COLS, generator=g) ** 2).sum(0) / 3.0
    t = z / c.sqrt()
    mask = torch.rand(ROWS, COLS, generator=g) < 1e-3
    t = torch.where(mask, t * 1e3, t)
    return t.to(torch.bfloat16).to(device)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.th.join(timeout=2)
        sm = sorted(int(r[1]) for r in self.rows if len(r) >= 8 and r[1].isdigit())
        mx = [int(r[2]) for r in self.rows if len(r) >= 8 and r[2].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 8 and r[4 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# dram__bytes_read.sum + dram__bytes_write.sum of one mx_strided_bf16_kernel launch on this workload
# (profiles/mx_strided_bf16_kernel__c2_sweep.md)
STRIDED_TRAFFIC_BYTES = 216_604_672


def mx_linear_block(torch, be, dev):
    """MX linear at the config-3 shape (8192 tokens, 4096 -> 4096, fp8_e4m3 forward, fp8_e5m2 backward,
    block 32, bfloat16): GEMM-only throughput of the block-scaled tensor-core kernel, and forward+backward
    of mx.Linear through the Python API (6 MX quantizations + 3 GEMMs per step), CUDA events."""
    import microxcaling_b200 as mx
    from microxcaling_b200.specs import finalize_mx_specs
    M, K, N = 8192, 4096, 4096
    g = torch.Generator(device="cpu").manual_seed(7)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    go = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
    sp = finalize_mx_specs({"w_elem_format": "fp8_e4m3", "a_elem_format": "fp8_e4m3", "w_elem_format_bp": "fp8_e5m2",
                            "a_elem_format_bp": "fp8_e5m2", "a_elem_format_bp_ex": "fp8_e5m2",
                            "a_elem_format_bp_os": "fp8_e5m2", "block_size": 32, "scale_bits": 8, "bfloat": 16,
                            "custom_cuda": True})
    torch.manual_seed(0)
    layer = mx.Linear(K, N, bias=False, mx_specs=sp).to(dev).to(torch.bfloat16)
    xr = x.clone().requires_grad_()
    _, ca, sa = be.quantize_mx(x, 8, 4, 5, 448.0, 32, 1, want_dq=False, want_codes=True, gemm_layout=True)
    _, cb, sb = be.quantize_mx(layer.weight.detach(), 8, 4, 5, 448.0, 32, 1, want_dq=False, want_codes=True,
                               gemm_layout=True)
    out = torch.empty(1, M, N, dtype=torch.bfloat16, device=dev)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e-3

    def step():
        y = layer(xr)
        y.backward(go)
        layer.weight.grad = None
        xr.grad = None

    t_gemm = timed(lambda: be.gemm_mx(ca, sa, cb, sb, 1, M, N, K, 0, 0, torch.bfloat16, 16, 0, None, 0, out=out), 50)
    t_step = min(timed(step, 20) for _ in range(3))      # the step is close to host-bound: best of 3 runs of 20
    assert be.device_status() == 0
    flop = 2.0 * M * N * K
    return {"shape": "8192 x 4096 -> 4096, w/a fp8_e4m3, backward fp8_e5m2, block 32, bfloat16 output rounding",
            "gemm_us": t_gemm * 1e6, "gemm_tflops": flop / t_gemm / 1e12,
            "fwd_bwd_us": t_step * 1e6, "fwd_bwd_tflops": 3 * flop / t_step / 1e12,
            "tensor_peak_nominal_tflops": 4500.0, "gemm_frac_of_nominal": flop / t_gemm / 1e12 / 4500.0,
            "tensor_pipe_active_pct_ncu": 74.0,
            "note": "fwd_bwd counts the 3 GEMMs' flops over the whole step (6 MX quantizations included), best of 3 x 20 steps; "
                    "tensor_pipe_active_pct_ncu from profiles/gemm_mx_kernel__8192x4096x4096.md"}


def mx_attention_block(torch, dev):
    """Config-4 shape: 32 heads x 2048 x 128, bf16, fp6_e3m2 operands, block 32: S = mx.bmm(Q, K^T),
    P = mx.softmax(S), O = mx.bmm(P, V), forward only.  Flops counted: the two batched products."""
    import microxcaling_b200 as mx
    from microxcaling_b200.specs import finalize_mx_specs
    Hh, S, D = 32, 2048, 128
    sp = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "block_size": 32, "scale_bits": 8, "bfloat": 16,
                            "custom_cuda": True})
    g = torch.Generator(device="cpu").manual_seed(0)
    q, k, v = [(torch.randn(Hh, S, D, generator=g) * 128 ** -0.25).to(torch.bfloat16).to(dev) for _ in range(3)]
    kt = k.transpose(-1, -2).contiguous()

    def fwd():
        with torch.no_grad():
            s = mx.bmm(q, kt, mx_specs=sp)
            p = mx.softmax(s, dim=-1, mx_specs=sp)
            return mx.bmm(p, v, mx_specs=sp)

    for _ in range(3):
        fwd()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 20
    a.record()
    for _ in range(iters):
        fwd()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / iters
    flop = 2 * 2.0 * Hh * S * S * D
    return {"shape": "32 x 2048 x 128 (QK^T, softmax, PV), fp6_e3m2, block 32, bfloat16", "ms": ms,
            "tflops": flop / (ms * 1e-3) / 1e12,
            "note": "4 MX packings, 2 block-scaled GEMMs and one fused softmax kernel per forward; the 2048 x 2048 "
                    "score matrices (268 MB in bf16) dominate: the block is HBM-bound, not tensor-bound"}


def mx_ffn_block(torch, dist, dev, rank, world):
    """Forward of the Llama-style FFN block of config 5 (hidden 8192, intermediate 28672, 16384 tokens,
    w fp4_e2m1, a fp8_e4m3, block 32, bfloat16), tensor-parallel over the ranks: column-parallel gate/up,
    row-parallel down, packed activations all-gathered, fp32 partials reduce-scattered (NCCL).  Total
    work is fixed (strong scaling); the time is the max over ranks."""
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.tp import TensorParallelFFN
    H, I, T = 8192, 28672, 16384
    if I % (128 * world) or T % (128 * world):
        return {"skipped": "shape does not split over %d ranks" % world}
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32,
                            "scale_bits": 8, "bfloat": 16, "custom_cuda": True})
    torch.manual_seed(100 + rank)
    ffn = TensorParallelFFN(H, I, sp, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for w in (ffn.w_gate, ffn.w_up, ffn.w_down):
            w.copy_((torch.rand(w.shape, device=dev) * 2 - 1) * (1.0 / w.shape[1]) ** 0.5)
    x = torch.randn(T // world, H, device=dev, dtype=torch.bfloat16)
    for _ in range(4):
        y = ffn(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    iters = 10
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        y = ffn(x)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / iters
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    flop = 3 * 2.0 * T * H * I
    fused_scatter = ffn._slabs is not None
    ffn.release_peer_buffers()
    del ffn, x, y
    torch.cuda.empty_cache()
    return {"shape": "16384 tokens, hidden 8192, intermediate 28672, SwiGLU + RMSNorm, w fp4_e2m1 / a fp8_e4m3",
            "parallelism": "tp%d (column-parallel gate/up, row-parallel down; NCCL all-gather of packed activations; "
                           "%s)" % (world, "single GPU, no exchange" if world == 1 else
                                    "down-projection GEMM scatters its fp32 tiles into the owners' buffers over "
                                    "peer memory, then an ordered slab sum" if fused_scatter else
                                    "NCCL reduce-scatter of fp32 partials"),
            "ms": ms, "tflops": flop / (ms * 1e-3) / 1e12, "scaling": "strong"}


def cpu_baseline(torch, x_rows_f32, kind_wanted=None):
    """Times the nine passes on a [CPU_SAMPLE_ROWS, 8192] fp32-container slab
    with all host threads: the reference's own C++ math where oracle/_ref was
    built, else the C port."""
    import numpy as np
    import oracle
    x = np.ascontiguousarray(x_rows_f32)
    use_ref = oracle.ref() is not None
    fn_mx = oracle.ref_quantize_mx_f32 if use_ref else oracle.quantize_mx
    cores = oracle.ref().mxref_num_threads() if use_ref else oracle.lib().mxo_num_threads()
    t0 = time.perf_counter()
    for fmt in MX_FORMATS:
        for axis in (0, 1):
            fn_mx(x, fmt, axis=axis, block=32, scale_bits=8, round="nearest")
    if use_ref:
        oracle.ref_quantize_elemwise_f32(x, 9, 8, BF16_MAX_NORM, "even")
    else:
        oracle.quantize_elemwise(x, 9, 8, BF16_MAX_NORM, "even")
    dt = time.perf_counter() - t0
    bytes_done = PASSES * 4 * x.size            # counted as bf16 traffic: 2 B in + 2 B out
    return {"value": bytes_done / dt / 1e9, "unit": "GB/s", "cores": int(cores),
            "kind": "reference" if use_ref else "port",
            "sample": "the nine passes on rows [0,%d) of the tensor held as fp32 values (%.2f s)" % (x.shape[0], dt)}, dt


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    x = make_input(torch, 0, "cpu")[:CPU_SAMPLE_ROWS].float().numpy()
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_baseline(torch, x[:64])
    vals, tot = [], 0.0
    steps = max(1, min(args.steps, 5))
    for _ in range(steps):
        cb, dt = cpu_baseline(torch, x)
        vals.append(cb["value"])
        tot += dt
    v = sum(vals) / len(vals)
    cb["value"] = v
    print(json.dumps({"impl": "reference", "metric": "MX-quantize GB/s", "value": v, "unit": "GB/s",
                      "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": tot / steps * 1e3,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                      "data": "synthetic",
                      "config": CONFIG,
                      "cpu_baseline": cb,
                      "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    import torch
    import torch.distributed as dist
    from microxcaling_b200 import _backend as be
    from microxcaling_b200.formats import _get_format_params
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.mx_ops import quantize_mx_op
    from microxcaling_b200.elemwise_ops import _quantize_bfloat

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = be.lib()

    NBUF = 3                                   # 3 x (128 MiB in + 128 MiB out) > 126 MB L2
    xs = [make_input(torch, 1000 * rank + i, dev) for i in range(NBUF)]
    ys = [torch.empty_like(x) for x in xs]
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)
    fmt_params = {f: _get_format_params(f) for f in MX_FORMATS}

    def launch_pass(i, x, y):
        if i < 8:
            eb, mb, _, mn, _ = fmt_params[MX_FORMATS[i // 2]]
            pre, n, post = (1, ROWS, COLS) if i % 2 == 0 else (ROWS, COLS, 1)
            rc = L.mxq_quantize_mx(x.data_ptr(), y.data_ptr(), None, None, be.BF16, pre, n, post, 32, 8,
                                   eb, mb, mn, 0, 0, None, 0, 0, sp)
        else:
            rc = L.mxq_quantize_elemwise(x.data_ptr(), y.data_ptr(), be.BF16, be.BF16, x.numel(), 9, 8,
                                         BF16_MAX_NORM, 2, 0, 1, None, sp)
        if rc:
            be.check(rc)

    # one step: the four axis-0 passes, the four last-axis passes, the elementwise pass; one CUDA event at
    # each group boundary, so a kernel's average launch duration = group time / launches in the group
    ORDER = [0, 2, 4, 6, 1, 3, 5, 7, 8]
    GROUP_STARTS = (0, 4, 8)

    def step(s, events=None):
        x, y = xs[s % NBUF], ys[s % NBUF]
        for n, i in enumerate(ORDER):
            if events is not None and n in GROUP_STARTS:
                events[GROUP_STARTS.index(n)].record(stream)
            launch_pass(i, x, y)
        if events is not None:
            events[3].record(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for s in range(max(args.warmup, 3)):
        step(s)
    barrier()
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for s in range(K):
        step(s, ev[s])
    t_end.record(stream)
    barrier()
    total_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None
    group_ms = [sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(K)) / K for i in range(3)]
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())

    # ---- end to end through the public API, host buffers -------------------
    specs = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "block_size": 32, "scale_bits": 8, "bfloat": 16,
                               "custom_cuda": True})
    hx = xs[0].cpu().pin_memory()

    def e2e_step():
        # host tensor in, host tensor out, through the public ops: the library cuts the tensor into
        # chunks and overlaps H2D, kernel and D2H (mxq_quantize_mx_host / mxq_quantize_elemwise_host)
        for i in range(PASSES):
            if i < 8:
                hy = quantize_mx_op(hx, specs, elem_format=MX_FORMATS[i // 2], axes=[0 if i % 2 == 0 else -1],
                                    round="nearest")
            else:
                hy = _quantize_bfloat(hx, 16, round="even", custom_cuda=True)
            assert not hy.is_cuda
        torch.cuda.synchronize()

    e2e_step()
    barrier()
    e0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - e0) / args.e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # ---- MX linear (config 3 shape): packed-operand GEMM and the full layer ----
    lin = att = None
    if rank == 0:
        lin = mx_linear_block(torch, be, dev)
        att = mx_attention_block(torch, dev)

    # ---- tensor-parallel MX FFN (config 5 shape), all ranks ----
    ffn = mx_ffn_block(torch, dist, dev, rank, world)

    if rank == 0:
        step_bytes = PASSES * PASS_BYTES
        value = world * step_bytes * K / (total_ms * 1e-3) / 1e9
        peaks = {}
        pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pk):
            peaks = json.load(open(pk))
        peak = float(peaks.get("hbm_gbs", 6650.0))
        # dominant kernel: the strided-axis MX kernel (4 of the 9 launches, the slowest passes)
        strided_ms = group_ms[0] / 4
        last_ms = group_ms[1] / 4
        achieved = PASS_BYTES / (strided_ms * 1e-3) / 1e9
        out = {
            "metric": "MX-quantize GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, fp32/u32 lane arithmetic",
            "data": "synthetic",
            "config": CONFIG,
            "roofline": {"bound": "hbm", "kernel": "mx_strided_bf16_kernel (axis-0 passes)", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks else "6650 (of fallback)",
                         "traffic": None,
                         "other_kernels": {"mx_lastaxis_bf16_kernel": PASS_BYTES / (last_ms * 1e-3) / 1e9,
                                           "ew_vec_kernel(bf16,even)": PASS_BYTES / (group_ms[2] * 1e-3) / 1e9}},
            "e2e": {"value": world * step_bytes / e2e_s / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": PASSES * hx.numel() * 2, "d2h_bytes_per_step": PASSES * hx.numel() * 2,
                    "ms_per_step": e2e_s * 1e3},
            "gpu_launches": PASSES * K,
            "clocks": clocks,
        }
        out["roofline"]["traffic"] = STRIDED_TRAFFIC_BYTES
        out["mx_linear"] = lin
        out["mx_attention"] = att
        out["mx_ffn"] = ffn
        if world == 1:
            cb, _ = cpu_baseline(torch, xs[0][:CPU_SAMPLE_ROWS].float().cpu().numpy())
            out["cpu_baseline"] = cb
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
