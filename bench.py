#!/usr/bin/env python
"""Benchmark of the MX quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--only quantize|config1|pack|vector|linear|attention|ffn]

Workload (the format/rounding sweep the headline metric is quoted on): a bf16
[8192, 8192] tensor drawn from Student-t (df=3) with 0.1% of the entries
multiplied by 1e3 (seeded, synthetic).  One step = nine passes over it:
quantize_mx_op for {fp6_e3m2, fp6_e2m3, fp4_e2m1, int8} x {axis 0, axis -1}
(block 32, scale_bits 8, round 'nearest'; 2 B read + 2 B written per element =
268 435 456 B per pass) plus the elementwise bfloat16 round-'even' pass on the
fp32 copy of the same values (4 B read + 2 B written = 402 653 184 B; on bf16
storage that pass is the identity and launches nothing, as in the reference).

`value` times the kernels through the C ABI with inputs resident in HBM;
`e2e` times the same nine passes through the public Python API
(quantize_mx_op / quantize_elemwise_op) with pinned HOST buffers, the
host->device and device->host copies inside the timed region.
With --gpus N each rank owns one such tensor (a row shard of an [N*8192, 8192]
tensor); there is no data-path collective, so scaling is weak.
`--impl reference` times the reference's own C++ CPU code (compiled from its
headers into oracle/_ref, else the C port under oracle/) on the host cores, on a
bounded row slab.  Further blocks of the same JSON line (they do not enter
`value`): config 1 (fp32 [4096,4096] fp8_e4m3), the packing kernels that feed the
GEMMs, MX linear (config 3), the attention-shaped block (config 4) and the FFN
block (config 5, tensor-parallel over the ranks, with a numerical check of the
sharded result against the unsharded block).  `--only X` runs one block alone
(for profiler captures).
"""
import argparse
import ctypes
import json
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 8192
MX_FORMATS = ["fp6_e3m2", "fp6_e2m3", "fp4_e2m1", "int8"]
MX_PASS_BYTES = 2 * 2 * ROWS * COLS            # bf16 in, bf16 out
EW_PASS_BYTES = (4 + 2) * ROWS * COLS          # fp32 in, bf16 out
PASSES = 2 * len(MX_FORMATS) + 1
STEP_BYTES = 2 * len(MX_FORMATS) * MX_PASS_BYTES + EW_PASS_BYTES
CPU_SAMPLE_ROWS = 8192
BF16_MAX_NORM = 3.3895313892515355e38
NBUF = 4                                       # buffer sets, rotated per launch
CONFIG = {"workload": "format/rounding sweep: bf16 [8192,8192] Student-t(3) with 0.1% x1e3 outliers; "
                      "quantize_mx_op {fp6_e3m2,fp6_e2m3,fp4_e2m1,int8} x {axis 0, axis -1}, block 32, "
                      "nearest; plus the bfloat16 round-even elementwise pass on the fp32 copy of the tensor",
          "passes_per_step": PASSES, "bytes_per_mx_pass": MX_PASS_BYTES, "bytes_elementwise_pass": EW_PASS_BYTES,
          "l2": "inputs and outputs rotate per launch over %d buffer sets of 256 MiB (bf16) / 384 MiB (fp32 pass), "
                "each larger than the 126 MB L2" % NBUF,
          "sharding": "one [8192,8192] row shard per GPU, no collective"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--only", default=None, choices=["quantize", "config1", "pack", "vector", "linear", "attention", "ffn"])
    ap.add_argument("--ffn-tokens", type=int, default=16384, help="token count of the FFN block (reduce for captures)")
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


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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


def peaks():
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    p = json.load(open(pk)) if os.path.exists(pk) else {}
    return {"hbm_gbs": float(p.get("hbm_gbs", 6650.0)), "bf16_tflops": float(p.get("bf16_tflops", 1590.0)),
            "source": "MEASURED_PEAKS.json (of measured)" if p else "6650 GB/s, 1590 TFLOP/s (of fallback)"}


def captured_traffic(kernel):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel`, read from the line
    'dram_bytes_per_launch: N' of the committed profiler summary for this workload; None if absent."""
    d = os.path.join(ROOT, "profiles")
    if not os.path.isdir(d):
        return None, None
    for name in sorted(os.listdir(d)):
        if name.startswith(kernel + "__"):
            m = re.search(r"dram_bytes_per_launch:\s*([0-9_]+)", open(os.path.join(d, name)).read())
            if m:
                return int(m.group(1).replace("_", "")), name
    return None, None


def timed(torch, fn, iters, warm=3):
    """Mean seconds per call of fn(i) over `iters` back-to-back calls (CUDA events on the current stream)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def rotated(torch, x, n):
    """n buffers with the value distribution of x (column rotations of it), so that consecutive launches
    never touch the same lines."""
    return [x if i == 0 else torch.roll(x, shifts=977 * i, dims=-1).contiguous() for i in range(n)]


# ------------------------------------------------------------------------------------------------
def config1_block(torch, be, dev, hbm):
    """Config 1: quantize_mx_op on fp32 [4096,4096] N(0,1), fp8_e4m3, block 32 along the last axis,
    scale_bits 8, nearest; 4 B read + 4 B written per element."""
    from microxcaling_b200.formats import _get_format_params
    g = torch.Generator(device="cpu").manual_seed(0)
    x0 = torch.randn(4096, 4096, generator=g).to(dev)
    xs = rotated(torch, x0, 8)                      # 8 x (64 MiB in + 64 MiB out) = 1 GiB
    ys = [torch.empty_like(x) for x in xs]
    eb, mb, _, mn, _ = _get_format_params("fp8_e4m3")
    L = be.lib()
    sp = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def f(i):
        x, y = xs[i % 8], ys[i % 8]
        be.check(L.mxq_quantize_mx(x.data_ptr(), y.data_ptr(), None, None, be.F32, 4096, 4096, 1, 32, 8, eb, mb, mn,
                                   0, 0, None, 0, 0, sp))
    t = timed(torch, f, 200, warm=8)
    nbytes = 2 * 4 * 4096 * 4096
    return {"shape": "fp32 [4096,4096] N(0,1), fp8_e4m3, block 32 along the last axis, nearest",
            "kernel": "mx_lastaxis_kernel<f32>", "bytes": nbytes, "us": t * 1e6, "gbs": nbytes / t / 1e9,
            "frac": nbytes / t / 1e9 / hbm, "buffers": "8 input/output pairs of 64 MiB rotated per launch"}


def pack_block(torch, be, dev, hbm):
    """The kernels that write the packed GEMM operand (one code byte per element + E8M0 scales in the
    GEMM's chunk layout, no dequantized output): along the last axis, along axis 0 with the codes written
    transposed, and SiLU(gate) * up fused into the packing (config-5 intermediate, 16384 x 28672)."""
    x0 = make_input(torch, 3, dev)
    xs = rotated(torch, x0, NBUF)
    out = {}
    n = ROWS * COLS
    for name, kw, kern in (("lastaxis_codes", dict(axis=1, transposed=False), "mx_lastaxis_bf16_kernel"),
                           ("strided_codes_transposed", dict(axis=0, transposed=True), "mx_strided_bf16_kernel")):
        def f(i, kw=kw):
            be.quantize_mx(xs[i % NBUF], 8, 4, 5, 448.0, 32, kw["axis"], want_dq=False, want_codes=True,
                           transposed=kw["transposed"], gemm_layout=True)
        t = timed(torch, f, 40)
        nbytes = n * 2 + n + n // 32
        out[name] = {"kernel": kern, "bytes": nbytes, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                     "frac": nbytes / t / 1e9 / hbm}
    del xs, x0
    T, I = 16384, 28672
    gs = [torch.randn(T, I, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    us_ = [torch.randn(T, I, device=dev, dtype=torch.bfloat16) for _ in range(2)]

    def f(i):
        be.swiglu_quantize_mx(gs[i % 2], us_[i % 2], 8, 4, 5, 448.0)
    t = timed(torch, f, 10)
    nbytes = T * I * 4 + T * I + T * I // 32
    out["swiglu_pack"] = {"kernel": "mx_lastaxis_bf16_kernel<PRO=1>", "shape": "16384 x 28672", "bytes": nbytes,
                          "us": t * 1e6, "gbs": nbytes / t / 1e9, "frac": nbytes / t / 1e9 / hbm}
    del gs, us_
    torch.cuda.empty_cache()
    return out


def vector_block(torch, be, dev, hbm):
    """The bfloat16 vector kernels between the GEMMs and the inner-dimension reductions, each on an input
    larger than L2: softmax over [65536, 2048] (the config-4 score matrices), the same fused with the MX
    packing of the probabilities (fp6_e3m2), RMSNorm over [16384, 8192] (config 5), sum / max over the inner
    dimension of fp32 [16384, 8192]."""
    out = {}
    xs = [torch.randn(32, 2048, 2048, device=dev).to(torch.bfloat16) for _ in range(2)]
    n = xs[0].numel()
    t = timed(torch, lambda i: be.softmax_bf16(xs[i % 2]), 20)
    out["softmax"] = {"kernel": "softmax_bf16_kernel", "bytes": 4 * n, "us": t * 1e6, "frac": 4 * n / t / 1e9 / hbm}
    t = timed(torch, lambda i: be.softmax_quantize_mx(xs[i % 2], 8, 3, 4, 28.0, False, 0, rows_per_batch=2048), 20)
    nb = 2 * n + 2 * n + n + n // 32
    out["softmax_pack"] = {"kernel": "softmax_quantize_kernel", "bytes": nb, "us": t * 1e6, "frac": nb / t / 1e9 / hbm,
                           "note": "probabilities written as bfloat16 and as the packed operand"}
    t = timed(torch, lambda i: be.softmax_quantize_mx(xs[i % 2], 8, 3, 4, 28.0, False, 0, rows_per_batch=2048,
                                                      want_probs=False), 20)
    nb = 2 * n + n + n // 32
    out["softmax_pack_only"] = {"kernel": "softmax_quantize_kernel", "bytes": nb, "us": t * 1e6, "frac": nb / t / 1e9 / hbm}
    del xs
    hs = [torch.randn(16384, 8192, device=dev).to(torch.bfloat16) for _ in range(2)]
    w = torch.ones(8192, device=dev, dtype=torch.bfloat16)
    b = torch.zeros(8192, device=dev, dtype=torch.bfloat16)
    n = hs[0].numel()
    t = timed(torch, lambda i: be.rmsnorm_bf16(hs[i % 2], w, b, 1e-5), 20)
    out["rmsnorm"] = {"kernel": "rmsnorm_bf16_kernel", "bytes": 4 * n, "us": t * 1e6, "frac": 4 * n / t / 1e9 / hbm}
    del hs
    fs = [torch.randn(16384, 8192, device=dev) for _ in range(2)]
    n = fs[0].numel()
    for nm in ("sum", "max"):
        fn = be.funcs.reduce_sum_inner_dim if nm == "sum" else be.funcs.reduce_max_inner_dim
        t = timed(torch, lambda i: fn(fs[i % 2]), 20)
        out["reduce_" + nm] = {"kernel": "reduce_%s_rows_kernel" % nm, "bytes": 4 * n, "us": t * 1e6,
                               "frac": 4 * n / t / 1e9 / hbm}
    del fs
    torch.cuda.empty_cache()
    return out


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

    def step(_):
        y = layer(xr)
        y.backward(go)
        layer.weight.grad = None
        xr.grad = None

    t_gemm = timed(torch, lambda _: be.gemm_mx(ca, sa, cb, sb, 1, M, N, K, 0, 0, torch.bfloat16, 16, 0, None, 0,
                                               out=out), 50)
    t_step = timed(torch, step, 20)
    assert be.device_status() == 0
    flop = 2.0 * M * N * K
    return {"shape": "8192 x 4096 -> 4096, w/a fp8_e4m3, backward fp8_e5m2, block 32, bfloat16 output rounding",
            "gemm_us": t_gemm * 1e6, "gemm_tflops": flop / t_gemm / 1e12,
            "fwd_bwd_us": t_step * 1e6, "fwd_bwd_tflops": 3 * flop / t_step / 1e12,
            "tensor_peak_nominal_tflops": 4500.0, "gemm_frac_of_nominal": flop / t_gemm / 1e12 / 4500.0,
            "note": "fwd_bwd counts the 3 GEMMs' flops over the whole step (6 MX quantizations included), mean of 20 "
                    "steps after 3 warm-up steps"}


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

    def fwd(_):
        with torch.no_grad():
            s = mx.bmm(q, kt, mx_specs=sp)
            p = mx.softmax(s, dim=-1, mx_specs=sp)
            return mx.bmm(p, v, mx_specs=sp)

    t = timed(torch, fwd, 20)
    flop = 2 * 2.0 * Hh * S * S * D
    floor_bytes = 4 * Hh * S * D * 2 + 2 * Hh * S * S * 2 + 2 * (Hh * S * S + Hh * S * S // 32)
    return {"shape": "32 x 2048 x 128 (QK^T, softmax, PV), fp6_e3m2, block 32, bfloat16; entries N(0, std 128^-1/4)",
            "ms": t * 1e3, "tflops": flop / t / 1e12, "hbm_floor_bytes": floor_bytes,
            "note": "4 MX packings, 2 block-scaled GEMMs and one fused softmax kernel per forward; the 2048 x 2048 "
                    "score matrices (268 MB in bf16) dominate: the block is HBM-bound, not tensor-bound"}


def _ffn_weights(torch, dev, H, I):
    """The same full weight matrices on every rank (seeded on the device), Kaiming-uniform-like."""
    g = torch.Generator(device=dev).manual_seed(100)
    mk = lambda r, c: ((torch.rand(r, c, device=dev, generator=g) * 2 - 1) * (1.0 / c) ** 0.5).to(torch.bfloat16)
    return mk(I, H), mk(I, H), mk(H, I)


def mx_ffn_block(torch, dist, dev, rank, world, T):
    """Forward of the Llama-style FFN block of config 5 (hidden 8192, intermediate 28672, T tokens,
    w fp4_e2m1, a fp8_e4m3, block 32, bfloat16), tensor-parallel over the ranks: column-parallel gate/up,
    row-parallel down, packed activations all-gathered, fp32 partials reduce-scattered.  Total work is
    fixed (strong scaling); the time is the max over ranks.  After the timing, 32 tokens of every rank's
    shard are recomputed by the unsharded block on rank 0 and compared."""
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.tp import TensorParallelFFN
    H, I = 8192, 28672
    if I % (128 * world) or T % (128 * world):
        return {"skipped": "shape does not split over %d ranks" % world}
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32,
                            "scale_bits": 8, "bfloat": 16, "custom_cuda": True})
    wg, wu, wd = _ffn_weights(torch, dev, H, I)
    ffn = TensorParallelFFN(H, I, sp, device=dev, dtype=torch.bfloat16)
    ffn.load_full(wg, wu, wd, torch.ones(H, device=dev, dtype=torch.bfloat16))
    with torch.no_grad():
        ffn.norm.bias.zero_()
    if world > 1:
        del wg, wu, wd
    gx = torch.Generator(device=dev).manual_seed(200 + rank)
    x = torch.randn(T // world, H, device=dev, dtype=torch.bfloat16, generator=gx)
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
    res = {"shape": "%d tokens, hidden 8192, intermediate 28672, SwiGLU + RMSNorm, w fp4_e2m1 / a fp8_e4m3" % T,
           "parallelism": "tp%d (column-parallel gate/up, row-parallel down; NCCL all-gather of packed activations; "
                          "%s)" % (world, "single GPU, no exchange" if world == 1 else
                                   "down-projection GEMM scatters its fp32 tiles into the owners' buffers over "
                                   "peer memory, then an ordered slab sum" if fused_scatter else
                                   "NCCL reduce-scatter of fp32 partials" +
                                   ("; %d token chunks, exchanges of a chunk under the GEMMs of its neighbours, "
                                    "%d SMs left to NCCL" % (ffn._token_chunks(T // world), ffn._comm_sms())
                                    if ffn._token_chunks(T // world) > 1 else "")),
           "ms": ms, "tflops": flop / (ms * 1e-3) / 1e12, "scaling": "strong",
           "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "library default")}
    # ---- numerics of the sharded block: 32 tokens per rank against the unsharded block on rank 0 ----
    if world > 1:
        n_chk = 32
        xs = [torch.empty(n_chk, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
        ys = [torch.empty(n_chk, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
        dist.all_gather(xs, x[:n_chk].contiguous())
        dist.all_gather(ys, y[:n_chk].contiguous())
        ffn.release_peer_buffers()
        del ffn
        torch.cuda.empty_cache()
        solo = [dist.new_group([r]) for r in range(world)]
        if rank == 0:
            wg, wu, wd = _ffn_weights(torch, dev, H, I)
            one = TensorParallelFFN(H, I, sp, group=solo[0], device=dev, dtype=torch.bfloat16)
            one.load_full(wg, wu, wd, torch.ones(H, device=dev, dtype=torch.bfloat16))
            with torch.no_grad():
                one.norm.bias.zero_()
            ref = one(torch.cat(xs, 0)).float()
            got = torch.cat(ys, 0).float()
            # bf16 spacing at each output, and at the size of the outputs of its token: an output that is a
            # near-cancelling sum of 28672 products legitimately moves by many of its own (tiny) ulps when the
            # fp32 partial sums are added in another order
            spacing = lambda t: torch.exp2(torch.floor(torch.log2(t.clamp_min(1e-30))) - 7)
            row = ref.pow(2).mean(dim=1, keepdim=True).sqrt()
            err = (got - ref).abs()
            res["numerics_vs_unsharded"] = {"tokens": n_chk * world,
                                            "frac_equal": float((got == ref).float().mean().item()),
                                            "max_ulp": float((err / spacing(ref.abs())).max().item()),
                                            "max_ulp_at_token_scale": float((err / spacing(torch.maximum(ref.abs(), row))).max().item())}
            del one, wg, wu, wd
        dist.barrier()
    else:
        del ffn
    del x, y
    torch.cuda.empty_cache()
    return res


def mx_ffn_injected(torch, dev, T):
    """Config 5 built the way it is specified: inject_pyt_ops first, then stock torch.nn.Linear, F.silu
    and torch.mul (plus the explicit mx.RMSNorm); one GPU, forward, weights re-quantized in every call as
    the reference does."""
    import torch.nn.functional as F
    import microxcaling_b200 as mx
    from microxcaling_b200 import mx_mapping
    from microxcaling_b200.specs import finalize_mx_specs
    H, I = 8192, 28672
    sp = finalize_mx_specs({"w_elem_format": "fp4_e2m1", "a_elem_format": "fp8_e4m3", "block_size": 32,
                            "scale_bits": 8, "bfloat": 16, "custom_cuda": True})

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = mx.RMSNorm(H, eps=1e-5, mx_specs=sp)
            self.gate = torch.nn.Linear(H, I, bias=False)
            self.up = torch.nn.Linear(H, I, bias=False)
            self.down = torch.nn.Linear(I, H, bias=False)

        def forward(self, x):
            h = self.norm(x)
            return self.down(torch.mul(F.silu(self.gate(h)), self.up(h)))

    with mx_mapping.injected(sp):
        torch.manual_seed(0)
        blk = Block().to(dev).to(torch.bfloat16).eval()
        x = torch.randn(T // 4096 if T >= 4096 else 1, min(T, 4096), H, device=dev, dtype=torch.bfloat16)

        def fwd(_):
            with torch.no_grad():
                return blk(x)
        t = timed(torch, fwd, 5, warm=2)
    flop = 3 * 2.0 * x.shape[0] * x.shape[1] * H * I
    del blk, x
    torch.cuda.empty_cache()
    return {"ms": t * 1e3, "tflops": flop / t / 1e12,
            "note": "stock torch.nn.Linear / F.silu / torch.mul after inject_pyt_ops; three weight packings, SiLU, "
                    "product and activation packing are separate kernels because every stock op returns its tensor"}


def cpu_baseline(torch, x_rows_f32):
    """Times the nine passes on a [rows, 8192] fp32-container slab with all host threads: the
    reference's own C++ math where oracle/_ref was built, else the C port."""
    import numpy as np
    import oracle
    x = np.ascontiguousarray(x_rows_f32)
    use_ref = oracle.ref() is not None
    fn_mx = oracle.ref_quantize_mx_f32 if use_ref else oracle.quantize_mx
    cores = host_threads()
    t0 = time.perf_counter()
    for fmt in MX_FORMATS:
        for axis in (0, 1):
            fn_mx(x, fmt, axis=axis, block=32, scale_bits=8, round="nearest", nthreads=cores)
    if use_ref:
        oracle.ref_quantize_elemwise_f32(x, 9, 8, BF16_MAX_NORM, "even", nthreads=cores)
    else:
        oracle.quantize_elemwise(x, 9, 8, BF16_MAX_NORM, "even", nthreads=cores)
    dt = time.perf_counter() - t0
    bytes_done = STEP_BYTES * x.shape[0] / ROWS          # counted like the GPU passes (bf16 / fp32+bf16 traffic)
    return {"value": bytes_done / dt / 1e9, "unit": "GB/s", "cores": int(cores),
            "kind": "reference" if use_ref else "port",
            "sample": "the nine passes on rows [0,%d) of the tensor held as fp32 values (%.2f s)" % (x.shape[0], dt)}, dt


def cpu_baseline_pytorch(torch, x_rows_f32):
    """The pure-PyTorch formulation of the same passes (what custom_cuda=False runs on CPU tensors),
    through this package's own torch-op path, on a small row slab with torch's host threads."""
    from microxcaling_b200.specs import finalize_mx_specs
    from microxcaling_b200.mx_ops import quantize_mx_op
    from microxcaling_b200.elemwise_ops import _quantize_bfloat
    sp = finalize_mx_specs({"a_elem_format": "fp6_e3m2", "block_size": 32, "scale_bits": 8, "custom_cuda": False})
    x = torch.as_tensor(x_rows_f32)
    t0 = time.perf_counter()
    for fmt in MX_FORMATS:
        for axis in (0, -1):
            quantize_mx_op(x, sp, elem_format=fmt, axes=[axis], round="nearest")
    _quantize_bfloat(x, 16, round="even", custom_cuda=False)
    dt = time.perf_counter() - t0
    return {"value": STEP_BYTES * x.shape[0] / ROWS / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": "the nine passes as torch ops (the custom_cuda=False formulation) on rows [0,%d), %.2f s"
                      % (x.shape[0], dt)}


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(host_threads())
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
    from microxcaling_b200.elemwise_ops import quantize_elemwise_op

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = be.lib()
    pk = peaks()
    hbm = pk["hbm_gbs"]
    only = args.only

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = {}
    if only in (None, "quantize"):
        x0 = make_input(torch, 1000 * rank, dev)
        xs = rotated(torch, x0, NBUF)
        ys = [torch.empty_like(x) for x in xs]
        xf = [x.float() for x in xs]                           # fp32 copies for the elementwise pass
        stream = torch.cuda.current_stream()
        sp = ctypes.c_void_p(stream.cuda_stream)
        fmt_params = {f: _get_format_params(f) for f in MX_FORMATS}
        launches = [0]

        def launch_pass(i):
            b = launches[0] % NBUF                             # buffers rotate per launch
            launches[0] += 1
            if i < 8:
                eb, mb, _, mn, _ = fmt_params[MX_FORMATS[i // 2]]
                pre, n, post = (1, ROWS, COLS) if i % 2 == 0 else (ROWS, COLS, 1)
                rc = L.mxq_quantize_mx(xs[b].data_ptr(), ys[b].data_ptr(), None, None, be.BF16, pre, n, post, 32, 8,
                                       eb, mb, mn, 0, 0, None, 0, 0, sp)
            else:
                rc = L.mxq_quantize_elemwise(xf[b].data_ptr(), ys[b].data_ptr(), be.F32, be.BF16, xf[b].numel(), 9, 8,
                                             BF16_MAX_NORM, 2, 0, 1, None, sp)
            if rc:
                be.check(rc)

        # one step: the four axis-0 passes, the four last-axis passes, the elementwise pass; one CUDA event at
        # each group boundary, so a kernel's average launch duration = group time / launches in the group
        ORDER = [0, 2, 4, 6, 1, 3, 5, 7, 8]
        GROUP_STARTS = (0, 4, 8)

        def step(events=None):
            for n, i in enumerate(ORDER):
                if events is not None and n in GROUP_STARTS:
                    events[GROUP_STARTS.index(n)].record(stream)
                launch_pass(i)
            if events is not None:
                events[3].record(stream)

        W = max(args.warmup, 3)
        for _ in range(W):
            step()
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
        launches[0] = 0
        t_start.record(stream)
        for s in range(K):
            step(ev[s])
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
                                   "round": "even", "custom_cuda": True})
        hx = xs[0].cpu().pin_memory()
        hxf = xf[0].cpu().pin_memory()
        del xf
        torch.cuda.empty_cache()

        def e2e_step():
            # host tensor in, host tensor out, through the public ops: the library cuts the tensor into
            # chunks and overlaps H2D, kernel and D2H (mxq_quantize_mx_host / mxq_quantize_elemwise_host)
            for i in range(PASSES):
                if i < 8:
                    hy = quantize_mx_op(hx, specs, elem_format=MX_FORMATS[i // 2], axes=[0 if i % 2 == 0 else -1],
                                        round="nearest")
                else:
                    hy = quantize_elemwise_op(hxf, specs, round="even")
                    assert hy.dtype == torch.bfloat16
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
        h2d = 8 * hx.numel() * 2 + hxf.numel() * 4
        d2h = 8 * hx.numel() * 2 + hxf.numel() * 2

        # what the host side allows: the same bytes as plain pinned copies, both directions at once on two
        # streams, no kernel -- every rank at the same time, so shared host memory and root ports show up
        def copies_only():
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            dx, dxf = torch.empty_like(hx, device=dev), torch.empty_like(hxf, device=dev)
            dy, hy = torch.empty_like(hx, device=dev), torch.empty_like(hx).pin_memory()
            assert hxf.numel() == hx.numel()

            def once():
                with torch.cuda.stream(s_in):
                    for _ in range(8):
                        dx.copy_(hx, non_blocking=True)
                    dxf.copy_(hxf, non_blocking=True)
                with torch.cuda.stream(s_out):
                    for _ in range(9):
                        hy.copy_(dy, non_blocking=True)
                torch.cuda.synchronize()
            once()
            barrier()
            c0 = time.perf_counter()
            for _ in range(2):
                once()
            barrier()
            return (time.perf_counter() - c0) / 2
        copy_s = copies_only()
        if world > 1:
            t = torch.tensor([copy_s], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            copy_s = float(t.item())

        value = world * STEP_BYTES * K / (total_ms * 1e-3) / 1e9
        strided_ms, last_ms = group_ms[0] / 4, group_ms[1] / 4
        achieved = MX_PASS_BYTES / (strided_ms * 1e-3) / 1e9
        traffic, traffic_from = captured_traffic("mx_strided_bf16_kernel")
        out = {
            "metric": "MX-quantize GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 / fp32 storage, fp32/u32 lane arithmetic",
            "data": "synthetic",
            "config": CONFIG,
            "roofline": {"bound": "hbm", "kernel": "mx_strided_bf16_kernel (axis-0 passes)", "achieved": achieved,
                         "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "peak_source": pk["source"],
                         "traffic": traffic, "traffic_from": traffic_from,
                         "other_kernels": {
                             "mx_lastaxis_bf16_kernel": {"gbs": MX_PASS_BYTES / (last_ms * 1e-3) / 1e9,
                                                         "frac": MX_PASS_BYTES / (last_ms * 1e-3) / 1e9 / hbm},
                             "ew_f32_to_bf16_rne_kernel": {"gbs": EW_PASS_BYTES / (group_ms[2] * 1e-3) / 1e9,
                                                                "frac": EW_PASS_BYTES / (group_ms[2] * 1e-3) / 1e9 / hbm}}},
            "e2e": {"value": world * STEP_BYTES / e2e_s / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3,
                    "copies_only": {"value": world * STEP_BYTES / copy_s / 1e9, "unit": "GB/s",
                                    "note": "the same metric with the step's bytes moved as plain pinned copies, "
                                            "both directions at once, by every rank at the same time: the host-side "
                                            "ceiling of e2e on this box"}},
            "gpu_launches": PASSES * K,
            "clocks": clocks,
        }
        cpu_slab = xs[0][:CPU_SAMPLE_ROWS].float().cpu().numpy() if rank == 0 and world == 1 else None
        del xs, ys, hx, hxf
        torch.cuda.empty_cache()
        if cpu_slab is not None:
            cb, _ = cpu_baseline(torch, cpu_slab)
            out["cpu_baseline"] = cb
            out["cpu_baseline_pytorch"] = cpu_baseline_pytorch(torch, cpu_slab[:512])
    else:
        out = {"only": only, "n_gpus": world}

    # ---- single-GPU blocks on rank 0 ----
    if rank == 0:
        if only in (None, "config1"):
            out["config1"] = config1_block(torch, be, dev, hbm)
        if only in (None, "pack"):
            out["pack"] = pack_block(torch, be, dev, hbm)
        if only in (None, "vector"):
            out["vector"] = vector_block(torch, be, dev, hbm)
        if only in (None, "linear"):
            out["mx_linear"] = mx_linear_block(torch, be, dev)
        if only in (None, "attention"):
            out["mx_attention"] = mx_attention_block(torch, dev)
        if only in (None, "ffn") and world == 1:
            out["mx_ffn_injected"] = mx_ffn_injected(torch, dev, args.ffn_tokens)
    # ---- tensor-parallel MX FFN (config 5 shape), all ranks ----
    if only in (None, "ffn"):
        ffn = mx_ffn_block(torch, dist, dev, rank, world, args.ffn_tokens)
        if rank == 0:
            out["mx_ffn"] = ffn
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
