"""Tensor-parallel MX feed-forward block (Llama style: RMSNorm -> gate/up ->
SiLU(gate) * up -> down) over the GPUs of one node.

The reference has no distributed code; this module adds the one exchange pattern
its FFN admits without changing results beyond fp32 accumulation order:

  * tokens are sharded across ranks for everything that is token-local
    (RMSNorm, MX quantization of the block input along `hidden`);
  * the packed input (one code byte per element + E8M0 scales) is all-gathered,
    4x fewer bytes than fp32 values;
  * gate/up are column-parallel: each rank owns `intermediate / p` output
    features, so every output element is a complete dot product and equals the
    single-GPU value bit for bit;
  * SiLU and the product are elementwise on the local columns;
  * down is row-parallel: each rank contracts over its slice of `intermediate`
    (a multiple of 32, so MX blocks never straddle ranks), the fp32 partial sums
    are reduce-scattered over tokens and rounded to bfloat once, after the sum.
    On GPUs with peer access the scatter is part of the GEMM: every finished
    128-row tile is stored straight into the receive buffer of the rank that
    owns those tokens (mxq_gemm_mx_scatter), one small NCCL all-reduce orders
    the ranks, and each rank adds the slabs it received in rank order
    (mxq_sum_slabs_f32).  This is the default for two ranks; for more ranks the
    NCCL reduce-scatter is faster (see _local_scatter_eligible) and is used unless
    MXQ_TP_FUSED_SCATTER=1.  The ranks agree on the branch collectively.

On CUDA tensors the GEMMs run on packed operands through libmxq; on CPU tensors
(used by the gloo tests of this logic) the same steps run on fake-quantized
values with torch's GEMM.  `world_size == 1` skips the collectives.
"""
import os

import torch
import torch.distributed as dist

from . import activations, layernorm, simd_ops
from ._mxgemm import _MODE, _fast_ok, _fmt, _pack, mx_gemm
from .elemwise_ops import quantize_elemwise_op
from .formats import _get_format_params
from .specs import apply_mx_specs
from .vector_ops import fused_bf16_ok

# SMs the token-chunked forward leaves to the collectives that run beside its GEMMs (MXQ_TP_COMM_SMS
# overrides; 0 = none).  NCCL's reduce-scatter of the fp32 partial sums wants about 32 CTAs: at 4 ranks
# 16384 tokens took 3.10 ms with no room, 3.03 ms with 32 SMs, 3.12 ms with 16.
_COMM_SMS = 32


def shard_bounds(n, rank, world, multiple=1):
    """[lo, hi) of rank's contiguous shard of n items; n must split evenly into
    shards that are multiples of `multiple`."""
    if n % world != 0 or (n // world) % multiple != 0:
        raise ValueError("cannot split %d items over %d ranks in multiples of %d" % (n, world, multiple))
    per = n // world
    return rank * per, (rank + 1) * per


class _PeerSlabs:
    """One fp32 receive buffer [world, rows, cols] per rank, each mapped into every
    other rank of the node through CUDA IPC (plain peer mappings opened under the
    importer's own device, no multicast object).  Slab s of a rank's buffer is
    written by rank s only."""

    def __init__(self, group, world, rank, rows, cols, device):
        from . import _backend as be
        self.rows, self.cols, self.world, self.device = rows, cols, world, device
        self.local, self.opened, self.my_slab_on = None, [], []
        slab_bytes = rows * cols * 4
        handle = None
        try:
            self.local, handle = be.peer_alloc(device, world * slab_bytes)
        except Exception:                                   # every rank still takes part in the exchange below
            pass
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        self.ok = all(h is not None for h in handles)
        if self.ok:
            try:
                self.opened = [None if r == rank else be.peer_open(device, h) for r, h in enumerate(handles)]
                self.my_slab_on = [(self.local if r == rank else p) + rank * slab_bytes
                                   for r, p in enumerate(self.opened)]
            except Exception:
                self.ok = False
        self.token = torch.zeros(1, dtype=torch.float32, device=device)

    def close(self):
        """Collective in spirit: every rank closes its mappings before any owner frees its buffer
        (call it on all ranks, with a barrier in between if the ranks are not already in step)."""
        from . import _backend as be
        for p in self.opened:
            if p is not None:
                be.peer_close(p)
        self.opened = []

    def free(self):
        from . import _backend as be
        if self.local:
            be.peer_free(self.local)
            self.local = None


def _local_scatter_eligible(device, world):
    """This rank's own view: may the scattering GEMM be used?  (The ranks then agree on the
    minimum over all views, see TensorParallelFFN._use_scatter.)
    Measured on B200 / NVSwitch (config-5 FFN forward) the scattering GEMM wins for two ranks and
    loses to the NCCL reduce-scatter beyond that, so it is the default only for two ranks;
    MXQ_TP_FUSED_SCATTER=1 asks for it at any size, =0 forbids it."""
    mode = os.environ.get("MXQ_TP_FUSED_SCATTER", "")
    if mode == "0" or world > 8 or (mode != "1" and world > 2):
        return False
    return device.type == "cuda"


class TensorParallelFFN(torch.nn.Module):
    def __init__(self, hidden, intermediate, mx_specs, group=None, eps=1e-5, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.hidden, self.intermediate = hidden, intermediate
        self.mx_specs = apply_mx_specs(mx_specs)
        lo, hi = shard_bounds(intermediate, self.rank, self.world, multiple=128)
        self.cols = (lo, hi)
        kw = dict(device=device, dtype=dtype)
        self.norm = layernorm.RMSNorm(hidden, eps=eps, mx_specs=mx_specs).to(**kw)
        self.w_gate = torch.nn.Parameter(torch.empty(hi - lo, hidden, **kw))
        self.w_up = torch.nn.Parameter(torch.empty(hi - lo, hidden, **kw))
        self.w_down = torch.nn.Parameter(torch.empty(hidden, hi - lo, **kw))
        self._packed = None                     # (key, packed weights), see _weights_packed
        self._slabs = None
        self._scatter = None                    # agreed by all ranks on the first multi-rank forward

    def _use_scatter(self, device):
        """Collective, once: every rank must take the same branch (scattering GEMM or NCCL
        reduce-scatter), or the collectives of the two branches would be mismatched.  Each rank
        contributes its own eligibility and its real device index; the answer is the minimum over
        ranks, with peer access checked between the devices the ranks really run on."""
        if self._scatter is None:
            mine = _local_scatter_eligible(device, self.world)
            idx = device.index if device.index is not None else (torch.cuda.current_device() if device.type == "cuda" else -1)
            info = [None] * self.world
            dist.all_gather_object(info, (bool(mine), int(idx)), group=self.group)
            ok = all(e for e, _ in info)
            if ok:
                devs = [d for _, d in info]
                ok = len(set(devs)) == self.world and all(
                    d == idx or (0 <= d < torch.cuda.device_count() and torch.cuda.can_device_access_peer(idx, d))
                    for d in devs)
            flag = torch.tensor([1.0 if ok else 0.0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            self._scatter = float(flag.item()) >= 1.0
        return self._scatter

    def _make_slabs(self, rows, device):
        """Collective: either every rank ends up with mapped receive buffers or none does (then the
        NCCL reduce-scatter is used from here on)."""
        slabs = _PeerSlabs(self.group, self.world, self.rank, rows, self.hidden, device)
        flag = torch.tensor([1.0 if slabs.ok else 0.0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if float(flag.item()) < 1.0:                        # no IPC / peer mapping somewhere: nobody uses it
            slabs.close()
            dist.barrier(group=self.group)
            slabs.free()
            self._scatter = False
            return None
        return slabs

    def release_peer_buffers(self):
        """Unmap and free the receive buffers of the scattering GEMM (all ranks call this together)."""
        if self._slabs is not None:
            torch.cuda.synchronize()
            self._slabs.close()
            if self.world > 1:
                dist.barrier(group=self.group)
            self._slabs.free()
            self._slabs = None

    @torch.no_grad()
    def load_full(self, w_gate, w_up, w_down, norm_weight=None):
        """Take this rank's shards out of full (unsharded) weight matrices."""
        lo, hi = self.cols
        self.w_gate.copy_(w_gate[lo:hi])
        self.w_up.copy_(w_up[lo:hi])
        self.w_down.copy_(w_down[:, lo:hi])
        if norm_weight is not None:
            self.norm.weight.copy_(norm_weight)
        self._packed = None

    # ------------------------------------------------------------------ helpers
    def _fast(self, x):
        sp = self.mx_specs
        return _fast_ok(x, self.w_gate, _fmt(sp["a_elem_format"]), _fmt(sp["w_elem_format"]), sp, self.hidden,
                        sp["round_mx_output"], sp["round_mx_output"], sp["round_output"]) and \
            (self.cols[1] - self.cols[0]) % 128 == 0

    def _weights_packed(self):
        """The three weight shards as packed MX operands, remade when a parameter's storage or version
        counter changes (an optimizer step, load_state_dict, load_full).  Writes that bypass the
        version counter (`w.data.mul_()`) are not seen: call invalidate_packed_weights() after them."""
        ws = (self.w_gate, self.w_up, self.w_down)
        key = tuple((w.data_ptr(), w._version) for w in ws)
        if self._packed is None or self._packed[0] != key:
            sp = self.mx_specs
            rnd = sp["round_mx_output"]
            wf = _fmt(sp["w_elem_format"])
            q = lambda w: _pack(quantize_elemwise_op(w.detach(), sp, round=sp["round_weight"]), wf, sp, rnd, True)
            self._packed = (key, tuple(q(w) for w in ws))
        return self._packed[1]

    def invalidate_packed_weights(self):
        self._packed = None

    def _all_gather_rows(self, t):
        if self.world == 1:
            return t
        out = torch.empty((t.shape[0] * self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def _reduce_scatter_rows(self, t):
        if self.world == 1:
            return t
        out = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t.contiguous(), op=dist.ReduceOp.SUM, group=self.group)
        return out

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, x_local):
        """x_local: this rank's [tokens / p, hidden] slice (tokens / p a multiple of 128 when p > 1).
        Returns the same slice of the block output."""
        sp = self.mx_specs
        if x_local.dim() != 2 or x_local.shape[1] != self.hidden:
            raise ValueError("expected a [tokens, hidden] tensor")
        if self.world > 1 and x_local.shape[0] % 128 != 0:
            raise ValueError("the per-rank token count must be a multiple of 128")
        h = self.norm(x_local)
        if self._fast(h):
            return self._forward_packed(h)
        return self._forward_values(h)

    def _forward_packed(self, h):
        from . import _backend as be
        sp = self.mx_specs
        af = _fmt(sp["a_elem_format"])
        rnd, out_rnd = sp["round_mx_output"], _MODE[sp["round_output"]]
        bits = sp["bfloat"] if sp["bfloat"] >= 10 else 0
        pg, pu, pd = self._weights_packed()
        h = quantize_elemwise_op(h, sp, round=sp["round_output"])
        px = _pack(h, af, sp, rnd, True)                               # local tokens
        n_chunks = self._token_chunks(h.shape[0])
        if n_chunks > 1 and not self._use_scatter(h.device):
            return self._forward_pipelined(h, px, pg, pu, pd, n_chunks)
        xc, xs, xk = self._all_gather_rows(px.codes.reshape(-1, self.hidden)), \
            self._all_gather_rows(px.scales.view(-1, 512)).view(-1), px.container
        T = xc.shape[0]
        Il = self.cols[1] - self.cols[0]
        gate = be.gemm_mx(xc, xs, pg.codes, pg.scales, 1, T, Il, self.hidden, xk, pg.container, out_dtype=h.dtype,
                          bfloat_bits=bits, round_mode=out_rnd)[0]
        up = be.gemm_mx(xc, xs, pu.codes, pu.scales, 1, T, Il, self.hidden, xk, pu.container, out_dtype=h.dtype,
                        bfloat_bits=bits, round_mode=out_rnd)[0]
        if fused_bf16_ok(sp, gate, up) and Il % 32 == 0 and sp["round_output"] in ("nearest", "floor", "even"):
            # SiLU(gate) * up and the MX packing of the product in one pass; the vector format leaves
            # bfloat16 values untouched, so the rounding between the two steps is the identity
            eb, mb, _, mn, _ = _get_format_params(af)
            ac, as_ = be.swiglu_quantize_mx(gate, up, sp["scale_bits"] or 8, eb, mb, mn, sp["mx_flush_fp32_subnorms"],
                                            _MODE[rnd])
            ak = 1 if eb == 5 else 0
        else:
            act = simd_ops.simd_mul(activations.silu(gate, mx_specs=sp), up, mx_specs=sp)
            act = quantize_elemwise_op(act, sp, round=sp["round_output"])
            pa = _pack(act, af, sp, rnd, True)
            ac, as_, ak = pa.codes, pa.scales, pa.container
        dc, ds, dk = pd.codes, pd.scales, pd.container
        if self.world == 1:
            return be.gemm_mx(ac, as_, dc, ds, 1, T, self.hidden, Il, ak, dk, out_dtype=h.dtype, bfloat_bits=bits,
                              round_mode=out_rnd)[0]
        rows = T // self.world
        if self._slabs is None and self._use_scatter(h.device):
            self._slabs = self._make_slabs(rows, h.device)
        sl = self._slabs
        if sl is not None and (sl.rows, sl.cols) == (rows, self.hidden):
            # GEMM + scatter in one kernel; the previous call's slabs were consumed before any rank
            # could get past this call's all-gather, so they may be overwritten now
            be.gemm_mx_scatter(ac, as_, dc, ds, sl.my_slab_on, rows, T, self.hidden, Il, ak, dk)
            dist.all_reduce(sl.token, group=self.group)           # every rank's tiles have landed
            out = be.sum_slabs(sl.local, self.world, (rows, self.hidden), h.device)
        else:
            out = self._down_chunked(ac, as_, ak, dc, ds, dk, T, Il, rows)
        out = quantize_elemwise_op(out, sp, round=sp["round_output"])
        return out.to(h.dtype)

    def _gemm_sms(self, device):
        """SMs the GEMMs keep while a collective runs beside them: the device's SMs less MXQ_TP_COMM_SMS
        (0 = all: the GEMM is persistent, one CTA per SM, so without room the collective's CTAs only
        start when the GEMM ends and nothing overlaps)."""
        reserve = self._comm_sms()
        if reserve <= 0:
            return 0
        return max(torch.cuda.get_device_properties(device).multi_processor_count - reserve, 2)

    @staticmethod
    def _comm_sms():
        return int(os.environ.get("MXQ_TP_COMM_SMS", str(_COMM_SMS)))

    def _token_chunks(self, local_tokens):
        """Token chunks of the pipelined forward: more than one only with several ranks, for whole
        128-row groups per chunk; MXQ_TP_TOKEN_CHUNKS overrides (1 = off)."""
        if self.world == 1:
            return 1
        want = int(os.environ.get("MXQ_TP_TOKEN_CHUNKS", "0")) or (4 if self.world >= 4 else 1)
        while want > 1 and (local_tokens % (128 * want) != 0):
            want -= 1
        return max(want, 1)

    def _forward_pipelined(self, h, px, pg, pu, pd, n_chunks):
        """The forward pass cut into token chunks (chunk c = the c-th part of EVERY rank's tokens, so each
        chunk's exchange is balanced): the all-gather of chunk c+1's packed input and the reduce-scatter of
        chunk c's fp32 partial sums run on NCCL's stream under the GEMMs of the neighbouring chunks.  Every
        output element sums the same per-rank partials as the unchunked pass."""
        from . import _backend as be
        sp = self.mx_specs
        af = _fmt(sp["a_elem_format"])
        rnd, out_rnd = sp["round_mx_output"], _MODE[sp["round_output"]]
        bits = sp["bfloat"] if sp["bfloat"] >= 10 else 0
        H, Il, W = self.hidden, self.cols[1] - self.cols[0], self.world
        Tl = h.shape[0]
        rc = Tl // n_chunks                                     # local rows per chunk (multiple of 128)
        sf_per_chunk = (rc // 128) * ((H + 127) // 128) * 512   # scale bytes of one local chunk (contiguous)
        codes = px.codes.reshape(Tl, H)
        scales = px.scales.view(-1)
        eb, mb, _, mn, _ = _get_format_params(af)
        fused = fused_bf16_ok(sp, h) and Il % 32 == 0 and sp["round_output"] in ("nearest", "floor", "even")

        def gather(c):
            xc = torch.empty((W * rc, H), dtype=torch.uint8, device=h.device)
            xs = torch.empty(W * sf_per_chunk, dtype=torch.uint8, device=h.device)
            w1 = dist.all_gather_into_tensor(xc, codes[c * rc:(c + 1) * rc], group=self.group, async_op=True)
            w2 = dist.all_gather_into_tensor(xs, scales[c * sf_per_chunk:(c + 1) * sf_per_chunk], group=self.group,
                                             async_op=True)
            return xc, xs, (w1, w2)

        nxt = gather(0)
        outs, works = [], []
        with be.gemm_sm_budget(self._gemm_sms(h.device)):      # every GEMM here has an exchange beside it
            for c in range(n_chunks):
                xc, xs, ws = nxt
                for w in ws:
                    w.wait()
                if c + 1 < n_chunks:
                    nxt = gather(c + 1)
                M = W * rc
                gate = be.gemm_mx(xc, xs, pg.codes, pg.scales, 1, M, Il, H, px.container, pg.container, out_dtype=h.dtype,
                                  bfloat_bits=bits, round_mode=out_rnd)[0]
                up = be.gemm_mx(xc, xs, pu.codes, pu.scales, 1, M, Il, H, px.container, pu.container, out_dtype=h.dtype,
                                bfloat_bits=bits, round_mode=out_rnd)[0]
                if fused:
                    ac, as_ = be.swiglu_quantize_mx(gate, up, sp["scale_bits"] or 8, eb, mb, mn, sp["mx_flush_fp32_subnorms"],
                                                    _MODE[rnd])
                    ak = 1 if eb == 5 else 0
                else:
                    act = simd_ops.simd_mul(activations.silu(gate, mx_specs=sp), up, mx_specs=sp)
                    pa = _pack(quantize_elemwise_op(act, sp, round=sp["round_output"]), af, sp, rnd, True)
                    ac, as_, ak = pa.codes, pa.scales, pa.container
                part = be.gemm_mx(ac, as_, pd.codes, pd.scales, 1, M, H, Il, ak, pd.container, out_dtype=torch.float32,
                                  bfloat_bits=0, round_mode=-1)[0]
                o = torch.empty((rc, H), dtype=torch.float32, device=h.device)
                works.append(dist.reduce_scatter_tensor(o, part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
                outs.append(o)
        for w in works:
            w.wait()
        out = quantize_elemwise_op(torch.cat(outs, dim=0), sp, round=sp["round_output"])
        return out.to(h.dtype)

    def _down_chunked(self, ac, as_, ak, dc, ds, dk, T, Il, rows):
        """Down projection + NCCL reduce-scatter, pipelined: the output features are cut into slabs (whole
        128-row groups of the packed weight, so codes and scale chunks of a slab are contiguous); the
        reduce-scatter of slab c runs on NCCL's stream while the GEMM of slab c + 1 runs on the compute
        stream.  Every output element still sums the same per-rank partials."""
        from . import _backend as be
        H = self.hidden
        n_slabs = 4 if H % (4 * 256) == 0 else 1
        slab = H // n_slabs
        kchunks = (Il + 127) // 128
        codes2d = dc.reshape(H, Il)
        outs, works = [], []
        for c in range(n_slabs):
            b_codes = codes2d[c * slab:(c + 1) * slab]
            b_scales = ds.view(-1)[(c * slab // 128) * kchunks * 512:((c + 1) * slab // 128) * kchunks * 512]
            part = be.gemm_mx(ac, as_, b_codes, b_scales, 1, T, slab, Il, ak, dk, out_dtype=torch.float32,
                              bfloat_bits=0, round_mode=-1)[0]
            o = torch.empty((rows, slab), dtype=torch.float32, device=part.device)
            works.append(dist.reduce_scatter_tensor(o, part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            outs.append(o)
        for w in works:
            w.wait()
        return outs[0] if n_slabs == 1 else torch.cat(outs, dim=1)

    def _forward_values(self, h):
        sp = self.mx_specs
        no_round = sp.copy()
        no_round["bfloat"], no_round["fp"] = 0, 0
        af, wf, rnd = sp["a_elem_format"], sp["w_elem_format"], sp["round_mx_output"]
        h = quantize_elemwise_op(h, sp, round=sp["round_output"])
        x = self._all_gather_rows(h)
        qw = lambda w: quantize_elemwise_op(w.detach().to(x.dtype), sp, round=sp["round_weight"])
        gate = mx_gemm(x, qw(self.w_gate), af, wf, sp, rnd, rnd, sp["round_output"], trans2=True)
        up = mx_gemm(x, qw(self.w_up), af, wf, sp, rnd, rnd, sp["round_output"], trans2=True)
        act = simd_ops.simd_mul(activations.silu(gate, mx_specs=sp), up, mx_specs=sp)
        act = quantize_elemwise_op(act, sp, round=sp["round_output"])
        if self.world == 1:
            return mx_gemm(act, qw(self.w_down), af, wf, sp, rnd, rnd, sp["round_output"], trans2=True)
        part = mx_gemm(act.float(), qw(self.w_down).float(), af, wf, no_round, rnd, rnd, "nearest", trans2=True)
        out = self._reduce_scatter_rows(part)
        return quantize_elemwise_op(out, sp, round=sp["round_output"]).to(h.dtype)
