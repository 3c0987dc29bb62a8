#!/usr/bin/env python
"""Benchmark of the scan hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--only c0|c1|c2|c3|c4]

One JSON line.  The headline (`metric`, `value`, `roofline`, `e2e`, `cpu_baseline`) is the Mamba-1 selective
scan at the 2.8B-layer shape (batch 8, d_inner 5120, seqlen 2048, d_state 16, bf16); `workloads` carries the
other configurations of the path with the same fields:

    c2  Mamba-2 SSD chunked scan        batch 8, seqlen 4096, 80 heads x 64, 1 group, d_state 128, chunk 256, gated
    c3  Mamba-2 SSD, long sequence      batch 1, seqlen 262144, 128 heads x 64, 8 groups, d_state 128, no gate
    c4  Mamba-2 decode state update     batch 256, 80 heads x 64, d_state 128, fp32 state, consecutive in-place steps

With N > 1 (torchrun, one rank per GPU) every workload is the SAME fixed problem, divided: c1 by batch rows,
c2 by heads, c4 by batch rows (independent units, no collective on the data path) and c3 by contiguous chunk
ranges of the sequence with the range states exchanged by NCCL.  `value` is whole-problem tokens per second,
timed on the device as the maximum over ranks ("scaling": "strong").

Timing: W warm-up steps, then R blocks of exactly K steps, each block bracketed by a barrier and a device
synchronisation and timed with CUDA events on the launching stream; the MEDIAN block sets the reported time.
R is chosen so that the timed blocks cover at least 0.3 s (5 <= R <= 400), long enough for the clock sampler.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC, UNIT = "scan_fwd_tokens_per_s", "tokens/s"

# DRAM bytes (read + write) per launch group of a full single-GPU step, from the committed ncu captures
NCU_TRAFFIC = {
    "c1": (659_956_992, "profiles/scan_stream_kernel__config1.md"),
    "c2": (1_735_000_000, "profiles/ssd_chunk_scan_forward__config2.md + profiles/ssd_state_stream_kernel__config2.md"),
    "c3": (20_734_000_000, "profiles/ssd_forward__config3_eighth.md (captured on an eighth of the sequence, scaled by 8: every kernel's traffic grows with the number of chunks)"),
    "c4": (1_291_591_424, "profiles/ssu_packet_kernel__config4.md"),
    "c1b": (3_002_000_000, "profiles/scan_bwd_kernels__config1_shape.md"),
}

WORKLOAD_DESC = {
    "c0": "mamba1_selective_scan_fwd fp32 b2 d256 L512 N16",
    "c1": "mamba1_selective_scan_fwd bf16 b8 d5120 L2048 N16 (2.8B layer)",
    "c1b": "mamba1_selective_scan_bwd bf16 b8 d5120 L2048 N16 (gradients of c1 for a seeded dout; --only c1b, not part of the default line)",
    "c2": "mamba2_ssd_chunk_scan_fwd bf16 b8 L4096 h80 P64 g1 N128 Q256 (+z, +final_states)",
    "c3": "mamba2_ssd_chunk_scan_fwd bf16 b1 L262144 h128 P64 g8 N128 Q256 (no z, +final_states)",
    "c4": "mamba2_selective_state_update b256 h80 P64 g1 N128, fp32 state, bf16 activations, consecutive steps",
}
PARTITION = {
    "c0": "replicas only (correctness configuration)",
    "c1": "batch rows divided over the GPUs, no collective",
    "c1b": "batch rows divided over the GPUs; parameter gradients (dA, dD, ddelta_bias) would be summed by the caller",
    "c2": "heads divided over the GPUs (B and C replicated), no collective",
    "c3": "contiguous chunk ranges of the sequence per GPU; range states exchanged by NCCL (all-gather + local fold)",
    "c4": "batch rows divided over the GPUs, each owning its slice of the state; no collective",
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def split_even(total, world, rank):
    """Contiguous share [lo, hi) of `total` units for `rank`."""
    per, extra = divmod(total, world)
    lo = rank * per + min(rank, extra)
    return lo, lo + per + (1 if rank < extra else 0)


# ----------------------------------------------------------------------------------------- inputs
def softplus_inv_dt(n, g):
    dt = torch.exp(torch.rand(n, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    return dt + torch.log(-torch.expm1(-dt))


def make_c1_rows(rows, dim=5120, L=2048, N=16, seed=1001, dtype=torch.bfloat16):
    """Host tensors of the given batch rows of config 1 (a row's data depends only on its index)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    par = dict(A=-torch.exp(r(dim, N)), D=r(dim), delta_bias=softplus_inv_dt(dim, g))
    cols = {k: [] for k in ("u", "delta", "z", "B", "C")}
    for row in rows:
        gr = torch.Generator().manual_seed(seed * 1000 + row)
        rr = lambda *s: torch.randn(*s, generator=gr)
        for k, shape in (("u", (1, dim, L)), ("delta", (1, dim, L)), ("z", (1, dim, L)), ("B", (1, 1, N, L)), ("C", (1, 1, N, L))):
            cols[k].append(rr(*shape).to(dtype))
    empty = {"u": (0, dim, L), "delta": (0, dim, L), "z": (0, dim, L), "B": (0, 1, N, L), "C": (0, 1, N, L)}
    par.update({k: (torch.cat(v) if v else torch.zeros(empty[k], dtype=dtype)) for k, v in cols.items()})
    return par


def make_c0(batch=2, dim=256, L=512, N=16, seed=1000):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return dict(u=r(batch, dim, L), delta=r(batch, dim, L), z=r(batch, dim, L), A=-torch.exp(r(dim, N)),
                B=r(batch, 1, N, L), C=r(batch, 1, N, L), D=r(dim), delta_bias=-4 + 2 * torch.rand(dim, generator=g))


def ssd_params(H, seed):
    g = torch.Generator().manual_seed(seed)
    return dict(A=-(1 + 15 * torch.rand(H, generator=g)), D=torch.randn(H, generator=g), dt_bias=softplus_inv_dt(H, g))


class Workload:
    """One configuration, this rank's share of it: device step, byte counts, CPU-baseline sample."""

    def __init__(self, name, dev, rank=0, world=1, batch=None):
        """`batch` shrinks the batch (profiling captures of a small case only; the JSON line then says so)."""
        import mamba_b200 as mb
        self.mb, self.name, self.dev, self.rank, self.world = mb, name, dev, rank, world
        self.reduced = batch is not None
        self.desc, self.partition = WORKLOAD_DESC[name], PARTITION[name]
        self.step_no = 0
        self.flops = None
        bf = torch.bfloat16
        if name in ("c1", "c0", "c1b"):
            if name != "c0":
                nb = batch or 8
                lo, hi = split_even(nb, world, rank)
                host = make_c1_rows(range(lo, hi))
                self.global_tokens = nb * 2048
            else:
                host = make_c0()
                self.global_tokens = 2 * 512
            b, d, L = host["u"].shape
            esz = host["u"].element_size()
            self.shape = dict(batch=b, d_inner=d, seqlen=L, d_state=16)
            self.dtype = "f32" if name == "c0" else "bf16"
            self.alg_bytes = 4 * b * d * L * esz + 2 * b * 16 * L * esz + d * 16 * 4 + 2 * d * 4 + b * d * 16 * 4
            self.launches_per_step = 1 if b > 0 else 0
            self.kernels = "scan_stream_kernel"
            self.host = host
            self.d = {k: v.to(dev) for k, v in host.items()}
            if name == "c1b":
                # reads u, delta, z, dout, B, C; writes du, ddelta, dz, fp32 dB and dC, and the parameter gradients
                g = torch.Generator().manual_seed(1001 + 7919 * rank)
                self.d["dout"] = torch.randn(b, d, L, generator=g).to(bf).to(dev)
                self.alg_bytes = 7 * b * d * L * esz + 2 * b * 16 * L * (esz + 4) + 2 * d * 16 * 4 + 4 * d * 4
                self.launches_per_step = 2 if b > 0 else 0
                self.kernels = "scan_bwd_states_kernel, scan_bwd_kernel (+ 5 memsets of the accumulators)"
        elif name == "c2":
            nb, L, Hall, P, N = batch or 8, 4096, 80, 64, 128
            lo, hi = split_even(Hall, world, rank)
            H = hi - lo
            g = torch.Generator(device=dev).manual_seed(1002)
            r = lambda *s: torch.randn(*s, generator=g, device=dev)
            par = ssd_params(Hall, 1002)
            # B and C belong to the one group and are the same on every rank; x, dt, z are this rank's heads
            Bc, Cc = r(nb, L, 1, N).to(bf), r(nb, L, 1, N).to(bf)
            g.manual_seed(100200 + rank)
            self.d = dict(x=r(nb, L, H, P).to(bf), dt=r(nb, L, H).to(bf), z=r(nb, L, H, P).to(bf), B=Bc, C=Cc,
                          **{k: v[lo:hi].to(dev) for k, v in par.items()})
            self.shape = dict(batch=nb, seqlen=L, nheads=H, headdim=P, ngroups=1, d_state=N, chunk_size=256)
            self.global_tokens = nb * L
            self.dtype = "bf16"
            self.alg_bytes = 3 * nb * L * H * P * 2 + nb * L * H * 2 + 2 * nb * L * N * 2 + nb * H * P * N * 4 + 3 * H * 4
            self.flops = nb * L * (2 * 256 * N + H * (2 * P * N + 2 * 256 * P + 2 * N * P))   # C.B^T, chunk state, intra-chunk (dense), C.state
            self.launches_per_step = 5 if H > 0 else 0
            self.kernels = "ssd_tc_cb, ssd_cumsum, ssd_tc_state_stream (pairs, singles), ssd_tc_chunk_scan"
        elif name == "c3":
            from mamba_b200.seqpar import split_sequence
            Ltot, H, P, G, N = (batch or 1) * 262144, 128, 64, 8, 128
            if self.reduced:
                Ltot = 262144 // 8
            lo, hi = split_sequence(Ltot, 256, world, rank)
            Lr = hi - lo
            g = torch.Generator(device=dev).manual_seed(1003 + rank)
            r = lambda *s: torch.randn(*s, generator=g, device=dev)
            self.d = dict(x=r(1, Lr, H, P).to(bf), dt=r(1, Lr, H).to(bf), B=r(1, Lr, G, N).to(bf), C=r(1, Lr, G, N).to(bf),
                          **{k: v.to(dev) for k, v in ssd_params(H, 1003).items()})
            self.shape = dict(batch=1, seqlen_total=Ltot, seqlen_this_gpu=Lr, nheads=H, headdim=P, ngroups=G, d_state=N, chunk_size=256)
            self.global_tokens = Ltot
            self.dtype = "bf16"
            self.alg_bytes = 2 * Lr * H * P * 2 + Lr * H * 2 + 2 * Lr * G * N * 2 + H * P * N * 4 + 3 * H * 4
            self.flops = Lr * (G * 2 * 256 * N + H * (2 * P * N + 2 * 256 * P + 2 * N * P))
            self.launches_per_step = 4 if world == 1 else 7
            self.kernels = ("ssd_tc_cb, ssd_cumsum, ssd_tc_state_stream, ssd_tc_chunk_scan" if world == 1 else
                            "ssd_cumsum, ssd_tc_state_stream, ssd_fold_ranges, ssd_incoming_state, ssd_tc_cb, ssd_tc_chunk_scan (+ NCCL all-gather)")
        elif name == "c4":
            nb_all, H, P, N, pool = batch or 256, 80, 64, 128, 4
            lo, hi = split_even(nb_all, world, rank)
            nb = hi - lo
            g = torch.Generator(device=dev).manual_seed(1004 + rank)
            r = lambda *s: torch.randn(*s, generator=g, device=dev)
            par = ssd_params(H, 1004)
            # `pool` distinct token inputs are rotated through the steps; the state is updated in place
            self.d = dict(state=0.1 * r(nb, H, P, N), x=r(pool, nb, H, P).to(bf), z=r(pool, nb, H, P).to(bf), dt=r(pool, nb, H).to(bf),
                          B=r(pool, nb, 1, N).to(bf), C=r(pool, nb, 1, N).to(bf), **{k: v.to(dev) for k, v in par.items()})
            self.A3 = self.d["A"][:, None, None].expand(H, P, N)
            self.D2 = self.d["D"][:, None].expand(H, P)
            self.bias2 = self.d["dt_bias"][:, None].expand(H, P)
            self.shape = dict(batch=nb, nheads=H, headdim=P, ngroups=1, d_state=N, consecutive_steps=True)
            self.global_tokens = nb_all
            self.dtype = "f32"
            self.alg_bytes = 2 * nb * H * P * N * 4 + 3 * nb * H * P * 2 + nb * H * 2 + 2 * nb * N * 2 + 3 * H * 4
            self.launches_per_step = 1 if nb > 0 else 0
            self.kernels = "ssu_packet_kernel"
        else:
            raise SystemExit(f"unknown workload {name}")

    # -- one pass with this rank's inputs already in HBM ---------------------------------------
    def step(self, src=None):
        d, mb = (self.d if src is None else src), self.mb
        if self.name == "c1b":
            return mb.selective_scan_bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["z"], d["delta_bias"], d["dout"], True)[0]
        if self.name in ("c1", "c0"):
            return mb.selective_scan_fn(d["u"], d["delta"], self.d["A"], d["B"], d["C"], self.d["D"], d["z"],
                                        self.d["delta_bias"], delta_softplus=True, return_last_state=True)[0]
        if self.name == "c2":
            return mb.mamba_chunk_scan_combined(d["x"], d["dt"], d["A"], d["B"], d["C"], 256, D=d["D"], z=d["z"],
                                                dt_bias=d["dt_bias"], dt_softplus=True, return_final_states=True)[0]
        if self.name == "c3":
            return self.c3_step()[0]
        i = self.step_no % d["x"].shape[0]
        self.step_no += 1
        b, H, P = self.shape["batch"], self.shape["nheads"], self.shape["headdim"]
        return mb.selective_state_update(d["state"], d["x"][i], d["dt"][i][..., None].expand(b, H, P), self.A3, d["B"][i], d["C"][i],
                                         self.D2, d["z"][i], self.bias2, dt_softplus=True)

    def c3_step(self, phases=None):
        d, mb = self.d, self.mb
        if self.world == 1:
            return mb.mamba_chunk_scan_combined(d["x"], d["dt"], d["A"], d["B"], d["C"], 256, D=d["D"], dt_bias=d["dt_bias"],
                                                dt_softplus=True, return_final_states=True)
        from mamba_b200.seqpar import mamba_chunk_scan_sequence_parallel
        return mamba_chunk_scan_sequence_parallel(d["x"], d["dt"], d["A"], d["B"], d["C"], 256, D=d["D"], dt_bias=d["dt_bias"],
                                                  dt_softplus=True, return_final_states=True, phases=phases)

    # -- c3 at N > 1: the split result against a one-GPU run of the same heads (outside the timed region) ----
    def c3_parity(self, heads=(5, 127)):
        """Normalised max error of `heads` of the N-GPU output (and of the final state) against ONE call of the
        operator over the whole sequence for those heads on rank 0."""
        import torch.distributed as dist
        d, dev, world = self.d, self.dev, self.world
        out, fin = self.c3_step()
        hs = list(heads)
        gs = [h // (128 // 8) for h in hs]
        L = self.shape["seqlen_this_gpu"]
        lens = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
        dist.all_gather(lens, torch.tensor([L], dtype=torch.int64, device=dev))
        if len({int(v.item()) for v in lens}) != 1:
            return {"skipped": "ranges of unequal length"}
        parts = dict(x=d["x"][:, :, hs], dt=d["dt"][:, :, hs], B=d["B"][:, :, gs], C=d["C"][:, :, gs], out=out[:, :, hs])
        full = {}
        for k, v in parts.items():
            v = v.contiguous()
            buf = torch.empty((world,) + tuple(v.shape), dtype=v.dtype, device=dev)
            dist.all_gather_into_tensor(buf, v)
            full[k] = torch.cat(list(buf.unbind(0)), dim=1)          # ranks own consecutive ranges
        fin_last = fin[:, hs].contiguous()
        dist.broadcast(fin_last, src=world - 1)
        res = None
        if self.rank == 0:
            want, wfin = self.mb.mamba_chunk_scan_combined(full["x"], full["dt"], d["A"][hs], full["B"], full["C"], 256, D=d["D"][hs],
                                                           dt_bias=d["dt_bias"][hs], dt_softplus=True, return_final_states=True)
            torch.cuda.synchronize()
            err = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1.0)).item()
            res = {"heads": hs, "out_norm_err": err(full["out"], want), "final_state_norm_err": err(fin_last, wfin),
                   "against": "one call over the whole sequence for these heads on rank 0", "tolerance": 2e-2}
        return res

    # -- pinned host buffers for the end-to-end leg (headline workload) -------------------------
    def pinned_inputs(self):
        return {k: self.host[k].contiguous().pin_memory() for k in ("u", "delta", "z", "B", "C")}


# ----------------------------------------------------------------------------------------- CPU baseline
def cpu_inputs(name):
    """Host tensors of the bounded sample of `name` the CPU baseline runs, and what that sample is."""
    bf = torch.bfloat16
    if name == "c1b":
        h = make_c1_rows([0])
        keep = 64    # autograd through the reference keeps every step's (channels x states) tensors alive
        h = {k: (v[:, :keep].contiguous() if k in ("u", "delta", "z") else v[:keep].contiguous() if k in ("A", "D", "delta_bias") else v)
             for k, v in h.items()}
        h["dout"] = torch.randn(h["u"].shape, generator=torch.Generator().manual_seed(7)).to(bf)
        return h, h["u"].shape[2] * keep / 5120, f"1 of 8 batch rows x {keep} of 5120 channels, full seqlen, forward + autograd backward"
    if name in ("c1", "c0"):
        h = make_c1_rows([0]) if name == "c1" else make_c0()
        nb = h["u"].shape[0]
        total = 8 if name == "c1" else nb
        return h, nb * h["u"].shape[2], f"{nb} of {total} batch rows, all channels, full seqlen"
    g = torch.Generator().manual_seed(2000)
    r = lambda *s: torch.randn(*s, generator=g)
    if name in ("c2", "c3"):
        L, nh = 4096, 16
        h = dict(x=r(1, L, nh, 64).to(bf), dt=r(1, L, nh).to(bf), B=r(1, L, 1, 128).to(bf), C=r(1, L, 1, 128).to(bf),
                 z=r(1, L, nh, 64).to(bf) if name == "c2" else None, **ssd_params(nh, 2000))
        if name == "c2":
            return h, L * nh / 80, f"1 of 8 batch rows x {nh} of 80 heads, full seqlen, fp32-widened inputs"
        return h, L * nh / 128, f"first {L} of 262144 tokens x {nh} of 128 heads (one B/C group), fp32-widened inputs"
    nb, H, P, N = 32, 80, 64, 128
    h = dict(state=0.1 * r(nb, H, P, N), x=r(nb, H, P).to(bf), z=r(nb, H, P).to(bf), dt=r(nb, H).to(bf), B=r(nb, 1, N).to(bf),
             C=r(nb, 1, N).to(bf), **ssd_params(H, 2000))
    return h, nb, f"{nb} of 256 batch rows, one step"


def cpu_callable(name, h):
    """The CPU form of workload `name` on sample `h`: the reference's own function when oracle/_ref holds it
    (kind "reference"), else the PyTorch-on-CPU restatement (kind "port")."""
    from oracle import make_ref
    from oracle import torch_port as tp
    ref = make_ref.load()
    kind = "reference" if ref else "port"
    f = lambda t: None if t is None else t.float()
    if name == "c1b":
        fn = ref["selective_scan"] if ref else tp.selective_scan

        def fwd_bwd():
            leaves = [h[k].detach().clone().requires_grad_() for k in ("u", "delta", "A", "B", "C", "D", "z", "delta_bias")]
            out = fn(*leaves, delta_softplus=True)
            out.backward(h["dout"].to(out.dtype))
            return leaves[0].grad
        return fwd_bwd, kind
    if name in ("c1", "c0"):
        fn = ref["selective_scan"] if ref else tp.selective_scan
        return (lambda: fn(h["u"], h["delta"], h["A"], h["B"], h["C"], h["D"], h["z"], h["delta_bias"], delta_softplus=True,
                           return_last_state=True)), kind
    if name in ("c2", "c3"):
        x, dt, B, C, z = f(h["x"]), f(h["dt"]), f(h["B"]), f(h["C"]), f(h["z"])
        if ref:
            return (lambda: ref["ssd_chunk_scan"](x, dt, h["A"], B, C, 256, D=h["D"], z=z, dt_bias=h["dt_bias"], dt_softplus=True)), kind
        return (lambda: tp.ssd_chunk_scan(x, dt, h["A"], B, C, 256, h["D"], z, h["dt_bias"], dt_softplus=True)), kind
    nb, H, P, N = h["state"].shape
    state = h["state"].clone()
    fn = ref["selective_state_update"] if ref else tp.selective_state_update
    return (lambda: fn(state, h["x"], h["dt"][..., None].expand(nb, H, P), h["A"][:, None, None].expand(H, P, N), h["B"], h["C"],
                       h["D"][:, None].expand(H, P), h["z"], h["dt_bias"][:, None].expand(H, P), dt_softplus=True)), kind


def time_cpu(name, budget_s):
    torch.set_num_threads(os.cpu_count())
    h, tokens, sample = cpu_inputs(name)
    fn, kind = cpu_callable(name, h)
    fn()  # warm-up (allocator, thread pool)
    reps, t0 = 0, time.perf_counter()
    while reps < 1 or (time.perf_counter() - t0 < budget_s and reps < 8):
        fn()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": tokens / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample, "reps": reps}


# ----------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (NVML; nvidia-smi as a fallback)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.sm, self.max_sm, self.reasons, self.stop = index, [], None, set(), threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and vis.split(",")[index].isdigit() else index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _poll_nvml(self):
        n = self.nvml
        self.sm.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
        bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        for name, flag in (("hw_slowdown", n.nvmlClocksThrottleReasonHwSlowdown),
                           ("hw_thermal_slowdown", n.nvmlClocksThrottleReasonHwThermalSlowdown),
                           ("sw_thermal_slowdown", n.nvmlClocksThrottleReasonSwThermalSlowdown),
                           ("sw_power_cap", n.nvmlClocksThrottleReasonSwPowerCap)):
            if bits & flag:
                self.reasons.add(name)

    def _poll_smi(self):
        out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        f = [x.strip() for x in out.split(",")]
        if f and f[0].isdigit():
            self.sm.append(int(f[0]))
            self.max_sm = int(f[1]) if f[1].isdigit() else self.max_sm
            for i, name in enumerate(self.NAMES):
                if len(f) > 2 + i and f[2 + i].lower().startswith("active"):
                    self.reasons.add(name)

    def _run(self):
        while not self.stop.is_set():
            try:
                self._poll_nvml() if self.nvml else self._poll_smi()
            except Exception:
                pass
            self.stop.wait(0.002 if self.nvml else 0.05)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm, "reasons": sorted(self.reasons),
                "samples": len(sm), "source": "nvml" if self.nvml else "nvidia-smi"}


# ----------------------------------------------------------------------------------------- timing
def all_max(values, dist, dev):
    if not dist:
        return list(values)
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t.tolist()


def fence(dist):
    torch.cuda.synchronize()
    if dist:
        torch.distributed.barrier()
        torch.cuda.synchronize()


BLOCKS_OVERRIDE = None      # --blocks: fixed number of timed blocks (profiling captures)


def time_blocks(w, steps, warmup, dist, clock_index, target_s=0.3):
    """Median (over R blocks) of the device time of exactly `steps` steps, maximum over ranks per block."""
    for _ in range(warmup):
        w.step()
    fence(dist)
    # a first block sizes R; it is a warm-up too and is not reported
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        w.step()
    e1.record()
    torch.cuda.synchronize()
    est = all_max([e0.elapsed_time(e1) / 1e3], dist, w.dev)[0]
    R = int(min(400, max(5, math.ceil(target_s / max(est, 1e-6))))) if BLOCKS_OVERRIDE is None else BLOCKS_OVERRIDE
    times = []
    with ClockSampler(clock_index) as clk:
        for _ in range(R):
            fence(dist)
            e0.record()
            for _ in range(steps):
                w.step()
            e1.record()
            fence(dist)
            times.append(e0.elapsed_time(e1) / 1e3)
    times = sorted(all_max(times, dist, w.dev))
    return times[len(times) // 2], {"blocks": R, "block_s_min": times[0], "block_s_max": times[-1]}, clk.summary()


def time_e2e(w, steps, warmup, dist):
    """The headline pass through the public API from pinned host buffers: H2D of the step's inputs, the
    kernel, D2H of the step's output, all inside the timed region, every step.  Fed one batch row at a time on
    three streams (copy-in, compute, copy-out), so the two PCIe directions and the kernels overlap."""
    pinned = w.pinned_inputs()
    nb = pinned["u"].shape[0]
    dev_in = {k: torch.empty_like(v, device=w.dev) for k, v in pinned.items()}
    h2d = sum(v.numel() * v.element_size() for v in pinned.values())
    res_host = torch.empty(pinned["u"].shape, dtype=pinned["u"].dtype).pin_memory()
    d2h = res_host.numel() * res_host.element_size()
    cur = torch.cuda.current_stream(w.dev)
    s_in, s_cmp, s_out = (torch.cuda.Stream(w.dev) for _ in range(3))
    done_prev = [None] * nb

    def one():
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(cur)
        for i in range(nb):
            sl = slice(i, i + 1)
            with torch.cuda.stream(s_in):
                if done_prev[i] is not None:
                    s_in.wait_event(done_prev[i])          # the previous step's kernel has consumed this row
                for k, v in pinned.items():
                    dev_in[k][sl].copy_(v[sl], non_blocking=True)
                ready = s_in.record_event()
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ready)
                out = w.step({k: v[sl] for k, v in dev_in.items()})
                done_prev[i] = s_cmp.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_prev[i])
                out.record_stream(s_out)
                res_host[sl].copy_(out, non_blocking=True)
        cur.wait_stream(s_out)
        cur.wait_stream(s_cmp)

    for _ in range(max(1, min(warmup, 3))):
        one()
    fence(dist)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    fence(dist)
    return e0.elapsed_time(e1) / 1e3, h2d, d2h


def measure(name, dev, rank, world, local, steps, warmup, batch, cpu_budget):
    """Times one workload; returns (this workload's JSON fields, the Workload)."""
    dist = world > 1
    peak_gbs, peak_tf, peak_src = measured_peaks()
    w = Workload(name, dev, rank, world, batch)
    t_blk, blocks, clocks = time_blocks(w, steps, warmup, dist, local)
    per_step = t_blk / steps
    achieved = w.alg_bytes / per_step / 1e9
    traffic = NCU_TRAFFIC.get(name) if (world == 1 and not w.reduced) else None
    out = {
        "workload": w.desc + (" [REDUCED SIZE: profiling run, not a benchmark result]" if w.reduced else ""),
        "value": w.global_tokens * steps / t_blk, "unit": UNIT, "ms_per_step": per_step * 1e3, "dtype": w.dtype,
        "this_gpu": w.shape, "partition": w.partition, "kernels": w.kernels,
        "gpu_launches": w.launches_per_step * steps, "timing": blocks,
        "l2_policy": "inputs_exceed_l2" if w.alg_bytes > 2 * 126e6 else "inputs_fit_l2_not_flushed",
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                     "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": w.alg_bytes,
                     "per": "this GPU's share of the problem, slowest rank's time"},
        "clocks": clocks,
    }
    if name == "c1" and world == 1 and not w.reduced:
        # the pipe this kernel leans on hardest is not HBM: the same count of special-function operations issued by
        # themselves takes 0.3764 ms on this part (tests/test_gpu_mufu_ceiling.py measures it)
        out["roofline"]["special_function_ceiling"] = {
            "ms_per_step": 0.3764, "operations": 8 * 5120 * 2048 * (16 + 3), "source": "tests/test_gpu_mufu_ceiling.py (measured on B200, 1965 MHz)",
            "frac_of_ceiling": 0.3764e-3 / per_step, "ceiling_as_frac_of_hbm_peak": w.alg_bytes / 0.3764e-3 / 1e9 / peak_gbs}
    if w.flops:
        tf = w.flops / per_step / 1e12
        out["roofline"]["tensor"] = {"flops_per_launch": w.flops, "achieved_tflops": tf, "peak_tflops": peak_tf,
                                     "frac": tf / peak_tf if peak_tf else None,
                                     "hbm_time_ms": w.alg_bytes / peak_gbs / 1e6, "tensor_time_ms": w.flops / peak_tf / 1e9 if peak_tf else None}
    if name == "c2" and not dist and not w.reduced:
        # the same launch group on packed input: `seqs` sequences of equal length per batch row (continuous batching)
        seqs = 8
        L = w.shape["seqlen"]
        seq_idx = (torch.arange(L, device=dev, dtype=torch.int32) // (L // seqs))[None].expand(w.shape["batch"], L).contiguous()
        d = w.d
        packed = lambda: w.mb.mamba_chunk_scan_combined(d["x"], d["dt"], d["A"], d["B"], d["C"], 256, D=d["D"], z=d["z"], dt_bias=d["dt_bias"],
                                                        seq_idx=seq_idx, dt_softplus=True, return_final_states=True)
        for _ in range(3):
            packed()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            packed()
        e1.record()
        torch.cuda.synchronize()
        out["packed_sequences"] = {"sequences_per_row": seqs, "ms_per_step": e0.elapsed_time(e1) / steps,
                                   "ratio_to_unpacked": e0.elapsed_time(e1) / steps / (per_step * 1e3)}
    if name == "c3" and dist:
        out["parity"] = w.c3_parity()
        phases = {}
        for _ in range(3):
            w.c3_step(phases=phases)
        torch.cuda.synchronize()
        if phases:
            out["phases_ms"] = {k: round(v, 4) for k, v in phases.items()}
    if rank == 0 and world == 1 and cpu_budget > 0 and not w.reduced:
        out["cpu_baseline"] = time_cpu(name, cpu_budget)
    return out, w


def reference_arm(args, rank):
    """The reference's own CPU implementation of the headline workload on this host's cores (rank 0 only)."""
    if rank != 0:
        return 0
    name = args.only or "c1"
    torch.set_num_threads(os.cpu_count())
    h, tokens, sample = cpu_inputs(name)
    fn, kind = cpu_callable(name, h)
    budget, t_start = 150.0, time.perf_counter()
    warm = 0
    for _ in range(max(1, args.warmup)):
        fn()
        warm += 1
        if time.perf_counter() - t_start > budget / 5:
            break
    steps, t0 = 0, time.perf_counter()
    while steps < args.steps and (steps == 0 or time.perf_counter() - t_start < budget):
        fn()
        steps += 1
    dt = (time.perf_counter() - t0) / steps
    val = tokens / dt
    note = (f"each step is the bounded sample below, not the whole batch; {steps} of the {args.steps} requested steps and "
            f"{warm} of the {args.warmup} requested warm-ups fit the wall-clock budget of {budget:.0f} s")
    print(json.dumps({
        "impl": "reference", "metric": METRIC if name != "c1b" else "scan_bwd_tokens_per_s", "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_DESC[name], "sample_per_step": sample, "note": note},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=["c0", "c1", "c1b", "c2", "c3", "c4"],
                    help="measure this one workload as the headline and skip the others")
    ap.add_argument("--workload", dest="only", choices=["c0", "c1", "c1b", "c2", "c3", "c4"], help=argparse.SUPPRESS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--blocks", type=int, default=None, help="fixed number of timed blocks instead of >= 0.3 s worth (profiling captures)")
    ap.add_argument("--batch", type=int, default=None,
                    help="shrink the problem (for ncu captures of a small case; not a benchmark result)")
    args = ap.parse_args()
    global BLOCKS_OVERRIDE
    BLOCKS_OVERRIDE = args.blocks
    warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        return reference_arm(args, rank)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: mamba_b200 has no CPU path")
    dist = world > 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if dist:
        torch.distributed.init_process_group("nccl", device_id=dev)

    head_name = args.only or "c1"
    cpu_budget = 0 if args.no_cpu_baseline else 8.0
    head, w = measure(head_name, dev, rank, world, local, args.steps, warmup, args.batch, cpu_budget)
    line = {
        "metric": METRIC if head_name != "c1b" else "scan_bwd_tokens_per_s", "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong" if head_name != "c0" else "weak",
        "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
        "config": {"workload": head["workload"], "this_gpu": head["this_gpu"], "partition": head["partition"],
                   "l2_policy": head["l2_policy"], "timing": dict(head["timing"], rule="median of `blocks` blocks of `steps` steps, max over ranks per block")},
        "gpu_launches": head["gpu_launches"], "kernels": head["kernels"], "roofline": head["roofline"], "clocks": head["clocks"],
    }
    if head_name in ("c1", "c0") and not args.no_e2e and w.shape["batch"] > 0:
        e2e_steps = max(3, min(args.steps, 10))
        t_e2e, h2d, d2h = time_e2e(w, e2e_steps, warmup, dist)
        t_e2e = all_max([t_e2e], dist, dev)[0]
        line["e2e"] = {"value": w.global_tokens * e2e_steps / t_e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "steps": e2e_steps, "bytes": "this GPU's share per step"}
    for k in ("cpu_baseline", "packed_sequences", "parity", "phases_ms"):
        if k in head:
            line[k] = head[k]
    del w
    torch.cuda.empty_cache()
    if not args.only:
        line["workloads"] = {}
        for name in ("c2", "c3", "c4"):
            res, wl = measure(name, dev, rank, world, local, args.steps, warmup, None, cpu_budget * 0.75)
            line["workloads"][name] = res
            del wl
            torch.cuda.empty_cache()
    if dist:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
