#!/usr/bin/env python
"""Benchmark of the scan hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c0] [--impl ours|reference]

Default workload (the one the headline metric is quoted on): the Mamba-1 selective scan at the
2.8B-layer shape -- batch 8, d_inner 5120, seqlen 2048, d_state 16, bf16 activations, one B/C group
(synthetic seeded inputs).  One "step" is one forward pass over that batch.  With N > 1 (launched by
torchrun, one rank per GPU) every rank runs the same per-GPU batch on its own data (no collective on
the data path; weak scaling) and the slowest rank sets the time.

Prints ONE JSON line: tokens/s with inputs resident in HBM (`value`), the same through the public
API with pinned host buffers and the copies timed (`e2e`), the roofline of the dominant kernel
against the measured HBM peak, and the CPU baseline (the PyTorch-on-CPU restatement of the
reference's definition) timed on this host.
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

# dram bytes (read + write) per launch of the dominant kernel from the committed ncu capture
# (profiles/), or None where no capture exists for that workload.
NCU_TRAFFIC_BYTES = {
    "c1": 659_956_992,      # scan_stream_kernel: 509.0 MB read + 151.0 MB written
    "c2": 1_735_000_000,    # the SSD launches summed (state stream 368 + 154 MB, chunk_scan 881 + 310 MB)
    "c4": 1_291_591_424,    # ssu_packet_kernel: 676.8 MB read + 614.7 MB written
    "c0": None, "c3": None,
}


# the names the GPU arm puts in config.workload; the reference arm reports under the same ones
WORKLOAD_DESC = {
    "c0": "mamba1_selective_scan_fwd fp32 b2 d256 L512 N16",
    "c1": "mamba1_selective_scan_fwd bf16 b8 d5120 L2048 N16 (2.8B layer)",
    "c2": "mamba2_ssd_chunk_scan_fwd bf16 b8 L4096 h80 P64 g1 N128 Q256 (+z, +final_states)",
    "c3": "mamba2_ssd_chunk_scan_fwd bf16 b1 L262144 h128 P64 g8 N128 Q256 (no z), sequence split over GPUs",
    "c4": "mamba2_selective_state_update b256 h80 P64 N128 fp32 state, bf16 activations",
}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", p.get("bf16_tflops", 0.0))), "measured"
    return 6650.0, 1590.0, "fallback"


# ----------------------------------------------------------------------------------------- inputs
def softplus_inv_dt(n, g):
    dt = torch.exp(torch.rand(n, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    return dt + torch.log(-torch.expm1(-dt))


def make_c1(batch, dim=5120, L=2048, N=16, seed=1001, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return dict(u=r(batch, dim, L).to(dtype), delta=r(batch, dim, L).to(dtype), z=r(batch, dim, L).to(dtype),
                A=-torch.exp(r(dim, N)), B=r(batch, 1, N, L).to(dtype), C=r(batch, 1, N, L).to(dtype), D=r(dim),
                delta_bias=softplus_inv_dt(dim, g))


def make_c0(batch=2, dim=256, L=512, N=16, seed=1000):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return dict(u=r(batch, dim, L), delta=r(batch, dim, L), z=r(batch, dim, L), A=-torch.exp(r(dim, N)),
                B=r(batch, 1, N, L), C=r(batch, 1, N, L), D=r(dim), delta_bias=-4 + 2 * torch.rand(dim, generator=g))


def make_c2(batch, H=80, L=4096, P=64, N=128, seed=1002):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    bf = torch.bfloat16
    return dict(x=r(batch, L, H, P).to(bf), dt=r(batch, L, H).to(bf), A=-(1 + 15 * torch.rand(H, generator=g)),
                B=r(batch, L, 1, N).to(bf), C=r(batch, L, 1, N).to(bf), D=r(H), z=r(batch, L, H, P).to(bf),
                dt_bias=softplus_inv_dt(H, g))


def make_c4(batch, H=80, P=64, N=128, seed=1004, pool=4):
    """`pool` distinct token inputs are rotated through the steps; the state is updated in place."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    bf = torch.bfloat16
    return dict(state=0.1 * r(batch, H, P, N), x=r(pool, batch, H, P).to(bf), z=r(pool, batch, H, P).to(bf),
                dt=r(pool, batch, H).to(bf), B=r(pool, batch, 1, N).to(bf), C=r(pool, batch, 1, N).to(bf),
                A=-(1 + 15 * torch.rand(H, generator=g)), D=r(H), dt_bias=softplus_inv_dt(H, g))


class Workload:
    """One benchmark configuration: device step, host-buffer step, CPU-baseline sample, byte counts."""

    def __init__(self, name, dev, batch=None):
        """`batch` shrinks the per-GPU batch (profiling captures only; the JSON line then says so)."""
        self.name, self.dev = name, dev
        self.reduced = batch is not None
        import mamba_b200 as mb
        self.mb = mb
        if name in ("c1", "c0"):
            host = make_c1(batch or 8) if name == "c1" else make_c0()
            self.shape = dict(batch=host["u"].shape[0], d_inner=host["u"].shape[1], seqlen=host["u"].shape[2], d_state=16)
            self.tokens = host["u"].shape[0] * host["u"].shape[2]
            self.desc = WORKLOAD_DESC[name]
            self.dtype = "bf16" if name == "c1" else "f32"
            self.step_inputs = ("u", "delta", "z", "B", "C")
            esz = host["u"].element_size()
            b, d, L = host["u"].shape
            self.alg_bytes = 4 * b * d * L * esz + 2 * b * 16 * L * esz + d * 16 * 4 + 2 * d * 4 + b * d * 16 * 4
            self.launches_per_step = 1
        elif name == "c2":
            host = make_c2(batch or 8)
            b, L, H, P = host["x"].shape
            self.shape = dict(batch=b, seqlen=L, nheads=H, headdim=P, ngroups=1, d_state=128, chunk_size=256)
            self.tokens = b * L
            self.desc = WORKLOAD_DESC[name]
            self.dtype = "bf16"
            self.step_inputs = ("x", "dt", "z", "B", "C")
            self.alg_bytes = 3 * b * L * H * P * 2 + b * L * H * 2 + 2 * b * L * 128 * 2 + b * H * P * 128 * 4 + 3 * H * 4
            self.launches_per_step = 5      # cumsum, state stream (head pairs, then single heads), C.B^T, chunk scan
        elif name == "c3":
            # long sequence split into contiguous chunk ranges, one per rank; the whole sequence at N=1
            from mamba_b200.seqpar import split_sequence
            world = int(os.environ.get("WORLD_SIZE", "1"))
            rank = int(os.environ.get("RANK", "0"))
            Ltot, H, P, G, N = 262144, 128, 64, 8, 128
            lo, hi = split_sequence(Ltot, 256, world, rank)
            Lr = hi - lo
            g = torch.Generator(device=dev).manual_seed(1003 + rank)
            r = lambda *sh: torch.randn(*sh, generator=g, device=dev)
            bf = torch.bfloat16
            gh = torch.Generator().manual_seed(1003)
            host = dict(A=-(1 + 15 * torch.rand(H, generator=gh)), D=torch.randn(H, generator=gh), dt_bias=softplus_inv_dt(H, gh))
            self.dev_only = dict(x=r(1, Lr, H, P).to(bf), dt=r(1, Lr, H).to(bf), B=r(1, Lr, G, N).to(bf), C=r(1, Lr, G, N).to(bf))
            self.shape = dict(batch=1, seqlen_total=Ltot, seqlen_this_gpu=Lr, nheads=H, headdim=P, ngroups=G, d_state=N, chunk_size=256)
            self.tokens = Lr
            self.desc = WORKLOAD_DESC[name]
            self.dtype = "bf16"
            self.step_inputs = ("x", "dt", "B", "C")
            self.alg_bytes = 2 * Lr * H * P * 2 + Lr * H * 2 + 2 * Lr * G * N * 2 + H * P * N * 4 + 3 * H * 4
            self.launches_per_step = 4 if world == 1 else 5
            self.world = world
        elif name == "c4":
            host = make_c4(batch or 256)
            b, H, P, N = host["state"].shape
            self.shape = dict(batch=b, nheads=H, headdim=P, ngroups=1, d_state=N, consecutive_steps=True)
            self.tokens = b
            self.desc = WORKLOAD_DESC[name]
            self.dtype = "f32"
            self.step_inputs = ("x", "dt", "z", "B", "C")
            self.alg_bytes = 2 * b * H * P * N * 4 + 3 * b * H * P * 2 + b * H * 2 + 2 * b * N * 2 + 3 * H * 4
            self.launches_per_step = 1
        else:
            raise SystemExit(f"unknown workload {name}")
        self.host = host
        self.d = {k: v.to(dev) for k, v in host.items()}
        if name == "c3":
            self.d.update(self.dev_only)
        self.step_no = 0
        if name == "c4":
            H, P, N = self.shape["nheads"], self.shape["headdim"], self.shape["d_state"]
            self.A3 = self.d["A"][:, None, None].expand(H, P, N)
            self.D2 = self.d["D"][:, None].expand(H, P)
            self.bias2 = self.d["dt_bias"][:, None].expand(H, P)

    # -- one pass with inputs already in HBM -------------------------------------------------
    def step(self, src=None):
        d = self.d if src is None else src
        mb = self.mb
        if self.name in ("c1", "c0"):
            return mb.selective_scan_fn(d["u"], d["delta"], self.d["A"], d["B"], d["C"], self.d["D"], d["z"],
                                        self.d["delta_bias"], delta_softplus=True, return_last_state=True)[0]
        if self.name == "c3":
            if self.world == 1:
                return mb.mamba_chunk_scan_combined(d["x"], d["dt"], self.d["A"], d["B"], d["C"], 256, D=self.d["D"],
                                                    dt_bias=self.d["dt_bias"], dt_softplus=True, return_final_states=True)[0]
            from mamba_b200.seqpar import mamba_chunk_scan_sequence_parallel
            return mamba_chunk_scan_sequence_parallel(d["x"], d["dt"], self.d["A"], d["B"], d["C"], 256, D=self.d["D"],
                                                      dt_bias=self.d["dt_bias"], dt_softplus=True, return_final_states=True,
                                                      handoff=os.environ.get("MB200_BENCH_HANDOFF") or None)[0]
        if self.name == "c2":
            return mb.mamba_chunk_scan_combined(d["x"], d["dt"], self.d["A"], d["B"], d["C"], 256, D=self.d["D"], z=d["z"],
                                                dt_bias=self.d["dt_bias"], dt_softplus=True, return_final_states=True)[0]
        i = self.step_no % self.d["x"].shape[0] if src is None else 0
        self.step_no += 1
        pick = (lambda k: d[k][i]) if src is None else (lambda k: d[k])
        b, H, P = self.shape["batch"], self.shape["nheads"], self.shape["headdim"]
        return mb.selective_state_update(self.d["state"], pick("x"), pick("dt")[..., None].expand(b, H, P), self.A3,
                                         pick("B"), pick("C"), self.D2, pick("z"), self.bias2, dt_softplus=True)

    # -- host buffers for the end-to-end leg ---------------------------------------------------
    def pinned_inputs(self):
        out = {}
        for k in self.step_inputs:
            if self.name == "c3":
                t = self.d[k].cpu()
            else:
                t = self.host[k] if self.name != "c4" else self.host[k][0]
            out[k] = t.contiguous().pin_memory()
        return out


# ----------------------------------------------------------------------------------------- CPU baseline
def cpu_sample(name, h):
    """A bounded sample of workload `name` (host tensors `h`) for the PyTorch-on-CPU restatement.
    Returns (callable, tokens the call processes, description of the sample)."""
    from oracle import torch_port as tp
    if name in ("c1", "c0"):
        nb = 1
        sl = {k: (h[k][:nb] if k in ("u", "delta", "z", "B", "C") else h[k]) for k in h}
        fn = lambda: tp.selective_scan(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"],
                                       sl["delta_bias"], delta_softplus=True, return_last_state=True)
        return fn, nb * h["u"].shape[2], f"{nb} of {h['u'].shape[0]} batch rows, all channels, full seqlen"
    if name == "c3":
        f = lambda t: t.float()
        fn = lambda: tp.ssd_chunk_scan(f(h["x"]), f(h["dt"]), h["A"], f(h["B"]), f(h["C"]), 256, h["D"], None, h["dt_bias"],
                                       dt_softplus=True)
        L, nh = h["x"].shape[1], h["x"].shape[2]
        return fn, L * nh / 128, f"first {L} of 262144 tokens x {nh} of 128 heads (one B/C group), fp32-widened inputs"
    if name == "c2":
        nh = 16
        f = lambda t: t.float()
        sl = dict(x=f(h["x"][:1, :, :nh]), dt=f(h["dt"][:1, :, :nh]), A=h["A"][:nh], B=f(h["B"][:1]), C=f(h["C"][:1]),
                  D=h["D"][:nh], z=f(h["z"][:1, :, :nh]), dt_bias=h["dt_bias"][:nh])
        fn = lambda: tp.ssd_chunk_scan(sl["x"], sl["dt"], sl["A"], sl["B"], sl["C"], 256, sl["D"], sl["z"], sl["dt_bias"],
                                       dt_softplus=True)
        frac = nh / h["x"].shape[2]
        return fn, h["x"].shape[1] * frac, f"1 of 8 batch rows x {nh} of 80 heads, full seqlen, fp32-widened inputs"
    nb = 32
    _, H, P, N = h["state"].shape
    state = h["state"][:nb].clone()
    fn = lambda: tp.selective_state_update(state, h["x"][0, :nb], h["dt"][0, :nb, :, None].expand(nb, H, P),
                                           h["A"][:, None, None].expand(H, P, N), h["B"][0, :nb], h["C"][0, :nb],
                                           h["D"][:, None].expand(H, P), h["z"][0, :nb],
                                           h["dt_bias"][:, None].expand(H, P), dt_softplus=True)
    return fn, nb, f"{nb} of 256 batch rows, one step"


def make_c3_sample(L=4096, H=16, P=64, N=128, seed=1003):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    bf = torch.bfloat16
    return dict(x=r(1, L, H, P).to(bf), dt=r(1, L, H).to(bf), A=-(1 + 15 * torch.rand(H, generator=g)), B=r(1, L, 1, N).to(bf),
                C=r(1, L, 1, N).to(bf), D=r(H), dt_bias=softplus_inv_dt(H, g))


HOST_INPUTS = {"c3": make_c3_sample, "c0": lambda: make_c0(), "c1": lambda: make_c1(8), "c2": lambda: make_c2(8), "c4": lambda: make_c4(256)}


# ----------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs.

    NVML is polled directly (a query costs well under a millisecond, so even a 20 ms timed region
    yields several samples); if the NVML binding is missing, `nvidia-smi` is polled instead."""
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


# ----------------------------------------------------------------------------------------- legs
def time_device(w, steps, warmup, dist, clock_index):
    for _ in range(warmup):
        w.step()
    torch.cuda.synchronize()
    if dist:
        torch.distributed.barrier()
        torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with ClockSampler(clock_index) as clk:       # samples are taken only while the timed steps run
        ev[0].record()
        for i in range(steps):
            w.step()
            ev[i + 1].record()
        torch.cuda.synchronize()
    if dist:
        torch.distributed.barrier()
        torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[steps]) / 1e3, clk.summary()


def time_e2e(w, steps, warmup, dist):
    """Same pass through the public API from pinned host buffers: H2D of the step's inputs, the
    kernels, D2H of the step's output, all inside the timed region.

    Batched workloads are fed one batch row at a time on three streams (copy-in, compute, copy-out), so
    the two PCIe directions and the kernels overlap; every byte of the step's inputs still crosses the
    bus inside the timed region, every step."""
    pinned = w.pinned_inputs()
    dev_in = {k: torch.empty_like(v, device=w.dev) for k, v in pinned.items()}
    h2d = sum(v.numel() * v.element_size() for v in pinned.values())
    probe = w.step({k: v.to(w.dev) for k, v in pinned.items()})
    res_host = torch.empty(probe.shape, dtype=probe.dtype).pin_memory()
    d2h = res_host.numel() * res_host.element_size()
    del probe
    nb = next(iter(pinned.values())).shape[0]
    sliceable = w.name in ("c0", "c1", "c2") and nb > 1 and all(v.shape[0] == nb for v in pinned.values())
    cur = torch.cuda.current_stream(w.dev)
    s_in, s_cmp, s_out = (torch.cuda.Stream(w.dev) for _ in range(3))
    done_prev = [None] * nb

    def one_simple():
        for k, v in pinned.items():
            dev_in[k].copy_(v, non_blocking=True)
        res_host.copy_(w.step(dev_in), non_blocking=True)

    def one_pipelined():
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(cur)
        for i in range(nb):
            sl = slice(i, i + 1)
            with torch.cuda.stream(s_in):
                if done_prev[i] is not None:
                    s_in.wait_event(done_prev[i])          # the previous step's kernels have consumed this row
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

    one = one_pipelined if sliceable else one_simple
    for _ in range(max(1, min(warmup, 3))):
        one()
    torch.cuda.synchronize()
    if dist:
        torch.distributed.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    if dist:
        torch.distributed.barrier()
    return e0.elapsed_time(e1) / 1e3, h2d, d2h


def time_cpu(w, budget_s=20.0, min_reps=1):
    torch.set_num_threads(os.cpu_count())
    fn, tokens, sample = cpu_sample(w.name, w.host)
    fn()  # warm-up (allocator, thread pool)
    reps, t0 = 0, time.perf_counter()
    while reps < min_reps or (time.perf_counter() - t0 < budget_s / 2 and reps < 8):
        fn()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return tokens / dt, sample, torch.get_num_threads()


def max_over_ranks(x, dist, dev):
    if not dist:
        return x
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c1", choices=["c0", "c1", "c2", "c3", "c4"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None,
                    help="shrink the per-GPU batch (for ncu captures of a small case; not a benchmark result)")
    args = ap.parse_args()
    warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    metric, unit = "scan_fwd_tokens_per_s", "tokens/s"

    if args.impl == "reference":
        # The reference's own CPU form of the path (PyTorch restatement), on this host's cores.
        if rank != 0:
            return 0
        torch.set_num_threads(os.cpu_count())
        fn, tokens, sample = cpu_sample(args.workload, HOST_INPUTS[args.workload]())
        for _ in range(min(warmup, 1)):
            fn()
        steps = min(args.steps, 3)
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        dt = (time.perf_counter() - t0) / steps
        val = tokens / dt
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": min(warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_DESC[args.workload], "sample_per_step": sample},
            "cpu_baseline": {"value": val, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: mamba_b200 has no CPU path")
    dist = world > 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if dist:
        torch.distributed.init_process_group("nccl", device_id=dev)
    w = Workload(args.workload, dev, args.batch)

    t_dev, clocks = time_device(w, args.steps, warmup, dist, local)
    t_dev = max_over_ranks(t_dev, dist, dev)
    t_e2e, h2d, d2h = time_e2e(w, max(3, min(args.steps, 10)), warmup, dist)
    e2e_steps = max(3, min(args.steps, 10))
    t_e2e = max_over_ranks(t_e2e, dist, dev)

    peak_gbs, _, peak_src = measured_peak_gbs()
    per_launch_s = t_dev / args.steps
    achieved = w.alg_bytes / per_launch_s / 1e9
    line = {
        "metric": metric, "value": world * w.tokens * args.steps / t_dev, "unit": unit, "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": per_launch_s * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.workload == "c3" else "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": w.desc + (" [REDUCED BATCH: profiling run, not a benchmark result]" if w.reduced else ""),
                   "per_gpu": w.shape,
                   "partition": ("contiguous chunk ranges per GPU, range states handed rank to rank by NCCL P2P"
                                 if args.workload == "c3" else "batch rows per GPU, no collective"),
                   "l2_policy": "inputs_exceed_l2" if w.alg_bytes > 2 * 126e6 else "inputs_fit_l2_not_flushed"},
        "e2e": {"value": world * w.tokens * e2e_steps / t_e2e, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": w.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                     "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": w.alg_bytes},
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload != "c3":
        v, sample, cores = time_cpu(w)
        line["cpu_baseline"] = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
    if dist:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
