"""Regenerates tests/golden/*.npz by running the REFERENCE's own pure-PyTorch
definitions on seeded inputs.

Run where the reference checkout is importable (it is not needed to run the
tests, only to regenerate the vectors):

    PYTHONPATH=/path/to/mamba python tests/golden/make_golden.py

Every fixture stores its inputs as well as the reference outputs, so the tests
never depend on a random-number generator reproducing the same stream.
bf16 cases store the bf16-rounded values widened to float32.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F
from einops import rearrange, repeat

from mamba_ssm.ops.selective_scan_interface import selective_scan_ref
from mamba_ssm.ops.triton.selective_state_update import selective_state_update_ref
from mamba_ssm.ops.triton.ssd_combined import ssd_chunk_scan_combined_ref
from mamba_ssm.ops.triton.ssd_chunk_state import chunk_state_ref
from mamba_ssm.ops.triton.ssd_state_passing import state_passing_ref
from mamba_ssm.ops.triton.ssd_chunk_scan import chunk_scan_ref
from mamba_ssm.ops.triton.layernorm_gated import rms_norm_ref

HERE = os.path.dirname(os.path.abspath(__file__))


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if v is None:
            continue
        if torch.is_tensor(v):
            v = v.detach().float().contiguous().numpy()
        out[k] = np.asarray(v)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def dt_bias_init(n, g):
    """softplus^-1 of dt drawn log-uniform in [1e-3, 1e-1] (the reference modules' init)."""
    dt = torch.exp(torch.rand(n, generator=g) * (np.log(0.1) - np.log(1e-3)) + np.log(1e-3))
    return dt + torch.log(-torch.expm1(-dt))


# ----------------------------------------------------------------------------- Mamba-1
def mamba1(name, seed, batch, dim, L, N, groups, dtype=torch.float32, has_z=True, has_D=True,
           const_bc=False, test_style=False):
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    if test_style:  # distributions of the reference's tests/ops/test_selective_scan.py:56-86
        A = -0.5 * torch.rand(dim, N, generator=g)
        delta = 0.5 * torch.rand(batch, dim, L, generator=g)
        bias = 0.5 * torch.rand(dim, generator=g)
    else:           # distributions of the benchmark's fp32 configuration
        A = -torch.exp(r(dim, N))
        delta = r(batch, dim, L)
        bias = -4 + 2 * torch.rand(dim, generator=g)
    u = r(batch, dim, L)
    if const_bc:
        B, C = r(dim, N), r(dim, N)
    else:
        B, C = r(batch, groups, N, L), r(batch, groups, N, L)
    D = r(dim) if has_D else None
    z = r(batch, dim, L) if has_z else None
    cast = lambda t: None if t is None else t.to(dtype)
    u, delta, z = cast(u), cast(delta), cast(z)
    if not const_bc:
        B, C = cast(B), cast(C)
    out, last = selective_scan_ref(u, delta, A, B, C, D, z, bias, delta_softplus=True, return_last_state=True)
    save(name, u=u, delta=delta, A=A, B=B, C=C, D=D, z=z, delta_bias=bias, out=out, last_state=last,
         is_bf16=np.int32(dtype == torch.bfloat16))


def mamba1_bwd(name, seed, batch, dim, L, N, groups, dtype=torch.float32, has_z=True, has_D=True, has_bias=True,
               const_b=False, const_c=False, softplus=True):
    """Gradients of selective_scan_ref by autograd for a seeded dout: the comparison the reference makes for its CUDA
    backward (tests/ops/test_selective_scan.py:56-147, whose input distributions these are)."""
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    A = -0.5 * torch.rand(dim, N, generator=g)
    delta = 0.5 * torch.rand(batch, dim, L, generator=g)
    bias = 0.5 * torch.rand(dim, generator=g) if has_bias else None
    u = r(batch, dim, L)
    B = r(dim, N) if const_b else r(batch, groups, N, L).to(dtype)
    C = r(dim, N) if const_c else r(batch, groups, N, L).to(dtype)
    D = r(dim) if has_D else None
    z = r(batch, dim, L).to(dtype) if has_z else None
    u, delta = u.to(dtype), delta.to(dtype)
    dout = r(batch, dim, L).to(dtype)
    leaves = [None if t is None else t.detach().clone().requires_grad_() for t in (u, delta, A, B, C, D, z, bias)]
    out = selective_scan_ref(*leaves[:5], leaves[5], leaves[6], leaves[7], delta_softplus=softplus)
    out.backward(dout.to(out.dtype))
    gr = [None if t is None else t.grad for t in leaves]
    save(name, u=u, delta=delta, A=A, B=B, C=C, D=D, z=z, delta_bias=bias, dout=dout, du=gr[0], ddelta=gr[1], dA=gr[2],
         dB=gr[3], dC=gr[4], dD=gr[5], dz=gr[6], ddelta_bias=gr[7], is_bf16=np.int32(dtype == torch.bfloat16),
         delta_softplus=np.int32(softplus))


# ----------------------------------------------------------------------------- decode update
def decode(name, seed, batch, nheads, dim, N, groups, dtype=torch.float32, tie=False, heads=True,
           has_z=True, steps=1):
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    if heads:
        state = (0.1 * r(batch, nheads, dim, N)).to(dtype)
        if tie:
            A = repeat(-torch.rand(nheads, generator=g) - 1.0, "h -> h p n", p=dim, n=N)
            bias = repeat(torch.rand(nheads, generator=g) - 4.0, "h -> h p", p=dim)
            D = repeat(r(nheads), "h -> h p", p=dim)
        else:
            A = -torch.rand(nheads, dim, N, generator=g) - 1.0
            bias = torch.rand(nheads, dim, generator=g) - 4.0
            D = r(nheads, dim)
        shp, bc = (batch, nheads, dim), (batch, groups, N)
    else:
        state = (0.1 * r(batch, dim, N)).to(dtype)
        A = -torch.rand(dim, N, generator=g) - 1.0
        bias = torch.rand(dim, generator=g) - 4.0
        D = r(dim)
        shp, bc = (batch, dim), (batch, N)
    state0 = state.clone()
    xs, dts, Bs, Cs, zs, outs = [], [], [], [], [], []
    for _ in range(steps):
        x = r(*shp).to(dtype)
        if heads and tie:
            dt = repeat(r(batch, nheads).to(dtype), "b h -> b h p", p=dim)
        else:
            dt = r(*shp).to(dtype)
        B, C = r(*bc).to(dtype), r(*bc).to(dtype)
        z = r(*shp).to(dtype) if has_z else None
        # widen first: the oracle target is the ref on the rounded inputs in fp32
        st32 = state.float()
        out = selective_state_update_ref(st32, x.float(), dt.float(), A, B.float(), C.float(), D,
                                         None if z is None else z.float(), bias, dt_softplus=True)
        state = st32.to(dtype)
        xs.append(x.float()); dts.append(dt.float()); Bs.append(B.float()); Cs.append(C.float())
        zs.append(None if z is None else z.float()); outs.append(out)
    stack = lambda l: None if l[0] is None else torch.stack(l)
    save(name, state0=state0, x=stack(xs), dt=stack(dts), A=A.contiguous(), B=stack(Bs), C=stack(Cs),
         D=D.contiguous(), z=stack(zs), dt_bias=bias.contiguous(), out=stack(outs), state_final=state,
         is_bf16=np.int32(dtype == torch.bfloat16), tie=np.int32(tie), heads=np.int32(heads))


# ----------------------------------------------------------------------------- SSD
def ssd(name, seed, batch, L, H, P, G, N, Q, dtype=torch.float32, has_z=True, D_hdim=False,
        with_init=False):
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    x = r(batch, L, H, P).to(dtype)
    dt = r(batch, L, H).to(dtype)
    A = -(1 + 15 * torch.rand(H, generator=g))
    B = r(batch, L, G, N).to(dtype)
    C = r(batch, L, G, N).to(dtype)
    D = r(H, P) if D_hdim else r(H)
    z = r(batch, L, H, P).to(dtype) if has_z else None
    bias = dt_bias_init(H, g)
    init = 0.5 * r(batch, H, P, N) if with_init else None
    f = lambda t: None if t is None else t.float()
    # the parity target is the reference evaluated on the (rounded) inputs in fp32
    xf, dtf, Bf, Cf, zf = f(x), f(dt), f(B), f(C), f(z)
    if L % Q == 0:
        dtc = F.softplus(rearrange(dtf, "b (c l) h -> b h c l", l=Q) + bias[:, None, None])
        cum = torch.cumsum(dtc * A[:, None, None], dim=-1)
        states = chunk_state_ref(Bf, xf, dtc, cum)
        prev, final = state_passing_ref(rearrange(states, "... p n -> ... (p n)"), cum[..., -1],
                                        None if init is None else rearrange(init, "... p n -> ... (p n)"))
        prev = rearrange(prev, "... (p n) -> ... p n", n=N)
        final = rearrange(final, "... (p n) -> ... p n", n=N)
        out = chunk_scan_ref(Bf, Cf, xf, dtc, cum, prev, D=D, z=zf)
        if init is None:
            whole = ssd_chunk_scan_combined_ref(xf, dtf, A, Bf, Cf, Q, D=D, z=zf, dt_bias=bias, dt_softplus=True)
            assert torch.equal(whole, out)
    else:
        # ragged tail: the chunked reference asserts full chunks, so use the plain recurrence
        # (the mapping of ssd_combined.py:744-776) which is the same mathematics for any L.
        assert init is None
        xs = rearrange(xf, "b l h p -> b (h p) l")
        dts = repeat(dtf, "b l h -> b (h p) l", p=P)
        As = repeat(A, "h -> (h p) n", p=P, n=N)
        Ds = rearrange(D, "h p -> (h p)") if D_hdim else repeat(D, "h -> (h p)", p=P)
        zs = None if zf is None else rearrange(zf, "b l h p -> b (h p) l")
        bs = repeat(bias, "h -> (h p)", p=P)
        out, final = selective_scan_ref(xs, dts, As, rearrange(Bf, "b l g n -> b g n l"),
                                        rearrange(Cf, "b l g n -> b g n l"), D=Ds, z=zs, delta_bias=bs,
                                        delta_softplus=True, return_last_state=True)
        out = rearrange(out, "b (h p) l -> b l h p", p=P)
        final = rearrange(final, "b (h p) n -> b h p n", p=P)
    save(name, x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=bias, initial_states=init, out=out,
         final_states=final, chunk_size=np.int32(Q), is_bf16=np.int32(dtype == torch.bfloat16))


# ----------------------------------------------------------------------------- the steps around the scan
def conv1d(name, seed, batch, dim, L, width, dtype=torch.float32, activation="silu", steps=0):
    """The reference's CPU form of the causal conv: a depthwise nn.Conv1d with left padding, cut to seqlen
    (mamba_ssm/modules/mamba2.py:232-234), and for `steps` further tokens the roll / multiply / sum of :309-315."""
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    conv = torch.nn.Conv1d(dim, dim, width, groups=dim, padding=width - 1, bias=True)
    with torch.no_grad():
        conv.weight.copy_(r(dim, 1, width) * 0.5)
        conv.bias.copy_(r(dim) * 0.1)
    x = r(batch, dim, L).to(dtype)
    act = F.silu if activation else (lambda t: t)
    with torch.no_grad():
        out = act(conv(x.float())[..., :L])
        state = F.pad(x.float(), (width - L, 0)) if L < width else x.float()[..., -width:].clone()     # (batch, dim, width), as Mamba2 keeps it
        state0 = state.clone()
        w2 = rearrange(conv.weight, "d 1 w -> d w")
        xs, outs = [], []
        for _ in range(steps):
            xt = r(batch, dim).to(dtype).float()
            state.copy_(torch.roll(state, shifts=-1, dims=-1))
            state[:, :, -1] = xt
            outs.append(act(torch.sum(state * w2, dim=-1) + conv.bias))
            xs.append(xt)
    save(name, x=x, weight=w2, bias=conv.bias, out=out, final_states=x.float()[..., -(width - 1):] if L >= width - 1 else None,
         state0=state0 if steps else None, x_steps=torch.stack(xs) if steps else None, out_steps=torch.stack(outs) if steps else None,
         state_final=state if steps else None, has_act=np.int32(bool(activation)), is_bf16=np.int32(dtype == torch.bfloat16))


def rmsnorm(name, seed, rows, cols, group, norm_before_gate, dtype=torch.float32, has_z=True, has_bias=False):
    g = gen(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    x, z = r(*rows, cols).to(dtype), (r(*rows, cols).to(dtype) if has_z else None)
    w, b = 1 + 0.1 * r(cols), (0.1 * r(cols) if has_bias else None)
    out = rms_norm_ref(x.float(), w, b, z=None if z is None else z.float(), eps=1e-5, group_size=group, norm_before_gate=norm_before_gate)
    save(name, x=x, z=z, weight=w, bias=b, out=out, group_size=np.int32(group or cols), norm_before_gate=np.int32(norm_before_gate),
         eps=np.float32(1e-5), is_bf16=np.int32(dtype == torch.bfloat16))


def main():
    torch.set_num_threads(os.cpu_count())
    conv1d("conv_fp32_w4", 41, 2, 24, 70, 4, steps=3)
    conv1d("conv_fp32_w3_noact", 42, 1, 8, 33, 3, activation=None)
    conv1d("conv_fp32_w2_short", 43, 2, 8, 1, 2, steps=2)
    conv1d("conv_bf16_w4", 44, 2, 64, 130, 4, dtype=torch.bfloat16, steps=2)
    rmsnorm("rms_fp32_group_gate_after", 51, (3, 5), 64, 16, True)
    rmsnorm("rms_fp32_nogroup_gate_before", 52, (7,), 96, None, False, has_bias=True)
    rmsnorm("rms_fp32_noz", 53, (4,), 40, 8, True, has_z=False)
    rmsnorm("rms_bf16_group_gate_before", 54, (2, 9), 256, 128, False, dtype=torch.bfloat16)
    mamba1("m1_fp32_g1", 11, 2, 4, 128, 8, 1, test_style=True)
    mamba1("m1_fp32_g2_odd", 12, 2, 4, 372, 8, 2, has_z=False, test_style=True)
    mamba1("m1_fp32_constbc", 13, 2, 6, 100, 4, 1, const_bc=True, has_D=False)
    mamba1("m1_fp32_bench_small", 14, 2, 16, 512, 16, 1)
    mamba1("m1_bf16", 15, 2, 8, 256, 16, 1, dtype=torch.bfloat16)
    mamba1("m1_fp32_long", 16, 1, 2, 2500, 16, 1, test_style=True)
    decode("ssu_flat_fp32", 21, 2, 1, 64, 16, 1, heads=False)
    decode("ssu_heads_tie_fp32", 22, 3, 4, 16, 32, 2, tie=True, steps=3)
    decode("ssu_heads_untied_fp32", 23, 2, 4, 8, 64, 4, has_z=False)
    decode("ssu_heads_tie_bf16", 24, 2, 4, 64, 128, 1, dtype=torch.bfloat16, tie=True, steps=4)
    ssd("ssd_fp32_z", 31, 2, 256, 4, 16, 2, 16, 64)
    ssd("ssd_fp32_dhp_noz", 32, 1, 192, 3, 8, 1, 32, 64, has_z=False, D_hdim=True)
    ssd("ssd_fp32_init", 33, 2, 128, 2, 16, 1, 16, 32, with_init=True)
    ssd("ssd_fp32_tail", 34, 1, 200, 2, 8, 2, 16, 64)
    ssd("ssd_bf16", 35, 1, 512, 2, 64, 1, 128, 256, dtype=torch.bfloat16)
    mamba1_bwd("m1b_fp32_g1", 61, 2, 4, 128, 8, 1)
    mamba1_bwd("m1b_fp32_g2_odd", 62, 2, 4, 372, 8, 2, has_z=False, has_bias=False, softplus=False)
    mamba1_bwd("m1b_fp32_constbc", 63, 2, 6, 100, 4, 1, const_b=True, const_c=True, has_D=False)
    mamba1_bwd("m1b_fp32_constb", 64, 1, 40, 77, 16, 1, const_b=True)
    mamba1_bwd("m1b_fp32_wide", 65, 2, 64, 200, 16, 2)
    mamba1_bwd("m1b_fp32_n40", 66, 1, 8, 60, 40, 1)
    mamba1_bwd("m1b_bf16", 67, 2, 64, 256, 16, 1, dtype=torch.bfloat16)


if __name__ == "__main__":
    sys.exit(main())
