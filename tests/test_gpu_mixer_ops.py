"""GPU parity of the steps either side of the scan (causal conv1d, gated RMSNorm) and of the fused Mamba-2 block
forward, through the C ABI, against the CPU oracle and the reference-generated fixtures."""
import math

import pytest
import torch
import torch.nn.functional as F

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close, golden_names, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _io(d):
    return (torch.bfloat16, TOL_BF16) if d["bf16"] else (torch.float32, TOL_FP32)


@pytest.mark.parametrize("layout", ["time_contiguous", "channels_contiguous"])
@pytest.mark.parametrize("name", golden_names("conv_"))
def test_conv1d_golden(name, layout):
    from mamba_b200 import causal_conv1d_fn, causal_conv1d_update
    d = load_golden(name)
    io, tol = _io(d)
    act = "silu" if d["has_act"] else None
    x = d["x"].to(DEV, io)
    if layout == "channels_contiguous":
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
    w, b = d["weight"].to(DEV), d["bias"].to(DEV)
    out, fin = causal_conv1d_fn(x, w, b, activation=act, return_final_states=True)
    assert out.stride() == x.stride() and out.dtype == io
    assert_close(out, d["out"], tol, name + " out")
    if "final_states" in d:
        assert_close(fin, d["final_states"], tol, name + " final_states")
    if "x_steps" in d:
        state = d["state0"].to(DEV, io)
        for s in range(d["x_steps"].shape[0]):
            o = causal_conv1d_update(d["x_steps"][s].to(DEV, io), state, w, b, act)
            assert_close(o, d["out_steps"][s], tol, f"{name} step {s}")
        assert_close(state, d["state_final"], tol, name + " state")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16)])
@pytest.mark.parametrize("batch,dim,L,W,layout", [(2, 5376, 300, 4, "cl"), (1, 264, 1000, 4, "cl"), (3, 100, 77, 3, "cl"), (2, 96, 513, 4, "cf"),
                                                  (1, 7, 19, 2, "cf"), (2, 64, 2, 4, "cl")])
def test_conv1d_shapes_and_options(dtype, tol, batch, dim, L, W, layout):
    """Mixer-sized and ragged shapes in both layouts, with a carried initial state, packed sequences and final states."""
    from mamba_b200 import causal_conv1d_fn
    g = torch.Generator().manual_seed(dim + L)
    x = torch.randn(batch, dim, L, generator=g).to(dtype)
    w, b = 0.5 * torch.randn(dim, W, generator=g), 0.1 * torch.randn(dim, generator=g)
    init = torch.randn(batch, dim, W - 1, generator=g).to(dtype)
    cut = sorted(set([0, L // 3, (2 * L) // 3, L]))
    seq_idx = torch.cat([torch.full((hi - lo,), i, dtype=torch.int32) for i, (lo, hi) in enumerate(zip(cut, cut[1:]))])[None].expand(batch, L)
    xd = x.to(DEV)
    if layout == "cl":
        xd = xd.transpose(1, 2).contiguous().transpose(1, 2)
    for kw in (dict(), dict(initial_states=init), dict(seq_idx=seq_idx)):
        want, wfin = oracle.causal_conv1d(x.float(), w, b, activation="silu", return_final_states=True, **{k: (v.float() if v.is_floating_point() else v) for k, v in kw.items()})
        got, fin = causal_conv1d_fn(xd, w.to(DEV), b.to(DEV), activation="silu", return_final_states=True, **{k: v.to(DEV) for k, v in kw.items()})
        assert_close(got, want, tol, f"conv {list(kw)} out")
        assert_close(fin, wfin, tol, f"conv {list(kw)} final_states")


def test_conv1d_reads_a_slice_of_the_projection_in_place():
    """The Mamba-2 mixer hands the conv a column slice of its input projection, viewed as (batch, dim, seqlen)."""
    from mamba_b200 import causal_conv1d_fn
    g = torch.Generator().manual_seed(9)
    b, L, lead, dim, tail = 2, 200, 64, 320, 24
    proj = torch.randn(b, L, lead + dim + tail, generator=g).bfloat16()
    w, bias = 0.5 * torch.randn(dim, 4, generator=g).bfloat16(), 0.1 * torch.randn(dim, generator=g).bfloat16()
    x = proj.to(DEV)[..., lead:lead + dim].transpose(1, 2)
    got = causal_conv1d_fn(x, w.to(DEV), bias.to(DEV), activation="silu")
    assert got.shape == (b, dim, L) and got.stride(1) == 1
    want = oracle.causal_conv1d(proj[..., lead:lead + dim].transpose(1, 2).float(), w.float(), bias.float(), activation="silu")
    assert_close(got, want, TOL_BF16, "conv on a projection slice")


def test_conv1d_errors_mirror_the_package():
    from mamba_b200 import causal_conv1d_fn
    x = torch.zeros(1, 8, 16, device=DEV)
    with pytest.raises(AssertionError, match="width between 2 and 4"):
        causal_conv1d_fn(x, torch.zeros(8, 5, device=DEV))
    with pytest.raises(NotImplementedError):
        causal_conv1d_fn(x, torch.zeros(8, 4, device=DEV), activation="relu")
    assert causal_conv1d_fn(x[:0], torch.zeros(8, 4, device=DEV)).shape == (0, 8, 16)


@pytest.mark.parametrize("name", golden_names("rms_"))
def test_rmsnorm_golden(name):
    from mamba_b200 import rmsnorm_fn
    d = load_golden(name)
    io, tol = _io(d)
    c = lambda k: None if k not in d else d[k].to(DEV)
    out = rmsnorm_fn(d["x"].to(DEV, io), c("weight"), c("bias"), z=None if "z" not in d else d["z"].to(DEV, io), eps=float(d["eps"]),
                     group_size=int(d["group_size"]), norm_before_gate=bool(d["norm_before_gate"]))
    assert out.dtype == io and out.shape == d["x"].shape
    assert_close(out, d["out"], tol, name)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16)])
@pytest.mark.parametrize("rows,cols,group,before", [((4, 300), 5120, 5120, False), ((2, 64), 5120, 640, False), ((1000,), 2048, 256, True),
                                                    ((33,), 72, 24, True), ((5,), 10, None, False), ((3,), 8192, None, True)])
def test_rmsnorm_shapes(dtype, tol, rows, cols, group, before):
    from mamba_b200 import rmsnorm_fn
    g = torch.Generator().manual_seed(cols)
    x, z = torch.randn(*rows, cols, generator=g).to(dtype), torch.randn(*rows, cols, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(cols, generator=g)
    want = oracle.rmsnorm_gated(x.float(), w, None, z.float(), eps=1e-5, group_size=group, norm_before_gate=before)
    got = rmsnorm_fn(x.to(DEV), w.to(DEV), None, z=z.to(DEV), eps=1e-5, group_size=group, norm_before_gate=before)
    assert_close(got, want, tol, "rmsnorm")


def _block_inputs(seed, b, L, nheads, headdim, ngroups, dstate, d_nonssm, d_model, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    dim = nheads * headdim
    conv_dim = dim + 2 * ngroups * dstate
    dtv = torch.exp(torch.rand(nheads, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    return dict(zxbcdt=r(b, L, 2 * d_nonssm + 2 * dim + 2 * ngroups * dstate + nheads).to(dtype), conv_w=(0.5 * r(conv_dim, 4)).to(dtype),
                conv_b=(0.1 * r(conv_dim)).to(dtype), dt_bias=dtv + torch.log(-torch.expm1(-dtv)), A=-(1 + 15 * torch.rand(nheads, generator=g)),
                D=r(nheads), norm_w=(1 + 0.1 * r(dim)).to(dtype), out_w=(r(d_model, d_nonssm + dim) / math.sqrt(dim)).to(dtype))


def _block_oracle(c, nheads, headdim, ngroups, dstate, d_nonssm, Q, rmsnorm, norm_before_gate):
    """The reference's composition (mamba_ssm/modules/mamba2.py:206-275), step by step on the CPU oracle."""
    f = lambda t: t.float()
    dim = nheads * headdim
    zx0, z, xBC, dt = torch.split(f(c["zxbcdt"]), [2 * d_nonssm, dim, dim + 2 * ngroups * dstate, nheads], dim=-1)
    io = c["zxbcdt"].dtype
    xBC = oracle.causal_conv1d(xBC.transpose(1, 2), f(c["conv_w"]), f(c["conv_b"]), activation="silu").transpose(1, 2).to(io).float()
    x, B, C = torch.split(xBC, [dim, ngroups * dstate, ngroups * dstate], dim=-1)
    b, L = x.shape[:2]
    y, fin = oracle.ssd_chunk_scan(x.reshape(b, L, nheads, headdim), dt, c["A"], B.reshape(b, L, ngroups, dstate), C.reshape(b, L, ngroups, dstate),
                                   Q, c["D"], None if rmsnorm else z.reshape(b, L, nheads, headdim), c["dt_bias"], dt_softplus=True)
    y = y.reshape(b, L, dim).to(io).float()
    if rmsnorm:
        y = oracle.rmsnorm_gated(y, f(c["norm_w"]), None, z, eps=1e-5, group_size=dim // ngroups, norm_before_gate=norm_before_gate).to(io).float()
    if d_nonssm > 0:
        x0, z0 = zx0.chunk(2, dim=-1)
        y = torch.cat([(F.silu(z0) * x0).to(io).float(), y], dim=-1)
    return F.linear(y, f(c["out_w"])), fin


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("rmsnorm,before,d_nonssm,ngroups", [(True, False, 0, 1), (True, True, 0, 2), (False, True, 0, 1), (True, False, 32, 2)])
def test_split_conv1d_scan_combined(dtype, tol, rmsnorm, before, d_nonssm, ngroups):
    """The fused Mamba-2 block forward (mamba_ssm/ops/triton/ssd_combined.py:983-1003).  bf16 runs take the tensor-core
    SSD kernels on strided views of the conv output; the tolerance allows for the three roundings to the storage
    dtype between the stages, which the oracle composition repeats."""
    from mamba_b200 import mamba_split_conv1d_scan_combined
    b, L, nheads, headdim, dstate, d_model, Q = 2, 512, 8, 64, 128, 256, 256
    c = _block_inputs(70 + d_nonssm + ngroups, b, L, nheads, headdim, ngroups, dstate, d_nonssm, d_model, dtype)
    want, wfin = _block_oracle(c, nheads, headdim, ngroups, dstate, d_nonssm, Q, rmsnorm, before)
    g = {k: v.to(DEV) for k, v in c.items()}
    out, fin = mamba_split_conv1d_scan_combined(g["zxbcdt"], g["conv_w"], g["conv_b"], g["dt_bias"], g["A"], g["D"], Q, return_final_states=True,
                                                activation="silu", rmsnorm_weight=g["norm_w"] if rmsnorm else None, rmsnorm_eps=1e-5,
                                                outproj_weight=g["out_w"], headdim=headdim, ngroups=ngroups, norm_before_gate=before)
    assert out.shape == (b, L, d_model) and out.dtype == dtype
    assert_close(out, want, tol, "block out")
    assert_close(fin, wfin, tol, "block final_states")


def _time_ms(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def test_streaming_rates_at_layer_size(capsys):
    """Both steps are pure streaming work: at the size of a Mamba-2 2.7B layer on 8 x 4096 tokens (inputs larger than
    L2) the achieved rate of algorithmic bytes (input read once + output written once) is reported and must be a
    sizeable share of what a device-to-device copy reaches on this part."""
    from mamba_b200 import causal_conv1d_fn, rmsnorm_fn
    b, L, d_ssm, ngroups, dstate = 8, 4096, 5120, 1, 128
    conv_dim = d_ssm + 2 * ngroups * dstate
    g = torch.Generator(device=DEV).manual_seed(0)
    xBC = torch.randn(b, L, conv_dim, generator=g, device=DEV).bfloat16()
    w, bias = torch.randn(conv_dim, 4, generator=g, device=DEV).bfloat16(), torch.randn(conv_dim, generator=g, device=DEV).bfloat16()
    y, z = torch.randn(b, L, d_ssm, generator=g, device=DEV).bfloat16(), torch.randn(b, L, d_ssm, generator=g, device=DEV).bfloat16()
    nw = torch.ones(d_ssm, device=DEV, dtype=torch.bfloat16)
    copy_src, copy_dst = torch.empty(1 << 28, device=DEV, dtype=torch.uint8), torch.empty(1 << 28, device=DEV, dtype=torch.uint8)
    t_copy = _time_ms(lambda: copy_dst.copy_(copy_src))
    t_conv = _time_ms(lambda: causal_conv1d_fn(xBC.transpose(1, 2), w, bias, activation="silu"))
    t_norm = _time_ms(lambda: rmsnorm_fn(y, nw, None, z=z, eps=1e-5, group_size=d_ssm // ngroups, norm_before_gate=False))
    copy_gbs = 2 * (1 << 28) / t_copy / 1e6
    conv_gbs = 2 * xBC.numel() * 2 / t_conv / 1e6
    norm_gbs = 3 * y.numel() * 2 / t_norm / 1e6
    with capsys.disabled():
        print(f"\n[mixer ops] copy {copy_gbs:.0f} GB/s; causal_conv1d (channels-last, {conv_dim} ch) {t_conv * 1e3:.1f} us = {conv_gbs:.0f} GB/s "
              f"({conv_gbs / copy_gbs:.2f} of copy); gated rmsnorm ({d_ssm} cols) {t_norm * 1e3:.1f} us = {norm_gbs:.0f} GB/s ({norm_gbs / copy_gbs:.2f} of copy)")
    assert conv_gbs > 0.3 * copy_gbs and norm_gbs > 0.3 * copy_gbs
