"""GPU parity of the single-token decode state update (through the C ABI)."""
import math

import pytest
import torch

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close, golden_names, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fn():
    from mamba_b200 import selective_state_update
    return selective_state_update


def _expand_tied(d, A, bias, D):
    """Golden fixtures store tied tensors densely; rebuild the stride-0 views the mixer passes."""
    if not d["tie"]:
        return A, bias, D
    return (A[:, :1, :1].expand_as(A), bias[:, :1].expand_as(bias), D[:, :1].expand_as(D))


@pytest.mark.parametrize("name", golden_names("ssu_"))
def test_golden(name):
    d = load_golden(name)
    io = torch.bfloat16 if d["bf16"] else torch.float32
    tol = TOL_BF16 if d["bf16"] else TOL_FP32
    state = d["state0"].to(DEV).to(io)
    A, bias, D = (d["A"].to(DEV), d["dt_bias"].to(DEV), d["D"].to(DEV))
    if d["heads"]:
        A, bias, D = _expand_tied(d, A, bias, D)
    for s in range(d["x"].shape[0]):
        dt = d["dt"][s].to(DEV).to(io)
        if d["heads"] and d["tie"]:
            dt = dt[..., :1].expand_as(dt)
        z = None if "z" not in d else d["z"][s].to(DEV).to(io)
        out = _fn()(state, d["x"][s].to(DEV).to(io), dt, A, d["B"][s].to(DEV).to(io), d["C"][s].to(DEV).to(io),
                    D, z, bias, dt_softplus=True)
        assert out.dtype == io
        assert_close(out, d["out"][s], tol, f"{name} out[{s}]")
    assert_close(state, d["state_final"], tol, name + " state")


def make(seed, batch, nheads, dim, N, groups, itype, tie, heads=True, nstates=None):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    nstates = nstates or batch
    if heads:
        state = r(nstates, nheads, dim, N).to(itype)
        x = r(batch, nheads, dim).to(itype)
        if tie:
            dt = r(batch, nheads, 1).to(itype).expand(batch, nheads, dim)
            bias = (torch.rand(nheads, 1, generator=g) - 4.0).expand(nheads, dim)
            A = (-torch.rand(nheads, 1, 1, generator=g) - 1.0).expand(nheads, dim, N)
            D = r(nheads, 1).expand(nheads, dim)
        else:
            dt = r(batch, nheads, dim).to(itype)
            bias = torch.rand(nheads, dim, generator=g) - 4.0
            A = -torch.rand(nheads, dim, N, generator=g) - 1.0
            D = r(nheads, dim)
        B, C = r(batch, groups, N), r(batch, groups, N)
        z = r(batch, nheads, dim).to(itype)
    else:
        state = r(nstates, dim, N).to(itype)
        x, dt, z = r(batch, dim).to(itype), r(batch, dim).to(itype), r(batch, dim).to(itype)
        bias = torch.rand(dim, generator=g) - 4.0
        A = -torch.rand(dim, N, generator=g) - 1.0
        B, C, D = r(batch, N), r(batch, N), r(dim)
    return dict(state=state, x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=bias)


def run_both(inp, tol, what, idx=None):
    f32 = lambda t: t.float()
    ref_state = f32(inp["state"]).clone()
    sel_state = ref_state if idx is None else ref_state[idx.clamp_min(0).long()].clone()
    want = oracle.selective_state_update(sel_state, f32(inp["x"]), f32(inp["dt"]), inp["A"], f32(inp["B"]), f32(inp["C"]),
                                         inp["D"], f32(inp["z"]), inp["dt_bias"], dt_softplus=True)
    c = {k: v.to(DEV) for k, v in inp.items()}
    state = c["state"].clone()
    got = _fn()(state, c["x"], c["dt"], c["A"], c["B"], c["C"], c["D"], c["z"], c["dt_bias"], dt_softplus=True,
                state_batch_indices=None if idx is None else idx.to(DEV))
    if idx is None:
        assert_close(got, want, tol, what + " out")
        assert_close(state, sel_state, tol, what + " state")
    else:
        live = idx >= 0
        assert_close(got[live.to(DEV)], want[live], tol, what + " out")
        assert torch.all(got[(~live).to(DEV)] == 0), "padding rows must produce zeros"
        expect = f32(inp["state"]).clone()
        expect[idx[live].long()] = sel_state[live]
        assert_close(state, expect, tol, what + " state")
    return got


ITYPES = [(torch.float32, TOL_FP32), (torch.float16, TOL_BF16), (torch.bfloat16, TOL_BF16)]


@pytest.mark.parametrize("itype,tol", ITYPES)
@pytest.mark.parametrize("dstate", [16, 32, 64])
@pytest.mark.parametrize("dim", [2048, 2064, 4096])
def test_flat(dim, dstate, itype, tol):
    """The no-heads (Mamba-1 step) form at the sizes of the reference's own test."""
    run_both(make(1, 2, 1, dim, dstate, 1, itype, False, heads=False), tol, f"flat dim{dim} n{dstate}")


@pytest.mark.parametrize("itype,tol", ITYPES)
@pytest.mark.parametrize("tie", [False, True])
@pytest.mark.parametrize("groups", [1, 2, 4])
@pytest.mark.parametrize("dstate", [16, 32, 64, 128])
def test_heads(dstate, groups, tie, itype, tol):
    run_both(make(2, 2, 8, 64, dstate, groups, itype, tie), tol, f"heads n{dstate} g{groups} tie{tie}")


@pytest.mark.parametrize("dstate,dim", [(5, 7), (24, 10), (256, 32), (320, 3)])
def test_odd_sizes_general_kernel(dstate, dim):
    run_both(make(3, 3, 2, dim, dstate, 1, torch.float32, False), TOL_FP32, f"odd n{dstate} dim{dim}")


@pytest.mark.parametrize("heads", [False, True])
def test_state_batch_indices(heads):
    """Gather through a larger state pool, with padding entries (< 0) producing zero rows."""
    batch, pool = 16, 40
    inp = make(4, batch, 4 if heads else 1, 64, 32, 1, torch.float32, False, heads=heads, nstates=pool)
    idx = torch.randperm(pool, generator=torch.Generator().manual_seed(0))[:batch].to(torch.int32)
    idx[3] = -1
    idx[9] = -1
    run_both(inp, TOL_FP32, "batch indices", idx=idx)


def test_strided_state_takes_the_general_kernel():
    inp = make(5, 2, 4, 16, 32, 1, torch.float32, True)
    big = torch.zeros(2, 4, 16, 64)
    big[..., ::2] = inp["state"]
    c = {k: v.to(DEV) for k, v in inp.items()}
    state = big.to(DEV)[..., ::2]
    assert state.stride(-1) == 2
    want_state = inp["state"].clone()
    want = oracle.selective_state_update(want_state, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["z"],
                                         inp["dt_bias"], dt_softplus=True)
    got = _fn()(state, c["x"], c["dt"], c["A"], c["B"], c["C"], c["D"], c["z"], c["dt_bias"], dt_softplus=True)
    assert_close(got, want, TOL_FP32, "strided out")
    assert_close(state, want_state, TOL_FP32, "strided state")


def test_tied_and_dense_views_agree():
    inp = make(6, 2, 8, 64, 128, 1, torch.bfloat16, True)
    c = {k: v.to(DEV) for k, v in inp.items()}
    s1, s2 = c["state"].float().clone(), c["state"].float().clone()
    o1 = _fn()(s1, c["x"], c["dt"], c["A"], c["B"], c["C"], c["D"], c["z"], c["dt_bias"], dt_softplus=True)
    o2 = _fn()(s2, c["x"], c["dt"].contiguous(), c["A"].contiguous(), c["B"], c["C"], c["D"].contiguous(), c["z"],
               c["dt_bias"].contiguous(), dt_softplus=True)
    assert_close(o1, o2, 1e-5, "tied vs dense out")
    assert_close(s1, s2, 1e-5, "tied vs dense state")


def bench_config4(batch, steps, seed=1004, nheads=80, P=64, N=128):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    state = 0.1 * r(batch, nheads, P, N)
    A = -(1 + 15 * torch.rand(nheads, generator=g))
    dtv = torch.exp(torch.rand(nheads, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    bias = dtv + torch.log(-torch.expm1(-dtv))
    D = r(nheads)
    xs = r(steps, batch, nheads, P).bfloat16()
    zs = r(steps, batch, nheads, P).bfloat16()
    dts = r(steps, batch, nheads).bfloat16()
    Bs, Cs = r(steps, batch, 1, N).bfloat16(), r(steps, batch, 1, N).bfloat16()
    return dict(state=state, A=A, dt_bias=bias, D=D, x=xs, z=zs, dt=dts, B=Bs, C=Cs)


def test_bench_config4_consecutive_steps():
    """Decode shape of the benchmark (80 heads x 64 x 128, fp32 state, bf16 activations, tied A/dt) for
    16 consecutive in-place steps on 4 batch rows, output checked every step."""
    batch, steps, H, P, N = 4, 16, 80, 64, 128
    d = bench_config4(batch, steps)
    ref_state = d["state"].clone()
    state = d["state"].to(DEV)
    A = d["A"].to(DEV)[:, None, None].expand(H, P, N)
    bias = d["dt_bias"].to(DEV)[:, None].expand(H, P)
    D = d["D"].to(DEV)[:, None].expand(H, P)
    for s in range(steps):
        dt = d["dt"][s].to(DEV)[..., None].expand(batch, H, P)
        got = _fn()(state, d["x"][s].to(DEV), dt, A, d["B"][s].to(DEV), d["C"][s].to(DEV), D, d["z"][s].to(DEV), bias,
                    dt_softplus=True)
        want = oracle.selective_state_update(ref_state, d["x"][s].float(), d["dt"][s].float()[..., None].expand(batch, H, P),
                                             d["A"][:, None, None].expand(H, P, N), d["B"][s].float(), d["C"][s].float(),
                                             d["D"][:, None].expand(H, P), d["z"][s].float(),
                                             d["dt_bias"][:, None].expand(H, P), dt_softplus=True)
        assert_close(got, want, TOL_BF16, f"step {s} out")
    assert_close(state, ref_state, TOL_FP32, "state after 16 steps")


def test_bench_config4_full_size():
    """The benchmark's own size: batch 256, 128 consecutive in-place steps.  Three batch rows are followed by the
    oracle through all 128 steps (rows are independent), and a second run from the same start gives the same
    bits (no atomics)."""
    batch, steps, H, P, N = 256, 128, 80, 64, 128
    d = bench_config4(batch, steps)
    rows = torch.tensor([3, 128, 255])
    A = d["A"].to(DEV)[:, None, None].expand(H, P, N)
    bias = d["dt_bias"].to(DEV)[:, None].expand(H, P)
    D = d["D"].to(DEV)[:, None].expand(H, P)
    dev = {k: d[k].to(DEV) for k in ("x", "z", "dt", "B", "C")}

    def run():
        state = d["state"].to(DEV)
        outs = []
        for s in range(steps):
            dt = dev["dt"][s][..., None].expand(batch, H, P)
            outs.append(_fn()(state, dev["x"][s], dt, A, dev["B"][s], dev["C"][s], D, dev["z"][s], bias, dt_softplus=True)[rows.to(DEV)])
        return state, torch.stack(outs)

    state1, outs1 = run()
    state2, outs2 = run()
    assert torch.equal(state1, state2) and torch.equal(outs1, outs2)
    ref_state = d["state"][rows].clone()
    nb = len(rows)
    for s in range(steps):
        want = oracle.selective_state_update(ref_state, d["x"][s][rows].float(), d["dt"][s][rows].float()[..., None].expand(nb, H, P),
                                             d["A"][:, None, None].expand(H, P, N), d["B"][s][rows].float(), d["C"][s][rows].float(),
                                             d["D"][:, None].expand(H, P), d["z"][s][rows].float(),
                                             d["dt_bias"][:, None].expand(H, P), dt_softplus=True)
        assert_close(outs1[s], want, TOL_BF16, f"step {s} out")
    assert_close(state1[rows.to(DEV)], ref_state, TOL_FP32, "state after 128 steps")


def test_decode_matches_scan_recurrence():
    """T decode steps equal the Mamba-1 scan over the same T tokens (out per step and final state)."""
    from mamba_b200 import selective_scan_fn
    b, d, N, T = 2, 32, 16, 24
    g = torch.Generator().manual_seed(8)
    u = torch.randn(b, d, T, generator=g).to(DEV)
    delta = torch.randn(b, d, T, generator=g).to(DEV)
    A = (-torch.rand(d, N, generator=g) - 0.5).to(DEV)
    B = torch.randn(b, N, T, generator=g).to(DEV)
    C = torch.randn(b, N, T, generator=g).to(DEV)
    D = torch.randn(d, generator=g).to(DEV)
    bias = (torch.rand(d, generator=g) - 3).to(DEV)
    out, last = selective_scan_fn(u, delta, A, B, C, D, None, bias, delta_softplus=True, return_last_state=True)
    state = torch.zeros(b, d, N, device=DEV)
    for t in range(T):
        o = _fn()(state, u[:, :, t].contiguous(), delta[:, :, t].contiguous(), A, B[:, :, t].contiguous(),
                  C[:, :, t].contiguous(), D, None, bias, dt_softplus=True)
        assert_close(o, out[:, :, t], TOL_FP32, f"token {t}")
    assert_close(state, last, TOL_FP32, "state vs last_state")
