"""Pins the CPU oracle (C restatement and PyTorch port) to golden outputs that
were produced by importing the reference's own pure-PyTorch definitions."""
import pytest
import torch

import oracle
from oracle import torch_port
from helpers import golden_names, load_golden, assert_close

PIN = 2e-5   # fp32 round-off between a double-precision loop and the reference's fp32 tensors


def _opt(d, k):
    return d.get(k)


@pytest.mark.parametrize("impl", ["c", "torch"])
@pytest.mark.parametrize("name", golden_names("m1_"))
def test_selective_scan_pinned(name, impl):
    d = load_golden(name)
    fn = oracle.selective_scan if impl == "c" else torch_port.selective_scan
    out, last = fn(d["u"], d["delta"], d["A"], d["B"], d["C"], _opt(d, "D"), _opt(d, "z"),
                   _opt(d, "delta_bias"), delta_softplus=True, return_last_state=True)
    # bf16 fixtures hold the reference output after its cast back to bf16
    tol = 4e-3 if d["bf16"] else PIN
    assert_close(out, d["out"], tol, name + " out")
    assert_close(last, d["last_state"], PIN, name + " last_state")


GRADS = ("du", "ddelta", "dA", "dB", "dC", "dD", "dz", "ddelta_bias")


@pytest.mark.parametrize("impl", ["c", "torch"])
@pytest.mark.parametrize("name", golden_names("m1b_"))
def test_selective_scan_bwd_pinned(name, impl):
    """The written-out adjoint (C) and autograd through the PyTorch port against autograd through the reference."""
    d = load_golden(name)
    ins = [_opt(d, k) for k in ("u", "delta", "A", "B", "C", "D", "z", "delta_bias")]
    sp = bool(d["delta_softplus"])
    if impl == "c":
        got = oracle.selective_scan_bwd(*ins, d["dout"], sp)
    else:
        leaves = [None if t is None else t.detach().clone().requires_grad_() for t in ins]
        out = torch_port.selective_scan(*leaves[:5], leaves[5], leaves[6], leaves[7], delta_softplus=sp)
        out.backward(d["dout"].to(out.dtype))
        got = [None if t is None else t.grad for t in leaves]
    # bf16 fixtures hold the gradients after autograd's cast back to the bf16 leaves, and the reference evaluates
    # silu(z) in bf16 there (selective_scan_interface.py:190-191), which reaches every gradient through dy: two
    # bf16 roundings
    tol = 8e-3 if d["bf16"] else PIN
    for k, g in zip(GRADS, got):
        if k not in d:
            assert g is None or k in ("dD", "dz", "ddelta_bias")
            continue
        assert_close(g, d[k], tol, f"{name} {k}")


@pytest.mark.parametrize("impl", ["c", "torch"])
@pytest.mark.parametrize("name", golden_names("ssu_"))
def test_state_update_pinned(name, impl):
    d = load_golden(name)
    fn = oracle.selective_state_update if impl == "c" else torch_port.selective_state_update
    state = d["state0"].clone()
    # a carried state narrowed to bf16 each step can flip one bf16 ulp between implementations
    tol = 4e-3 if d["bf16"] else PIN
    for s in range(d["x"].shape[0]):
        z = None if "z" not in d else d["z"][s]
        out = fn(state, d["x"][s], d["dt"][s], d["A"], d["B"][s], d["C"][s], d["D"], z, d["dt_bias"],
                 dt_softplus=True)
        if d["bf16"]:   # the fixture narrows the carried state to bf16 after each step
            state = state.bfloat16().float()
        assert_close(out, d["out"][s], tol, f"{name} out[{s}]")
    assert_close(state, d["state_final"], tol, name + " state")


@pytest.mark.parametrize("impl", ["c", "torch"])
@pytest.mark.parametrize("name", golden_names("ssd_"))
def test_ssd_pinned(name, impl):
    d = load_golden(name)
    Q = int(d["chunk_size"])
    if impl == "torch" and d["x"].shape[1] % Q != 0:
        pytest.skip("the PyTorch port, like the reference's chunked definition, needs whole chunks")
    fn = oracle.ssd_chunk_scan if impl == "c" else torch_port.ssd_chunk_scan
    out, fin = fn(d["x"], d["dt"], d["A"], d["B"], d["C"], Q, _opt(d, "D"), _opt(d, "z"), d["dt_bias"],
                  _opt(d, "initial_states"), dt_softplus=True)
    assert_close(out, d["out"], PIN, name + " out")
    assert_close(fin, d["final_states"], PIN, name + " final_states")


def test_oracle_ssd_equals_recurrence():
    """Cross-check inside the oracle: SSD with scalar A per head is the Mamba-1 recurrence."""
    g = torch.Generator().manual_seed(5)
    b, L, H, P, G, N, Q = 1, 96, 2, 4, 1, 8, 32
    x = torch.randn(b, L, H, P, generator=g)
    dt = torch.rand(b, L, H, generator=g)
    A = -torch.rand(H, generator=g) - 0.5
    B = torch.randn(b, L, G, N, generator=g)
    C = torch.randn(b, L, G, N, generator=g)
    out, fin = oracle.ssd_chunk_scan(x, dt, A, B, C, Q)
    u = x.permute(0, 2, 3, 1).reshape(b, H * P, L)
    dl = dt.permute(0, 2, 1).repeat_interleave(P, dim=1)
    A1 = A.repeat_interleave(P)[:, None].expand(H * P, N).contiguous()
    o1, l1 = oracle.selective_scan(u, dl, A1, B.permute(0, 2, 3, 1), C.permute(0, 2, 3, 1),
                                   return_last_state=True)
    assert_close(out.permute(0, 2, 3, 1).reshape(b, H * P, L), o1, 1e-6, "ssd vs scan")
    assert_close(fin.reshape(b, H * P, N), l1, 1e-6, "final vs last")


@pytest.mark.parametrize("name", golden_names("conv_"))
def test_causal_conv1d_pinned(name):
    """Prefill conv and the single-token steps that follow it, against the reference's nn.Conv1d / roll-and-sum forms."""
    d = load_golden(name)
    act = "silu" if d["has_act"] else None
    out, fin = oracle.causal_conv1d(d["x"], d["weight"], d["bias"], activation=act, return_final_states=True)
    assert_close(out, d["out"], PIN, name + " out")
    if "final_states" in d:
        assert_close(fin, d["final_states"], PIN, name + " final_states")
    if "x_steps" in d:
        state = d["state0"].clone()
        for s in range(d["x_steps"].shape[0]):
            o = oracle.causal_conv1d_update(d["x_steps"][s], state, d["weight"], d["bias"], act)
            assert_close(o, d["out_steps"][s], PIN, f"{name} step {s}")
        assert_close(state, d["state_final"], PIN, name + " state")


def test_causal_conv1d_options_agree_with_their_definition():
    """Carried state = the conv of the concatenated input; packed sequences = each sequence on its own."""
    g = torch.Generator().manual_seed(3)
    x, w, b = torch.randn(1, 5, 40, generator=g), torch.randn(5, 4, generator=g), torch.randn(5, generator=g)
    whole = oracle.causal_conv1d(x, w, b, activation="silu")
    first, fin = oracle.causal_conv1d(x[..., :17], w, b, activation="silu", return_final_states=True)
    second = oracle.causal_conv1d(x[..., 17:], w, b, initial_states=fin, activation="silu")
    assert_close(torch.cat([first, second], dim=-1), whole, 1e-6, "carried state")
    seq_idx = torch.cat([torch.zeros(17), torch.ones(23)]).int()[None]
    packed = oracle.causal_conv1d(x, w, b, seq_idx=seq_idx, activation="silu")
    alone = oracle.causal_conv1d(x[..., 17:], w, b, activation="silu")
    assert_close(packed[..., 17:], alone, 1e-6, "packed second sequence")
    assert_close(packed[..., :17], first, 1e-6, "packed first sequence")


@pytest.mark.parametrize("name", golden_names("rms_"))
def test_rmsnorm_gated_pinned(name):
    d = load_golden(name)
    out = oracle.rmsnorm_gated(d["x"], d["weight"], d.get("bias"), d.get("z"), eps=float(d["eps"]), group_size=int(d["group_size"]),
                               norm_before_gate=bool(d["norm_before_gate"]))
    assert_close(out, d["out"], PIN, name)
