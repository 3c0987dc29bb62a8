"""PyTorch-on-CPU restatement of the reference's pure-PyTorch scan definitions.

TEST / BASELINE INFRASTRUCTURE ONLY.  This is the form of the path the
reference itself can run on a CPU, so it is what the benchmark times as the
CPU baseline ("port"): the same tensor operations in the same order of
materialisation (dense ``exp(dt*A)`` tensors, a Python loop over time for
Mamba-1, per-chunk decay matrices for SSD), written independently.

Reference definitions followed:
  selective_scan        <- mamba_ssm/ops/selective_scan_interface.py:127-193
  selective_state_update<- mamba_ssm/ops/triton/selective_state_update.py:224-285
  ssd_chunk_scan        <- mamba_ssm/ops/triton/ssd_combined.py:687-725,
                           ssd_chunk_state.py:1094-1122, ssd_state_passing.py:327-350,
                           ssd_chunk_scan.py:1846-1887
"""
import torch
import torch.nn.functional as F


def _per_channel(t, dim):
    """(b, g, n, l) -> (b, dim, n, l) by repeating each group over its channels."""
    return t.repeat_interleave(dim // t.shape[1], dim=1)


def selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False,
                   return_last_state=False):
    in_dtype = u.dtype
    u, delta = u.float(), delta.float()
    if delta_bias is not None:
        delta = delta + delta_bias.float()[:, None]
    if delta_softplus:
        delta = F.softplus(delta)
    batch, dim, L = u.shape
    N = A.shape[1]
    B, C = B.float(), C.float()
    decay = torch.exp(delta[..., None] * A[None, :, None, :])              # (b, d, l, n)
    du = delta * u                                                         # (b, d, l)
    if B.dim() == 2:
        drive = du[..., None] * B[None, :, None, :]
    else:
        if B.dim() == 3:
            B = B[:, None]
        drive = du[..., None] * _per_channel(B, dim).transpose(2, 3)        # (b, d, l, n)
    if C.dim() == 3:
        C = C[:, None]
    Cc = _per_channel(C, dim) if C.dim() == 4 else None                    # (b, d, n, l)
    h = torch.zeros(batch, dim, N, dtype=torch.float32)
    ys = []
    for t in range(L):
        h = decay[:, :, t] * h + drive[:, :, t]
        ys.append((h * (C if Cc is None else Cc[..., t])).sum(-1))
    y = torch.stack(ys, dim=2)
    if D is not None:
        y = y + u * D.float()[:, None]
    if z is not None:
        y = y * F.silu(z.float())
    y = y.to(in_dtype)
    return (y, h) if return_last_state else y


def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False):
    heads = state.dim() > 3
    if not heads:
        state_v, x, dt, A = state[:, None], x[:, None], dt[:, None], A[None]
        B, C = B[:, None], C[:, None]
        D = None if D is None else D[None]
        z = None if z is None else z[:, None]
        dt_bias = None if dt_bias is None else dt_bias[None]
    else:
        state_v = state
    nheads, ngroups = state_v.shape[1], B.shape[1]
    if dt_bias is not None:
        dt = dt + dt_bias
    if dt_softplus:
        dt = F.softplus(dt)
    Bh = B.repeat_interleave(nheads // ngroups, dim=1)                     # (b, h, n)
    Ch = C.repeat_interleave(nheads // ngroups, dim=1)
    decay = torch.exp(dt[..., None] * A)                                   # (b, h, p, n)
    drive = dt[..., None] * Bh[:, :, None, :] * x[..., None]
    state_v.copy_(state_v * decay + drive)
    out = (state_v.to(Ch.dtype) * Ch[:, :, None, :]).sum(-1)
    if D is not None:
        out = out + (x * D).to(out.dtype)
    if z is not None:
        out = out * F.silu(z)
    out = out.to(x.dtype)
    return out if heads else out[:, 0]


def ssd_chunk_scan(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                   dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """Returns ``(out, final_states)``; seqlen must be a multiple of ``chunk_size``."""
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    Q = chunk_size
    assert L % Q == 0
    nc = L // Q
    dtf = dt.float().view(b, nc, Q, H).permute(0, 3, 1, 2)                 # (b, h, c, q)
    if dt_bias is not None:
        dtf = dtf + dt_bias.float()[None, :, None, None]
    if dt_softplus:
        dtf = F.softplus(dtf)
    if dt_limit != (0.0, float("inf")):
        dtf = dtf.clamp(dt_limit[0], dt_limit[1])
    cum = torch.cumsum(dtf * A.float()[None, :, None, None], dim=-1)       # (b, h, c, q)
    xc = x.view(b, nc, Q, H, P)
    Bc = B.repeat_interleave(H // G, dim=2).view(b, nc, Q, H, N)
    Cc = C.repeat_interleave(H // G, dim=2).view(b, nc, Q, H, N)
    cdt = x.dtype
    # chunk states: sum_k exp(cum_last - cum_k) dt_k x_k (outer) B_k
    w = (torch.exp(cum[..., -1:] - cum) * dtf).to(cdt)                      # (b, h, c, q)
    states = torch.einsum("bcqhn,bhcq,bcqhp->bchpn", Bc.to(cdt), w, xc).float()
    # inter-chunk recurrence (sequential form of the reference's decay-matrix einsum)
    carry = torch.exp(cum[..., -1])                                        # (b, h, c)
    h = torch.zeros(b, H, P, N) if initial_states is None else initial_states.float().clone()
    prev = []
    for c in range(nc):
        prev.append(h)
        h = carry[:, :, c, None, None] * h + states[:, c]
    prev = torch.stack(prev, dim=1).to(cdt)                                # (b, c, h, p, n)
    # chunk outputs
    cb = torch.einsum("bcqhn,bcshn->bchqs", Cc, Bc)
    decay = torch.exp(cum[..., :, None] - cum[..., None, :]).permute(0, 2, 1, 3, 4)
    mask = torch.tril(torch.ones(Q, Q, dtype=torch.bool))
    scores = (cb * decay).masked_fill(~mask, 0)
    y = torch.einsum("bchqs,bhcs,bcshp->bcqhp", scores.to(cdt), dtf.to(cdt), xc)
    y_prev = torch.einsum("bcqhn,bchpn->bcqhp", Cc, prev.to(Cc.dtype)) * torch.exp(cum).permute(0, 2, 3, 1)[..., None]
    y = (y + y_prev).reshape(b, L, H, P)
    if D is not None:
        y = y + x * (D[:, None] if D.dim() == 1 else D)
    if z is not None:
        y = y * F.silu(z)
    return y, h
