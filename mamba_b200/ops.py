"""The three scan operators of state-spaces/mamba, served by libmamba_b200.so.

Signatures, argument meaning, return values and error behaviour mirror the reference:

* ``selective_scan_fn``          mamba_ssm/ops/selective_scan_interface.py:118-124 (forward of :36-68)
* ``mamba_chunk_scan_combined``  mamba_ssm/ops/triton/ssd_combined.py:628-648 (forward :343-394)
* ``selective_state_update``     mamba_ssm/ops/triton/selective_state_update.py:135-221

The SSD and decode operators are forward only (their outputs carry no autograd graph); the Mamba-1 scan also has
its backward (``selective_scan_bwd``).  PyTorch supplies device memory and the current stream; all arithmetic
happens in the library's CUDA kernels.
"""
import ctypes
import math
import os

import torch

from . import _lib as L


def _last_dim_contiguous(t):
    return t if t is None or t.stride(-1) == 1 else t.contiguous()


def _fp32(t):
    return t if t is None or t.dtype == torch.float32 else t.float()


# --------------------------------------------------------------------------------------- Mamba-1
def selective_scan_fn(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False,
                      return_last_state=False):
    """Mamba-1 selective scan.

    u, delta, z: (batch, dim, seqlen).  A: (dim, dstate) fp32.  B, C: (batch, dstate, seqlen),
    (batch, ngroups, dstate, seqlen) or constant (dim, dstate).  D, delta_bias: (dim) fp32.
    Returns ``out`` (gated by silu(z) when z is given) or ``(out, last_state)`` with
    ``last_state`` (batch, dim, dstate) fp32.

    When gradients are enabled and an input requires them, the result carries an autograd node whose backward is
    the library's backward kernel (the role of SelectiveScanFn.backward, selective_scan_interface.py:70-100); as in
    the reference, no gradient flows through ``last_state``.
    """
    tensors = (u, delta, A, B, C, D, z, delta_bias)
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        return _SelectiveScanFn.apply(u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)
    return _selective_scan(u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)


def _scan_inputs(u, delta, A, B, C, D, z, delta_bias):
    """The contiguity fix-ups and shape checks of SelectiveScanFn.forward (selective_scan_interface.py:40-57) and of the
    extension (selective_scan.cpp:233-305).  Returns the tensors the library reads plus (B_var, C_var, ngroups)."""
    if A.is_complex():
        raise NotImplementedError("mamba_b200: complex A is not supported")
    u, delta, z = _last_dim_contiguous(u), _last_dim_contiguous(delta), _last_dim_contiguous(z)
    B, C = _last_dim_contiguous(B), _last_dim_contiguous(C)
    D = None if D is None else _fp32(D).contiguous()
    delta_bias = None if delta_bias is None else _fp32(delta_bias).contiguous()
    A = _fp32(A)
    assert u.dim() == 3 and delta.shape == u.shape, "u and delta must both be (batch, dim, seqlen)"
    assert delta.dtype == u.dtype, "u and delta must have the same dtype"
    batch, dim, seqlen = u.shape
    assert A.dim() == 2 and A.shape[0] == dim, "A must be (dim, dstate)"
    dstate = A.shape[1]
    B_var, C_var = B.dim() >= 3, C.dim() >= 3
    if B_var and B.dim() == 3:
        B = B.unsqueeze(1)
    if C_var and C.dim() == 3:
        C = C.unsqueeze(1)
    ngroups = B.shape[1] if B_var else (C.shape[1] if C_var else 1)
    for name, t, var in (("B", B, B_var), ("C", C, C_var)):
        if var:
            assert t.shape == (batch, ngroups, dstate, seqlen), f"{name} must be (batch, ngroups, dstate, seqlen)"
            assert t.dtype == u.dtype, f"variable {name} must have the dtype of u"
        else:
            assert t.shape == (dim, dstate), f"constant {name} must be (dim, dstate)"
    if not B_var:
        B = _fp32(B)
    if not C_var:
        C = _fp32(C)
    if z is not None:
        assert z.shape == u.shape and z.dtype == u.dtype, "z must match u"
    if D is not None:
        assert D.shape == (dim,)
    if delta_bias is not None:
        assert delta_bias.shape == (dim,)
    return (u, delta, A, B, C, D, z, delta_bias), (B_var, C_var, ngroups)


def _selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, return_last_state=False,
                    out=None):
    """selective_scan_fn with an optional caller-provided ``out`` (batch, dim, seqlen; last stride 1)."""
    L.require_cuda(u, delta, A, B, C, D, z, delta_bias, out)
    (u, delta, A, B, C, D, z, delta_bias), (B_var, C_var, ngroups) = _scan_inputs(u, delta, A, B, C, D, z, delta_bias)
    batch, dim, seqlen = u.shape
    dstate = A.shape[1]
    if out is None:
        out = torch.empty_like(delta)
    assert out.shape == u.shape and out.dtype == u.dtype and out.stride(-1) == 1, "out must match u, last stride 1"
    last_state = torch.empty(batch, dim, dstate, device=u.device, dtype=torch.float32) if return_last_state else None

    a = L.ScanArgs()
    a.u, a.delta, a.A, a.B, a.C = L.ptr(u), L.ptr(delta), L.ptr(A), L.ptr(B), L.ptr(C)
    a.D, a.z, a.delta_bias = L.ptr(D), L.ptr(z), L.ptr(delta_bias)
    a.out, a.out_pregate, a.last_state = L.ptr(out), None, L.ptr(last_state)
    a.batch, a.dim, a.seqlen, a.dstate, a.ngroups = batch, dim, seqlen, dstate, ngroups
    a.io_dtype = L.dtype_code(u.dtype)
    a.B_variable, a.C_variable, a.delta_softplus = int(B_var), int(C_var), int(bool(delta_softplus))
    a.device = u.device.index
    L.set_strides(a.u_stride, u, 2)
    L.set_strides(a.delta_stride, delta, 2)
    L.set_strides(a.out_stride, out, 2)
    if z is not None:
        L.set_strides(a.z_stride, z, 2)
    L.set_strides(a.A_stride, A, 2)
    L.set_strides(a.B_stride, B, 3 if B_var else 2)
    L.set_strides(a.C_stride, C, 3 if C_var else 2)
    # few (batch, channel) rows: lend the library scratch so that it can cut the sequence into segments that run side by side
    need = ctypes.c_size_t(0)
    L.check(L.lib().mb200_scan_scratch_bytes(ctypes.byref(a), ctypes.byref(need)))
    scratch = torch.empty(need.value, dtype=torch.uint8, device=u.device) if need.value else None
    a.scratch, a.scratch_bytes = L.ptr(scratch), need.value
    L.check(L.lib().mb200_selective_scan_fwd(ctypes.byref(a), L.stream_ptr(u.device)))
    return out if not return_last_state else (out, last_state)


def selective_scan_bwd(u, delta, A, B, C, D, z, delta_bias, dout, delta_softplus=False, scratch_bytes=None, outputs=None):
    """Gradients of selective_scan_fn for ``dout`` = dL/d(out): the call ``selective_scan_cuda.bwd`` serves in the
    reference (selective_scan_interface.py:83-86, selective_scan.cpp:338-492).  The scan is recomputed from the inputs,
    so nothing of the forward is needed.  Returns ``(du, ddelta, dA, dB, dC, dD, dz, ddelta_bias)``: du, ddelta, dz in
    the dtype of u, dA, dD, ddelta_bias fp32, dB and dC in the dtype and shape of B and C (accumulated in fp32);
    None where the input is None.  ``scratch_bytes`` caps the temporary buffer (default: what the library asks for, at
    most 1 GiB): with less than the whole batch needs, the batch is walked in slices (one row's worth is the minimum).
    ``outputs`` = (du, ddelta, dz) lets the caller provide these three (shape and dtype of u, last stride 1; dz None
    without z), as the extension accepts a preallocated dz (selective_scan.cpp:434-441)."""
    L.require_cuda(u, delta, A, B, C, D, z, delta_bias, dout)
    squeeze_B, squeeze_C = B.dim() == 3, C.dim() == 3
    B_dtype, C_dtype = B.dtype, C.dtype
    (u, delta, A, B, C, D, z, delta_bias), (B_var, C_var, ngroups) = _scan_inputs(u, delta, A, B, C, D, z, delta_bias)
    batch, dim, seqlen = u.shape
    dstate = A.shape[1]
    dout = _last_dim_contiguous(dout)
    assert dout.shape == u.shape and dout.dtype == u.dtype, "dout must match u"
    dev = u.device
    if outputs is None:
        du, ddelta = torch.empty_like(u), torch.empty_like(delta)
        dz = torch.empty_like(z) if z is not None else None
    else:
        du, ddelta, dz = outputs
        for t in (du, ddelta) + ((dz,) if z is not None else ()):
            assert t is not None and t.shape == u.shape and t.dtype == u.dtype and t.stride(-1) == 1, \
                "outputs must have the shape and dtype of u and a unit last stride"
        L.require_cuda(du, ddelta, dz)
    f32 = dict(device=dev, dtype=torch.float32)
    dA = torch.empty(dim, dstate, **f32)
    dB = torch.empty(B.shape, **f32)
    dC = torch.empty(C.shape, **f32)
    dD = torch.empty(dim, **f32) if D is not None else None
    dbias = torch.empty(dim, **f32) if delta_bias is not None else None

    a = L.ScanBwdArgs()
    a.u, a.delta, a.A, a.B, a.C = L.ptr(u), L.ptr(delta), L.ptr(A), L.ptr(B), L.ptr(C)
    a.D, a.z, a.delta_bias, a.dout = L.ptr(D), L.ptr(z), L.ptr(delta_bias), L.ptr(dout)
    a.du, a.ddelta, a.dz = L.ptr(du), L.ptr(ddelta), L.ptr(dz)
    a.dA, a.dB, a.dC, a.dD, a.ddelta_bias = L.ptr(dA), L.ptr(dB), L.ptr(dC), L.ptr(dD), L.ptr(dbias)
    a.batch, a.dim, a.seqlen, a.dstate, a.ngroups = batch, dim, seqlen, dstate, ngroups
    a.io_dtype = L.dtype_code(u.dtype)
    a.B_variable, a.C_variable, a.delta_softplus = int(B_var), int(C_var), int(bool(delta_softplus))
    a.device = dev.index
    for field, t in ((a.u_stride, u), (a.delta_stride, delta), (a.dout_stride, dout), (a.du_stride, du),
                     (a.ddelta_stride, ddelta)):
        L.set_strides(field, t, 2)
    if z is not None:
        L.set_strides(a.z_stride, z, 2)
        L.set_strides(a.dz_stride, dz, 2)
    L.set_strides(a.A_stride, A, 2)
    L.set_strides(a.B_stride, B, 3 if B_var else 2)
    L.set_strides(a.C_stride, C, 3 if C_var else 2)
    need = ctypes.c_size_t(0)
    L.check(L.lib().mb200_scan_bwd_scratch_bytes(ctypes.byref(a), ctypes.byref(need)))
    nbytes = need.value if scratch_bytes is None else min(need.value, int(scratch_bytes))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    a.scratch, a.scratch_bytes = L.ptr(scratch), nbytes
    L.check(L.lib().mb200_selective_scan_bwd(ctypes.byref(a), L.stream_ptr(dev)))
    dB, dC = dB.to(B_dtype), dC.to(C_dtype)       # selective_scan.cpp:487
    if squeeze_B:
        dB = dB.squeeze(1)
    if squeeze_C:
        dC = dC.squeeze(1)
    return du, ddelta, dA, dB, dC, dD, dz, dbias


class _SelectiveScanFn(torch.autograd.Function):
    """Autograd node of selective_scan_fn.  Unlike SelectiveScanFn (selective_scan_interface.py:34-100) it saves only the
    inputs: the backward kernel recomputes the scan, so neither the prefix tensor nor the pre-gate output is kept."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state):
        res = _selective_scan(u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)
        ctx.delta_softplus = delta_softplus
        ctx.save_for_backward(u, delta, A, B, C, D, z, delta_bias)
        if return_last_state:
            ctx.mark_non_differentiable(res[1])
        return res

    @staticmethod
    def backward(ctx, dout, *unused):
        u, delta, A, B, C, D, z, delta_bias = ctx.saved_tensors
        du, ddelta, dA, dB, dC, dD, dz, dbias = selective_scan_bwd(u, delta, A, B, C, D, z, delta_bias, dout,
                                                                   ctx.delta_softplus)
        as_of = lambda g, t: None if g is None else g.to(t.dtype).reshape(t.shape)
        return (du, ddelta, as_of(dA, A), dB, dC, as_of(dD, D) if D is not None else None, dz,
                as_of(dbias, delta_bias) if delta_bias is not None else None, None, None)


# --------------------------------------------------------------------------------------- decode
def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False,
                           state_batch_indices=None):
    """Single-token decode update; ``state`` is modified in place.

    state: (batch, dim, dstate) or (batch, nheads, dim, dstate); x, dt, z: (batch, dim) or
    (batch, nheads, dim); A: (dim, dstate) or (nheads, dim, dstate); B, C: (batch, dstate) or
    (batch, ngroups, dstate); D, dt_bias: (dim,) or (nheads, dim).  Stride-0 (broadcast) views of
    A, dt, dt_bias and D are used as they are.  Returns out with the shape and dtype of x.
    """
    L.require_cuda(state, x, dt, A, B, C, D, z, dt_bias, state_batch_indices)
    has_heads = state.dim() > 3
    if state.dim() == 3:
        state = state.unsqueeze(1)
    if x.dim() == 2:
        x = x.unsqueeze(1)
    if dt.dim() == 2:
        dt = dt.unsqueeze(1)
    if A.dim() == 2:
        A = A.unsqueeze(0)
    if B.dim() == 2:
        B = B.unsqueeze(1)
    if C.dim() == 2:
        C = C.unsqueeze(1)
    if D is not None and D.dim() == 1:
        D = D.unsqueeze(0)
    if z is not None and z.dim() == 2:
        z = z.unsqueeze(1)
    if dt_bias is not None and dt_bias.dim() == 1:
        dt_bias = dt_bias.unsqueeze(0)
    _, nheads, dim, dstate = state.shape
    batch = x.shape[0]
    assert x.shape == (batch, nheads, dim)
    assert dt.shape == x.shape
    assert A.shape == (nheads, dim, dstate)
    ngroups = B.shape[1]
    assert nheads % ngroups == 0, "nheads must be divisible by ngroups"
    assert B.shape == (batch, ngroups, dstate)
    assert C.shape == B.shape and C.dtype == B.dtype
    if D is not None:
        assert D.shape == (nheads, dim)
    if z is not None:
        assert z.shape == x.shape and z.dtype == x.dtype
    if dt_bias is not None:
        assert dt_bias.shape == (nheads, dim)
    if state_batch_indices is not None:
        assert state_batch_indices.shape == (batch,)
        if state_batch_indices.dtype != torch.int32:
            state_batch_indices = state_batch_indices.to(torch.int32)
        state_batch_indices = state_batch_indices.contiguous()
    else:
        assert state.shape[0] == batch
    A, D, dt_bias = _fp32(A), _fp32(D), _fp32(dt_bias)
    out = torch.empty_like(x)

    a = L.SsuArgs()
    a.state, a.x, a.dt, a.A, a.B, a.C = L.ptr(state), L.ptr(x), L.ptr(dt), L.ptr(A), L.ptr(B), L.ptr(C)
    a.D, a.z, a.dt_bias, a.out = L.ptr(D), L.ptr(z), L.ptr(dt_bias), L.ptr(out)
    a.state_batch_indices = L.ptr(state_batch_indices)
    a.batch, a.nheads, a.dim, a.dstate, a.ngroups = batch, nheads, dim, dstate, ngroups
    a.state_dtype, a.x_dtype = L.dtype_code(state.dtype), L.dtype_code(x.dtype)
    a.dt_dtype, a.bc_dtype = L.dtype_code(dt.dtype), L.dtype_code(B.dtype)
    a.dt_softplus = int(bool(dt_softplus))
    a.device = x.device.index
    L.set_strides(a.state_stride, state, 4)
    L.set_strides(a.x_stride, x, 3)
    L.set_strides(a.dt_stride, dt, 3)
    L.set_strides(a.out_stride, out, 3)
    L.set_strides(a.A_stride, A, 3)
    L.set_strides(a.B_stride, B, 3)
    L.set_strides(a.C_stride, C, 3)
    if z is not None:
        L.set_strides(a.z_stride, z, 3)
    if D is not None:
        L.set_strides(a.D_stride, D, 2)
    if dt_bias is not None:
        L.set_strides(a.dt_bias_stride, dt_bias, 2)
    L.check(L.lib().mb200_selective_state_update(ctypes.byref(a), L.stream_ptr(x.device)))
    return out if has_heads else out.squeeze(1)


# --------------------------------------------------------------------------------------- SSD
def _ssd_args(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus, dt_limit):
    batch, seqlen, nheads, headdim = x.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, seqlen, nheads)
    assert A.shape == (nheads,)
    assert C.shape == B.shape
    assert B.dtype == x.dtype and C.dtype == x.dtype, "B and C must have the dtype of x"
    if z is not None:
        assert z.shape == x.shape and z.dtype == x.dtype
    if D is not None:
        assert D.shape == (nheads, headdim) or D.shape == (nheads,)
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, headdim, dstate)
    a = L.SsdArgs()
    a.batch, a.seqlen, a.nheads, a.headdim = batch, seqlen, nheads, headdim
    a.ngroups, a.dstate, a.chunk_size = ngroups, dstate, int(chunk_size)
    a.io_dtype, a.dt_dtype = L.dtype_code(x.dtype), L.dtype_code(dt.dtype)
    a.dt_softplus = int(bool(dt_softplus))
    a.D_has_hdim = int(D is not None and D.dim() == 2)
    a.dt_min, a.dt_max = float(dt_limit[0]), min(float(dt_limit[1]), 3.0e38)
    a.device = x.device.index
    return a


# What ssd_status() needs of the most recent SSD call: the 256-byte tail of its scratch buffer -- the buffer itself
# while it is small, a copy of the tail made on the stream when holding the buffer would pin a lot of memory until
# the next call -- or the argument struct of a call that used the library's built-in buffer.
_PIN_SCRATCH_BELOW = 64 << 20
_last_ssd_status = None
_last_ssd_static_args = None
# MB200_CHECK_STATUS=1: every SSD call synchronises and raises if a kernel abandoned a bounded wait (debugging aid).
_CHECK_STATUS = os.environ.get("MB200_CHECK_STATUS", "0") not in ("", "0")


def scan_status(device=None):
    """Status word of the TMA-fed selective-scan kernel on `device` (synchronises the device).

    0 means no bounded wait of that kernel has ever run out on the device.  Meant for tests and
    debugging; the operators themselves never synchronise."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    st = ctypes.c_int32(0)
    L.check(L.lib().mb200_scan_status(dev, ctypes.byref(st)))
    return int(st.value)


def ssd_status():
    """Status word of the most recent SSD call on this process (synchronises the device).

    0 means every kernel ran to completion.  A non-zero value means a kernel abandoned one of its
    bounded waits (its code is the value) and the outputs of that call must not be used.  Meant for
    tests and debugging; the operators themselves never synchronise."""
    if _last_ssd_static_args is not None:
        st = ctypes.c_int32(0)
        L.check(L.lib().mb200_ssd_static_status(ctypes.byref(_last_ssd_static_args), ctypes.byref(st)))
        return int(st.value)
    if _last_ssd_status is None:
        return 0
    return int(_last_ssd_status[:4].view(torch.int32).item())


def seqlen_of(x):
    return x.shape[1]


def _ssd_launch(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus, dt_limit,
                phases, out=None, final_states=None, range_decay=None, scratch=None, builtin_scratch=False,
                cu_seqlens=None, varlen_states=None):
    L.require_cuda(x, dt, A, B, C, D, z, dt_bias, initial_states, seq_idx)
    if builtin_scratch:
        # this path must not create device tensors: the caller supplies everything in its final form
        for name, t, want in (("A", A, torch.float32), ("dt_bias", dt_bias, torch.float32), ("D", D, torch.float32),
                              ("initial_states", initial_states, torch.float32)):
            assert t is None or (t.dtype == want and t.is_contiguous()), f"{name} must be contiguous {want}"
        for name, t in (("x", x), ("z", z), ("B", B), ("C", C)):
            assert t is None or t.stride(-1) == 1, f"{name} must have a unit last stride"
        assert out is not None, "out must be supplied"
        assert seq_idx is None
    B, C = _last_dim_contiguous(B), _last_dim_contiguous(C)
    x, z = _last_dim_contiguous(x), _last_dim_contiguous(z)
    A, dt_bias = _fp32(A).contiguous(), None if dt_bias is None else _fp32(dt_bias).contiguous()
    D = None if D is None else _fp32(D).contiguous()
    initial_states = None if initial_states is None else _fp32(initial_states).contiguous()
    if seq_idx is not None:
        seq_idx = seq_idx.to(torch.int32).contiguous()
    a = _ssd_args(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus, dt_limit)
    a.phases = phases
    need = ctypes.c_size_t(0)
    L.check(L.lib().mb200_ssd_scratch_bytes(ctypes.byref(a), ctypes.byref(need)))
    if scratch is None and not builtin_scratch:
        scratch = torch.empty(max(need.value, 256), dtype=torch.uint8, device=x.device)
    if out is None and phases & L.PHASE_OUTPUT:
        out = torch.empty_like(x)
    a.x, a.dt, a.A, a.B, a.C = L.ptr(x), L.ptr(dt), L.ptr(A), L.ptr(B), L.ptr(C)
    a.D, a.z, a.dt_bias, a.seq_idx = L.ptr(D), L.ptr(z), L.ptr(dt_bias), L.ptr(seq_idx)
    a.initial_states, a.out, a.final_states = L.ptr(initial_states), L.ptr(out), L.ptr(final_states)
    a.range_decay = L.ptr(range_decay)
    if cu_seqlens is not None:
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        a.cu_seqlens, a.varlen_states, a.num_seqs = L.ptr(cu_seqlens), L.ptr(varlen_states), cu_seqlens.numel() - 1
    a.scratch, a.scratch_bytes = (None, 0) if builtin_scratch else (L.ptr(scratch), scratch.numel())
    L.set_strides(a.x_stride, x, 3)
    L.set_strides(a.dt_stride, dt, 3)
    L.set_strides(a.B_stride, B, 3)
    L.set_strides(a.C_stride, C, 3)
    if out is not None:
        L.set_strides(a.out_stride, out, 3)
    if z is not None:
        L.set_strides(a.z_stride, z, 3)
    entry = L.lib().mb200_ssd_chunk_scan_fwd_static if builtin_scratch else L.lib().mb200_ssd_chunk_scan_fwd
    L.check(entry(ctypes.byref(a), L.stream_ptr(x.device)))
    global _last_ssd_status, _last_ssd_static_args
    if builtin_scratch:
        _last_ssd_status, _last_ssd_static_args = None, a        # no device tensor is created on this path
    else:
        _last_ssd_static_args = None
        if seqlen_of(x) == 0:
            _last_ssd_status = None
        else:
            tail = scratch[-256:]
            _last_ssd_status = tail if scratch.numel() <= _PIN_SCRATCH_BELOW else tail.clone()
    if _CHECK_STATUS:
        st = ssd_status()
        if st:
            raise RuntimeError(f"mamba_b200: an SSD kernel abandoned a bounded wait (status {st}); the outputs are invalid")
    return out, scratch


def mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                              seq_idx=None, cu_seqlens=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                              return_final_states=False, return_varlen_states=False, state_dtype=None):
    """Mamba-2 SSD chunked scan forward.

    x, z: (batch, seqlen, nheads, headdim); dt: (batch, seqlen, nheads); A, dt_bias: (nheads);
    B, C: (batch, seqlen, ngroups, dstate); D: (nheads,) or (nheads, headdim);
    initial_states: (batch, nheads, headdim, dstate).  seq_idx: int (batch, seqlen) ids of packed sequences
    (non-decreasing, starting at 0); cu_seqlens: int (num_sequences + 1), read only with
    ``return_varlen_states`` (batch must then be 1).
    Returns ``out``, ``(out, final_states)``, ``(out, varlen_states)`` or ``(out, final_states, varlen_states)``
    like the reference; final_states fp32 (batch, nheads, headdim, dstate), varlen_states fp32
    (num_sequences, nheads, headdim, dstate).  ``state_dtype`` is accepted for signature compatibility and not
    used: the running inter-chunk state is fp32 on chip; the copy of it that the chunk-output stage multiplies by C
    is rounded to the input dtype on the tensor-core path (as the reference's default does) and stays fp32 on the
    general path.
    """
    if not return_varlen_states:
        cu_seqlens = None
    else:
        assert cu_seqlens is not None, "cu_seqlens must be provided if return_varlen_states is True"
        assert x.shape[0] == 1, "passing cu_seqlens to get the varlen states is only supported if batch dimension is 1"
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[-1]
    final_states = (torch.empty(batch, nheads, headdim, dstate, device=x.device, dtype=torch.float32)
                    if return_final_states else None)
    varlen_states = (torch.empty(cu_seqlens.numel() - 1, nheads, headdim, dstate, device=x.device, dtype=torch.float32)
                     if cu_seqlens is not None else None)
    out, _ = _ssd_launch(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus,
                         dt_limit, L.PHASE_ALL, final_states=final_states, cu_seqlens=cu_seqlens,
                         varlen_states=varlen_states)
    if not return_varlen_states:
        return out if not return_final_states else (out, final_states)
    return (out, varlen_states) if not return_final_states else (out, final_states, varlen_states)


def mamba_chunk_scan_combined_noalloc(x, dt, A, B, C, chunk_size, out, D=None, z=None, dt_bias=None, initial_states=None,
                                      dt_softplus=False, dt_limit=(0.0, float("inf")), final_states=None):
    """SSD chunked scan for callers that cannot allocate device memory (mb200_ssd_chunk_scan_fwd_static).

    Some callers have no allocator to turn to at the point where the scan runs: a plugin inside an
    engine that planned all of its memory up front, a callback that runs on a stream, a process that
    has already handed every byte of its budget to a pool.  For them the library carries a fixed
    32 MiB buffer for the scan's intermediates.  This wrapper creates no device tensor either: ``out``
    (and ``final_states`` fp32 (batch, nheads, headdim, dstate) if wanted) come from the caller, and
    the parameter tensors must already be contiguous fp32.  Problems whose intermediates exceed the
    buffer raise AssertionError.  The first call on a device performs a one-time address look-up
    and should happen before any stream capture.  All calls share the buffer, so two calls that
    overlap on the GPU (different streams or threads) corrupt each other: keep them in order.
    """
    assert out.shape == x.shape and out.dtype == x.dtype and out.stride(-1) == 1
    if final_states is not None:
        assert final_states.dtype == torch.float32 and final_states.is_contiguous()
    _ssd_launch(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, None, dt_softplus, dt_limit, L.PHASE_ALL,
                out=out, final_states=final_states, builtin_scratch=True)
    return out


def ssd_local_states(x, dt, A, B, chunk_size, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf")), C=None):
    """First half of a sequence-split SSD scan on this device's contiguous chunk range.

    Returns ``(range_state, range_decay, scratch)``: the state at the end of the range given a zero
    incoming state (batch, nheads, headdim, dstate) fp32, the product of the range's chunk decays
    (batch, nheads) fp32, and an opaque scratch handle that ``ssd_finish`` must be handed back unchanged.
    The recurrence of this half does not read C; when C is given anyway, C.B^T -- which needs nothing from the
    exchange that follows -- is formed here too, so that it is off the critical path after the exchange.
    """
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[-1]
    range_state = torch.empty(batch, nheads, headdim, dstate, device=x.device, dtype=torch.float32)
    range_decay = torch.empty(batch, nheads, device=x.device, dtype=torch.float32)
    cb_early = C is not None and seqlen > 0
    _, scratch = _ssd_launch(x, dt, A, B, C if cb_early else B, chunk_size, None, None, dt_bias, None, None, dt_softplus, dt_limit,
                             L.PHASE_LOCAL | (L.PHASE_CB if cb_early else 0), final_states=range_state, range_decay=range_decay)
    return range_state, range_decay, (scratch, cb_early)


def ssd_finish(x, dt, A, B, C, chunk_size, scratch, D=None, z=None, dt_bias=None, incoming_state=None,
               dt_softplus=False, dt_limit=(0.0, float("inf")), return_final_states=False):
    """Second half of a sequence-split SSD scan: inter-chunk recurrence from ``incoming_state`` and
    the chunk outputs, reusing the scratch ``ssd_local_states`` filled."""
    batch, seqlen, nheads, headdim = x.shape
    dstate = B.shape[-1]
    final_states = (torch.empty(batch, nheads, headdim, dstate, device=x.device, dtype=torch.float32)
                    if return_final_states else None)
    scratch, cb_ready = scratch if isinstance(scratch, tuple) else (scratch, False)
    out, _ = _ssd_launch(x, dt, A, B, C, chunk_size, D, z, dt_bias, incoming_state, None, dt_softplus, dt_limit,
                         L.PHASE_OUTPUT | (L.PHASE_CB_READY if cb_ready else 0), final_states=final_states, scratch=scratch)
    return out if not return_final_states else (out, final_states)


def ssd_fold_state(incoming_state, range_decay, range_state):
    """``range_decay[..., None, None] * incoming_state + range_state`` on the device (fp32)."""
    L.require_cuda(range_decay, range_state, incoming_state)
    out = torch.empty_like(range_state)
    rows = range_decay.numel()
    row = range_state.numel() // max(rows, 1)
    # the converted tensors stay bound to names until the launch has been enqueued
    s_in = None if incoming_state is None else _fp32(incoming_state).contiguous()
    decay, local = _fp32(range_decay).contiguous(), _fp32(range_state).contiguous()
    L.check(L.lib().mb200_ssd_fold_state(L.ptr(s_in), L.ptr(decay), L.ptr(local), L.ptr(out), rows, row,
                                         range_state.device.index, L.stream_ptr(range_state.device)))
    return out


def ssd_fold_ranges(summaries, first, last, state_shape):
    """Folds the range summaries ``first..last`` (rows of ``summaries``: a flattened state followed by its
    (batch, nheads) decays, as the all-gather hand-off lays them out) into the state after range ``last``,
    in one launch: ``s = state[first]; s = decay[r] * s + state[r]`` for r = first+1 .. last."""
    L.require_cuda(summaries)
    assert summaries.dim() == 2 and summaries.dtype == torch.float32 and summaries.stride(1) == 1
    out = torch.empty(state_shape, device=summaries.device, dtype=torch.float32)
    rows = int(state_shape[0]) * int(state_shape[1])
    row = out.numel() // max(rows, 1)
    L.check(L.lib().mb200_ssd_fold_ranges(L.ptr(summaries), summaries.stride(0), int(first), int(last), L.ptr(out), rows, row,
                                          summaries.device.index, L.stream_ptr(summaries.device)))
    return out
