"""The steps either side of the scan inside the Mamba mixers, served by libmamba_b200.so.

Signatures and argument meaning follow what the reference calls at these places:

* ``causal_conv1d_fn`` / ``causal_conv1d_update``   the causal-conv1d package (not vendored by the reference) as used
  at mamba_ssm/modules/mamba2.py:236-242, 298-304 and mamba_ssm/modules/mamba_simple.py:172-177, 223-229; the
  reference's own CPU form is the depthwise ``nn.Conv1d`` at mamba2.py:232-234 and the roll / sum at :309-315
* ``rmsnorm_fn``                                     mamba_ssm/ops/triton/layernorm_gated.py (``RMSNorm.forward`` :415-437)
* ``mamba_split_conv1d_scan_combined``               mamba_ssm/ops/triton/ssd_combined.py:983-1003 (forward :820-899)

Forward only.  PyTorch supplies device memory, the current stream and the output projection (a plain library GEMM).
"""
import ctypes

import torch
import torch.nn.functional as F

from . import _lib as L
from . import ops


def _activation_code(activation):
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    return 0 if activation is None else 1


def causal_conv1d_fn(x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False,
                     final_states_out=None, activation=None):
    """Causal depthwise conv1d: x (batch, dim, seqlen) in either memory layout, weight (dim, width), bias (dim).

    ``out[b, c, t] = act(bias[c] + sum_k weight[c, k] * x[b, c, t - (width - 1) + k])`` with zeros (or
    ``initial_states`` (batch, dim, width-1)) before the start; ``seq_idx`` (batch, seqlen) keeps packed sequences
    apart.  Returns ``out`` laid out like x, or ``(out, final_states)`` with the last width-1 inputs.
    """
    L.require_cuda(x, weight, bias, seq_idx, initial_states, final_states_out)
    act = _activation_code(activation)
    assert x.dim() == 3, "x must be (batch, dim, seqlen)"
    batch, dim, seqlen = x.shape
    assert weight.dim() == 2 and weight.shape[0] == dim, "weight must be (dim, width)"
    width = weight.shape[1]
    if x.stride(2) != 1 and x.stride(1) != 1:
        x = x.contiguous()
    weight = weight.contiguous()
    bias = None if bias is None else bias.contiguous()
    assert bias is None or (bias.shape == (dim,) and bias.dtype == weight.dtype), "bias must be (dim,) with the dtype of weight"
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
        seq_idx = seq_idx.to(torch.int32).contiguous()
    if initial_states is not None:
        assert initial_states.shape == (batch, dim, width - 1) and initial_states.dtype == x.dtype
    out = torch.empty_like(x)       # keeps the layout of x (channels-last input gives channels-last output)
    final = None
    if return_final_states:
        final = final_states_out if final_states_out is not None else torch.empty(batch, width - 1, dim, device=x.device, dtype=x.dtype).transpose(1, 2)
        assert final.shape == (batch, dim, width - 1) and final.dtype == x.dtype
    a = L.Conv1dArgs()
    a.x, a.weight, a.bias, a.seq_idx = L.ptr(x), L.ptr(weight), L.ptr(bias), L.ptr(seq_idx)
    a.initial_states, a.final_states, a.out = L.ptr(initial_states), L.ptr(final), L.ptr(out)
    a.batch, a.dim, a.seqlen, a.width = batch, dim, seqlen, width
    a.io_dtype, a.w_dtype, a.activation, a.device = L.dtype_code(x.dtype), L.dtype_code(weight.dtype), act, x.device.index
    L.set_strides(a.x_stride, x, 3)
    L.set_strides(a.out_stride, out, 3)
    if initial_states is not None:
        L.set_strides(a.init_stride, initial_states, 3)
    if final is not None:
        L.set_strides(a.final_stride, final, 3)
    L.check(L.lib().mb200_causal_conv1d_fwd(ctypes.byref(a), L.stream_ptr(x.device)))
    return out if not return_final_states else (out, final)


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, cache_seqlens=None):
    """Single-token causal conv1d: x (batch, dim); conv_state (batch, dim, state_len >= width-1) is shifted left by
    one and x appended, in place.  Returns out (batch, dim)."""
    L.require_cuda(x, conv_state, weight, bias)
    if cache_seqlens is not None:
        raise NotImplementedError("mamba_b200: the circular-buffer form (cache_seqlens) is not supported")
    act = _activation_code(activation)
    squeeze = x.dim() == 3
    if squeeze:
        assert x.shape[2] == 1, "one token per call"
        x = x[:, :, 0]
    batch, dim = x.shape
    width = weight.shape[1]
    assert weight.shape == (dim, width) and conv_state.shape[:2] == (batch, dim) and conv_state.dtype == x.dtype
    weight = weight.contiguous()
    bias = None if bias is None else bias.contiguous()
    assert bias is None or (bias.shape == (dim,) and bias.dtype == weight.dtype)
    out = torch.empty_like(x)
    a = L.Conv1dUpdateArgs()
    a.x, a.weight, a.bias, a.conv_state, a.out = L.ptr(x), L.ptr(weight), L.ptr(bias), L.ptr(conv_state), L.ptr(out)
    a.batch, a.dim, a.width, a.state_len = batch, dim, width, conv_state.shape[2]
    a.io_dtype, a.w_dtype, a.activation, a.device = L.dtype_code(x.dtype), L.dtype_code(weight.dtype), act, x.device.index
    L.set_strides(a.x_stride, x, 2)
    L.set_strides(a.out_stride, out, 2)
    L.set_strides(a.state_stride, conv_state, 3)
    L.check(L.lib().mb200_causal_conv1d_update(ctypes.byref(a), L.stream_ptr(x.device)))
    return out.unsqueeze(-1) if squeeze else out


def rmsnorm_fn(x, weight, bias=None, z=None, eps=1e-6, group_size=None, norm_before_gate=True, out=None):
    """Gated RMSNorm over the last dimension (per group of ``group_size`` columns when given):
    ``norm(x) * silu(z)`` if ``norm_before_gate`` else ``norm(x * silu(z))``.  Returns a tensor shaped like x."""
    L.require_cuda(x, weight, bias, z, out)
    shape = x.shape
    ncols = shape[-1]
    x2 = x.reshape(-1, ncols)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    z2 = None
    if z is not None:
        assert z.shape == shape and z.dtype == x.dtype, "z must match x"
        z2 = z.reshape(-1, ncols)
        if z2.stride(-1) != 1:
            z2 = z2.contiguous()
    weight = weight.contiguous()
    bias = None if bias is None else bias.contiguous()
    assert weight.shape == (ncols,) and (bias is None or (bias.shape == (ncols,) and bias.dtype == weight.dtype))
    group = ncols if group_size is None else int(group_size)
    assert ncols % group == 0, "the row length must be a multiple of group_size"
    if out is None:
        out2 = torch.empty(x2.shape, device=x.device, dtype=x.dtype)
    else:
        assert out.shape == shape and out.dtype == x.dtype and out.stride(-1) == 1
        out2 = out.view(-1, ncols) if out.dim() != 2 else out
    a = L.RmsNormArgs()
    a.x, a.z, a.weight, a.bias, a.out = L.ptr(x2), L.ptr(z2), L.ptr(weight), L.ptr(bias), L.ptr(out2)
    a.nrows, a.ncols, a.group_size = x2.shape[0], ncols, group
    a.io_dtype, a.w_dtype, a.norm_before_gate = L.dtype_code(x.dtype), L.dtype_code(weight.dtype), int(bool(norm_before_gate))
    a.eps, a.device = float(eps), x.device.index
    a.x_stride, a.out_stride = x2.stride(0), out2.stride(0)
    a.z_stride = 0 if z2 is None else z2.stride(0)
    L.check(L.lib().mb200_rmsnorm_gated_fwd(ctypes.byref(a), L.stream_ptr(x.device)))
    return out if out is not None else out2.view(shape)


def mamba_split_conv1d_scan_combined(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, initial_states=None,
                                     seq_idx=None, dt_limit=(0.0, float("inf")), return_final_states=False, activation="silu",
                                     rmsnorm_weight=None, rmsnorm_eps=1e-6, outproj_weight=None, outproj_bias=None, headdim=None,
                                     ngroups=1, norm_before_gate=True, state_dtype=None):
    """The Mamba-2 block after its input projection, forward only: split -> causal conv1d (+ activation) -> SSD chunked
    scan -> gated RMSNorm (or the plain gate) -> output projection.

    zxbcdt: (batch, seqlen, 2 * d_nonssm + 2 * dim + 2 * ngroups * dstate + nheads), dim = nheads * headdim;
    conv1d_weight: (dim + 2 * ngroups * dstate, width); D: (nheads,) with ``headdim`` given, or (nheads, headdim).
    Returns out (batch, seqlen, out_dim or d_nonssm + dim) and, if asked, final_states (batch, nheads, headdim, dstate).
    """
    assert activation in [None, "silu", "swish"]
    if D.dim() == 1:
        assert headdim is not None
        nheads, = D.shape
    else:
        nheads, headdim = D.shape
    batch, seqlen, _ = zxbcdt.shape
    dim = nheads * headdim
    assert nheads % ngroups == 0
    dstate = (conv1d_weight.shape[0] - dim) // ngroups // 2
    d_nonssm = (zxbcdt.shape[-1] - 2 * dim - 2 * ngroups * dstate - nheads) // 2
    assert d_nonssm >= 0
    assert zxbcdt.shape == (batch, seqlen, 2 * d_nonssm + 2 * dim + 2 * ngroups * dstate + nheads)
    assert dt_bias.shape == (nheads,)
    assert A.shape == (nheads,)
    zx0, z, xBC, dt = torch.split(zxbcdt, [2 * d_nonssm, dim, dim + ngroups * dstate * 2, nheads], dim=-1)
    # the conv reads its slice of zxbcdt in place (channels contiguous) and writes a dense (batch, seqlen, channels) tensor
    xBC_conv = causal_conv1d_fn(xBC.transpose(1, 2), conv1d_weight, conv1d_bias, seq_idx=seq_idx, activation=activation).transpose(1, 2)
    x, B, C = torch.split(xBC_conv, [dim, ngroups * dstate, ngroups * dstate], dim=-1)
    x = x.unflatten(-1, (nheads, headdim))
    B = B.unflatten(-1, (ngroups, dstate))
    C = C.unflatten(-1, (ngroups, dstate))
    z4 = z.unflatten(-1, (nheads, headdim))
    gate_in_scan = rmsnorm_weight is None
    res = ops.mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=D, z=z4 if gate_in_scan else None, dt_bias=dt_bias,
                                        initial_states=initial_states, seq_idx=seq_idx, dt_softplus=True, dt_limit=dt_limit,
                                        return_final_states=return_final_states, state_dtype=state_dtype)
    y, final_states = res if return_final_states else (res, None)
    y = y.flatten(-2)
    if d_nonssm > 0:
        out = torch.empty(batch, seqlen, d_nonssm + dim, device=y.device, dtype=y.dtype)
        x0, z0 = zx0.chunk(2, dim=-1)
        out[..., :d_nonssm] = F.silu(z0) * x0
        if gate_in_scan:
            out[..., d_nonssm:] = y
        else:
            rmsnorm_fn(y, rmsnorm_weight, None, z=z, eps=rmsnorm_eps, group_size=dim // ngroups, norm_before_gate=norm_before_gate,
                       out=out[..., d_nonssm:])
    elif gate_in_scan:
        out = y
    else:
        out = rmsnorm_fn(y, rmsnorm_weight, None, z=z, eps=rmsnorm_eps, group_size=dim // ngroups, norm_before_gate=norm_before_gate)
    if outproj_weight is not None:
        out = F.linear(out, outproj_weight, outproj_bias)
    else:
        assert outproj_bias is None
    return out if not return_final_states else (out, final_states)
