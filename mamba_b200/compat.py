"""Stand-in for the reference's compiled extension module ``selective_scan_cuda``.

The reference's ``SelectiveScanFn.forward`` (mamba_ssm/ops/selective_scan_interface.py:36-68) calls
``selective_scan_cuda.fwd(u, delta, A, B, C, D, z, delta_bias, delta_softplus)`` and expects
``[out, x]`` or ``[out, x, out_z]`` back (csrc/selective_scan/selective_scan.cpp:226-336), where ``x``
is ``(batch, dim, n_chunks, 2 * dstate)`` holding, per 2048-step chunk and state, the product of the decays from the
first step to the chunk's end (even positions) and the state there (odd positions); the reference's forward only ever
reads ``x[:, :, -1, 1::2]``, its backward kernel reads all of it.  Installing this object under that name lets the
reference's own Python run unmodified on top of libmamba_b200 for inference:

    import sys, mamba_b200.compat
    sys.modules["selective_scan_cuda"] = mamba_b200.compat.selective_scan_cuda

``bwd`` serves the reference's ``SelectiveScanFn.backward`` (:70-100) from the library's backward kernel.
"""
import ctypes

import torch

from . import _lib as L

_CHUNK = 2048   # the reference extension's chunk length (selective_scan.cpp:307)


class _SelectiveScanCuda:
    @staticmethod
    def fwd(u, delta, A, B, C, D_, z_, delta_bias_, delta_softplus):
        L.require_cuda(u, delta, A, B, C, D_, z_, delta_bias_)
        if A.is_complex():
            raise NotImplementedError("mamba_b200: complex A is not supported")
        assert u.stride(-1) == 1 and delta.stride(-1) == 1, "u and delta must have a unit last stride"
        batch, dim, seqlen = u.shape
        dstate = A.shape[1]
        B_var, C_var = B.dim() >= 3, C.dim() >= 3
        assert (not B_var or B.dim() == 4) and (not C_var or C.dim() == 4), "variable B/C must be (batch, groups, dstate, seqlen)"
        ngroups = B.shape[1] if B_var else (C.shape[1] if C_var else 1)
        out = torch.empty_like(delta)
        out_z = torch.empty_like(z_) if z_ is not None else None
        n_chunks = (seqlen + _CHUNK - 1) // _CHUNK
        x = torch.zeros(batch, dim, n_chunks, 2 * dstate, device=u.device, dtype=torch.float32)
        last = torch.empty(batch, dim, dstate, device=u.device, dtype=torch.float32)
        # converted copies are bound to names so that they outlive the launch, and their own strides are passed
        A = A.float()
        D32 = None if D_ is None else D_.float().contiguous()
        bias32 = None if delta_bias_ is None else delta_bias_.float().contiguous()
        if not B_var:
            B = B.float()
        if not C_var:
            C = C.float()
        a = L.ScanArgs()
        a.u, a.delta, a.A, a.B, a.C = L.ptr(u), L.ptr(delta), L.ptr(A), L.ptr(B), L.ptr(C)
        a.D = L.ptr(D32)
        a.delta_bias = L.ptr(bias32)
        a.z = L.ptr(z_)
        # with a gate the extension returns the ungated result as `out` and the gated one as `out_z`
        a.out, a.out_pregate = (L.ptr(out_z), L.ptr(out)) if z_ is not None else (L.ptr(out), None)
        a.last_state = L.ptr(last)
        a.batch, a.dim, a.seqlen, a.dstate, a.ngroups = batch, dim, seqlen, dstate, ngroups
        a.io_dtype = L.dtype_code(u.dtype)
        a.B_variable, a.C_variable, a.delta_softplus = int(B_var), int(C_var), int(bool(delta_softplus))
        a.device = u.device.index
        L.set_strides(a.u_stride, u, 2)
        L.set_strides(a.delta_stride, delta, 2)
        L.set_strides(a.A_stride, A, 2)
        L.set_strides(a.B_stride, B, 3 if B_var else 2)
        L.set_strides(a.C_stride, C, 3 if C_var else 2)
        if z_ is not None:
            L.set_strides(a.z_stride, z_, 2)
            L.set_strides(a.out_stride, out_z, 2)
            L.set_strides(a.pregate_stride, out, 2)
        else:
            L.set_strides(a.out_stride, out, 2)
        L.check(L.lib().mb200_selective_scan_fwd(ctypes.byref(a), L.stream_ptr(u.device)))
        # x[b, d, c] = (product of exp(dt A) from the first step to the end of chunk c, state there) per state, interleaved:
        # the running prefix of selective_scan_fwd_kernel.cuh:240-258, which the extension's own backward reads.  The
        # library's kernels do not need it, so it is assembled here, off the hot path: the decay products from a running
        # sum of dt, the states before the last chunk end from forward calls over the prefixes (none up to 2048 steps).
        x[:, :, -1, 1::2] = last
        dt = delta.float() if bias32 is None else delta.float() + bias32[:, None]
        if delta_softplus:
            dt = torch.nn.functional.softplus(dt)
        ends = [min((c + 1) * _CHUNK, seqlen) for c in range(n_chunks)]
        sums = dt.cumsum(-1)[..., [e - 1 for e in ends]] if seqlen > 0 else dt.new_zeros(batch, dim, n_chunks)
        x[..., 0::2] = torch.exp(sums[..., None] * A[None, :, None, :])
        from . import ops
        for c, e in enumerate(ends[:-1]):
            cut = lambda t, var: t[..., :e] if var else t
            x[:, :, c, 1::2] = ops._selective_scan(u[..., :e], delta[..., :e], A, cut(B, B_var), cut(C, C_var), D32, None, bias32,
                                                   delta_softplus, return_last_state=True)[1]
        return [out, x] if z_ is None else [out, x, out_z]

    @staticmethod
    def bwd(u, delta, A, B, C, D_, z_, delta_bias_, dout, x_, out_, dz_, delta_softplus, recompute_out_z):
        """``selective_scan_cuda.bwd`` (csrc/selective_scan/selective_scan.cpp:338-492): returns
        ``[du, ddelta, dA, dB, dC, dD, ddelta_bias]`` followed by ``dz`` when z is given and ``out_z`` when asked for.
        ``x_`` and ``out_`` are accepted and ignored: the library's backward recomputes the scan from the inputs."""
        from . import ops
        assert (B.dim() != 3) and (C.dim() != 3), "variable B/C must be (batch, groups, dstate, seqlen)"
        du, ddelta, dA, dB, dC, dD, dz, dbias = ops.selective_scan_bwd(u, delta, A, B, C, D_, z_, delta_bias_, dout,
                                                                       delta_softplus)
        result = [du, ddelta, dA, dB, dC, dD, dbias]
        if z_ is not None:
            if dz_ is not None:        # a preallocated dz is filled in place, as the extension does
                dz_.copy_(dz)
                dz = dz_
            result.append(dz)
            if recompute_out_z:
                result.append(ops._selective_scan(u, delta, A, B, C, D_, z_, delta_bias_, delta_softplus))
        return result


selective_scan_cuda = _SelectiveScanCuda()
