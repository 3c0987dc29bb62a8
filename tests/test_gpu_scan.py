"""GPU parity of the Mamba-1 selective scan (through the C ABI) against the golden vectors and the oracle."""
import math

import pytest
import torch

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close, golden_names, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fn():
    from mamba_b200 import selective_scan_fn
    return selective_scan_fn


def _cuda(d, k, dtype=None):
    t = d.get(k)
    if t is None:
        return None
    t = t.to(DEV)
    return t.to(dtype) if dtype is not None else t


@pytest.mark.parametrize("name", golden_names("m1_"))
def test_golden(name):
    d = load_golden(name)
    io = torch.bfloat16 if d["bf16"] else torch.float32
    const_bc = d["B"].dim() == 2
    out, last = _fn()(_cuda(d, "u", io), _cuda(d, "delta", io), _cuda(d, "A"),
                      _cuda(d, "B", None if const_bc else io), _cuda(d, "C", None if const_bc else io),
                      _cuda(d, "D"), _cuda(d, "z", io), _cuda(d, "delta_bias"), delta_softplus=True,
                      return_last_state=True)
    tol = TOL_BF16 if d["bf16"] else TOL_FP32
    assert out.dtype == io and last.dtype == torch.float32
    assert_close(out, d["out"], tol, name + " out")
    assert_close(last, d["last_state"], tol, name + " last_state")


def make_inputs(seed, batch, dim, L, N, groups, dtype, has_z=True, has_D=True, bench_style=False, const_b=False,
                const_c=False):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    if bench_style:
        A = -torch.exp(r(dim, N))
        delta = r(batch, dim, L)
        bias = -4 + 2 * torch.rand(dim, generator=g)
    else:
        A = -0.5 * torch.rand(dim, N, generator=g)
        delta = 0.5 * torch.rand(batch, dim, L, generator=g)
        bias = 0.5 * torch.rand(dim, generator=g)
    u = r(batch, dim, L).to(dtype)
    delta = delta.to(dtype)
    B = r(dim, N) if const_b else r(batch, groups, N, L).to(dtype)
    C = r(dim, N) if const_c else r(batch, groups, N, L).to(dtype)
    D = r(dim) if has_D else None
    z = r(batch, dim, L).to(dtype) if has_z else None
    return dict(u=u, delta=delta, A=A, B=B, C=C, D=D, z=z, delta_bias=bias)


def run_both(inp, tol, what):
    want, want_last = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(),
                                            inp["C"].float(), inp["D"], None if inp["z"] is None else inp["z"].float(),
                                            inp["delta_bias"], delta_softplus=True, return_last_state=True)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    got, got_last = _fn()(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"],
                          delta_softplus=True, return_last_state=True)
    assert_close(got, want, tol, what + " out")
    assert_close(got_last, want_last, tol, what + " last_state")
    return got, got_last


@pytest.mark.parametrize("L", [128, 256, 512, 1024, 2048, 4096, 372, 784, 1134, 1, 17])
@pytest.mark.parametrize("groups", [1, 2])
def test_reference_test_shapes_fp32(L, groups):
    """batch 2, dim 4, dstate 8 and the sequence lengths of the reference's own scan test."""
    run_both(make_inputs(100 + L, 2, 4, L, 8, groups, torch.float32), TOL_FP32, f"L{L} g{groups}")


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16)])
@pytest.mark.parametrize("L", [512, 1000])
def test_half_dtypes(dtype, tol, L):
    run_both(make_inputs(7, 2, 24, L, 16, 1, dtype, bench_style=True), tol, f"{dtype} L{L}")


@pytest.mark.parametrize("N", [1, 5, 16, 24, 64, 256])
def test_state_sizes(N):
    run_both(make_inputs(9 + N, 1, 20, 600, N, 2, torch.float32), TOL_FP32, f"N{N}")


@pytest.mark.parametrize("const_b,const_c", [(True, True), (True, False), (False, True)])
def test_constant_bc(const_b, const_c):
    run_both(make_inputs(21, 2, 12, 300, 8, 1, torch.float32, const_b=const_b, const_c=const_c), TOL_FP32, "const B/C")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16)])
@pytest.mark.parametrize("L,N,groups", [(700, 16, 1), (333, 8, 2), (64, 5, 1), (1, 16, 1), (1030, 12, 4)])
def test_many_channels(dtype, tol, L, N, groups):
    """Enough independent channels (batch x dim >= 2 x 32 x 148) for the one-lane-per-channel kernel:
    ragged lengths, dstate below 16, several groups, a channel count that is not a multiple of 32."""
    run_both(make_inputs(60 + L, 2, 4744, L, N, groups, dtype, bench_style=True), tol, f"many L{L} N{N} g{groups}")


def _row_padded(t, mult=8):
    """Same values in a buffer whose rows are padded to a multiple of `mult` elements (16-byte row strides with a
    ragged length, as a slice of a larger activation buffer has)."""
    L = t.shape[-1]
    Lp = (L + mult - 1) // mult * mult
    buf = t.new_zeros(*t.shape[:-1], Lp)
    buf[..., :L] = t
    return buf[..., :L]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16)])
@pytest.mark.parametrize("L,N,groups,gated", [(704, 16, 1, True), (328, 8, 2, True), (8, 16, 1, False), (1, 16, 1, True),
                                              (1032, 12, 1, True), (333, 8, 2, True), (23, 3, 2, False)])
def test_tma_fed_kernel(dtype, tol, L, N, groups, gated):
    """Whole groups of 32 channels with 16-byte aligned rows that end on a 16-byte boundary take the warp-specialised
    TMA-fed kernel: lengths that leave the last tile ragged (328, 1032, 8), dstate below 8 and 16, two groups, with and
    without gate; rows that end inside a 16-byte unit (333, 23, 1) must take another kernel and still be right."""
    from mamba_b200 import ops
    inp = make_inputs(90 + L, 2, 4800, L, N, groups, dtype, has_z=gated, has_D=gated, bench_style=True)
    want, want_last = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(),
                                            inp["C"].float(), inp["D"], None if inp["z"] is None else inp["z"].float(),
                                            inp["delta_bias"], delta_softplus=True, return_last_state=True)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    for k in ("u", "delta", "z", "B", "C"):
        if c[k] is not None:
            c[k] = _row_padded(c[k])
    out = _row_padded(torch.empty_like(c["u"]))      # aligned rows for every tensor, so the TMA path is eligible
    got, got_last = ops._selective_scan(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"],
                                        delta_softplus=True, return_last_state=True, out=out)
    assert ops.scan_status() == 0
    assert_close(got, want, tol, "tma-fed out")
    assert_close(got_last, want_last, tol, "tma-fed last_state")


@pytest.mark.parametrize("batch", [2, 5, 7])
def test_tma_fed_kernel_layouts_by_grid_size(batch):
    """300, 750 and 1050 CTAs: the six-warp, the four-warp and the three-warp layout of the TMA-fed kernel."""
    from mamba_b200 import ops
    inp = make_inputs(95, batch, 4800, 264, 16, 1, torch.bfloat16, bench_style=True)
    want, want_last = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(), inp["C"].float(),
                                            inp["D"], inp["z"].float(), inp["delta_bias"], delta_softplus=True, return_last_state=True)
    c = {k: v.to(DEV) for k, v in inp.items()}
    got, got_last = _fn()(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"], delta_softplus=True,
                          return_last_state=True)
    assert ops.scan_status() == 0
    assert_close(got, want, TOL_BF16, f"layout for {batch * 150} CTAs out")
    assert_close(got_last, want_last, TOL_BF16, f"layout for {batch * 150} CTAs last_state")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16)])
@pytest.mark.parametrize("batch,dim,L,N,gated", [(1, 5120, 2048, 16, True), (1, 1024, 2100, 16, True), (2, 512, 4096, 8, False), (1, 2048, 1030, 12, True)])
def test_few_channel_rows_cut_the_sequence_into_segments(dtype, tol, batch, dim, L, N, gated):
    """Few (batch, channel) rows -- one batch row of a divided batch -- make the library cut the sequence into segments
    that run side by side (summary launch, fold, full launch).  Output and last state equal the oracle's, which walks
    every row from end to end; ragged lengths leave the last segment short or empty."""
    from mamba_b200 import _lib, ops
    import ctypes
    inp = make_inputs(300 + L, batch, dim, L, N, 1, dtype, has_z=gated, has_D=gated, bench_style=True)
    a = _lib.ScanArgs()
    a.batch, a.dim, a.seqlen, a.dstate, a.ngroups = batch, dim, L, N, 1
    need = ctypes.c_size_t(0)
    _lib.check(_lib.lib().mb200_scan_scratch_bytes(ctypes.byref(a), ctypes.byref(need)))
    assert need.value > 0, "this shape is meant to take the segmented path"
    want, want_last = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(),
                                            inp["C"].float(), inp["D"], None if inp["z"] is None else inp["z"].float(),
                                            inp["delta_bias"], delta_softplus=True, return_last_state=True)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    for k in ("u", "delta", "z", "B", "C"):
        if c[k] is not None:
            c[k] = _row_padded(c[k])
    out = _row_padded(torch.empty_like(c["u"]))
    got, got_last = ops._selective_scan(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"],
                                        delta_softplus=True, return_last_state=True, out=out)
    assert ops.scan_status() == 0
    assert_close(got, want, tol, "segmented out")
    assert_close(got_last, want_last, tol, "segmented last_state")


def test_tma_fed_kernel_plain_delta():
    """The same kernel without softplus, bias, skip and gate (delta used as given)."""
    from mamba_b200 import ops
    inp = make_inputs(97, 2, 4800, 200, 16, 1, torch.bfloat16, has_z=False, has_D=False)
    want, want_last = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(), inp["C"].float(),
                                            None, None, None, delta_softplus=False, return_last_state=True)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    got, got_last = _fn()(c["u"], c["delta"], c["A"], c["B"], c["C"], return_last_state=True)
    assert ops.scan_status() == 0
    assert_close(got, want, TOL_BF16, "plain delta out")
    assert_close(got_last, want_last, TOL_BF16, "plain delta last_state")


def test_many_channels_unaligned_and_ungated():
    inp = make_inputs(71, 2, 4800, 77, 16, 1, torch.bfloat16, has_z=False, has_D=False)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    pad = lambda t: torch.cat([t.new_zeros(*t.shape[:-1], 1), t], dim=-1)[..., 1:]
    got, last = _fn()(pad(c["u"]), pad(c["delta"]), c["A"], pad(c["B"]), pad(c["C"]), None, None, c["delta_bias"],
                      delta_softplus=True, return_last_state=True)
    want, wl = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(), inp["C"].float(),
                                     None, None, inp["delta_bias"], delta_softplus=True, return_last_state=True)
    assert_close(got, want, TOL_BF16, "unaligned many out")
    assert_close(last, wl, TOL_BF16, "unaligned many last")


def test_optional_tensors_absent():
    inp = make_inputs(23, 2, 8, 200, 8, 1, torch.float32, has_z=False, has_D=False)
    inp["delta_bias"] = None
    want = oracle.selective_scan(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], delta_softplus=False)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    got = _fn()(c["u"], c["delta"], c["A"], c["B"], c["C"])
    assert_close(got, want, TOL_FP32, "no D/z/bias")


def test_bench_config0_full():
    """batch 2, d_inner 256, seqlen 512, d_state 16, fp32: the CPU-runnable benchmark configuration."""
    run_both(make_inputs(1000, 2, 256, 512, 16, 1, torch.float32, bench_style=True), TOL_FP32, "config 0")


def test_output_row_inside_a_wider_buffer_is_not_overrun():
    """A caller-provided `out` whose rows are the first 100 steps of 200-step buffers (16-bit, aligned strides): the bytes
    after a row's end stay untouched (a tile store would clip at a 16-byte unit, not at the element)."""
    from mamba_b200 import ops
    L = 100
    inp = make_inputs(91, 2, 2400, L, 16, 1, torch.bfloat16)
    wide = lambda t: torch.cat([t, torch.ones_like(t)], dim=2).to(DEV)[:, :, :L]
    out = torch.full((2, 2400, 2 * L), 7.0, dtype=torch.bfloat16, device=DEV)[:, :, :L]
    got = ops._selective_scan(wide(inp["u"]), wide(inp["delta"]), inp["A"].to(DEV), inp["B"].to(DEV), inp["C"].to(DEV),
                              inp["D"].to(DEV), wide(inp["z"]), inp["delta_bias"].to(DEV), True, out=out)
    want = oracle.selective_scan(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["z"], inp["delta_bias"],
                                 delta_softplus=True)
    assert_close(got, want, TOL_BF16, "row view")
    assert float((out._base[:, :, L:].float() - 7.0).abs().max()) == 0.0


def test_strided_views_like_the_mixer():
    """u and z as the two halves of one xz buffer and delta as a permuted view, as Mamba.forward passes
    them (mamba_ssm/modules/mamba_simple.py:141-200); out inherits delta's strides."""
    b, d, L, N = 2, 16, 256, 16
    g = torch.Generator().manual_seed(3)
    xz = torch.randn(b, 2 * d, L, generator=g).to(DEV)
    u, z = xz.chunk(2, dim=1)
    delta_flat = (0.5 * torch.rand(d, b * L, generator=g)).to(DEV)
    delta = delta_flat.view(d, b, L).permute(1, 0, 2)
    A = (-0.5 * torch.rand(d, N, generator=g)).to(DEV)
    B = torch.randn(b, N, L, generator=g).to(DEV)
    C = torch.randn(b, N, L, generator=g).to(DEV)
    assert not delta.is_contiguous() and not u.is_contiguous()
    got, last = _fn()(u, delta, A, B, C, None, z, None, delta_softplus=True, return_last_state=True)
    assert got.stride() == delta.stride()
    want, wl = oracle.selective_scan(u.cpu(), delta.cpu(), A.cpu(), B.cpu(), C.cpu(), None, z.cpu(), None,
                                     delta_softplus=True, return_last_state=True)
    assert_close(got, want, TOL_FP32, "strided out")
    assert_close(last, wl, TOL_FP32, "strided last")


def test_unaligned_rows_take_the_scalar_path():
    inp = make_inputs(31, 1, 6, 333, 8, 1, torch.bfloat16)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    # shift every row by one element so no 16-byte packet is aligned
    pad = lambda t: torch.cat([t.new_zeros(*t.shape[:-1], 1), t], dim=-1)[..., 1:]
    got = _fn()(pad(c["u"]), pad(c["delta"]), c["A"], pad(c["B"]), pad(c["C"]), c["D"], pad(c["z"]), c["delta_bias"],
                delta_softplus=True)
    want = oracle.selective_scan(inp["u"].float(), inp["delta"].float(), inp["A"], inp["B"].float(), inp["C"].float(),
                                 inp["D"], inp["z"].float(), inp["delta_bias"], delta_softplus=True)
    assert_close(got, want, TOL_BF16, "unaligned")


def test_softplus_threshold_and_large_decay():
    """delta straddling the softplus threshold of 20 and strongly negative dt*A."""
    inp = make_inputs(41, 1, 8, 64, 8, 1, torch.float32)
    inp["delta"] = torch.linspace(-30, 30, 64).repeat(1, 8, 1).contiguous()
    inp["delta_bias"] = None
    inp["A"] = -torch.linspace(0.01, 40.0, 8).repeat(8, 1).contiguous()
    run_both(inp, TOL_FP32, "softplus threshold")


def test_errors_mirror_the_reference():
    inp = make_inputs(51, 1, 4, 32, 8, 1, torch.float32)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    with pytest.raises(AssertionError, match="256"):
        A_big = torch.zeros(4, 257, device=DEV)
        _fn()(c["u"], c["delta"], A_big, torch.zeros(1, 1, 257, 32, device=DEV), torch.zeros(1, 1, 257, 32, device=DEV))
    with pytest.raises(NotImplementedError):
        _fn()(c["u"], c["delta"], torch.zeros(4, 8, dtype=torch.complex64, device=DEV), c["B"], c["C"])
    with pytest.raises(AssertionError):
        _fn()(c["u"], c["delta"].half(), c["A"], c["B"], c["C"])


@pytest.mark.parametrize("many", [False, True])
def test_extension_module_stand_in(many):
    """mamba_b200.compat.selective_scan_cuda.fwd returns what the reference's SelectiveScanFn.forward consumes:
    [out, x, out_z] with the ungated result in `out`, the gated one in `out_z`, and the last state at
    x[:, :, -1, 1::2] (mamba_ssm/ops/selective_scan_interface.py:58-68)."""
    from mamba_b200.compat import selective_scan_cuda
    inp = make_inputs(81, 2, 4800 if many else 12, 300, 16, 1, torch.float32)
    c = {k: v.to(DEV) for k, v in inp.items()}
    out, x, out_z = selective_scan_cuda.fwd(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"], True)
    want_z, want_last = oracle.selective_scan(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["z"],
                                              inp["delta_bias"], delta_softplus=True, return_last_state=True)
    want = oracle.selective_scan(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], None, inp["delta_bias"],
                                 delta_softplus=True)
    assert x.shape == (2, inp["u"].shape[1], 1, 32)
    assert_close(out, want, TOL_FP32, "ungated out")
    assert_close(out_z, want_z, TOL_FP32, "gated out_z")
    assert_close(x[:, :, -1, 1::2], want_last, TOL_FP32, "last state slice")
    out2, x2 = selective_scan_cuda.fwd(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], None, c["delta_bias"], True)
    assert_close(out2, want, TOL_FP32, "no gate")
    # the backward of the same module, called the way SelectiveScanFn.backward does (:83-86): x and out are handed
    # over (and not needed), dz comes back last
    g = torch.Generator().manual_seed(181)
    dout = torch.randn(inp["u"].shape, generator=g)
    res = selective_scan_cuda.bwd(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"], dout.to(DEV), x, out,
                                  None, True, False)
    want_g = oracle.selective_scan_bwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["z"], inp["delta_bias"],
                                       dout, True)
    for k, got, ref in zip(("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dz"), res,
                           (want_g[0], want_g[1], want_g[2], want_g[3], want_g[4], want_g[5], want_g[7], want_g[6])):
        assert_close(got, ref, TOL_FP32, "stand-in bwd " + k)


def test_extension_module_stand_in_prefix_tensor():
    """x of the stand-in holds what the extension's forward leaves for its backward (selective_scan_fwd_kernel.cuh:240-258):
    per 2048-step chunk the decay product from the first step and the state at the chunk's end."""
    from mamba_b200.compat import selective_scan_cuda
    inp = make_inputs(83, 1, 8, 5000, 8, 1, torch.float32, has_z=False)
    c = {k: (None if v is None else v.to(DEV)) for k, v in inp.items()}
    out, x = selective_scan_cuda.fwd(c["u"], c["delta"], c["A"], c["B"], c["C"], c["D"], None, c["delta_bias"], True)
    assert x.shape == (1, 8, 3, 16)
    dt = torch.nn.functional.softplus(inp["delta"].double() + inp["delta_bias"].double()[:, None])
    for ch, end in enumerate((2048, 4096, 5000)):
        want_state = oracle.selective_scan(inp["u"][..., :end], inp["delta"][..., :end], inp["A"], inp["B"][..., :end],
                                           inp["C"][..., :end], inp["D"], None, inp["delta_bias"], delta_softplus=True,
                                           return_last_state=True)[1]
        want_prod = torch.exp(dt[..., :end].sum(-1)[..., None] * inp["A"].double()[None]).float()
        assert_close(x[:, :, ch, 1::2], want_state, TOL_FP32, f"state at the end of chunk {ch}")
        assert_close(x[:, :, ch, 0::2], want_prod, TOL_FP32, f"decay product to the end of chunk {ch}")


def test_extension_module_stand_in_converts_parameter_dtypes():
    """D and delta_bias in bf16 and a non-contiguous A: the stand-in converts them, and every converted copy must
    still be alive (and described by its own strides) when the kernel runs."""
    from mamba_b200.compat import selective_scan_cuda
    inp = make_inputs(82, 2, 64, 200, 16, 1, torch.float32)
    c = {k: v.to(DEV) for k, v in inp.items()}
    D16, bias16 = c["D"].bfloat16(), c["delta_bias"].bfloat16()
    A_t = c["A"].t().contiguous().t()                  # (dim, dstate) with strides (1, dim)
    assert not A_t.is_contiguous()
    out, x, out_z = selective_scan_cuda.fwd(c["u"], c["delta"], A_t, c["B"], c["C"], D16, c["z"], bias16, True)
    want_z, want_last = oracle.selective_scan(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], D16.float().cpu(), inp["z"],
                                              bias16.float().cpu(), delta_softplus=True, return_last_state=True)
    assert_close(out_z, want_z, TOL_FP32, "gated out_z (converted D / bias)")
    assert_close(x[:, :, -1, 1::2], want_last, TOL_FP32, "last state slice (converted D / bias)")


def test_empty_batch():
    out = _fn()(torch.zeros(0, 4, 16, device=DEV), torch.zeros(0, 4, 16, device=DEV), torch.zeros(4, 8, device=DEV),
                torch.zeros(0, 1, 8, 16, device=DEV), torch.zeros(0, 1, 8, 16, device=DEV))
    assert out.shape == (0, 4, 16)


def bench_config1_inputs(batch, dim, L=2048, N=16, seed=1001):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    u, delta, z = r(batch, dim, L).bfloat16(), r(batch, dim, L).bfloat16(), r(batch, dim, L).bfloat16()
    A = -torch.exp(r(dim, N))
    B, C = r(batch, 1, N, L).bfloat16(), r(batch, 1, N, L).bfloat16()
    D = r(dim)
    dt = torch.exp(torch.rand(dim, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    bias = dt + torch.log(-torch.expm1(-dt))
    return dict(u=u, delta=delta, A=A, B=B, C=C, D=D, z=z, delta_bias=bias)


def test_bench_config1_slice_against_oracle():
    """bf16 2.8B-layer shape (seqlen 2048, d_state 16) on 96 channels of 2 batch rows."""
    run_both(bench_config1_inputs(2, 96), TOL_BF16, "config 1 slice")


def test_bench_config1_full_size_properties():
    """Full benchmark size (batch 8, d_inner 5120): a channel subset against the oracle, run-to-run
    bit identity (the forward has no atomics), and linearity in u."""
    inp = bench_config1_inputs(8, 5120)
    c = {k: v.to(DEV) for k, v in inp.items()}
    f = _fn()
    args = (c["delta"], c["A"], c["B"], c["C"], c["D"], c["z"], c["delta_bias"])
    out1, last1 = f(c["u"], *args, delta_softplus=True, return_last_state=True)
    out2, last2 = f(c["u"], *args, delta_softplus=True, return_last_state=True)
    assert torch.equal(out1, out2) and torch.equal(last1, last2)
    sel = torch.arange(0, 5120, 97)
    sub = {k: (v[:, sel] if k in ("u", "delta", "z") else (v[sel] if k in ("A", "D", "delta_bias") else v))
           for k, v in inp.items()}
    want, wl = oracle.selective_scan(sub["u"].float(), sub["delta"].float(), sub["A"], sub["B"].float(),
                                     sub["C"].float(), sub["D"], sub["z"].float(), sub["delta_bias"],
                                     delta_softplus=True, return_last_state=True)
    assert_close(out1[:, sel.to(DEV)], want, TOL_BF16, "full-size subset out")
    assert_close(last1[:, sel.to(DEV)], wl, TOL_BF16, "full-size subset last")
    # linearity in u (D and the gate are linear in u too): f(2u) == 2 f(u) exactly up to bf16 rounding
    out3 = f(2 * c["u"], *args, delta_softplus=True)
    assert_close(out3, 2 * out1.float(), TOL_BF16, "linearity")
