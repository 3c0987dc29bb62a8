"""GPU parity of the Mamba-1 selective-scan backward (through the C ABI) against gradients that autograd derived from
the reference's selective_scan_ref (golden vectors) and against the oracle's written-out adjoint."""
import pytest
import torch

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close, golden_names, load_golden
from test_gpu_scan import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"
GRADS = ("du", "ddelta", "dA", "dB", "dC", "dD", "dz", "ddelta_bias")
KEYS = ("u", "delta", "A", "B", "C", "D", "z", "delta_bias")


def _bwd():
    from mamba_b200 import selective_scan_bwd
    return selective_scan_bwd


def _dev(t):
    return None if t is None else t.to(DEV)


def _check(got, want, tol, what):
    for k, g, w in zip(GRADS, got, want):
        if w is None:
            assert g is None, f"{what} {k}: expected None"
            continue
        assert_close(g, w, tol, f"{what} {k}")


@pytest.mark.parametrize("name", golden_names("m1b_"))
def test_golden(name):
    d = load_golden(name)
    io = torch.bfloat16 if d["bf16"] else torch.float32
    ins = []
    for k in KEYS:
        t = d.get(k)
        if t is not None and (k in ("u", "delta", "z") or (k in ("B", "C") and t.dim() > 2)):
            t = t.to(io)
        ins.append(_dev(t))
    got = _bwd()(*ins, _dev(d["dout"].to(io)), bool(d["delta_softplus"]))
    assert got[0].dtype == io and got[2].dtype == torch.float32
    # bf16 fixtures carry two bf16 roundings of the reference (its gate and the cast of the gradients)
    _check(got, [d.get(k) for k in GRADS], TOL_BF16 if d["bf16"] else TOL_FP32, name)


CASES = [
    # seed, batch, dim, L, N, groups, dtype, kwargs
    (1, 2, 4, 128, 8, 1, torch.float32, {}),                                   # the reference test's shape
    (2, 2, 4, 1134, 8, 2, torch.float32, dict(has_z=False)),                   # odd length, two groups
    (3, 1, 96, 250, 16, 3, torch.float32, {}),                                 # whole warps of channels, ragged tail block
    (4, 2, 40, 77, 16, 1, torch.float32, dict(const_b=True)),
    (5, 2, 40, 64, 12, 1, torch.float32, dict(const_c=True, has_D=False)),
    (6, 1, 33, 50, 5, 1, torch.float32, dict(const_b=True, const_c=True)),
    (7, 1, 16, 90, 40, 2, torch.float32, {}),                                  # three passes over the states
    (8, 1, 8, 33, 256, 1, torch.float32, dict(has_z=False)),                   # the largest state size
    (9, 2, 128, 512, 16, 1, torch.bfloat16, {}),
    (10, 2, 64, 300, 16, 2, torch.float16, dict(has_z=False)),
    (11, 1, 64, 4096, 16, 1, torch.float32, dict(bench_style=True)),           # long sequence, steep decays
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"s{c[0]}_b{c[1]}d{c[2]}L{c[3]}n{c[4]}g{c[5]}_{str(c[6])[6:]}")
def test_against_oracle(case):
    seed, batch, dim, L, N, groups, dtype, kw = case
    x = make_inputs(seed, batch, dim, L, N, groups, dtype, **kw)
    g = torch.Generator().manual_seed(100 + seed)
    dout = torch.randn(batch, dim, L, generator=g).to(dtype)
    ins = [x[k] for k in KEYS]
    want = oracle.selective_scan_bwd(*ins, dout, True)
    got = _bwd()(*[_dev(t) for t in ins], _dev(dout), True)
    _check(got, want, TOL_FP32 if dtype == torch.float32 else TOL_BF16, f"case{seed}")


def test_no_softplus_no_bias_strided():
    """Identity dt, rows that are views with a batch stride larger than dim * seqlen, B/C as (batch, dstate, seqlen)."""
    x = make_inputs(21, 2, 48, 100, 16, 1, torch.float32, has_D=False)
    g = torch.Generator().manual_seed(121)
    dout = torch.randn(2, 48, 100, generator=g)
    B3, C3 = x["B"].squeeze(1), x["C"].squeeze(1)
    want = oracle.selective_scan_bwd(x["u"], x["delta"], x["A"], B3, C3, None, x["z"], None, dout, False)
    wide = lambda t: torch.cat([t, torch.zeros_like(t)], dim=2).to(DEV)[:, :, :100]       # last stride 1, row stride 200
    got = _bwd()(wide(x["u"]), wide(x["delta"]), _dev(x["A"]), _dev(B3), _dev(C3), None, wide(x["z"]), None, wide(dout), False)
    assert got[3].shape == B3.shape and got[4].shape == C3.shape
    _check(got, want, TOL_FP32, "strided")


@pytest.mark.parametrize("dim,groups", [(64, 2), (48, 1)])
def test_tiles_through_the_copy_engine_ragged(dim, groups):
    """16-bit rows with aligned strides arrive as tiles through the copy engine: a sequence that ends inside a block of eight
    steps, rows that are views of wider buffers (nothing may be written past a row's end: tile stores clip in 16-byte
    units, so these outputs must leave by plain stores), and a channel count that leaves a tile ragged."""
    L = 100
    x = make_inputs(71, 2, dim, L, 16, groups, torch.bfloat16)
    g = torch.Generator().manual_seed(171)
    dout = torch.randn(2, dim, L, generator=g).bfloat16()
    want = oracle.selective_scan_bwd(*[x[k] for k in KEYS], dout, True)
    wide = lambda t: torch.cat([t, torch.ones_like(t)], dim=2).to(DEV)[:, :, :L]        # row stride 200, last stride 1
    outs = tuple(torch.full((2, dim, 2 * L), 7.0, dtype=torch.bfloat16, device=DEV)[:, :, :L] for _ in range(3))
    got = _bwd()(wide(x["u"]), wide(x["delta"]), _dev(x["A"]), _dev(x["B"]), _dev(x["C"]), _dev(x["D"]), wide(x["z"]),
                 _dev(x["delta_bias"]), wide(dout), True, outputs=outs)
    _check(got, want, TOL_BF16, f"tiles d{dim}")
    for t in outs:      # nothing was written past the end of a row
        assert float((t._base[:, :, L:].float() - 7.0).abs().max()) == 0.0
    from mamba_b200 import ops
    assert ops.scan_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_autograd_matches_reference_style_check(dtype):
    """selective_scan_fn(...).backward(g) fills .grad of every input, as tests/ops/test_selective_scan.py:119-147 checks."""
    from mamba_b200 import selective_scan_fn
    x = make_inputs(31, 2, 64, 256, 16, 1, dtype)
    leaves = {k: (None if t is None else t.to(DEV).requires_grad_()) for k, t in x.items()}
    out, last = selective_scan_fn(leaves["u"], leaves["delta"], leaves["A"], leaves["B"], leaves["C"], leaves["D"], leaves["z"],
                                  leaves["delta_bias"], delta_softplus=True, return_last_state=True)
    assert out.requires_grad and not last.requires_grad
    g = torch.Generator().manual_seed(131)
    dout = torch.randn(out.shape, generator=g).to(dtype)
    out.backward(dout.to(DEV))
    want = oracle.selective_scan_bwd(*[x[k] for k in KEYS], dout, True)
    got = [leaves[k].grad for k in KEYS]
    for k, t in zip(KEYS, got):
        assert t.dtype == leaves[k].dtype and t.shape == leaves[k].shape
    _check(got, want, TOL_FP32 if dtype == torch.float32 else TOL_BF16, "autograd")


def test_batch_walked_in_slices_when_scratch_is_short():
    """Scratch for one or two of five batch rows: the library walks the batch in slices and the gradients are the same."""
    x = make_inputs(61, 5, 64, 130, 16, 2, torch.float32)
    g = torch.Generator().manual_seed(161)
    dout = torch.randn(5, 64, 130, generator=g)
    ins = [_dev(x[k]) for k in KEYS]
    full = _bwd()(*ins, _dev(dout), True)
    per_row = 4 * ((130 + 7) // 8) * 16 * 64
    for rows in (1, 2):
        got = _bwd()(*ins, _dev(dout), True, scratch_bytes=rows * per_row + 8)
        _check(got, [t.cpu() if t is not None else None for t in full], 2e-6, f"slices of {rows}")
    with pytest.raises(AssertionError):
        _bwd()(*ins, _dev(dout), True, scratch_bytes=per_row - 16)


def test_compat_bwd_list():
    """The stand-in for the compiled extension returns the extension's list (selective_scan.cpp:487-490)."""
    from mamba_b200.compat import selective_scan_cuda
    x = make_inputs(41, 1, 32, 64, 8, 1, torch.float32)
    g = torch.Generator().manual_seed(141)
    dout = torch.randn(1, 32, 64, generator=g)
    want = oracle.selective_scan_bwd(*[x[k] for k in KEYS], dout, True)
    res = selective_scan_cuda.bwd(*[_dev(x[k]) for k in KEYS], _dev(dout), None, None, None, True, False)
    assert len(res) == 8
    du, ddelta, dA, dB, dC, dD, dbias, dz = res
    _check((du, ddelta, dA, dB, dC, dD, dz, dbias), want, TOL_FP32, "compat")


def test_empty_and_bad_arguments():
    from mamba_b200 import selective_scan_bwd
    x = make_inputs(51, 1, 8, 16, 4, 1, torch.float32)
    ins = [_dev(x[k]) for k in KEYS]
    with pytest.raises(AssertionError):
        selective_scan_bwd(*ins, torch.zeros(1, 8, 15, device=DEV), True)
    empty = [t[:0] if t is not None and t.dim() >= 3 else t for t in ins]
    got = selective_scan_bwd(*empty, torch.zeros(0, 8, 16, device=DEV), True)
    assert got[0].shape == (0, 8, 16) and float(got[2].abs().max()) == 0.0
