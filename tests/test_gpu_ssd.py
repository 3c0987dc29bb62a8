"""GPU parity of the Mamba-2 SSD chunked scan (through the C ABI)."""
import math

import pytest
import torch

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close, golden_names, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fn():
    from mamba_b200 import mamba_chunk_scan_combined
    return mamba_chunk_scan_combined


def _status():
    from mamba_b200 import ops
    return ops.ssd_status()


def _c(t, dtype=None):
    if t is None:
        return None
    t = t.to(DEV)
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("name", golden_names("ssd_"))
def test_golden(name):
    d = load_golden(name)
    io = torch.bfloat16 if d["bf16"] else torch.float32
    tol = TOL_BF16 if d["bf16"] else TOL_FP32
    out, fin = _fn()(_c(d["x"], io), _c(d["dt"], io), _c(d["A"]), _c(d["B"], io), _c(d["C"], io), int(d["chunk_size"]),
                     D=_c(d.get("D")), z=_c(d.get("z"), io), dt_bias=_c(d["dt_bias"]),
                     initial_states=_c(d.get("initial_states")), dt_softplus=True, return_final_states=True)
    assert out.dtype == io and fin.dtype == torch.float32
    assert _status() == 0
    assert_close(out, d["out"], tol, name + " out")
    assert_close(fin, d["final_states"], tol, name + " final_states")


def make(seed, b, L, H, P, G, N, dtype, has_z=True, D_hdim=False, init=False):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    dtv = torch.exp(torch.rand(H, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    return dict(x=r(b, L, H, P).to(dtype), dt=r(b, L, H).to(dtype), A=-(1 + 15 * torch.rand(H, generator=g)),
                B=r(b, L, G, N).to(dtype), C=r(b, L, G, N).to(dtype), D=r(H, P) if D_hdim else r(H),
                z=r(b, L, H, P).to(dtype) if has_z else None, dt_bias=dtv + torch.log(-torch.expm1(-dtv)),
                initial_states=0.5 * r(b, H, P, N) if init else None)


def run_both(inp, Q, tol, what, **kw):
    f = lambda t: None if t is None else t.float()
    want, wfin = oracle.ssd_chunk_scan(f(inp["x"]), f(inp["dt"]), inp["A"], f(inp["B"]), f(inp["C"]), Q, inp["D"], f(inp["z"]),
                                       inp["dt_bias"], inp["initial_states"], dt_softplus=True, **kw)
    c = {k: _c(v) for k, v in inp.items()}
    got, fin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                     initial_states=c["initial_states"], dt_softplus=True, return_final_states=True, **kw)
    assert _status() == 0, f"a kernel gave up a bounded wait (code {_status()})"
    assert_close(got, want, tol, what + " out")
    assert_close(fin, wfin, tol, what + " final_states")
    return got, fin


@pytest.mark.parametrize("P", [64, 128])
def test_determinism_test_shapes(P):
    """batch 2, seqlen 2048, 8 heads, dstate 64, chunk 256 (tests/test_determinism.py in the reference)."""
    run_both(make(1, 2, 2048, 8, P, 1, 64, torch.float32), 256, TOL_FP32, f"P{P}")


def test_ssd_minimal_shape():
    """batch 1, seqlen 2048, chunk 64, 32 heads x 64, dstate 64 (modules/ssd_minimal.py in the reference)."""
    run_both(make(2, 1, 2048, 32, 64, 1, 64, torch.float32, has_z=False), 64, TOL_FP32, "minimal")


@pytest.mark.parametrize("L,Q", [(1, 64), (63, 64), (65, 64), (200, 64), (300, 128), (257, 256)])
def test_ragged_lengths(L, Q):
    run_both(make(3 + L, 2, L, 4, 16, 2, 16, torch.float32), Q, TOL_FP32, f"L{L} Q{Q}")


@pytest.mark.parametrize("P,N,G,H", [(8, 8, 1, 3), (40, 24, 2, 6), (96, 80, 3, 3), (64, 128, 4, 8)])
def test_odd_head_and_state_sizes(P, N, G, H):
    run_both(make(9, 1, 192, H, P, G, N, torch.float32, D_hdim=True, init=True), 64, TOL_FP32, f"P{P} N{N}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_dtypes(dtype):
    run_both(make(10, 2, 512, 4, 64, 1, 128, dtype), 256, TOL_BF16, str(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L,G,H,init,D_hdim,has_z", [(256, 1, 2, False, False, True), (1024, 2, 4, True, True, False),
                                                       (700, 1, 3, True, False, True), (100, 1, 1, False, False, True)])
def test_tensor_core_shapes(dtype, L, G, H, init, D_hdim, has_z):
    """headdim 64, dstate 128, chunk 256, 16-bit inputs: the shapes the tcgen05 kernels serve, with ragged
    tails, several groups, initial states and both D layouts."""
    run_both(make(40 + L, 2, L, H, 64, G, 128, dtype, has_z=has_z, D_hdim=D_hdim, init=init), 256, TOL_BF16,
             f"tc L{L} G{G} H{H}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,L,G,H,init,has_z", [(2, 1024, 1, 40, False, True), (1, 700, 8, 80, True, False),
                                                 (3, 256, 2, 26, True, True), (2, 100, 1, 37, False, True)])
def test_fused_state_stream_shapes(dtype, b, L, G, H, init, has_z):
    """Enough (batch, head) pairs (>= 74) for the kernel that fuses the chunk states with the inter-chunk
    recurrence: several chunks, a ragged tail, a single short chunk, groups, initial states."""
    run_both(make(140 + L, b, L, H, 64, G, 128, dtype, has_z=has_z, init=init), 256, TOL_BF16,
             f"stream b{b} L{L} G{G} H{H}")


def test_fused_state_stream_options():
    """The fused path with a per-(head, column) D, a dt clamp and no softplus."""
    inp = make(171, 2, 768, 40, 64, 2, 128, torch.bfloat16, has_z=True, D_hdim=True, init=True)
    inp["dt"] = (inp["dt"].float().abs() * 0.1).to(torch.bfloat16)
    inp["dt_bias"] = None
    f = lambda t: None if t is None else t.float()
    want, wfin = oracle.ssd_chunk_scan(f(inp["x"]), f(inp["dt"]), inp["A"], f(inp["B"]), f(inp["C"]), 256, inp["D"], f(inp["z"]), None,
                                       inp["initial_states"], dt_softplus=False, dt_limit=(0.01, 0.1))
    c = {k: _c(v) for k, v in inp.items()}
    got, fin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, D=c["D"], z=c["z"], initial_states=c["initial_states"],
                     dt_limit=(0.01, 0.1), return_final_states=True)
    assert _status() == 0
    assert_close(got, want, TOL_BF16, "fused options out")
    assert_close(fin, wfin, TOL_BF16, "fused options final")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tensor_core_steep_decay(dtype):
    """dt*|A| of several units per step: the decay over a 32-step range exceeds what the factorised mask may
    span, so the element-by-element mask path of the tensor-core chunk scan runs (and rows far apart decay to 0)."""
    inp = make(181, 2, 512, 4, 64, 1, 128, dtype, has_z=True)
    g = torch.Generator().manual_seed(182)
    inp["dt"] = (0.3 + 0.7 * torch.rand(2, 512, 4, generator=g)).to(dtype)
    inp["A"] = -(8 + 8 * torch.rand(4, generator=g))
    inp["dt_bias"] = None
    f = lambda t: None if t is None else t.float()
    want, wfin = oracle.ssd_chunk_scan(f(inp["x"]), f(inp["dt"]), inp["A"], f(inp["B"]), f(inp["C"]), 256, inp["D"], f(inp["z"]), None,
                                       None, dt_softplus=False)
    c = {k: _c(v) for k, v in inp.items()}
    got, fin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, D=c["D"], z=c["z"], return_final_states=True)
    assert _status() == 0
    assert_close(got, want, TOL_BF16, "steep out")
    assert_close(fin, wfin, TOL_BF16, "steep final")


def test_dt_limit_and_no_softplus():
    inp = make(11, 1, 128, 2, 16, 1, 16, torch.float32)
    inp["dt"] = inp["dt"].abs() * 0.1
    inp["dt_bias"] = None
    f = lambda t: None if t is None else t.float()
    want, wfin = oracle.ssd_chunk_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], 64, inp["D"], inp["z"], None, None,
                                       dt_softplus=False, dt_limit=(0.01, 0.1))
    c = {k: _c(v) for k, v in inp.items()}
    got, fin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 64, D=c["D"], z=c["z"], dt_limit=(0.01, 0.1),
                     return_final_states=True)
    assert_close(got, want, TOL_FP32, "dt_limit out")
    assert_close(fin, wfin, TOL_FP32, "dt_limit final")


def test_strided_views_like_the_mixer():
    """x, B, C as slices of one xBC buffer and z, dt as slices of zxbcdt (mamba_ssm/modules/mamba2.py:210-260)."""
    b, L, H, P, G, N = 2, 256, 4, 32, 1, 64
    g = torch.Generator().manual_seed(12)
    xBC = torch.randn(b, L, H * P + 2 * G * N, generator=g).to(DEV)
    zdt = torch.randn(b, L, H * P + H, generator=g).to(DEV)
    x = xBC[..., :H * P].view(b, L, H, P)
    B = xBC[..., H * P:H * P + G * N].view(b, L, G, N)
    C = xBC[..., H * P + G * N:].view(b, L, G, N)
    z = zdt[..., :H * P].view(b, L, H, P)
    dt = zdt[..., H * P:]
    A = -(1 + torch.rand(H, generator=g)).to(DEV)
    D = torch.randn(H, generator=g).to(DEV)
    bias = (torch.rand(H, generator=g) - 4).to(DEV)
    assert not x.is_contiguous() and not dt.is_contiguous()
    got, fin = _fn()(x, dt, A, B, C, 128, D=D, z=z, dt_bias=bias, dt_softplus=True, return_final_states=True)
    want, wfin = oracle.ssd_chunk_scan(x.cpu(), dt.cpu(), A.cpu(), B.cpu(), C.cpu(), 128, D.cpu(), z.cpu(), bias.cpu(), None,
                                       dt_softplus=True)
    assert_close(got, want, TOL_FP32, "strided out")
    assert_close(fin, wfin, TOL_FP32, "strided final")


def test_prefill_state_continues_in_decode():
    """final_states of a prefill over L tokens, advanced by one decode step, equals the prefill over
    L+1 tokens: last output row and final state."""
    from mamba_b200 import selective_state_update
    b, L, H, P, G, N, Q = 2, 130, 4, 16, 2, 32, 64
    inp = make(13, b, L + 1, H, P, G, N, torch.float32)
    c = {k: _c(v) for k, v in inp.items()}
    full, fin_full = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                           dt_softplus=True, return_final_states=True)
    part, fin = _fn()(c["x"][:, :L], c["dt"][:, :L], c["A"], c["B"][:, :L], c["C"][:, :L], Q, D=c["D"], z=c["z"][:, :L],
                      dt_bias=c["dt_bias"], dt_softplus=True, return_final_states=True)
    assert_close(part, full[:, :L], TOL_FP32, "prefix")
    o = selective_state_update(fin, c["x"][:, L], c["dt"][:, L, :, None].expand(b, H, P), c["A"][:, None, None].expand(H, P, N),
                               c["B"][:, L], c["C"][:, L], c["D"][:, None].expand(H, P), c["z"][:, L],
                               c["dt_bias"][:, None].expand(H, P), dt_softplus=True)
    assert_close(o, full[:, L], TOL_FP32, "decode token")
    assert_close(fin, fin_full, TOL_FP32, "decode state")


@pytest.mark.parametrize("shape,dtype,tol", [((1, 512, 4, 32, 2, 64, 64), torch.float32, TOL_FP32),
                                             ((2, 1024, 40, 64, 2, 128, 256), torch.bfloat16, TOL_BF16),
                                             ((1, 1300, 80, 64, 8, 128, 256), torch.float16, TOL_BF16)])
@pytest.mark.parametrize("cb_early", [False, True])
def test_sequence_split_in_two_ranges(shape, dtype, tol, cb_early):
    """The two-phase entry used when a sequence is split across devices: both ranges run LOCAL, the
    first range's summary is folded and handed to the second, then both run OUTPUT.  Equal to one call.
    The 16-bit shapes have enough (batch, head) pairs for the fused state-stream path, where the OUTPUT half
    adds the incoming state's share to the entering states the LOCAL half stored.  With `cb_early` the LOCAL
    half is given C and forms C.B^T ahead of the exchange."""
    from mamba_b200 import ssd_finish, ssd_fold_state, ssd_local_states
    b, L, H, P, G, N, Q = shape
    inp = make(14, b, L, H, P, G, N, dtype, has_z=False)
    c = {k: _c(v) for k, v in inp.items()}
    TOL_FP32_ = tol
    whole, wfin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], dt_bias=c["dt_bias"], dt_softplus=True,
                        return_final_states=True)
    half = (L // 2) // Q * Q
    sl = [slice(0, half), slice(half, L)]
    loc = [ssd_local_states(c["x"][:, s], c["dt"][:, s], c["A"], c["B"][:, s], Q, dt_bias=c["dt_bias"], dt_softplus=True,
                            C=c["C"][:, s] if cb_early else None)
           for s in sl]
    incoming = [None, ssd_fold_state(None, loc[0][1], loc[0][0])]
    outs, fin = [], None
    for r, s in enumerate(sl):
        o, fin = ssd_finish(c["x"][:, s], c["dt"][:, s], c["A"], c["B"][:, s], c["C"][:, s], Q, loc[r][2], D=c["D"],
                            dt_bias=c["dt_bias"], incoming_state=incoming[r], dt_softplus=True, return_final_states=True)
        assert _status() == 0
        outs.append(o)
    assert_close(torch.cat(outs, dim=1), whole, TOL_FP32_, "split out")
    assert_close(fin, wfin, TOL_FP32_, "split final")
    assert_close(ssd_fold_state(incoming[1], loc[1][1], loc[1][0]), wfin, TOL_FP32_, "folded summary")


def test_sequence_split_when_only_the_output_half_is_misaligned():
    """The LOCAL half sees x, B and dt only and takes the streaming tensor-core launch; the OUTPUT half is handed a
    gate whose rows start 2 bytes off a 16-byte boundary, which the tensor-core chunk scan cannot take.  The OUTPUT
    half must notice that LOCAL left no fp32 chunk states and form them itself.  Equal to the single call."""
    from mamba_b200 import ssd_finish, ssd_fold_state, ssd_local_states
    b, L, H, P, G, N, Q = 2, 1024, 40, 64, 2, 128, 256          # 80 (batch, head) units: the streaming launch
    inp = make(21, b, L, H, P, G, N, torch.bfloat16)
    c = {k: _c(v) for k, v in inp.items()}
    zbuf = torch.zeros(b, L, H, P + 8, device=DEV, dtype=torch.bfloat16)
    zbuf[..., 1:P + 1] = c["z"]
    z_off = zbuf[..., 1:P + 1]                                  # unit last stride, strides multiples of 8, base 2 bytes off
    assert z_off.data_ptr() % 16 == 2
    whole, wfin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"], dt_softplus=True,
                        return_final_states=True)
    assert _status() == 0
    half = L // 2
    sl = [slice(0, half), slice(half, L)]
    # C goes to the LOCAL half too: its early tensor-core C.B^T is then of no use to the general chunk scan of the
    # OUTPUT half, which must form its own
    loc = [ssd_local_states(c["x"][:, s], c["dt"][:, s], c["A"], c["B"][:, s], Q, dt_bias=c["dt_bias"], dt_softplus=True, C=c["C"][:, s])
           for s in sl]
    incoming = [None, ssd_fold_state(None, loc[0][1], loc[0][0])]
    outs, fin = [], None
    for r, s in enumerate(sl):
        o, fin = ssd_finish(c["x"][:, s], c["dt"][:, s], c["A"], c["B"][:, s], c["C"][:, s], Q, loc[r][2], D=c["D"], z=z_off[:, s],
                            dt_bias=c["dt_bias"], incoming_state=incoming[r], dt_softplus=True, return_final_states=True)
        assert _status() == 0
        outs.append(o)
    assert_close(torch.cat(outs, dim=1), whole, TOL_BF16, "split out (misaligned gate)")
    assert_close(fin, wfin, TOL_BF16, "split final (misaligned gate)")
    # the whole operator with the same gate takes the general kernels throughout and agrees too
    got, gfin = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=z_off, dt_bias=c["dt_bias"], dt_softplus=True,
                      return_final_states=True)
    assert_close(got, whole, TOL_BF16, "single call (misaligned gate)")
    assert_close(gfin, wfin, TOL_BF16, "single call final (misaligned gate)")


def test_empty_range_of_a_sequence_split_is_the_identity():
    """A LOCAL call on zero tokens (a rank that owns no chunk) returns state 0 and decay 1; the OUTPUT call hands
    the incoming state on as the final state."""
    from mamba_b200 import ssd_finish, ssd_local_states
    b, H, P, G, N, Q = 2, 3, 64, 1, 128, 256
    inp = make(22, b, 0, H, P, G, N, torch.bfloat16, has_z=False, init=True)
    c = {k: _c(v) for k, v in inp.items()}
    state, decay, scratch = ssd_local_states(c["x"], c["dt"], c["A"], c["B"], Q, dt_bias=c["dt_bias"], dt_softplus=True)
    assert torch.equal(state, torch.zeros_like(state)) and torch.equal(decay, torch.ones_like(decay))
    out, fin = ssd_finish(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, scratch, D=c["D"], dt_bias=c["dt_bias"],
                          incoming_state=c["initial_states"], dt_softplus=True, return_final_states=True)
    assert out.shape == (b, 0, H, P) and torch.equal(fin, c["initial_states"])


def _packed(seed, lens, H, P, G, N, dtype):
    total = sum(lens)
    inp = make(seed, 1, total, H, P, G, N, dtype)
    seq_idx = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)])[None]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return inp, seq_idx, cu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16)])
@pytest.mark.parametrize("Q,lens", [(64, [201, 56, 5]), (128, [1, 130, 127, 64, 300]), (256, [256, 512, 100]), (64, [64, 64])])
def test_packed_sequences(dtype, tol, Q, lens):
    """seq_idx: packed sequences must not interact -- equal to running every sequence on its own; and the
    per-sequence end states (cu_seqlens / return_varlen_states) equal each run's final state.  This is how
    the reference tests its varlen path (tests/ops/triton/test_ssd.py:30-78)."""
    H, P, G, N = 4, 64, 2, 128
    inp, seq_idx, cu = _packed(50 + Q, lens, H, P, G, N, dtype)
    c = {k: _c(v) for k, v in inp.items()}
    out, fin, var = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                          seq_idx=seq_idx.to(DEV), cu_seqlens=cu.to(DEV), dt_softplus=True, return_final_states=True,
                          return_varlen_states=True)
    assert var.shape == (len(lens), H, P, N)
    f = lambda t: None if t is None else t.float()
    for i in range(len(lens)):
        sl = slice(int(cu[i]), int(cu[i + 1]))
        want, wfin = oracle.ssd_chunk_scan(f(inp["x"][:, sl]), f(inp["dt"][:, sl]), inp["A"], f(inp["B"][:, sl]), f(inp["C"][:, sl]),
                                           Q, inp["D"], f(inp["z"][:, sl]), inp["dt_bias"], None, dt_softplus=True)
        assert_close(out[:, sl], want, tol, f"packed out seq {i}")
        assert_close(var[i:i + 1], wfin, tol, f"varlen state seq {i}")
    assert_close(fin, var[-1:], tol, "final state is the last sequence's")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_packed_sequences_on_the_streaming_tensor_core_path(dtype):
    """Enough heads for the fused state-stream launch, sequences that start and end inside chunks, at chunk borders and
    that span several chunks; with an initial state for the first sequence.  Each sequence equals its own run."""
    H, P, G, N, Q = 80, 64, 2, 128, 256
    lens = [300, 212, 256, 700, 1, 67]                      # boundaries at 300, 512 (chunk border), 768 (border), 1468, 1469
    inp, seq_idx, cu = _packed(77, lens, H, P, G, N, dtype)
    g = torch.Generator().manual_seed(78)
    init = 0.5 * torch.randn(1, H, P, N, generator=g)
    c = {k: _c(v) for k, v in inp.items()}
    out, fin, var = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"], initial_states=init.to(DEV),
                          seq_idx=seq_idx.to(DEV), cu_seqlens=cu.to(DEV), dt_softplus=True, return_final_states=True, return_varlen_states=True)
    assert _status() == 0
    f = lambda t: None if t is None else t.float()
    for i in (0, 1, 3, 4, 5):
        sl = slice(int(cu[i]), int(cu[i + 1]))
        # every ninth head keeps the oracle's share of the test short; heads 0, 9, ... 72 cover both groups
        hs = list(range(0, H, 9))
        gs = sorted({h // (H // G) for h in hs})
        for gi in gs:
            hg = [h for h in hs if h // (H // G) == gi]
            want, wfin = oracle.ssd_chunk_scan(f(inp["x"][:, sl][:, :, hg]), f(inp["dt"][:, sl][:, :, hg]), inp["A"][hg], f(inp["B"][:, sl, gi:gi + 1]),
                                               f(inp["C"][:, sl, gi:gi + 1]), Q, inp["D"][hg], f(inp["z"][:, sl][:, :, hg]), inp["dt_bias"][hg],
                                               init[:, hg] if i == 0 else None, dt_softplus=True)
            assert_close(out[:, sl][:, :, hg], want, TOL_BF16, f"packed out seq {i} group {gi}")
            assert_close(var[i:i + 1][:, hg], wfin, TOL_BF16, f"varlen state seq {i} group {gi}")
    assert_close(fin, var[-1:], TOL_BF16, "final state is the last sequence's")


def test_seq_idx_without_varlen_states():
    inp, seq_idx, cu = _packed(61, [100, 92], 2, 16, 1, 16, torch.float32)
    c = {k: _c(v) for k, v in inp.items()}
    out = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 64, D=c["D"], z=c["z"], dt_bias=c["dt_bias"], seq_idx=seq_idx.to(DEV),
                dt_softplus=True)
    for i in range(2):
        sl = slice(int(cu[i]), int(cu[i + 1]))
        want, _ = oracle.ssd_chunk_scan(inp["x"][:, sl], inp["dt"][:, sl], inp["A"], inp["B"][:, sl], inp["C"][:, sl], 64, inp["D"],
                                        inp["z"][:, sl], inp["dt_bias"], None, dt_softplus=True)
        assert_close(out[:, sl], want, TOL_FP32, f"seq {i}")


def test_unsupported_features_raise():
    inp = make(15, 1, 64, 2, 8, 1, 8, torch.float32)
    c = {k: _c(v) for k, v in inp.items()}
    with pytest.raises(AssertionError, match="cu_seqlens must be provided"):
        _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 64, return_varlen_states=True)
    with pytest.raises(AssertionError):
        _fn()(c["x"], c["dt"], c["A"][:1], c["B"], c["C"], 64)
    two = make(15, 2, 64, 2, 8, 1, 8, torch.float32)
    t = {k: _c(v) for k, v in two.items()}
    with pytest.raises(AssertionError, match="batch dimension is 1"):
        _fn()(t["x"], t["dt"], t["A"], t["B"], t["C"], 64, cu_seqlens=torch.tensor([0, 64], device=DEV), return_varlen_states=True)


def bench_config2_inputs(b, H, L=4096, P=64, N=128, seed=1002):
    return make(seed, b, L, H, P, 1, N, torch.bfloat16)


def test_bench_config2_slice_against_oracle():
    """bf16, seqlen 4096, headdim 64, dstate 128, chunk 256, one group: 1 batch row x 4 heads."""
    run_both(bench_config2_inputs(1, 4), 256, TOL_BF16, "config 2 slice")


def test_bench_config2_full_size_properties():
    """Full benchmark size (batch 8, 80 heads, seqlen 4096): the fused state-stream path.  Three heads of one batch
    row against the oracle (heads are independent given their group's B and C), run-to-run bit identity (no
    atomics anywhere), and agreement with the two-launch path that a sequence split takes."""
    from mamba_b200 import ops
    inp = bench_config2_inputs(8, 80)
    c = {k: _c(v) for k, v in inp.items()}
    kw = dict(D=c["D"], z=c["z"], dt_bias=c["dt_bias"], dt_softplus=True, return_final_states=True)
    out1, fin1 = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, **kw)
    assert _status() == 0
    out2, fin2 = _fn()(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, **kw)
    assert torch.equal(out1, out2) and torch.equal(fin1, fin2)
    row, heads = 5, torch.tensor([0, 41, 79])
    f = lambda t: t.float()
    want, wfin = oracle.ssd_chunk_scan(f(inp["x"][row:row + 1, :, heads]), f(inp["dt"][row:row + 1, :, heads]), inp["A"][heads],
                                       f(inp["B"][row:row + 1]), f(inp["C"][row:row + 1]), 256, inp["D"][heads],
                                       f(inp["z"][row:row + 1, :, heads]), inp["dt_bias"][heads], None, dt_softplus=True)
    hd = heads.to(DEV)
    assert_close(out1[row:row + 1, :, hd], want, TOL_BF16, "full-size subset out")
    assert_close(fin1[row:row + 1, hd], wfin, TOL_BF16, "full-size subset final_states")
    # the same operator in two phases (chunk states kept in memory, separate state passing)
    st, dec, scratch = ops.ssd_local_states(c["x"], c["dt"], c["A"], c["B"], 256, dt_bias=c["dt_bias"], dt_softplus=True)
    out3, fin3 = ops.ssd_finish(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, scratch, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                                incoming_state=None, dt_softplus=True, return_final_states=True)
    assert _status() == 0
    assert_close(out3, out1.float(), TOL_BF16, "fused vs two-launch out")
    assert_close(fin3, fin1, TOL_BF16, "fused vs two-launch final_states")
    assert_close(st, fin1, TOL_BF16, "range state vs final state")


def test_bench_config3_full_size_properties():
    """Full length of the long-sequence configuration (batch 1, 262144 steps, 128 heads, 8 groups, no gate) on one
    GPU: two heads against the oracle over the whole sequence (output and final state), and the two-phase split
    into two ranges against the single call."""
    from mamba_b200 import ops
    L, H, P, G, N, Q = 262144, 128, 64, 8, 128, 256
    g = torch.Generator(device=DEV).manual_seed(1003)
    r = lambda *sh: torch.randn(*sh, generator=g, device=DEV)
    bf = torch.bfloat16
    x, dt, B, C = r(1, L, H, P).to(bf), r(1, L, H).to(bf), r(1, L, G, N).to(bf), r(1, L, G, N).to(bf)
    gh = torch.Generator().manual_seed(1003)
    A = -(1 + 15 * torch.rand(H, generator=gh))
    D = torch.randn(H, generator=gh)
    dtv = torch.exp(torch.rand(H, generator=gh) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    bias = dtv + torch.log(-torch.expm1(-dtv))
    Ad, Dd, bd = A.to(DEV), D.to(DEV), bias.to(DEV)
    out, fin = _fn()(x, dt, Ad, B, C, Q, D=Dd, dt_bias=bd, dt_softplus=True, return_final_states=True)
    assert _status() == 0
    for h in (5, 127):
        grp = h // (H // G)
        f = lambda t: t.float().cpu()
        want, wfin = oracle.ssd_chunk_scan(f(x[:, :, h:h + 1]), f(dt[:, :, h:h + 1]), A[h:h + 1], f(B[:, :, grp:grp + 1]),
                                           f(C[:, :, grp:grp + 1]), Q, D[h:h + 1], None, bias[h:h + 1], None, dt_softplus=True)
        assert_close(out[:, :, h:h + 1], want, TOL_BF16, f"head {h} out")
        assert_close(fin[:, h:h + 1], wfin, TOL_BF16, f"head {h} final_states")
    half = L // 2
    loc, outs, f2 = [], [], None
    for sl in (slice(0, half), slice(half, L)):
        loc.append(ops.ssd_local_states(x[:, sl], dt[:, sl], Ad, B[:, sl], Q, dt_bias=bd, dt_softplus=True))
    incoming = [None, ops.ssd_fold_state(None, loc[0][1], loc[0][0])]
    for i, sl in enumerate((slice(0, half), slice(half, L))):
        o, f2 = ops.ssd_finish(x[:, sl], dt[:, sl], Ad, B[:, sl], C[:, sl], Q, loc[i][2], D=Dd, dt_bias=bd,
                               incoming_state=incoming[i], dt_softplus=True, return_final_states=True)
        assert _status() == 0
        outs.append(o)
    assert_close(torch.cat(outs, dim=1), out.float(), TOL_BF16, "split out")
    assert_close(f2, fin, TOL_BF16, "split final_states")


def test_fold_ranges_equals_range_by_range_folds():
    """One launch over several gathered summaries gives the bits of folding them one at a time."""
    from mamba_b200 import ssd_fold_ranges, ssd_fold_state
    g = torch.Generator().manual_seed(5)
    world, b, h, p, n = 5, 2, 3, 8, 16
    states = torch.randn(world, b, h, p, n, generator=g)
    decays = torch.rand(world, b, h, generator=g)
    rec = torch.cat([states.reshape(world, -1), decays.reshape(world, -1)], dim=1).to(DEV)
    for last in (0, 1, 4):
        want = states[0].to(DEV)
        for r in range(1, last + 1):
            want = ssd_fold_state(want, decays[r].to(DEV), states[r].to(DEV))
        got = ssd_fold_ranges(rec, 0, last, (b, h, p, n))
        assert torch.equal(got, want)
