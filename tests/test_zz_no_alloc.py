"""The SSD entry point that allocates nothing (mb200_ssd_chunk_scan_fwd_static).

The buffer it uses lives in the library image and keeps whatever the previous call left in it, so these
tests must pass both on their own in a fresh process and after every other test of the suite has used
the library (this file is collected last).
"""
import math

import pytest
import torch

import oracle
from helpers import TOL_BF16, TOL_FP32, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, b, L, H, P, G, N, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    dtv = torch.exp(torch.rand(H, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    d = dict(x=r(b, L, H, P).to(dtype), dt=r(b, L, H).to(dtype), A=-(1 + 15 * torch.rand(H, generator=g)),
             B=r(b, L, G, N).to(dtype), C=r(b, L, G, N).to(dtype), D=r(H), z=r(b, L, H, P).to(dtype),
             dt_bias=dtv + torch.log(-torch.expm1(-dtv)), init=0.3 * r(b, H, P, N))
    return {k: v.to(DEV) for k, v in d.items()}


@pytest.mark.parametrize("dtype,tol,shape", [
    (torch.bfloat16, TOL_BF16, (2, 700, 4, 64, 1, 128, 256)),     # tensor-core stages, ragged tail
    (torch.float32, TOL_FP32, (1, 300, 3, 32, 1, 16, 64)),        # general stages
])
def test_static_scratch_matches_caller_scratch_twice(dtype, tol, shape):
    """Two calls in a row through the no-allocation entry point, each on different data, each compared
    with the ordinary entry point (which gets fresh caller-owned scratch) and with the CPU oracle."""
    from mamba_b200 import mamba_chunk_scan_combined, mamba_chunk_scan_combined_noalloc, ops
    b, L, H, P, G, N, Q = shape
    for rep in range(2):
        c = _inputs(900 + rep, b, L, H, P, G, N, dtype)
        want, want_fin = mamba_chunk_scan_combined(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"],
                                                   dt_bias=c["dt_bias"], initial_states=c["init"], dt_softplus=True,
                                                   return_final_states=True)
        out = torch.full_like(c["x"], float("nan"))
        fin = torch.full((b, H, P, N), float("nan"), device=DEV)
        allocations = lambda: torch.cuda.memory_stats()["allocation.all.allocated"]   # count of allocator requests so far
        before = allocations()
        got = mamba_chunk_scan_combined_noalloc(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, out, D=c["D"], z=c["z"],
                                                dt_bias=c["dt_bias"], initial_states=c["init"], dt_softplus=True,
                                                final_states=fin)
        assert allocations() == before, "the no-allocation path asked the allocator for device memory"
        torch.cuda.synchronize()
        assert got is out
        assert ops.ssd_status() == 0, "a kernel of the no-allocation call abandoned a bounded wait"
        assert_close(out, want, tol, f"static scratch out (call {rep})")
        assert_close(fin, want_fin, tol, f"static scratch final_states (call {rep})")
        f = lambda t: t.float().cpu()
        o_out, o_fin = oracle.ssd_chunk_scan(f(c["x"]), f(c["dt"]), f(c["A"]), f(c["B"]), f(c["C"]), Q, f(c["D"]), f(c["z"]),
                                             f(c["dt_bias"]), initial_states=f(c["init"]), dt_softplus=True)
        assert_close(out, o_out, tol, f"static scratch out vs oracle (call {rep})")
        assert_close(fin, o_fin, tol, f"static scratch final_states vs oracle (call {rep})")


def test_problem_larger_than_the_buffer_is_refused():
    from mamba_b200 import mamba_chunk_scan_combined_noalloc
    c = _inputs(7, 4, 4096, 16, 64, 1, 128, torch.bfloat16)   # 4*16*16 chunk states of 32 KiB in fp32 alone exceed 32 MiB
    out = torch.empty_like(c["x"])
    with pytest.raises(AssertionError, match="built-in buffer"):
        mamba_chunk_scan_combined_noalloc(c["x"], c["dt"], c["A"], c["B"], c["C"], 256, out, dt_softplus=True)
