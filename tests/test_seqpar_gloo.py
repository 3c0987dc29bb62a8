"""Host logic of the sequence-split SSD scan, exercised by CPU ranks over gloo (world size 2 and 3).

The ranks run the real hand-off code of mamba_b200/seqpar.py; the three compute steps are supplied by
the CPU oracle, so no GPU is involved.  A missing predecessor must surface as SequenceHandoffError on
the waiting rank (bounded by the process-group timeout), not as a hang.
"""
import datetime
import math
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(seed, b, L, H, P, G, N):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    dtv = torch.exp(torch.rand(H, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    return dict(x=r(b, L, H, P), dt=r(b, L, H), A=-(1 + 3 * torch.rand(H, generator=g)), B=r(b, L, G, N), C=r(b, L, G, N),
                D=r(H), z=r(b, L, H, P), dt_bias=dtv + torch.log(-torch.expm1(-dtv)), init=0.5 * r(b, H, P, N))


def _oracle_steps():
    import oracle
    import torch.nn.functional as F
    from mamba_b200.seqpar import SsdSteps

    def local(x, dt, A, B, Q, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf")), C=None):
        if x.shape[1] == 0:      # an empty range is summarised by the identity, as the library does
            return torch.zeros(x.shape[0], x.shape[2], x.shape[3], B.shape[3]), torch.ones(x.shape[0], x.shape[2]), None
        _, state = oracle.ssd_chunk_scan(x, dt, A, B, B, Q, dt_bias=dt_bias, dt_softplus=dt_softplus, dt_limit=dt_limit)
        d = dt.float() + (0 if dt_bias is None else dt_bias)
        d = F.softplus(d) if dt_softplus else d
        decay = torch.exp((d * A).sum(dim=1))                      # (batch, nheads)
        return state, decay, None

    def fold(incoming, decay, state):
        return state if incoming is None else decay[..., None, None] * incoming + state

    def finish(x, dt, A, B, C, Q, scratch, D=None, z=None, dt_bias=None, incoming_state=None, dt_softplus=False,
               dt_limit=(0.0, float("inf")), return_final_states=False):
        if x.shape[1] == 0:
            fin = incoming_state if incoming_state is not None else torch.zeros(x.shape[0], x.shape[2], x.shape[3], B.shape[3])
            return (x.float(), fin) if return_final_states else x.float()
        out, fin = oracle.ssd_chunk_scan(x, dt, A, B, C, Q, D, z, dt_bias, incoming_state, dt_softplus=dt_softplus,
                                         dt_limit=dt_limit)
        return (out, fin) if return_final_states else out

    return SsdSteps(local=local, fold=fold, finish=finish)


def _worker(rank, world, store, mode, result_dir):
    sys.path.insert(0, ROOT)
    from mamba_b200.seqpar import SequenceHandoffError, mamba_chunk_scan_sequence_parallel, split_sequence
    dist.init_process_group("gloo", init_method=f"file://{store}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    try:
        b, L, H, P, G, N, Q = 1, 448, 3, 8, 1, 16, 64
        mode, _, handoff = mode.partition(":")
        if mode == "short":      # fewer chunks than ranks: the last ranks own nothing
            L = 128
        inp = _inputs(5, b, L, H, P, G, N)
        lo, hi = split_sequence(L, Q, world, rank)
        sl = slice(lo, hi)
        if mode == "dead_predecessor" and rank == 0:
            return                                                  # leaves without handing its state on
        try:
            out, fin = mamba_chunk_scan_sequence_parallel(
                inp["x"][:, sl], inp["dt"][:, sl], inp["A"], inp["B"][:, sl], inp["C"][:, sl], Q, D=inp["D"], z=inp["z"][:, sl],
                dt_bias=inp["dt_bias"], initial_states=inp["init"], dt_softplus=True, return_final_states=True,
                steps=_oracle_steps(), handoff=handoff or None)
            torch.save({"out": out, "fin": fin, "range": (lo, hi)}, os.path.join(result_dir, f"rank{rank}.pt"))
        except SequenceHandoffError as e:
            torch.save({"error": str(e)}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(world, mode):
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        mp.spawn(_worker, args=(world, store, mode, tmp), nprocs=world, join=True)
        return {r: torch.load(os.path.join(tmp, f"rank{r}.pt")) for r in range(world) if os.path.exists(os.path.join(tmp, f"rank{r}.pt"))}


@pytest.mark.parametrize("world,handoff", [(2, "chain"), (3, "chain"), (2, "gather"), (3, "gather"), (3, "")])
def test_sequence_split_equals_single_rank(world, handoff):
    """Point-to-point chain, all-gather of the range summaries, and the default choice give the single-rank result."""
    import oracle
    res = _run(world, "ok:" + handoff)
    inp = _inputs(5, 1, 448, 3, 8, 1, 16)
    want, wfin = oracle.ssd_chunk_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], 64, inp["D"], inp["z"], inp["dt_bias"],
                                       inp["init"], dt_softplus=True)
    assert sorted(res) == list(range(world))
    got = torch.cat([res[r]["out"] for r in range(world)], dim=1)
    assert [res[r]["range"] for r in range(world)][0][0] == 0 and res[world - 1]["range"][1] == 448
    assert (got - want).abs().max() <= 1e-5 * want.abs().max()
    assert (res[world - 1]["fin"] - wfin).abs().max() <= 1e-5 * wfin.abs().max().clamp_min(1)


@pytest.mark.parametrize("handoff", ["chain", "gather"])
def test_more_ranks_than_chunks(handoff):
    """Ranks that own no chunk pass the state through unchanged: the last rank still returns the final state."""
    import oracle
    world = 4
    res = _run(world, "short:" + handoff)
    inp = _inputs(5, 1, 128, 3, 8, 1, 16)
    want, wfin = oracle.ssd_chunk_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], 64, inp["D"], inp["z"], inp["dt_bias"],
                                       inp["init"], dt_softplus=True)
    assert [res[r]["range"] for r in range(world)] == [(0, 64), (64, 128), (128, 128), (128, 128)]
    got = torch.cat([res[r]["out"] for r in range(world)], dim=1)
    assert (got - want).abs().max() <= 1e-5 * want.abs().max()
    for r in (1, 2, 3):
        assert (res[r]["fin"] - wfin).abs().max() <= 1e-5 * wfin.abs().max().clamp_min(1)


def test_missing_predecessor_is_reported_not_hung():
    res = _run(2, "dead_predecessor:chain")
    assert 0 not in res
    assert "error" in res[1] and "no state from rank 0" in res[1]["error"]


def test_missing_rank_is_reported_by_the_gather_too():
    res = _run(3, "dead_predecessor:gather")
    assert 0 not in res
    for r in (1, 2):
        assert "error" in res[r] and "gathering the range summaries failed" in res[r]["error"]


def test_split_sequence_covers_every_chunk_once():
    from mamba_b200.seqpar import split_sequence
    for L, Q, W in [(262144, 256, 8), (1000, 256, 3), (256, 256, 4), (700, 64, 5)]:
        edges = [split_sequence(L, Q, W, r) for r in range(W)]
        assert edges[0][0] == 0 and edges[-1][1] == L
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 <= a1
            assert a1 % Q == 0 or a1 == L
