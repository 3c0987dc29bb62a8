"""SSD chunked scan with the SEQUENCE split across ranks (one process per GPU).

The reference always runs the SSD scan on one device; its inter-chunk recurrence
``H_{c+1} = exp(sum dA_c) H_c + S_c`` (mamba_ssm/ops/triton/ssd_state_passing.py:72-80) is linear, so a
contiguous range of chunks can be summarised by ``(range_state, range_decay)`` and
``initial_states`` (already an input of the operator, ssd_combined.py:368-381) carries the rest:

    rank r:  1. local pass      range_state_r, range_decay_r   (zero incoming state; all ranks in parallel)
             2. hand-off        recv S_in from r-1;  send  range_decay_r * S_in + range_state_r  to r+1
             3. output pass     inter-chunk recurrence from S_in, chunk outputs

Step 2 is the only communication.  Two forms, same result bit for bit:

    "chain"   one (batch, nheads, headdim, dstate) fp32 tensor per hop, point to point (NCCL P2P over
              NVLink between GPUs): world-1 hops one after the other;
    "gather"  one all-gather of every rank's (range_state, range_decay) -- rank 0 contributes its
              OUTGOING state, so initial_states never has to travel -- and each rank folds the
              summaries of its predecessors itself, in rank order: one collective instead of a
              serial chain (the default above two ranks).

Received data lands in this rank's own memory before any kernel reads it.  Every wait is bounded by
the process group's timeout; a missing peer surfaces as ``SequenceHandoffError`` instead of a hang.

The compute steps are injectable so that the hand-off logic can be exercised by CPU ranks (gloo) in
tests; the defaults are this package's CUDA operators.
"""
import time
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import ops


class SequenceHandoffError(RuntimeError):
    """The state hand-off between neighbouring ranks failed (peer missing, timed out, or mismatched)."""


@dataclass
class SsdSteps:
    """The compute steps of a rank; defaults are the CUDA operators of this package.  ``fold_ranges`` (optional)
    folds several gathered summaries in one call; without it ``fold`` is applied range by range."""
    local: Callable = ops.ssd_local_states
    fold: Callable = ops.ssd_fold_state
    finish: Callable = ops.ssd_finish
    fold_ranges: Optional[Callable] = ops.ssd_fold_ranges


def split_sequence(seqlen: int, chunk_size: int, world: int, rank: int):
    """Contiguous range of whole chunks ``[start, stop)`` (in tokens) that `rank` owns."""
    nchunks = (seqlen + chunk_size - 1) // chunk_size
    per, extra = divmod(nchunks, world)
    first = rank * per + min(rank, extra)
    count = per + (1 if rank < extra else 0)
    return min(first * chunk_size, seqlen), min((first + count) * chunk_size, seqlen)


def _recv_state(like: torch.Tensor, src: int, group) -> torch.Tensor:
    buf = torch.empty_like(like)
    try:
        dist.recv(buf, src=src, group=group)
    except Exception as e:  # timeout, peer gone, transport error
        raise SequenceHandoffError(f"rank {dist.get_rank(group)}: no state from rank {src}: {e}") from e
    return buf


def _send_state(t: torch.Tensor, dst: int, group) -> None:
    try:
        dist.send(t.contiguous(), dst=dst, group=group)
    except Exception as e:
        raise SequenceHandoffError(f"rank {dist.get_rank(group)}: could not hand the state to rank {dst}: {e}") from e


def _gather_summaries(state: torch.Tensor, decay: torch.Tensor, group):
    """Every rank's (state, decay) as two lists indexed by rank; one collective carries both."""
    world = dist.get_world_size(group)
    ns, nd = state.numel(), decay.numel()
    mine = torch.cat([state.reshape(-1), decay.reshape(-1).to(state.dtype)])
    everyone = torch.empty(world, ns + nd, dtype=state.dtype, device=state.device)
    try:
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(everyone, mine, group=group)
        else:
            dist.all_gather(list(everyone.unbind(0)), mine, group=group)
    except Exception as e:  # timeout, peer gone, transport error
        raise SequenceHandoffError(f"rank {dist.get_rank(group)}: gathering the range summaries failed: {e}") from e
    states = [everyone[r, :ns].view(state.shape) for r in range(world)]          # views, nothing is copied
    decays = [everyone[r, ns:].view(decay.shape).to(decay.dtype) for r in range(world)]
    return states, decays, everyone


class _PhaseClock:
    """Device time stamps between the phases of one call (CUDA events on the current stream) plus the host time the
    call spent enqueueing; fills a caller-supplied dict with milliseconds when the call ends (synchronises)."""

    def __init__(self, sink, cuda):
        self.sink, self.cuda, self.marks = sink, cuda and sink is not None, []
        self.t_host = time.perf_counter()
        self.mark("start")

    def mark(self, name):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def finish(self):
        if self.sink is None:
            return
        self.sink["host_enqueue"] = (time.perf_counter() - self.t_host) * 1e3
        if self.cuda:
            torch.cuda.synchronize()
            for (_, a), (name, b) in zip(self.marks, self.marks[1:]):
                self.sink[name] = a.elapsed_time(b)
            self.sink["total_device"] = self.marks[0][1].elapsed_time(self.marks[-1][1])


def mamba_chunk_scan_sequence_parallel(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                                       dt_softplus=False, dt_limit=(0.0, float("inf")), return_final_states=False,
                                       group=None, steps: Optional[SsdSteps] = None, handoff: Optional[str] = None,
                                       phases: Optional[dict] = None):
    """Run this rank's slice of a sequence that is split over the ranks of `group`.

    x, dt, B, C, z hold THIS rank's contiguous tokens (a whole number of chunks on every rank but the
    last); A, D, dt_bias are replicated; ``initial_states`` (state before the first token of the whole
    sequence) is only read on rank 0.  ``handoff`` is "chain", "gather" or None (gather above two ranks).
    Returns this rank's ``out`` and, if asked, the state after this rank's last token -- on the last
    rank that is the final state of the whole sequence.  ``phases`` (a dict) receives the device time of every
    phase of this call in milliseconds and the host time spent enqueueing it; asking for it synchronises.
    """
    steps = steps or SsdSteps()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    clock = _PhaseClock(phases, x.is_cuda)
    if rank < world - 1:
        assert x.shape[1] % chunk_size == 0, "every rank but the last must hold whole chunks"
    # C goes along so that C.B^T, which needs nothing from the exchange, is formed ahead of it
    range_state, range_decay, scratch = steps.local(x, dt, A, B, chunk_size, dt_bias=dt_bias, dt_softplus=dt_softplus,
                                                    dt_limit=dt_limit, C=C)
    clock.mark("local")
    if handoff is None:
        handoff = "gather" if world > 2 else "chain"
    assert handoff in ("chain", "gather"), "handoff must be 'chain' or 'gather'"
    first = None if (rank != 0 or initial_states is None) else initial_states.to(range_state.dtype)
    if world == 1:
        incoming = first
    elif handoff == "chain":
        incoming = first if rank == 0 else _recv_state(range_state, rank - 1, group)
        if rank < world - 1:
            _send_state(steps.fold(incoming, range_decay, range_state), rank + 1, group)
    else:
        mine = steps.fold(first, range_decay, range_state) if rank == 0 else range_state
        states, decays, everyone = _gather_summaries(mine, range_decay, group)
        incoming = first
        if rank == 1:
            incoming = states[0]                       # the state rank 0 hands on
        elif rank > 1 and steps.fold_ranges is not None and everyone.is_cuda and everyone.dtype == torch.float32:
            incoming = steps.fold_ranges(everyone, 0, rank - 1, tuple(range_state.shape))    # one launch
        elif rank > 1:
            incoming = states[0]
            for r in range(1, rank):
                incoming = steps.fold(incoming, decays[r], states[r])
    clock.mark("handoff")
    res = steps.finish(x, dt, A, B, C, chunk_size, scratch, D=D, z=z, dt_bias=dt_bias, incoming_state=incoming,
                       dt_softplus=dt_softplus, dt_limit=dt_limit, return_final_states=return_final_states)
    clock.mark("output")
    clock.finish()
    return res
