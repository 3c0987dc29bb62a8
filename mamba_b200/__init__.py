"""mamba_b200 -- B200 (sm_100a) kernels behind the scan operators of state-spaces/mamba.

    from mamba_b200 import selective_scan_fn, mamba_chunk_scan_combined, selective_state_update

are drop-in replacements (forward / inference) for the reference's functions of the same name (the Mamba-1 scan is
differentiable too: its backward kernel serves autograd and ``selective_scan_bwd``); so are the steps
either side of the scan in the mixers (``causal_conv1d_fn``, ``causal_conv1d_update``, ``rmsnorm_fn``) and the fused
Mamba-2 block forward ``mamba_split_conv1d_scan_combined``.
All work is done by hand-written CUDA in ``libmamba_b200.so`` (C ABI: include/mamba_b200.h);
there is no CPU path and no fallback -- a missing library raises on first use.
"""
from .mixer_ops import (  # noqa: F401
    causal_conv1d_fn,
    causal_conv1d_update,
    mamba_split_conv1d_scan_combined,
    rmsnorm_fn,
)
from .ops import (  # noqa: F401
    mamba_chunk_scan_combined,
    mamba_chunk_scan_combined_noalloc,
    selective_scan_bwd,
    selective_scan_fn,
    selective_state_update,
    ssd_finish,
    ssd_fold_ranges,
    ssd_fold_state,
    ssd_local_states,
)

__version__ = "0.1.0"
