"""Shared helpers for the parity tests: golden loading and the error norms."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Parity tolerances of the path: fp32 inputs 1e-4, bf16 inputs 2e-2 (fp32 accumulation).
TOL_FP32 = 1e-4
TOL_BF16 = 2e-2


def golden_names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def load_golden(name, device="cpu"):
    """Returns a dict of tensors; inputs of bf16 cases are narrowed back to bf16."""
    d = np.load(os.path.join(GOLDEN, name + ".npz"))
    bf16 = bool(d["is_bf16"]) if "is_bf16" in d else False
    out = {}
    for k in d.files:
        v = d[k]
        out[k] = torch.from_numpy(v).to(device) if v.ndim > 0 else v.item()
    out["bf16"] = bf16
    return out


def norm_err(a, b):
    """max|a-b| / max(|b|, 1): the normalised error the tolerances are stated in."""
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1.0)).item()


def rel_err(a, b, floor_frac=1e-2):
    """Largest element-wise relative error |a-b| / |b| over the elements whose magnitude is at least
    `floor_frac` of the output range (below that a relative error measures rounding of near-cancelled sums)."""
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    keep = b.abs() >= floor_frac * b.abs().max().clamp_min(1e-30)
    if not keep.any():
        return 0.0
    return ((a - b).abs()[keep] / b.abs()[keep]).max().item()


# (what, normalised max error, element-wise relative error) of every comparison made, for the end-of-run report
ERROR_LOG = []


def assert_close(a, b, tol, what=""):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    e = norm_err(a, b)
    ERROR_LOG.append((what, e, rel_err(a, b)))
    assert e <= tol, f"{what}: normalised max error {e:.3e} > {tol:.1e}"
    # element-wise form with rtol = atol = tol scaled by the output range
    scale = b.abs().max().clamp_min(1.0)
    assert torch.allclose(a / scale, b / scale, rtol=tol, atol=tol), f"{what}: allclose(rtol=atol={tol}) failed"
