"""Places the reference's OWN CPU implementation of the path under oracle/_ref/ -- TEST / BASELINE INFRASTRUCTURE ONLY.

The reference's definitions of the three operators (selective_scan_ref, ssd_chunk_scan_combined_ref,
selective_state_update_ref) are pure PyTorch and live in its Python package.  This recipe copies that
package, unmodified, from the reference checkout where it lies into oracle/_ref/mamba_ssm (git-ignored: the
copy never enters history), so that it can travel to a machine that has no reference checkout and be timed
there as the CPU baseline (bench.py, `cpu_baseline.kind: "reference"`).  Nothing in the product imports it.

    python oracle/make_ref.py [path-to-reference-checkout]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make(reference_root="/root/reference"):
    """Returns the destination directory, or None when no reference checkout is present."""
    src = os.path.join(reference_root, "mamba_ssm")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "mamba_ssm")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


def load():
    """The copied package's three reference functions, or None when oracle/_ref is absent or does not import."""
    if not os.path.isdir(os.path.join(DEST, "mamba_ssm")):
        return None
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    try:
        from mamba_ssm.ops.selective_scan_interface import selective_scan_ref
        from mamba_ssm.ops.triton.selective_state_update import selective_state_update_ref
        from mamba_ssm.ops.triton.ssd_combined import ssd_chunk_scan_combined_ref
    except Exception:
        return None
    return dict(selective_scan=selective_scan_ref, ssd_chunk_scan=ssd_chunk_scan_combined_ref,
                selective_state_update=selective_state_update_ref)


if __name__ == "__main__":
    print(make(*sys.argv[1:2]))
