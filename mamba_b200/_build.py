"""Builds libmamba_b200.so in-tree with nvcc for sm_100a.

    python -m mamba_b200._build [--force] [--verbose]

The shared library is the product's only native artefact: a C-ABI (include/mamba_b200.h) over
the CUDA kernels in mamba_b200/csrc.  It links the CUDA runtime statically, so loading it needs
nothing but the driver.
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libmamba_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr", "--extended-lambda",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(PKG), "include", "mamba_b200.h"))
    return hs


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ and link libmamba_b200.so; returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    # the image exports CC/CXX to a wrapper; nvcc needs the system host compiler
    host = ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []
    newest_hdr = max(os.path.getmtime(h) for h in _headers())
    objs, logs = [], []
    procs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_hdr)
        if stale:
            cmd = [nvcc, *host, *NVCC_FLAGS, "-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        logs.append((src, out))
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src}")
        if verbose:
            sys.stderr.write(out)
    if procs or force or not os.path.exists(LIB):
        cmd = [nvcc, *host, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.check_call(cmd, env=env)
    if logs:
        with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
            for src, out in logs:
                f.write(f"==== {os.path.basename(src)}\n{out}\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
