"""The C-ABI library loads and exports every symbol include/mamba_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from mamba_b200 import _build
    return _build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mamba_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mb200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built):
    lib = ctypes.CDLL(built)
    names = declared_symbols()
    assert "mb200_selective_scan_fwd" in names and "mb200_ssd_chunk_scan_fwd" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mamba_b200.h but not exported"


def test_binding_covers_header(built):
    from mamba_b200 import _lib
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared_symbols()
    assert _lib.lib().mb200_version() >= 100


def test_struct_sizes_match_header(built, tmp_path):
    """ctypes mirrors must have the C compiler's layout of the argument structs."""
    import subprocess
    from mamba_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "mamba_b200.h"\nint main(void){printf("%zu %zu %zu\\n",'
                   'sizeof(mb200_scan_args),sizeof(mb200_ssu_args),sizeof(mb200_ssd_args));'
                   'printf(" %zu %zu %zu %zu\\n",sizeof(mb200_scan_bwd_args),sizeof(mb200_conv1d_args),'
                   'sizeof(mb200_conv1d_update_args),sizeof(mb200_rmsnorm_args));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["/usr/bin/gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    sizes = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    assert sizes == [ctypes.sizeof(t) for t in (_lib.ScanArgs, _lib.SsuArgs, _lib.SsdArgs, _lib.ScanBwdArgs, _lib.Conv1dArgs,
                                                _lib.Conv1dUpdateArgs, _lib.RmsNormArgs)]


def test_argument_errors_without_gpu(built):
    """Argument validation happens before any CUDA call, so it is testable on a CPU-only host."""
    from mamba_b200 import _lib
    a = _lib.ScanArgs()
    rc = _lib.lib().mb200_selective_scan_fwd(ctypes.byref(a), None)
    assert rc == _lib.ERR_BAD_ARG and b"sizes" in _lib.lib().mb200_last_error()
    a.batch, a.dim, a.seqlen, a.dstate, a.ngroups = 1, 4, 8, 4, 1
    rc = _lib.lib().mb200_selective_scan_fwd(ctypes.byref(a), None)
    assert rc == _lib.ERR_BAD_ARG and b"NULL" in _lib.lib().mb200_last_error()
    a.dstate = 300
    rc = _lib.lib().mb200_selective_scan_fwd(ctypes.byref(a), None)
    assert rc == _lib.ERR_BAD_ARG and b"256" in _lib.lib().mb200_last_error()
    with pytest.raises(AssertionError):
        _lib.check(rc)
    rc = _lib.lib().mb200_scan_status(0, None)
    assert rc == _lib.ERR_BAD_ARG and b"status is NULL" in _lib.lib().mb200_last_error()
    # backward of the scan: the scratch size is pure arithmetic (states at every eighth step, 16 states per pass, plus the
    # partial sums above 16 states), capped at 1 GiB by walking the batch in slices
    g = _lib.ScanBwdArgs()
    need = ctypes.c_size_t(0)
    rc = _lib.lib().mb200_scan_bwd_scratch_bytes(ctypes.byref(g), ctypes.byref(need))
    assert rc == _lib.ERR_BAD_ARG
    g.batch, g.dim, g.seqlen, g.dstate, g.ngroups = 3, 64, 100, 16, 1
    assert _lib.lib().mb200_scan_bwd_scratch_bytes(ctypes.byref(g), ctypes.byref(need)) == _lib.OK
    assert need.value == 3 * 13 * 16 * 64 * 4 + 16
    g.dstate = 40
    assert _lib.lib().mb200_scan_bwd_scratch_bytes(ctypes.byref(g), ctypes.byref(need)) == _lib.OK
    assert need.value == 3 * (13 * 16 * 64 + 3 * 64 * 100) * 4 + 16
    g.batch, g.dim, g.seqlen, g.dstate = 64, 5120, 2048, 16
    assert _lib.lib().mb200_scan_bwd_scratch_bytes(ctypes.byref(g), ctypes.byref(need)) == _lib.OK
    per_row = 256 * 16 * 5120 * 4
    assert need.value == ((1 << 30) // per_row) * per_row + 16 and need.value <= (1 << 30) + 16
    g.dstate = 300
    rc = _lib.lib().mb200_selective_scan_bwd(ctypes.byref(g), None)
    assert rc == _lib.ERR_BAD_ARG and b"256" in _lib.lib().mb200_last_error()
    s = _lib.SsdArgs()
    s.batch, s.seqlen, s.nheads, s.headdim, s.ngroups, s.dstate, s.chunk_size = 64, 1 << 16, 64, 64, 1, 128, 256
    s.phases = _lib.PHASE_ALL
    rc = _lib.lib().mb200_ssd_chunk_scan_fwd_static(ctypes.byref(s), None)
    assert rc == _lib.ERR_BAD_ARG and b"built-in buffer" in _lib.lib().mb200_last_error()


def test_cpu_tensors_are_rejected():
    import torch
    from mamba_b200 import selective_state_update
    s = torch.zeros(1, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        selective_state_update(s, torch.zeros(1, 4), torch.zeros(1, 4), torch.zeros(4, 8), torch.zeros(1, 8), torch.zeros(1, 8))
