"""ctypes binding of libmamba_b200.so (the C ABI declared in include/mamba_b200.h).

There is no fallback: if the shared library is missing or a call fails, the caller gets an
exception.  Nothing here computes anything.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmamba_b200.so")

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_NO_DEVICE = 0, -1, -2, -3, -4
PHASE_LOCAL, PHASE_OUTPUT, PHASE_ALL, PHASE_CB, PHASE_CB_READY = 1, 2, 3, 4, 8
SSD_STATIC_SCRATCH_BYTES = 32 << 20

c_i32, c_i64, c_vp, c_f = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float


class ScanArgs(ctypes.Structure):
    _fields_ = [
        ("u", c_vp), ("delta", c_vp), ("A", c_vp), ("B", c_vp), ("C", c_vp), ("D", c_vp), ("z", c_vp),
        ("delta_bias", c_vp), ("out", c_vp), ("out_pregate", c_vp), ("last_state", c_vp),
        ("batch", c_i32), ("dim", c_i32), ("seqlen", c_i32), ("dstate", c_i32), ("ngroups", c_i32),
        ("io_dtype", c_i32), ("B_variable", c_i32), ("C_variable", c_i32), ("delta_softplus", c_i32),
        ("device", c_i32),
        ("u_stride", c_i64 * 2), ("delta_stride", c_i64 * 2), ("z_stride", c_i64 * 2),
        ("out_stride", c_i64 * 2), ("pregate_stride", c_i64 * 2), ("A_stride", c_i64 * 2),
        ("B_stride", c_i64 * 3), ("C_stride", c_i64 * 3),
        ("scratch", c_vp), ("scratch_bytes", ctypes.c_size_t),
    ]


class ScanBwdArgs(ctypes.Structure):
    _fields_ = [
        ("u", c_vp), ("delta", c_vp), ("A", c_vp), ("B", c_vp), ("C", c_vp), ("D", c_vp), ("z", c_vp),
        ("delta_bias", c_vp), ("dout", c_vp), ("du", c_vp), ("ddelta", c_vp), ("dz", c_vp),
        ("dA", c_vp), ("dB", c_vp), ("dC", c_vp), ("dD", c_vp), ("ddelta_bias", c_vp),
        ("batch", c_i32), ("dim", c_i32), ("seqlen", c_i32), ("dstate", c_i32), ("ngroups", c_i32),
        ("io_dtype", c_i32), ("B_variable", c_i32), ("C_variable", c_i32), ("delta_softplus", c_i32),
        ("device", c_i32),
        ("u_stride", c_i64 * 2), ("delta_stride", c_i64 * 2), ("z_stride", c_i64 * 2), ("dout_stride", c_i64 * 2),
        ("du_stride", c_i64 * 2), ("ddelta_stride", c_i64 * 2), ("dz_stride", c_i64 * 2),
        ("A_stride", c_i64 * 2), ("B_stride", c_i64 * 3), ("C_stride", c_i64 * 3),
        ("scratch", c_vp), ("scratch_bytes", ctypes.c_size_t),
    ]


class SsuArgs(ctypes.Structure):
    _fields_ = [
        ("state", c_vp), ("x", c_vp), ("dt", c_vp), ("A", c_vp), ("B", c_vp), ("C", c_vp), ("D", c_vp),
        ("z", c_vp), ("dt_bias", c_vp), ("out", c_vp), ("state_batch_indices", c_vp),
        ("batch", c_i32), ("nheads", c_i32), ("dim", c_i32), ("dstate", c_i32), ("ngroups", c_i32),
        ("state_dtype", c_i32), ("x_dtype", c_i32), ("dt_dtype", c_i32), ("bc_dtype", c_i32),
        ("dt_softplus", c_i32), ("device", c_i32),
        ("state_stride", c_i64 * 4), ("x_stride", c_i64 * 3), ("dt_stride", c_i64 * 3),
        ("z_stride", c_i64 * 3), ("out_stride", c_i64 * 3), ("A_stride", c_i64 * 3),
        ("B_stride", c_i64 * 3), ("C_stride", c_i64 * 3), ("D_stride", c_i64 * 2),
        ("dt_bias_stride", c_i64 * 2),
    ]


class SsdArgs(ctypes.Structure):
    _fields_ = [
        ("x", c_vp), ("dt", c_vp), ("A", c_vp), ("B", c_vp), ("C", c_vp), ("D", c_vp), ("z", c_vp),
        ("dt_bias", c_vp), ("seq_idx", c_vp), ("initial_states", c_vp), ("out", c_vp),
        ("final_states", c_vp), ("range_decay", c_vp), ("scratch", c_vp), ("scratch_bytes", ctypes.c_size_t),
        ("batch", c_i32), ("seqlen", c_i32), ("nheads", c_i32), ("headdim", c_i32), ("ngroups", c_i32),
        ("dstate", c_i32), ("chunk_size", c_i32), ("io_dtype", c_i32), ("dt_dtype", c_i32),
        ("dt_softplus", c_i32), ("D_has_hdim", c_i32), ("dt_min", c_f), ("dt_max", c_f),
        ("phases", c_i32), ("device", c_i32),
        ("x_stride", c_i64 * 3), ("z_stride", c_i64 * 3), ("out_stride", c_i64 * 3),
        ("dt_stride", c_i64 * 3), ("B_stride", c_i64 * 3), ("C_stride", c_i64 * 3),
        ("cu_seqlens", c_vp), ("varlen_states", c_vp), ("num_seqs", c_i32), ("reserved_", c_i32),
    ]


class Conv1dArgs(ctypes.Structure):
    _fields_ = [
        ("x", c_vp), ("weight", c_vp), ("bias", c_vp), ("seq_idx", c_vp), ("initial_states", c_vp), ("final_states", c_vp),
        ("out", c_vp),
        ("batch", c_i32), ("dim", c_i32), ("seqlen", c_i32), ("width", c_i32), ("io_dtype", c_i32), ("w_dtype", c_i32),
        ("activation", c_i32), ("device", c_i32),
        ("x_stride", c_i64 * 3), ("out_stride", c_i64 * 3), ("init_stride", c_i64 * 3), ("final_stride", c_i64 * 3),
    ]


class Conv1dUpdateArgs(ctypes.Structure):
    _fields_ = [
        ("x", c_vp), ("weight", c_vp), ("bias", c_vp), ("conv_state", c_vp), ("out", c_vp),
        ("batch", c_i32), ("dim", c_i32), ("width", c_i32), ("state_len", c_i32), ("io_dtype", c_i32), ("w_dtype", c_i32),
        ("activation", c_i32), ("device", c_i32),
        ("x_stride", c_i64 * 2), ("out_stride", c_i64 * 2), ("state_stride", c_i64 * 3),
    ]


class RmsNormArgs(ctypes.Structure):
    _fields_ = [
        ("x", c_vp), ("z", c_vp), ("weight", c_vp), ("bias", c_vp), ("out", c_vp),
        ("nrows", c_i64), ("ncols", c_i32), ("group_size", c_i32), ("io_dtype", c_i32), ("w_dtype", c_i32),
        ("norm_before_gate", c_i32), ("eps", c_f), ("device", c_i32), ("reserved_", c_i32),
        ("x_stride", c_i64), ("z_stride", c_i64), ("out_stride", c_i64),
    ]


# every symbol include/mamba_b200.h declares, with its prototype
_PROTOTYPES = {
    "mb200_version": (ctypes.c_int, []),
    "mb200_last_error": (ctypes.c_char_p, []),
    "mb200_selective_scan_fwd": (ctypes.c_int, [ctypes.POINTER(ScanArgs), c_vp]),
    "mb200_scan_scratch_bytes": (ctypes.c_int, [ctypes.POINTER(ScanArgs), ctypes.POINTER(ctypes.c_size_t)]),
    "mb200_scan_status": (ctypes.c_int, [c_i32, ctypes.POINTER(c_i32)]),
    "mb200_scan_bwd_scratch_bytes": (ctypes.c_int, [ctypes.POINTER(ScanBwdArgs), ctypes.POINTER(ctypes.c_size_t)]),
    "mb200_selective_scan_bwd": (ctypes.c_int, [ctypes.POINTER(ScanBwdArgs), c_vp]),
    "mb200_selective_state_update": (ctypes.c_int, [ctypes.POINTER(SsuArgs), c_vp]),
    "mb200_ssd_scratch_bytes": (ctypes.c_int, [ctypes.POINTER(SsdArgs), ctypes.POINTER(ctypes.c_size_t)]),
    "mb200_ssd_chunk_scan_fwd": (ctypes.c_int, [ctypes.POINTER(SsdArgs), c_vp]),
    "mb200_ssd_chunk_scan_fwd_static": (ctypes.c_int, [ctypes.POINTER(SsdArgs), c_vp]),
    "mb200_ssd_static_status": (ctypes.c_int, [ctypes.POINTER(SsdArgs), ctypes.POINTER(c_i32)]),
    "mb200_ssd_fold_state": (ctypes.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_vp]),
    "mb200_ssd_fold_ranges": (ctypes.c_int, [c_vp, c_i64, c_i32, c_i32, c_vp, c_i64, c_i64, c_i32, c_vp]),
    "mb200_causal_conv1d_fwd": (ctypes.c_int, [ctypes.POINTER(Conv1dArgs), c_vp]),
    "mb200_causal_conv1d_update": (ctypes.c_int, [ctypes.POINTER(Conv1dUpdateArgs), c_vp]),
    "mb200_rmsnorm_gated_fwd": (ctypes.c_int, [ctypes.POINTER(RmsNormArgs), c_vp]),
}
EXPORTED_SYMBOLS = tuple(_PROTOTYPES)

_lib = None


def lib():
    """The loaded shared library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mamba_b200._build` "
                "(nvcc, sm_100a). mamba_b200 has no other execution path.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[t]
    except KeyError:
        raise RuntimeError(f"mamba_b200 supports float32, float16 and bfloat16, not {t}") from None


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def set_strides(field, t, n):
    for i in range(n):
        field[i] = t.stride(i)


def check(rc: int):
    """Turns a C-ABI status into the exception the reference would have raised."""
    if rc == OK:
        return
    msg = lib().mb200_last_error().decode("utf-8", "replace")
    if rc == ERR_BAD_ARG:
        raise AssertionError(msg)
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"mamba_b200 error {rc}: {msg}")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mamba_b200 runs on CUDA tensors only (there is no CPU path)")


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
