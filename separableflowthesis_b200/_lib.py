"""ctypes binding of the C ABI in ``include/sepflow_b200.h``.

There is no fallback: if the CUDA library has not been built, importing the ops fails with a
message that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "csrc", "libsepflow_b200.so")

SFB_OK = 0
SFB_ERR_INVALID_ARGUMENT = 1
SFB_ERR_UNSUPPORTED_SHAPE = 2
SFB_ERR_WORKSPACE_TOO_SMALL = 3
SFB_ERR_CUDA = 4
SFB_ERR_DEVICE_TIMEOUT = 5

OP_MAX_AVG_FORWARD = 0
OP_COMPRESSION_FORWARD = 1
OP_MAX_ARGMAX_AVG_BACKWARD = 2
OP_COMPRESSION_BACKWARD = 3
OP_CORR_VOLUME = 4
OP_SEPARATION_BACKWARD = 5
OP_MAX_AVG_FORWARD_CF = 6
OP_COMPRESSION_CF = 7
OP_SEPARATION_FEATURE_BACKWARD_CF = 8
OP_SEPARATION_LEVEL_FORWARD = 9
OP_SEPARATION_LEVEL_BACKWARD = 10

# Every symbol include/sepflow_b200.h declares.
EXPORTED_SYMBOLS = (
    "sfb_workspace_bytes", "sfb_max_avg_forward", "sfb_max_argmax_avg_forward",
    "sfb_max_argmax_avg_backward", "sfb_compression_forward", "sfb_compression_backward",
    "sfb_corr_volume", "sfb_device_status", "sfb_status_string", "sfb_last_error", "sfb_version",
    "sfb_kernel_timing_enable", "sfb_kernel_timing_count", "sfb_kernel_timing_read",
    "sfb_max_avg_forward_static", "sfb_static_scratch_bytes", "sfb_static_device_status", "sfb_separation_backward",
    "sfb_compression_attention_backward", "sfb_separation_feature_backward",
    "sfb_max_argmax_avg_forward_cf", "sfb_compression_forward_cf", "sfb_compression_attention_backward_cf",
    "sfb_separation_feature_backward_cf", "sfb_attention_forward", "sfb_attention_backward_workspace_bytes",
    "sfb_attention_backward", "sfb_separation_level_forward", "sfb_separation_level_backward",
    "sfb_separation_level_forward_fmaps", "sfb_separation_level_backward_fmaps",
    "sfb_upsample_displacement", "sfb_upsample_displacement_backward", "sfb_lookup_pyramid_bytes",
    "sfb_set_sweep_operands", "sfb_get_sweep_operands", "sfb_lookup_build_pyramid", "sfb_lookup_forward", "sfb_lookup_backward",
    "sfb_lookup4d_forward", "sfb_lookup4d_backward", "sfb_debug_wait_timeout",
)


class SfbShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "H1", "W1", "H2", "W2", "C", "Kc")]


_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and declare the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m separableflowthesis_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these ops)")
    lib = ctypes.CDLL(LIB_PATH)
    P, SZ, SH = ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(SfbShape)
    tail = [SH, P, SZ, P]  # shape, workspace, workspace_bytes, stream
    lib.sfb_workspace_bytes.restype = SZ
    lib.sfb_workspace_bytes.argtypes = [ctypes.c_int, SH]
    for name, nptr in (("sfb_max_avg_forward", 4), ("sfb_max_argmax_avg_forward", 6),
                       ("sfb_max_argmax_avg_backward", 8), ("sfb_compression_forward", 6),
                       ("sfb_compression_backward", 10), ("sfb_corr_volume", 3),
                       ("sfb_separation_backward", 14), ("sfb_compression_attention_backward", 6),
                       ("sfb_separation_feature_backward", 12), ("sfb_max_argmax_avg_forward_cf", 6),
                       ("sfb_compression_forward_cf", 6), ("sfb_compression_attention_backward_cf", 6),
                       ("sfb_separation_feature_backward_cf", 12), ("sfb_separation_level_forward", 12),
                       ("sfb_separation_level_backward", 18)):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [P] * nptr + tail
    I32, I64 = ctypes.c_int32, ctypes.c_int64
    lib.sfb_attention_forward.restype = ctypes.c_int
    lib.sfb_attention_forward.argtypes = [P, I64, P, P, P, I32, I32, I32, I32, I32, P]
    lib.sfb_attention_backward_workspace_bytes.restype = SZ
    lib.sfb_attention_backward_workspace_bytes.argtypes = [I32] * 5
    lib.sfb_attention_backward.restype = ctypes.c_int
    lib.sfb_attention_backward.argtypes = [P, I64, P, P, P, P, I64, P, P, P, I32, I32, I32, I32, I32, P, SZ, P]
    lib.sfb_set_sweep_operands.restype = ctypes.c_int
    lib.sfb_set_sweep_operands.argtypes = [ctypes.c_int]
    lib.sfb_get_sweep_operands.restype = ctypes.c_int
    lib.sfb_get_sweep_operands.argtypes = []
    lib.sfb_upsample_displacement.restype = ctypes.c_int
    lib.sfb_upsample_displacement.argtypes = [P, P, I64] + [I32] * 6 + [P]
    lib.sfb_upsample_displacement_backward.restype = ctypes.c_int
    lib.sfb_upsample_displacement_backward.argtypes = [P, I64, P] + [I32] * 6 + [P]
    lib.sfb_lookup_pyramid_bytes.restype = SZ
    lib.sfb_lookup_pyramid_bytes.argtypes = [I32] * 6
    lib.sfb_lookup_build_pyramid.restype = ctypes.c_int
    lib.sfb_lookup_build_pyramid.argtypes = [P, P] + [I32] * 6 + [P]
    lib.sfb_lookup_forward.restype = ctypes.c_int
    lib.sfb_lookup_forward.argtypes = [P, P, P, I64, P] + [I32] * 8 + [P]
    lib.sfb_lookup_backward.restype = ctypes.c_int
    lib.sfb_lookup_backward.argtypes = [P, P, I64, P, P] + [I32] * 8 + [P]
    lib.sfb_lookup4d_forward.restype = ctypes.c_int
    lib.sfb_lookup4d_forward.argtypes = [P, P, P, P, I32, P, P] + [I32] * 5 + [ctypes.c_float, P]
    lib.sfb_lookup4d_backward.restype = ctypes.c_int
    lib.sfb_lookup4d_backward.argtypes = [P, P, P, P, I32, P, P, P, P] + [I32] * 5 + [ctypes.c_float, P]
    lib.sfb_separation_level_forward_fmaps.restype = ctypes.c_int
    lib.sfb_separation_level_forward_fmaps.argtypes = [P, P, ctypes.c_float] + [P] * 6 + [I32, I32] + [P] * 4 + tail
    lib.sfb_separation_level_backward_fmaps.restype = ctypes.c_int
    lib.sfb_separation_level_backward_fmaps.argtypes = [P, P, ctypes.c_float] + [P] * 4 + [I32, I32] + [P] * 12 + tail
    lib.sfb_max_avg_forward_static.restype = ctypes.c_int
    lib.sfb_max_avg_forward_static.argtypes = [P, P, P, P, SH, P]
    lib.sfb_static_scratch_bytes.restype = SZ
    lib.sfb_static_scratch_bytes.argtypes = []
    lib.sfb_static_device_status.restype = ctypes.c_int
    lib.sfb_static_device_status.argtypes = [P, ctypes.POINTER(ctypes.c_int32)]
    lib.sfb_debug_wait_timeout.restype = ctypes.c_int
    lib.sfb_debug_wait_timeout.argtypes = [ctypes.c_uint64, ctypes.c_int]
    lib.sfb_device_status.restype = ctypes.c_int
    lib.sfb_device_status.argtypes = [P, P, ctypes.POINTER(ctypes.c_int32)]
    lib.sfb_status_string.restype = ctypes.c_char_p
    lib.sfb_status_string.argtypes = [ctypes.c_int]
    lib.sfb_last_error.restype = ctypes.c_char_p
    lib.sfb_last_error.argtypes = []
    lib.sfb_version.restype = ctypes.c_int
    lib.sfb_version.argtypes = []
    lib.sfb_kernel_timing_enable.restype = ctypes.c_int
    lib.sfb_kernel_timing_enable.argtypes = [ctypes.c_int]
    lib.sfb_kernel_timing_count.restype = ctypes.c_int
    lib.sfb_kernel_timing_count.argtypes = []
    lib.sfb_kernel_timing_read.restype = ctypes.c_int
    lib.sfb_kernel_timing_read.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                           ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int64)]
    _lib = lib
    return lib


def kernel_timing(enable: bool) -> None:
    """Start (True) or stop (False) a fresh per-kernel timing measurement."""
    load().sfb_kernel_timing_enable(1 if enable else 0)


def kernel_timing_report():
    """[(kernel name, total device ms, launches)] for every kernel that ran since timing was enabled."""
    lib = load()
    rows = []
    for i in range(lib.sfb_kernel_timing_count()):
        name, ms, n = ctypes.c_char_p(), ctypes.c_double(), ctypes.c_int64()
        lib.sfb_kernel_timing_read(i, ctypes.byref(name), ctypes.byref(ms), ctypes.byref(n))
        if n.value:
            rows.append((name.value.decode(), ms.value, n.value))
    return rows
