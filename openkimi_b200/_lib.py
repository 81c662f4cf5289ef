"""ctypes binding of ``libkda_b200.so`` (the C ABI declared in include/kda_b200.h).

There is no fallback: if the library is missing or fails to load, every op raises.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libkda_b200.so")

DTYPE_F32, DTYPE_BF16 = 0, 1
FLAG_QK_L2NORM, FLAG_GATE, FLAG_BETA_SIGMOID, FLAG_STATE_V_FIRST, FLAG_FORCE_SIMT = 1, 2, 4, 8, 16
FLAG_NO_SAVE = 1024
FLAG_ROW_COPIES = 2048
CHUNK = 64
ERR_DEVICE_WAIT = 7


class KdaParams(C.Structure):
    """Field-for-field mirror of ``struct KdaParams`` in include/kda_b200.h."""

    _fields_ = [
        ("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("dk", C.c_int32), ("dv", C.c_int32),
        ("N", C.c_int32), ("NT", C.c_int32), ("dtype", C.c_int32), ("flags", C.c_int32),
        ("scale", C.c_float), ("guard_span", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("h0", C.c_void_p),
        ("cu_seqlens", C.c_void_p), ("chunk_seq", C.c_void_p), ("seq_chunk_off", C.c_void_p),
        ("o", C.c_void_p), ("ht", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("grad_o", C.c_void_p), ("grad_ht", C.c_void_p),
        ("grad_q", C.c_void_p), ("grad_k", C.c_void_p), ("grad_v", C.c_void_p), ("grad_g", C.c_void_p),
        ("grad_beta", C.c_void_p), ("grad_A_log", C.c_void_p), ("grad_dt_bias", C.c_void_p),
        ("grad_h0", C.c_void_p),
        ("bwd_scratch", C.c_void_p), ("bwd_scratch_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("conv_q", C.c_void_p), ("conv_k", C.c_void_p), ("conv_v", C.c_void_p), ("conv_ksize", C.c_int32),
        ("chunk_tab", C.c_void_p),
        ("status_host", C.c_void_p),
        ("grad_conv_q", C.c_void_p), ("grad_conv_k", C.c_void_p), ("grad_conv_v", C.c_void_p),
    ]


EXPORTS = {
    "kda_abi_version": (C.c_int, []),
    "kda_guard_version": (C.c_int, []),
    "kda_guard_max_span": (C.c_float, []),
    "kda_guard_dot_precision": (C.c_char_p, []),
    "kda_status_string": (C.c_char_p, [C.c_int]),
    "kda_status_publish": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "kda_last_cuda_error": (C.c_char_p, []),
    "kda_profile_begin": (C.c_int, [C.c_int]),
    "kda_profile_read": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.c_int]),
    "kda_guarded_diagonal_tiles": (C.c_int, [C.c_void_p] * 10 + [C.c_int, C.c_float, C.c_void_p]),
    "kda_gate_tile_spans": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int32] * 5 + [C.c_void_p]),
    "kda_selftest_mma": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 12 + [C.c_void_p, C.c_void_p]),
    "kda_selftest_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "kda_workspace_bytes": (C.c_int, [C.POINTER(KdaParams), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "kda_fwd": (C.c_int, [C.POINTER(KdaParams), C.c_void_p]),
    "kda_bwd": (C.c_int, [C.POINTER(KdaParams), C.c_void_p]),
    "kda_recurrent_step": (C.c_int, [C.c_void_p] * 10 + [C.c_int32] * 6 + [C.c_float, C.c_void_p, C.c_void_p]),
    "kda_short_conv_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                     C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "kda_short_conv_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     C.c_void_p, C.c_int32, C.c_void_p]),
    "kda_short_conv_bwd_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                            C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                            C.c_void_p]),
    "kda_norm_gate_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_int32, C.c_float, C.c_int32, C.c_void_p]),
    "kda_norm_gate_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_float,
                                    C.c_int32, C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and declare the signatures of every export."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m openkimi_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the KDA kernels.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.kda_status_string(status).decode()
        extra = lib.kda_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed: {msg}" + (f" ({extra})" if extra and status == 6 else ""))
