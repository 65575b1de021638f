"""ctypes binding of libflashlinear_sm100.so (C ABI in include/flashlinear_sm100.h).

There is no fallback: if the library is missing the import fails with an error that says how to
build it, and every call fails loudly when the current device is not an sm_100 GPU.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashlinear_sm100.so")

FLA_ABI_VERSION = 9
FLA_DEBUG_WITHHOLD_FIRST_TILE = 1
FLA_DEBUG_NO_FUSED_SEGMENTS = 2
FLA_DEBUG_FORCE_SINGLE_SWEEP = 4
FLA_MAX_RANKS = 8
FLA_DTYPE_BF16 = 0
FLA_DTYPE_F16 = 1


class FlaTensor(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("stride_b", ctypes.c_int64),
        ("stride_h", ctypes.c_int64),
        ("stride_n", ctypes.c_int64),
    ]


class FlaArgs(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("seqlen", ctypes.c_int32),
        ("dk", ctypes.c_int32),
        ("dv", ctypes.c_int32),
        ("q", FlaTensor),
        ("k", FlaTensor),
        ("v", FlaTensor),
        ("o", FlaTensor),
        ("d_o", FlaTensor),
        ("d_q", FlaTensor),
        ("d_k", FlaTensor),
        ("d_v", FlaTensor),
        ("s_init", ctypes.c_void_p),
        ("s_final", ctypes.c_void_p),
        ("r_init", ctypes.c_void_p),
        ("r_final", ctypes.c_void_p),
        ("s_last", ctypes.c_void_p),
        ("segments", ctypes.c_int32),
        ("segment_states_ready", ctypes.c_int32),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
        ("seg_states", ctypes.c_void_p),
        ("seg_states_bytes", ctypes.c_size_t),
        ("dtype", ctypes.c_int32),
        ("wait_limit_us", ctypes.c_uint32),
        ("debug_flags", ctypes.c_uint32),
    ]


class FlaExchange(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int32),
        ("world", ctypes.c_int32),
        ("reverse", ctypes.c_int32),
        ("epoch", ctypes.c_uint32),
        ("inbox", ctypes.c_void_p * 8),
        ("flags", ctypes.c_void_p * 8),
        ("remote_out", ctypes.c_void_p),
        ("inclusive_out", ctypes.c_void_p),
        ("epoch_counter", ctypes.c_void_p),
        ("wait_limit_us", ctypes.c_uint32),
    ]


EXPORTED_SYMBOLS = (
    "fla_sm100_abi_version",
    "fla_sm100_timeout_records",
    "fla_sm100_strerror",
    "fla_sm100_workspace_bytes",
    "fla_sm100_auto_segments",
    "fla_sm100_seg_states_bytes",
    "fla_sm100_bwd_uses_final_state",
    "fla_sm100_fwd",
    "fla_sm100_bwd",
    "fla_sm100_state",
    "fla_sm100_fwd_static_scratch",
    "fla_sm100_product",
    "fla_sm100_normalize_workspace_bytes",
    "fla_sm100_normalize_fwd",
    "fla_sm100_normalize_bwd_prepare",
    "fla_sm100_normalize_bwd_sweep",
    "fla_sm100_taylor_dims",
    "fla_sm100_taylor_features",
    "fla_sm100_taylor_features_bwd",
    "fla_sm100_pad_rows",
    "fla_sm100_unpad_rows",
    "fla_sm100_exchange_bytes",
    "fla_sm100_exchange_workspace_bytes",
    "fla_sm100_state_exchange",
    "fla_sm100_enable_peer_access",
    "fla_sm100_exchange_alloc",
    "fla_sm100_exchange_open",
    "fla_sm100_exchange_close",
    "fla_sm100_exchange_free",
    "fla_sm100_last_launch_count",
)

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises ImportError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m flashy_linear_attention_b200.build` "
            "(needs nvcc); there is no CPU or PyTorch fallback for these kernels."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.fla_sm100_abi_version.restype = ctypes.c_int
    lib.fla_sm100_timeout_records.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fla_sm100_timeout_records.restype = ctypes.c_int
    lib.fla_sm100_strerror.restype = ctypes.c_char_p
    lib.fla_sm100_strerror.argtypes = [ctypes.c_int]
    lib.fla_sm100_workspace_bytes.restype = ctypes.c_size_t
    lib.fla_sm100_workspace_bytes.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int]
    lib.fla_sm100_auto_segments.restype = ctypes.c_int
    lib.fla_sm100_auto_segments.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int]
    lib.fla_sm100_seg_states_bytes.restype = ctypes.c_size_t
    lib.fla_sm100_seg_states_bytes.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_bwd_uses_final_state.restype = ctypes.c_int
    lib.fla_sm100_bwd_uses_final_state.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_fwd.restype = ctypes.c_int
    lib.fla_sm100_fwd.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_bwd.restype = ctypes.c_int
    lib.fla_sm100_bwd.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_state.restype = ctypes.c_int
    lib.fla_sm100_state.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int]
    lib.fla_sm100_fwd_static_scratch.restype = ctypes.c_int
    lib.fla_sm100_fwd_static_scratch.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_product.restype = ctypes.c_int
    lib.fla_sm100_product.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int]
    for name in ("fla_sm100_pad_rows", "fla_sm100_unpad_rows"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                       ctypes.c_void_p]
    lib.fla_sm100_normalize_workspace_bytes.restype = ctypes.c_size_t
    lib.fla_sm100_normalize_workspace_bytes.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_normalize_fwd.restype = ctypes.c_int
    lib.fla_sm100_normalize_fwd.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_float, ctypes.c_void_p]
    lib.fla_sm100_normalize_bwd_prepare.restype = ctypes.c_int
    lib.fla_sm100_normalize_bwd_prepare.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_void_p, ctypes.c_void_p]
    lib.fla_sm100_normalize_bwd_sweep.restype = ctypes.c_int
    lib.fla_sm100_normalize_bwd_sweep.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_void_p]
    lib.fla_sm100_taylor_dims.restype = ctypes.c_int
    lib.fla_sm100_taylor_dims.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    lib.fla_sm100_taylor_features.restype = ctypes.c_int
    lib.fla_sm100_taylor_features.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                              ctypes.c_void_p]
    lib.fla_sm100_taylor_features_bwd.restype = ctypes.c_int
    lib.fla_sm100_taylor_features_bwd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                  ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    lib.fla_sm100_exchange_bytes.restype = ctypes.c_int
    lib.fla_sm100_exchange_bytes.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int,
                                             ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    lib.fla_sm100_exchange_workspace_bytes.restype = ctypes.c_size_t
    lib.fla_sm100_exchange_workspace_bytes.argtypes = [ctypes.POINTER(FlaArgs)]
    lib.fla_sm100_exchange_alloc.restype = ctypes.c_int
    lib.fla_sm100_exchange_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
    lib.fla_sm100_exchange_open.restype = ctypes.c_int
    lib.fla_sm100_exchange_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.fla_sm100_exchange_close.restype = ctypes.c_int
    lib.fla_sm100_exchange_close.argtypes = [ctypes.c_void_p]
    lib.fla_sm100_exchange_free.restype = ctypes.c_int
    lib.fla_sm100_exchange_free.argtypes = [ctypes.c_void_p]
    lib.fla_sm100_enable_peer_access.restype = ctypes.c_int
    lib.fla_sm100_enable_peer_access.argtypes = [ctypes.c_int]
    lib.fla_sm100_state_exchange.restype = ctypes.c_int
    lib.fla_sm100_state_exchange.argtypes = [ctypes.POINTER(FlaArgs), ctypes.c_int, ctypes.POINTER(FlaExchange)]
    lib.fla_sm100_last_launch_count.restype = ctypes.c_int
    if lib.fla_sm100_abi_version() != FLA_ABI_VERSION:
        raise ImportError("libflashlinear_sm100.so has a different ABI version; rebuild it")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().fla_sm100_strerror(code).decode()
