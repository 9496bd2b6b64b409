"""ctypes binding of ``include/akgb.h`` — the only way Python reaches the kernels.

There is no Python or CPU implementation behind this module: if the shared
library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libakgb.so"

AKGB_OK = 0
AKGB_INVALID_JSON = 1
AKGB_UNSUPPORTED = 2
AKGB_INVALID_ARG = 3
AKGB_CUDA_ERROR = 4
AKGB_MISALIGNED = 5
AKGB_DEVICE_TIMEOUT = 6
AKGB_TOO_LARGE = 7

STATUS_NAMES = {
    0: "AKGB_OK", 1: "AKGB_INVALID_JSON", 2: "AKGB_UNSUPPORTED", 3: "AKGB_INVALID_ARG",
    4: "AKGB_CUDA_ERROR", 5: "AKGB_MISALIGNED", 6: "AKGB_DEVICE_TIMEOUT", 7: "AKGB_TOO_LARGE", 8: "AKGB_OUT_OF_RANGE",
}

# akgb_dtype code -> numpy dtype name
DTYPE_NAMES = {0: "bool", 1: "int8", 2: "int16", 3: "int32", 4: "int64",
               5: "float16", 6: "float32", 7: "float64", 8: "bfloat16"}

SHARD_REPLICATED, SHARD_SPLIT_AXIS0, SHARD_PARTIAL_SUM, SHARD_PARTIAL_MAX, SHARD_PARTIAL_MIN, SHARD_PARTIAL_PROD = range(6)

EXCHANGE_NAMES = {0: "none", 1: "nccl", 2: "peer-kernel", 3: "in-reduction"}

AKGB_MAX_RANK = 8
AKGB_FLAG_NO_JIT = 1
AKGB_FLAG_FOLD_IN_LAUNCH = 2
AKGB_FLAG_STAGE_LONG_ROWS = 4


class TensorDesc(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 64),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("shape", ctypes.c_int64 * AKGB_MAX_RANK),
        ("nbytes", ctypes.c_int64),
        ("is_output", ctypes.c_int32),
        ("shard_kind", ctypes.c_int32),
        ("written_in_place", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class Options(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("shard_rank", ctypes.c_int32),
        ("shard_world", ctypes.c_int32),
        ("flags", ctypes.c_int32),
    ]


class AkgbError(RuntimeError):
    """A C-ABI call returned a status other than AKGB_OK."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class UnsupportedError(AkgbError):
    """The fused region is valid but no kernel template covers it."""


_lib = None

COMM_ID_BYTES = 128
COMM_HANDLE_BYTES = 64

# every symbol include/akgb.h declares: (name, restype, argtypes)
_vp = ctypes.c_void_p
_SIGNATURES = [
    ("akgb_compile", ctypes.c_int, [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(Options), ctypes.POINTER(_vp)]),
    ("akgb_release", None, [_vp]),
    ("akgb_num_tensors", ctypes.c_int32, [_vp]),
    ("akgb_num_inputs", ctypes.c_int32, [_vp]),
    ("akgb_tensor_info", ctypes.c_int, [_vp, ctypes.c_int32, ctypes.POINTER(TensorDesc)]),
    ("akgb_workspace_size", ctypes.c_size_t, [_vp]),
    ("akgb_launch_count", ctypes.c_int32, [_vp]),
    ("akgb_launch", ctypes.c_int, [_vp, ctypes.POINTER(_vp), _vp, ctypes.c_size_t, _vp]),
    ("akgb_bind_shapes", ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_int64), ctypes.c_size_t,
                                         ctypes.POINTER(ctypes.c_size_t)]),
    ("akgb_launch_dynamic", ctypes.c_int, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_int64), ctypes.c_size_t,
                                            _vp, ctypes.c_size_t, _vp]),
    ("akgb_run_host", ctypes.c_int, [_vp, ctypes.POINTER(_vp)]),
    ("akgb_profile_host", ctypes.c_int, [_vp, ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32,
                                          ctypes.POINTER(ctypes.c_double)]),
    ("akgb_kernel_meta", ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]),
    ("akgb_prepare", ctypes.c_int, [_vp]),
    ("akgb_export_kernel", ctypes.c_int, [_vp, ctypes.c_char_p]),
    ("akgb_comm_unique_id", ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t]),
    ("akgb_comm_create", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                        ctypes.POINTER(ctypes.c_void_p)]),
    ("akgb_comm_wrap", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                      ctypes.POINTER(ctypes.c_void_p)]),
    ("akgb_comm_destroy", None, [ctypes.c_void_p]),
    ("akgb_comm_create_local", ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]),
    ("akgb_comm_set_peer_exchange", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
    ("akgb_comm_exchange_handle", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]),
    ("akgb_comm_attach_peers", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]),
    ("akgb_comm_set_timeout_ms", ctypes.c_int, [ctypes.c_void_p, ctypes.c_double]),
    ("akgb_comm_set_exchange_in_reduction", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
    ("akgb_allreduce_partials", ctypes.c_int, [_vp, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]),
    ("akgb_launch_sharded", ctypes.c_int, [_vp, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p,
                                           ctypes.c_size_t, ctypes.c_void_p]),
    ("akgb_sharded_exchange_kind", ctypes.c_int32, [_vp, ctypes.c_void_p]),
    ("akgb_set_cache_dir", ctypes.c_int, [ctypes.c_char_p]),
    ("akgb_jit_cache_stats", ctypes.c_int, [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    ("akgb_dump_jit_source", ctypes.c_int, [_vp, ctypes.c_int32, ctypes.c_char_p, ctypes.c_size_t,
                                             ctypes.POINTER(ctypes.c_size_t)]),
    ("akgb_kernel_class", ctypes.c_char_p, [_vp]),
    ("akgb_kernel_bytes", ctypes.c_int64, [_vp]),
    ("akgb_kernel_flops", ctypes.c_int64, [_vp]),
    ("akgb_check_device_error", ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_uint32)]),
    ("akgb_checked_shrink_for_test", None, [ctypes.c_int]),
    ("akgb_reduce_sum_axis0_f32_noalloc", ctypes.c_int, [_vp, _vp, ctypes.c_int64, ctypes.c_int64, _vp]),
    ("akgb_last_error", ctypes.c_char_p, []),
    ("akgb_version", ctypes.c_char_p, []),
]


def load() -> ctypes.CDLL:
    """Load ``libakgb.so`` (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("AKGB_LIBRARY", LIB_PATH))
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m akg_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(str(path))
    for name, restype, argtypes in _SIGNATURES:
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    if status == AKGB_OK:
        return
    msg = load().akgb_last_error().decode("utf-8", "replace")
    if status == AKGB_UNSUPPORTED:
        raise UnsupportedError(status, msg)
    raise AkgbError(status, msg)
