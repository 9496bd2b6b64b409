"""ctypes loader of the C restatement in ``cpu_ref.c`` — test infrastructure and
timed CPU baseline only (see the header of ``cpu_ref.c``)."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "libakg_cpu_ref.so"
_lib = None


def build() -> Path:
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return LIB


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.akg_ref_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(load().akg_ref_num_threads())


def use_all_host_threads() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (not to an inherited OMP_NUM_THREADS)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    fn = load().akg_ref_set_num_threads
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int]
    return int(fn(n))


def call(name: str, tensors, dims, scal=(), variant: str = "r1"):
    """Runs ``akg_ref_<name>_<variant>(void** tensors, const int64_t* dims, const double* scal)``."""
    fn = getattr(load(), f"akg_ref_{name}_{variant}")
    fn.restype = None
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.ctypes.data if t is not None else None for t in tensors])
    d = (ctypes.c_int64 * max(1, len(dims)))(*dims)
    s = (ctypes.c_double * max(1, len(scal)))(*scal)
    fn(ptrs, d, s)


def layernorm(x, gamma, beta, eps=1e-5, variant="r1"):
    rows, cols = x.shape
    y = np.empty_like(x)
    mean = np.empty(rows, np.float32)
    var = np.empty(rows, np.float32)
    call("layernorm_f32", [x, gamma, beta, y, mean, var], [rows, cols], [1.0 / cols, eps], variant)
    return y, mean, var


def gelu_chain(x, bias, y, consts=(0.044715, 0.7978845608, 0.5, 1.0), variant="r1"):
    out = np.empty(x.shape, np.float32)
    call("gelu_chain_f16", [x, bias, y, out], [x.size, bias.size], list(consts), variant)
    return out


def softmax(scores, mask, scale, variant="r1"):
    cols = scores.shape[-1]
    rows = scores.size // cols
    out = np.empty_like(scores)
    call("softmax_f16", [scores, mask, out], [rows, cols, mask.size // cols], [scale], variant)
    return out


def reduce_sum_axis0(x, variant="r1"):
    out = np.empty(x.shape[1], np.float32)
    call("reduce_sum_axis0_f32", [x, out], list(x.shape), [], variant)
    return out


def reduce_max_all(x, variant="r1"):
    out = np.empty(1, np.float32)
    call("reduce_max_all_f32", [x, out], [x.size], [], variant)
    return out


def matmul_bias_relu(a, b, bias, variant="r1"):
    """a, b, bias: bfloat16 arrays (ml_dtypes) or their uint16 views; returns uint16 bits of bf16."""
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), np.uint16)
    call("matmul_bias_relu_bf16", [a.view(np.uint16), b.view(np.uint16), bias.view(np.uint16), out], [m, k, n], [],
         variant)
    return out


def transpose4(x, perm, variant="r1"):
    assert x.ndim == 4 and x.dtype.itemsize == 2
    out = np.empty([x.shape[p] for p in perm], x.dtype)
    call("transpose4_b2", [x.view(np.uint16), out.view(np.uint16)], list(x.shape) + list(perm), [], variant)
    return out
