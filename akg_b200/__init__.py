"""akg_b200 — B200 (sm_100a) kernels behind AKG-MLIR's fused-operator interface.

The input is the MindSpore graph-kernel fused-op description (``.info`` JSON);
the output tensors are the ones AKG-MLIR's GPU lowering + launch path returns.
All computation happens in ``lib/libakgb.so`` (hand-written CUDA, C ABI in
``include/akgb.h``); this package is the thin host-side mirror of the
reference's Python driver.
"""
from ._capi import AkgbError, UnsupportedError  # noqa: F401
from .driver import FusedKernel, MlirDriver, compile_info  # noqa: F401

__all__ = ["FusedKernel", "MlirDriver", "compile_info", "AkgbError", "UnsupportedError"]
