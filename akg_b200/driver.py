"""Host-side mirror of the reference's Python driver for the GPU path.

``MlirDriver(kernel_name, input_file, backend="gpu")`` with ``compile()`` and
``run(input_for_mod, output_indexes)`` has the surface of
``akg-mlir/python/akg_mlir/mlir_driver.py:255-322``; ``run`` takes the same
list the reference harness builds (inputs then output placeholders, numpy
arrays, ``akg-mlir/python/akg_mlir/utils/composite_op_helper.py:645-708``) and
fills the outputs in place, like ``cuda_runtime_exec`` does.

``FusedKernel`` is the object underneath: one compiled description, launchable
on device tensors (``launch``) or host arrays (``run_host``).
"""
from __future__ import annotations

import ctypes
import json
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from . import _capi


@dataclass
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    nbytes: int
    is_output: bool
    shard_kind: int
    written_in_place: bool = False


def _np_dtype(name: str):
    if name == "bfloat16":
        import ml_dtypes
        return np.dtype(ml_dtypes.bfloat16)
    return np.dtype(name)


class FusedKernel:
    """One fused-op description compiled to a launch plan (``akgb_compile``)."""

    def __init__(self, info_json: str | bytes | dict, device: int = -1, shard_rank: int = 0, shard_world: int = 1,
                 flags: int = 0):
        lib = _capi.load()
        if isinstance(info_json, dict):
            info_json = json.dumps(info_json)
        if isinstance(info_json, str):
            info_json = info_json.encode("utf-8")
        self._lib = lib
        self._handle = ctypes.c_void_p()
        opt = _capi.Options(ctypes.sizeof(_capi.Options), device, shard_rank, shard_world, flags)
        _capi.check(lib.akgb_compile(info_json, len(info_json), ctypes.byref(opt), ctypes.byref(self._handle)))
        self.tensors: list[TensorInfo] = []
        for i in range(lib.akgb_num_tensors(self._handle)):
            d = _capi.TensorDesc()
            _capi.check(lib.akgb_tensor_info(self._handle, i, ctypes.byref(d)))
            self.tensors.append(TensorInfo(d.name.decode(), _capi.DTYPE_NAMES[d.dtype],
                                           tuple(d.shape[j] for j in range(d.rank)), int(d.nbytes),
                                           bool(d.is_output), int(d.shard_kind), bool(d.written_in_place)))
        self.num_inputs = lib.akgb_num_inputs(self._handle)
        self.workspace_size = int(lib.akgb_workspace_size(self._handle))
        self.op_class = lib.akgb_kernel_class(self._handle).decode()
        self.bytes = int(lib.akgb_kernel_bytes(self._handle))
        self.flops = int(lib.akgb_kernel_flops(self._handle))
        self.is_dynamic = any(e < 0 for t in self.tensors for e in t.shape)
        self._workspace = None

    # -- lifetime ---------------------------------------------------------------
    def close(self):
        if getattr(self, "_handle", None) and self._handle.value:
            self._lib.akgb_release(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- queries ----------------------------------------------------------------
    @property
    def inputs(self) -> list[TensorInfo]:
        return self.tensors[: self.num_inputs]

    @property
    def outputs(self) -> list[TensorInfo]:
        return self.tensors[self.num_inputs:]

    @property
    def launch_count(self) -> int:
        return int(self._lib.akgb_launch_count(self._handle))

    def meta(self) -> dict:
        """The launch metadata JSON (keys of the reference's ``<kernel>.json``)."""
        need = ctypes.c_size_t(0)
        _capi.check(self._lib.akgb_kernel_meta(self._handle, None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        _capi.check(self._lib.akgb_kernel_meta(self._handle, buf, need.value, ctypes.byref(need)))
        return json.loads(buf.value.decode())

    def jit_source(self, vectorised: bool = True) -> str:
        """CUDA C++ compiled at run time for the first generic elementwise group ('' if none)."""
        need = ctypes.c_size_t(0)
        _capi.check(self._lib.akgb_dump_jit_source(self._handle, int(vectorised), None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        _capi.check(self._lib.akgb_dump_jit_source(self._handle, int(vectorised), buf, need.value, ctypes.byref(need)))
        return buf.value.decode()

    def check_device_error(self) -> int:
        word = ctypes.c_uint32(0)
        _capi.check(self._lib.akgb_check_device_error(self._handle, ctypes.byref(word)))
        return int(word.value)

    def export(self, directory: str) -> None:
        """``akgb_export_kernel``: ``<kernel>.cubin`` + ``<kernel>.json`` for a region that runs as one generated
        kernel (raises ``UnsupportedError`` for the others)."""
        _capi.check(self._lib.akgb_export_kernel(self._handle, str(directory).encode()))

    def prepare(self):
        """``akgb_prepare``: device tables and generated kernels ahead of the first launch (needed before the launches
        are captured into a CUDA graph)."""
        _capi.check(self._lib.akgb_prepare(self._handle))

    # -- execution ----------------------------------------------------------------
    def launch_ptrs(self, ptrs: Sequence[int], workspace_ptr: int = 0, workspace_bytes: int = 0, stream: int = 0):
        """``akgb_launch`` on raw device addresses (inputs then outputs)."""
        arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        _capi.check(self._lib.akgb_launch(self._handle, arr, ctypes.c_void_p(workspace_ptr), workspace_bytes,
                                          ctypes.c_void_p(stream)))

    def launch(self, tensors: Sequence, stream=None):
        """Enqueue on torch CUDA tensors (inputs then outputs), asynchronously.

        torch is used for device memory and streams only; the workspace is a
        torch byte tensor owned by this object.
        """
        import torch
        if len(tensors) != len(self.tensors):
            raise ValueError(f"expected {len(self.tensors)} tensors, got {len(tensors)}")
        if self.is_dynamic:
            return self._launch_dynamic(tensors, stream)
        for t, d in zip(tensors, self.tensors):
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"tensor '{d.name}' must be a contiguous CUDA tensor")
            if t.numel() * t.element_size() != d.nbytes:
                raise ValueError(f"tensor '{d.name}' has {t.numel() * t.element_size()} bytes, expected {d.nbytes}")
        ws_ptr = 0
        if self.workspace_size:
            if self._workspace is None or self._workspace.device != tensors[0].device:
                self._workspace = torch.empty(self.workspace_size + 256, dtype=torch.uint8, device=tensors[0].device)
            ws_ptr = (self._workspace.data_ptr() + 255) // 256 * 256
        s = stream if stream is not None else torch.cuda.current_stream(tensors[0].device)
        self.launch_ptrs([t.data_ptr() for t in tensors], ws_ptr, self.workspace_size, s.cuda_stream)

    def bind_shapes(self, shapes: Sequence[Sequence[int]]) -> int:
        """``akgb_bind_shapes``: plans a dynamic-shape region for these extents; returns the workspace bytes."""
        flat = [int(e) for s in shapes for e in s]
        arr = (ctypes.c_int64 * len(flat))(*flat)
        ws = ctypes.c_size_t(0)
        _capi.check(self._lib.akgb_bind_shapes(self._handle, arr, len(flat), ctypes.byref(ws)))
        return int(ws.value)

    def _launch_dynamic(self, tensors: Sequence, stream=None):
        import torch
        for t, d in zip(tensors, self.tensors):
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"tensor '{d.name}' must be a contiguous CUDA tensor")
            if t.dim() != len(d.shape):
                raise ValueError(f"tensor '{d.name}' has rank {t.dim()}, expected {len(d.shape)}")
        flat = [int(e) for t in tensors for e in t.shape]
        arr = (ctypes.c_int64 * len(flat))(*flat)
        need = ctypes.c_size_t(0)
        _capi.check(self._lib.akgb_bind_shapes(self._handle, arr, len(flat), ctypes.byref(need)))
        ws_ptr = 0
        if need.value:
            if self._workspace is None or self._workspace.numel() < need.value + 256:
                self._workspace = torch.empty(need.value + 256, dtype=torch.uint8, device=tensors[0].device)
            ws_ptr = (self._workspace.data_ptr() + 255) // 256 * 256
        s = stream if stream is not None else torch.cuda.current_stream(tensors[0].device)
        ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        _capi.check(self._lib.akgb_launch_dynamic(self._handle, ptrs, arr, len(flat), ctypes.c_void_p(ws_ptr),
                                                  need.value, ctypes.c_void_p(s.cuda_stream)))

    def _host_ptrs(self, arrays: Sequence[np.ndarray]):
        if len(arrays) != len(self.tensors):
            raise ValueError(f"expected {len(self.tensors)} arrays, got {len(arrays)}")
        for a, d in zip(arrays, self.tensors):
            if not isinstance(a, np.ndarray) or not a.flags["C_CONTIGUOUS"]:
                raise ValueError(f"argument '{d.name}' must be a C-contiguous numpy array")
            if a.nbytes != d.nbytes:
                raise ValueError(f"argument '{d.name}' has {a.nbytes} bytes, expected {d.nbytes}")
        return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])

    def run_host(self, arrays: Sequence[np.ndarray]):
        """``akgb_run_host``: host arrays in, outputs written in place, synchronous."""
        _capi.check(self._lib.akgb_run_host(self._handle, self._host_ptrs(arrays)))

    def profile_host(self, arrays: Sequence[np.ndarray], number: int = 10, repeat: int = 1) -> float:
        """``akgb_profile_host``: average device time of one launch in microseconds."""
        us = ctypes.c_double(0.0)
        _capi.check(self._lib.akgb_profile_host(self._handle, self._host_ptrs(arrays), number, repeat,
                                                ctypes.byref(us)))
        return float(us.value)

    def empty_outputs(self) -> list[np.ndarray]:
        return [np.empty(d.shape, dtype=_np_dtype(d.dtype)) for d in self.outputs]


def compile_info(info_json, **kw) -> FusedKernel:
    return FusedKernel(info_json, **kw)


def set_cache_dir(path: str | None):
    """``akgb_set_cache_dir``: where run-time compiled kernels are kept between processes (None: the environment's
    choice, "": no disk cache)."""
    _capi.check(_capi.load().akgb_set_cache_dir(None if path is None else os.fsencode(path)))


def jit_cache_stats() -> tuple[int, int]:
    """(kernels compiled by this process, kernels loaded from the on-disk cache)."""
    a, b = ctypes.c_uint64(0), ctypes.c_uint64(0)
    _capi.check(_capi.load().akgb_jit_cache_stats(ctypes.byref(a), ctypes.byref(b)))
    return int(a.value), int(b.value)


def get_kernel_meta_path() -> str:
    """Directory of the kernel metadata files, resolved from the same environment variables as the reference
    (``KERNEL_META_DIR``, ``MS_COMPILER_CACHE_PATH``; ``akg-mlir/python/akg_mlir/mlir_driver.py:47-53``)."""
    kernel_meta_dir = os.getenv("KERNEL_META_DIR", default=os.path.expanduser("~/.akg"))
    return os.path.join(os.path.realpath(os.getenv("MS_COMPILER_CACHE_PATH", "")), kernel_meta_dir)


class MlirDriver:
    """Drop-in for the GPU branch of the reference's ``MlirDriver``."""

    def __init__(self, kernel_name: str, input_file: str, output_dir: str = "", dynamic_shape: bool = False,
                 profiling_trails: int = 0, backend: str = "gpu", device: int = -1, **_ignored):
        if backend != "gpu":
            raise RuntimeError("Unsupported backend: " + backend + "!\n")
        self.dynamic_shape = dynamic_shape
        self.kernel_name = kernel_name
        self.input_file = input_file
        self.output_dir = get_kernel_meta_path() if output_dir == "" else str(output_dir)
        self.profiling_trails = profiling_trails
        self.backend = backend
        self.device = device
        self.kernel: FusedKernel | None = None
        self.last_profile_us: float | None = None

    def compile(self):
        with open(self.input_file, "r", encoding="utf-8") as f:
            text = f.read()
        self.kernel = FusedKernel(text, device=self.device)
        # <kernel>.json beside where the reference writes <kernel>.ptx/.json: launch dims, kernelName, sha256 ...
        # (the launch dims are those of the planned template and are refined at the first launch)
        # kernels generated at the first launch are cached there too, as the reference's <kernel>.ptx is
        os.makedirs(self.output_dir, exist_ok=True)
        set_cache_dir(self.output_dir)
        meta = self.kernel.meta()
        # a region that runs as one generated kernel also leaves <kernel>.cubin there: the pair a runtime that loads
        # kernels from the meta directory needs (entry point, launch dims and sha256 then describe that image)
        own_name = json.loads(text).get("op", self.kernel_name)
        try:
            self.kernel.export(self.output_dir)
            with open(os.path.join(self.output_dir, own_name + ".json"), "r", encoding="utf-8") as f:
                meta.update(json.load(f))
        except (_capi.UnsupportedError, OSError):
            pass
        with open(os.path.join(self.output_dir, self.kernel_name + ".json"), "w", encoding="utf-8") as f:
            json.dump(meta, f)

    def run(self, input_for_mod, output_indexes=None):
        if self.kernel is None:
            raise RuntimeError("compile() must be called before run()")
        if self.kernel.is_dynamic:
            # extents come with the arrays (the reference passes them as extra kernel arguments,
            # python/akg_mlir/utils/gen_runtime_code.py:39-58); device memory and copies through torch
            import torch
            dev = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in input_for_mod]
            self.kernel.launch(dev)
            torch.cuda.synchronize()
            for a, t, d in zip(input_for_mod, dev, self.kernel.tensors):
                if d.is_output or d.written_in_place:
                    a[...] = t.cpu().numpy()
        elif self.profiling_trails > 0:
            self.last_profile_us = self.kernel.profile_host(input_for_mod, number=10, repeat=self.profiling_trails)
        else:
            self.kernel.run_host(input_for_mod)
        return input_for_mod
