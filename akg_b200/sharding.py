"""Host-side plumbing of leading-axis sharding over the GPUs of one box.

A fused op compiled with ``shard_rank``/``shard_world`` (see ``akgb_options``) reports, per argument, whether
the rank passes its slice of axis 0, the whole tensor, or receives a per-rank partial that must be all-reduced.
The reference has no multi-device notion (AKG compiles single kernels); this layer is what a data-parallel
caller needs around the kernels: slice, launch, all-reduce the partials.  The only collective is an all-reduce
of small partial results (NCCL on GPUs, gloo in CPU tests), and only when a reduction runs over the split axis.
"""
from __future__ import annotations

from typing import Sequence

from . import _capi


def slice_for_rank(kernel, global_arrays: Sequence, rank: int, world: int) -> list:
    """Cuts the GLOBAL input arrays/tensors down to what rank `rank` passes to its kernel."""
    if len(global_arrays) != kernel.num_inputs:
        raise ValueError(f"expected {kernel.num_inputs} inputs, got {len(global_arrays)}")
    out = []
    for a, d in zip(global_arrays, kernel.inputs):
        if d.shard_kind == _capi.SHARD_SPLIT_AXIS0:
            n = d.shape[0]
            if a.shape[0] != n * world:
                raise ValueError(f"input '{d.name}': axis 0 is {a.shape[0]}, expected {n * world}")
            out.append(a[rank * n:(rank + 1) * n])
        else:
            out.append(a)
    return out


def reduce_ops():
    import torch.distributed as dist
    return {_capi.SHARD_PARTIAL_SUM: dist.ReduceOp.SUM, _capi.SHARD_PARTIAL_MAX: dist.ReduceOp.MAX,
            _capi.SHARD_PARTIAL_MIN: dist.ReduceOp.MIN, _capi.SHARD_PARTIAL_PROD: dist.ReduceOp.PRODUCT}


def all_reduce_partials(kernel, outputs: Sequence, group=None) -> None:
    """All-reduces, in place, every output the kernel marks as a per-rank partial (torch tensors)."""
    import torch.distributed as dist
    ops = reduce_ops()
    for t, d in zip(outputs, kernel.outputs):
        if d.shard_kind in ops:
            dist.all_reduce(t, op=ops[d.shard_kind], group=group)


def gather_split_outputs(kernel, outputs: Sequence, world: int, group=None) -> list:
    """Full outputs on every rank: split outputs are all-gathered along axis 0, the rest passed through."""
    import torch
    import torch.distributed as dist
    res = []
    for t, d in zip(outputs, kernel.outputs):
        if d.shard_kind == _capi.SHARD_SPLIT_AXIS0:
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous(), group=group)
            res.append(torch.cat(parts, dim=0))
        else:
            res.append(t)
    return res


class Communicator:
    """``akgb_comm``: the library's own NCCL communicator for the exchange step, one per process (one process per GPU).

    `Communicator.from_process_group()` does the rendezvous over an initialised ``torch.distributed`` group (rank 0
    creates the id, a broadcast carries its 128 bytes); after that the data path does not go through torch:
    `launch_sharded` enqueues the kernel and the all-reduce of its partial outputs on one stream."""

    def __init__(self, id_bytes: bytes | None, rank: int, world: int, device: int = -1):
        """`id_bytes` None: a communicator without NCCL (``akgb_comm_create_local``), peer-memory exchange only."""
        import ctypes
        self._lib = _capi.load()
        self._handle = ctypes.c_void_p()
        if id_bytes is None:
            _capi.check(self._lib.akgb_comm_create_local(rank, world, device, ctypes.byref(self._handle)))
        else:
            buf = ctypes.create_string_buffer(bytes(id_bytes), _capi.COMM_ID_BYTES)
            _capi.check(self._lib.akgb_comm_create(buf, rank, world, device, ctypes.byref(self._handle)))
        self.rank, self.world = rank, world
        self.peer_exchange = False

    def attach_loopback(self):
        """Peer-memory exchange with every slot owner mapped to this rank's own buffer (single-rank use, tests)."""
        _capi.check(self._lib.akgb_comm_attach_peers(self._handle, None, 0))
        self.peer_exchange = True

    def disable_peer_exchange(self):
        """Back to NCCL for every partial (all ranks must do the same)."""
        _capi.check(self._lib.akgb_comm_set_peer_exchange(self._handle, 0))
        self.peer_exchange = False

    def restart_peer_exchange(self):
        """After a bounded wait ran out (AKGB_DEVICE_TIMEOUT): clears the refusal and restarts the call counters.
        Every rank must call it, and the ranks must synchronise before their next sharded launch."""
        _capi.check(self._lib.akgb_comm_set_peer_exchange(self._handle, 1))
        self.peer_exchange = True

    def exchange_kind(self, kernel) -> str:
        """How the partial outputs of `kernel` travel with this communicator as it is set up now:
        'none', 'nccl', 'peer-kernel' (one exchange kernel after the launch) or 'in-reduction' (the reduction's own
        launch completes the exchange)."""
        return _capi.EXCHANGE_NAMES[int(self._lib.akgb_sharded_exchange_kind(kernel._handle, self._handle))]

    def set_exchange_in_reduction(self, enabled: bool):
        """Whether reductions complete the exchange in their own launch (all ranks must choose the same)."""
        _capi.check(self._lib.akgb_comm_set_exchange_in_reduction(self._handle, 1 if enabled else 0))

    def set_timeout_ms(self, ms: float):
        _capi.check(self._lib.akgb_comm_set_timeout_ms(self._handle, float(ms)))

    def enable_peer_exchange(self, group=None) -> bool:
        """Maps the exchange buffers of all ranks of the (initialised) process group into one another; small float32
        partials then go through one kernel over NVLink instead of NCCL.  All ranks end up on the same path: if the
        mapping fails anywhere it is turned off everywhere.  Returns whether it is on."""
        import ctypes
        import torch
        import torch.distributed as dist
        on_gpu = dist.get_backend(group) == "nccl"
        dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
        h = ctypes.create_string_buffer(_capi.COMM_HANDLE_BYTES)
        ok = self._lib.akgb_comm_exchange_handle(self._handle, h, _capi.COMM_HANDLE_BYTES) == _capi.AKGB_OK
        mine = torch.frombuffer(bytearray(h.raw), dtype=torch.uint8).to(dev)
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=group)
        blob = b"".join(p.cpu().numpy().tobytes() for p in parts)
        if ok:
            ok = self._lib.akgb_comm_attach_peers(self._handle, blob, len(blob)) == _capi.AKGB_OK
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.peer_exchange = bool(flag.item())
        if ok and not self.peer_exchange:
            self._lib.akgb_comm_set_peer_exchange(self._handle, 0)
        return self.peer_exchange

    @staticmethod
    def unique_id() -> bytes:
        import ctypes
        buf = ctypes.create_string_buffer(_capi.COMM_ID_BYTES)
        _capi.check(_capi.load().akgb_comm_unique_id(buf, _capi.COMM_ID_BYTES))
        return buf.raw

    @classmethod
    def from_process_group(cls, device: int = -1, group=None):
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        on_gpu = dist.get_backend(group) == "nccl"
        dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
        t = torch.zeros(_capi.COMM_ID_BYTES, dtype=torch.uint8, device=dev)
        if rank == 0:
            t.copy_(torch.frombuffer(bytearray(cls.unique_id()), dtype=torch.uint8))
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(bytes(t.cpu().numpy().tobytes()), rank, world, device)

    def close(self):
        if getattr(self, "_handle", None) and self._handle.value:
            self._lib.akgb_comm_destroy(self._handle)
            self._handle.value = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def launch_sharded(self, kernel, tensors: Sequence, stream=None):
        """``akgb_launch_sharded`` on contiguous torch CUDA tensors (inputs then outputs)."""
        import ctypes
        import torch
        ws_ptr = 0
        if kernel.workspace_size:
            if kernel._workspace is None or kernel._workspace.device != tensors[0].device:
                kernel._workspace = torch.empty(kernel.workspace_size + 256, dtype=torch.uint8, device=tensors[0].device)
            ws_ptr = (kernel._workspace.data_ptr() + 255) // 256 * 256
        s = stream if stream is not None else torch.cuda.current_stream(tensors[0].device)
        ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        _capi.check(self._lib.akgb_launch_sharded(kernel._handle, self._handle, ptrs, ctypes.c_void_p(ws_ptr),
                                                  kernel.workspace_size, ctypes.c_void_p(s.cuda_stream)))
