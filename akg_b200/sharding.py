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
