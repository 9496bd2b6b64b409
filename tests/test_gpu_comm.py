"""The library's own communicator (akgb_comm): argument checks on the CPU, the all-reduce of partial outputs on one GPU
(a one-rank communicator) and across two GPUs where the box has them."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from akg_b200 import _capi


def test_comm_argument_checks():
    lib = _capi.load()
    small = ctypes.create_string_buffer(16)
    assert lib.akgb_comm_unique_id(small, 16) == _capi.AKGB_INVALID_ARG
    assert lib.akgb_comm_unique_id(None, 128) == _capi.AKGB_INVALID_ARG
    h = ctypes.c_void_p()
    ident = ctypes.create_string_buffer(128)
    assert lib.akgb_comm_create(ident, 2, 2, -1, ctypes.byref(h)) == _capi.AKGB_INVALID_ARG  # rank outside the world
    assert lib.akgb_comm_create(None, 0, 1, -1, ctypes.byref(h)) == _capi.AKGB_INVALID_ARG
    assert lib.akgb_comm_wrap(None, 0, 1, ctypes.byref(h)) == _capi.AKGB_INVALID_ARG
    lib.akgb_comm_destroy(None)  # accepted


@pytest.mark.gpu
def test_partials_all_reduce_on_a_one_rank_communicator():
    import torch
    from akg_b200 import FusedKernel, descs
    from akg_b200.sharding import Communicator
    comm = Communicator(Communicator.unique_id(), 0, 1, 0)
    # compiled as rank 0 of 2: the output is a partial over this rank's 256 of 512 rows
    k = FusedKernel(descs.reduce_sum_axis0(512, 300), device=0, shard_rank=0, shard_world=2)
    assert k.outputs[0].shard_kind == _capi.SHARD_PARTIAL_SUM and k.inputs[0].shape == (256, 300)
    x = torch.randn(256, 300, device="cuda")
    out = torch.empty(300, device="cuda")
    comm.launch_sharded(k, [x, out])
    torch.cuda.synchronize()
    torch.testing.assert_close(out.double().cpu(), x.double().sum(0).cpu(), rtol=1e-5, atol=1e-4)
    # a kernel without partial outputs: the exchange step is empty
    k2 = FusedKernel(descs.gelu_chain([4, 8, 64]), device=0)
    ins = [torch.randn(t.shape, device="cuda").half() for t in k2.inputs]
    o2 = torch.empty(k2.outputs[0].shape, device="cuda")
    comm.launch_sharded(k2, ins + [o2])
    torch.cuda.synchronize()
    assert bool(torch.isfinite(o2).all())
    comm.close()


@pytest.mark.gpu
def test_two_ranks_reduce_through_the_communicator():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29641", os.path.join(here, "comm_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "COMM_OK" in r.stdout
