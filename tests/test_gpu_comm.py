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
def test_peer_memory_exchange_on_one_rank_and_its_bounded_wait():
    """The one-kernel exchange with every slot mapped to this rank's own buffer, then a two-rank communicator whose
    second rank never arrives: the wait runs out, the error word reports it, the output is untouched and the device
    keeps working."""
    import ctypes
    import torch
    from akg_b200 import FusedKernel, descs
    from akg_b200.sharding import Communicator
    lib = _capi.load()
    k = FusedKernel(descs.reduce_sum_axis0(512, 300), device=0, shard_rank=0, shard_world=2)
    x = torch.randn(256, 300, device="cuda")
    want = x.double().sum(0).cpu()
    # one rank: the fold over a single slot returns the partial itself
    solo = Communicator(None, 0, 1, 0)
    solo.attach_loopback()
    out = torch.empty(300, device="cuda")
    for _ in range(3):  # both parities of the exchange buffer
        solo.launch_sharded(k, [x, out])
    torch.cuda.synchronize()
    torch.testing.assert_close(out.double().cpu(), want, rtol=1e-5, atol=1e-4)
    assert k.check_device_error() == 0
    # two ranks, nobody plays rank 1: its flag is never raised
    lonely = Communicator(None, 0, 2, 0)
    lonely.attach_loopback()
    lonely.set_timeout_ms(50.0)
    out2 = torch.full((300,), float("nan"), device="cuda")
    lonely.launch_sharded(k, [x, out2])
    torch.cuda.synchronize()
    word = ctypes.c_uint32(0)
    status = lib.akgb_check_device_error(k._handle, ctypes.byref(word))
    assert status == _capi.AKGB_DEVICE_TIMEOUT and word.value & 256
    torch.testing.assert_close(out2.double().cpu(), want, rtol=1e-5, atol=1e-4)  # the partial, not folded
    assert lonely.exchange_kind(k) == "in-reduction"  # the reduction's own launch carried (and bounded) the exchange
    # once a wait has run out the ranks' call counters may disagree: further exchanges of a multi-rank communicator on
    # this device are refused until the path is restarted (on all ranks)
    with pytest.raises(_capi.AkgbError) as refused:
        lonely.launch_sharded(k, [x, out2])
    assert refused.value.status == _capi.AKGB_DEVICE_TIMEOUT
    lonely.restart_peer_exchange()
    lonely.launch_sharded(k, [x, out2])  # accepted again (and, with nobody playing rank 1, runs out again)
    torch.cuda.synchronize()
    status = lib.akgb_check_device_error(k._handle, ctypes.byref(word))
    assert status == _capi.AKGB_DEVICE_TIMEOUT and word.value & 256
    lonely.disable_peer_exchange()  # clears the refusal as well
    # the same bound inside the exchange kernel that runs after a launch (two reductions produce the partials)
    lonely.restart_peer_exchange()
    kb = FusedKernel(descs.layer_norm_backward(512, 256), device=0, shard_rank=0, shard_world=2)
    assert lonely.exchange_kind(kb) == "peer-kernel"
    ins_b = [torch.randn(t.shape, device="cuda") for t in kb.inputs]
    outs_b = [torch.empty(t.shape, device="cuda") for t in kb.outputs]
    lonely.launch_sharded(kb, ins_b + outs_b)
    torch.cuda.synchronize()
    status = lib.akgb_check_device_error(kb._handle, ctypes.byref(word))
    assert status == _capi.AKGB_DEVICE_TIMEOUT and word.value & 256
    lonely.disable_peer_exchange()
    # the device and the library keep working
    solo.launch_sharded(k, [x, out])
    torch.cuda.synchronize()
    assert k.check_device_error() == 0
    torch.testing.assert_close(out.double().cpu(), want, rtol=1e-5, atol=1e-4)
    # a communicator without NCCL refuses what the exchange cannot carry
    big = FusedKernel(descs.reduce_sum_axis0(512, 32768), device=0, shard_rank=0, shard_world=2)
    xb = torch.randn(256, 32768, device="cuda")
    ob = torch.empty(32768, device="cuda")
    with pytest.raises(_capi.UnsupportedError):
        solo.launch_sharded(big, [xb, ob])
    solo.close()
    lonely.close()


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
