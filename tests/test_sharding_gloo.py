"""The N>1 host path on CPU: two gloo ranks plan their shards through the C ABI, slice the global inputs, produce
their local results (with the CPU oracle standing in for the kernels, which need a GPU), all-reduce the partials
and must reproduce the oracle's result on the unsplit input."""
import json
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from akg_b200 import FusedKernel, descs, sharding
        from helpers import KINDS, make_inputs
        from oracle import akg_oracle as O
        name, gdesc, kinds, local_desc_fn = case
        gdesc = json.loads(gdesc)
        ins = make_inputs(gdesc, 7, kinds)  # same seed on every rank: the global inputs
        k = FusedKernel(gdesc, shard_rank=rank, shard_world=world)
        local_ins = sharding.slice_for_rank(k, ins, rank, world)
        for a, d in zip(local_ins, k.inputs):
            assert tuple(a.shape) == d.shape, (d.name, a.shape, d.shape)
        # the local computation: the same op on the local shapes
        local_desc = eval(local_desc_fn)(descs, world)
        local_out = [torch.from_numpy(np.ascontiguousarray(o)) for o in O.evaluate(local_desc, local_ins)]
        for t, d in zip(local_out, k.outputs):
            assert tuple(t.shape) == d.shape, (d.name, t.shape, d.shape)
        sharding.all_reduce_partials(k, local_out)
        full = sharding.gather_split_outputs(k, local_out, world)
        want = O.evaluate(gdesc, ins, accum="float64")
        for g, w in zip(full, want):
            g = g.numpy()
            if name == "colsum":
                assert np.all(np.abs(g - w) <= 1e-5 * np.abs(ins[0]).sum(axis=0))
            else:
                np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=2e-3, atol=1e-6)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, "FAIL " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


CASES = [
    ("colsum", "reduce_sum_axis0(64, 48)", {}, "lambda d, w: d.reduce_sum_axis0(64 // w, 48)"),
    ("gmax", "reduce_max_all(64, 48)", {}, "lambda d, w: d.reduce_max_all(64 // w, 48)"),
    ("both", "reduce_sum_and_max(64, 48)", {}, "lambda d, w: d.reduce_sum_and_max(64 // w, 48)"),
    ("layernorm", "layernorm(32, 64)", {"gamma": "gamma", "beta": "beta"}, "lambda d, w: d.layernorm(32 // w, 64)"),
    ("softmax", "masked_softmax(4, 16, 32)", {"mask": "causal"}, "lambda d, w: d.masked_softmax(4 // w, 16, 32)"),
    ("gelu", "gelu_chain([8, 4, 64])", {"bias": "normal_small"}, "lambda d, w: d.gelu_chain([8 // w, 4, 64])"),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_two_rank_plan_slice_allreduce(lib, case):
    from akg_b200 import descs
    name, expr, kinds, local_fn = case
    gdesc = json.dumps(eval("descs." + expr))
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, (name, gdesc, kinds, local_fn), q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(r[1] == "ok" for r in results), results
