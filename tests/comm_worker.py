"""Worker of tests/test_gpu_comm.py: one process per GPU (launched by torch.distributed.run).  Every rank reduces its
slice of a [rows, cols] tensor with a sharded kernel, the library's communicator all-reduces the partials, and rank 0
checks the result against the whole-tensor reduction."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from akg_b200 import FusedKernel, descs  # noqa: E402
from akg_b200.sharding import Communicator  # noqa: E402


def random_staged_region(seed, rows):
    """A random region whose reductions over axis 0 (or over all elements) feed later ops: planned as stages when axis 0
    is split over ranks.  Bounded ops only, so that the values stay finite."""
    import numpy as np
    from akg_b200.descs import _Builder, _reduce_attr
    rng = np.random.default_rng(seed)
    cols = int(rng.choice([40, 256, 1000]))
    f = "float32"
    b = _Builder("Fused_fuzz_stage_%d_1" % seed)
    x = b.input("x", [rows, cols], f)
    w = b.input("w", [cols], f) if rng.random() < 0.5 else None
    cur, results = x, []
    for _ in range(int(rng.integers(1, 4))):
        for _ in range(int(rng.integers(0, 3))):
            op = str(rng.choice(["Abs", "Neg", "Tanh", "Mul", "Add"]))
            if op in ("Mul", "Add"):
                other = w if (w is not None and rng.random() < 0.5) else b.const(float(rng.uniform(-1.5, 1.5)), f)
                cur = b.emit(op, [cur, other], [rows, cols], f)
            else:
                cur = b.emit(op, [cur], [rows, cols], f)
        keep = bool(rng.random() < 0.7)
        axes = [0] if rng.random() < 0.8 else [0, 1]
        shp = ([1, cols] if keep else [cols]) if axes == [0] else ([1, 1] if keep else [1])
        red = b.emit(str(rng.choice(["ReduceSum", "ReduceMax", "ReduceMin"])), [cur], shp, f, _reduce_attr(axes, keep))
        if rng.random() < 0.3:
            results.append(red)
        small = red
        for _ in range(int(rng.integers(0, 3))):
            small = b.emit("Mul", [small, b.const(float(rng.uniform(0.05, 0.5)), f)], shp, f)
        cur = b.emit(str(rng.choice(["Sub", "Mul", "Add"])), [cur if rng.random() < 0.7 else x, small], [rows, cols], f)
    results.append(cur)
    for r in results:
        b.output(r)
    return b.build()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator.from_process_group(device=local)
    rows, cols = 512 * world, 1000
    g = torch.Generator().manual_seed(7)
    x = torch.randn(rows, cols, generator=g)  # the same on every rank
    mine = x[rank * (rows // world):(rank + 1) * (rows // world)].contiguous().cuda()
    ok = True
    for build, ref in ((descs.reduce_sum_axis0, lambda t: t.double().sum(0)),
                       (descs.reduce_max_all, lambda t: t.max().reshape(1))):
        k = FusedKernel(build(rows, cols), device=local, shard_rank=rank, shard_world=world)
        assert any(t.shard_kind >= 2 for t in k.outputs)
        out = torch.empty(k.outputs[0].shape, dtype=torch.float32, device="cuda")
        for _ in range(2):
            comm.launch_sharded(k, [mine, out])
        torch.cuda.synchronize()
        want = ref(x)
        got = out.cpu().double().reshape(want.shape)
        ok = ok and bool(torch.allclose(got, want.double(), rtol=1e-5, atol=1e-5 * float(x.abs().sum(0).max())))
    # data-parallel LayerNorm backward: dx stays with the rank's rows, the weight and bias gradients are partial sums
    rows_ln, cols_ln = 256 * world, 512
    dy_all, x_all = torch.randn(rows_ln, cols_ln, generator=g), torch.randn(rows_ln, cols_ln, generator=g) * 2 + 0.5
    gamma = torch.rand(cols_ln, generator=g) + 0.5
    k = FusedKernel(descs.layer_norm_backward(rows_ln, cols_ln), device=local, shard_rank=rank, shard_world=world)
    lo, hi = rank * (rows_ln // world), (rank + 1) * (rows_ln // world)
    outs = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in k.outputs]
    comm.launch_sharded(k, [dy_all[lo:hi].contiguous().cuda(), x_all[lo:hi].contiguous().cuda(), gamma.cuda()] + outs)
    torch.cuda.synchronize()
    xd, dyd = x_all.double(), dy_all.double()
    xhat = (xd - xd.mean(1, keepdim=True)) / torch.sqrt(xd.var(1, unbiased=False, keepdim=True) + 1e-5)
    gd = dyd * gamma.double()
    dx = (gd - gd.mean(1, keepdim=True) - xhat * (gd * xhat).mean(1, keepdim=True)) / torch.sqrt(xd.var(1, unbiased=False, keepdim=True) + 1e-5)
    ok = ok and bool(torch.allclose(outs[0].cpu().double(), dx[lo:hi], rtol=1e-4, atol=1e-4))
    ok = ok and bool(torch.allclose(outs[1].cpu().double(), (dyd * xhat).sum(0), rtol=1e-4, atol=1e-3))
    ok = ok and bool(torch.allclose(outs[2].cpu().double(), dyd.sum(0), rtol=1e-4, atol=1e-3))
    # the same reductions with the exchange over the ranks' mapped buffers instead of NCCL: inside the reduction's own
    # launch (the CTA that folds a tile exchanges it), and as one exchange kernel after the launch
    peer = comm.enable_peer_exchange()
    timings = {}
    if peer:
        big = torch.randn(65536 // world, 4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3 + rank))
        # three ways: the reduction's fold launch carries the exchange (default), the last CTA of the reduction itself
        # does (AKGB_FLAG_FOLD_IN_LAUNCH), one exchange kernel after the kernel's own launches
        for label, in_reduction, flags in (("fold launch", True, 0), ("last CTA", True, 2), ("exchange kernel", False, 0)):
            comm.set_exchange_in_reduction(in_reduction)
            for build, ref in ((descs.reduce_sum_axis0, lambda t: t.double().sum(0)),
                               (descs.reduce_max_all, lambda t: t.max().reshape(1)),
                               (descs.reduce_sum_and_max, None)):
                k = FusedKernel(build(rows, cols), device=local, shard_rank=rank, shard_world=world, flags=flags)
                ok = ok and comm.exchange_kind(k) == ("in-reduction" if in_reduction else "peer-kernel")
                outs = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in k.outputs]
                for _ in range(5):  # several calls, both parities of the exchange buffer
                    comm.launch_sharded(k, [mine] + outs)
                torch.cuda.synchronize()
                ok = ok and k.check_device_error() == 0
                wants = [ref(x)] if ref else [x.double().sum(0), x.max().reshape(1)]
                for o, w in zip(outs, wants):
                    ok = ok and bool(torch.allclose(o.cpu().double().reshape(w.shape), w.double(), rtol=1e-5,
                                                    atol=1e-5 * float(x.abs().sum(0).max())))
                # every rank holds the same bits
                for o in outs:
                    gathered = [torch.empty_like(o) for _ in range(world)]
                    dist.all_gather(gathered, o)
                    ok = ok and all(bool(torch.equal(g_, gathered[0])) for g_ in gathered)
                # the benchmark's split: [65536 / world, 4096] per rank, replayed from a CUDA graph
                kb = FusedKernel(build(65536, 4096), device=local, shard_rank=rank, shard_world=world, flags=flags)
                ob = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in kb.outputs]
                s = torch.cuda.Stream()
                with torch.cuda.stream(s):
                    for _ in range(3):
                        comm.launch_sharded(kb, [big] + ob, s)
                    s.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=s):
                        for _ in range(10):
                            comm.launch_sharded(kb, [big] + ob, torch.cuda.current_stream())
                    graph.replay()
                    torch.cuda.synchronize()
                    dist.barrier()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record(s)
                    graph.replay()
                    t1.record(s)
                    torch.cuda.synchronize()
                ok = ok and kb.check_device_error() == 0
                timings[(build.__name__, label)] = t0.elapsed_time(t1) / 10 * 1e3
                for o, d in zip(ob, kb.outputs):
                    if d.shard_kind == 2:  # column sums
                        part = big.double().sum(0)
                        dist.all_reduce(part)
                        ok = ok and bool(torch.allclose(o.double(), part, rtol=1e-5, atol=1e-2))
                    else:  # the maximum of all elements, bit for bit
                        mx = big.max().reshape(1).clone()
                        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                        ok = ok and bool(torch.equal(o.reshape(1), mx))
        comm.set_exchange_in_reduction(True)
    # a BatchMatMul whose operands both carry the batch: every rank multiplies its own batch entries
    bsz = 2 * world
    a_all = (torch.randn(bsz, 128, 64, generator=g) * 0.1).bfloat16()
    b_all = (torch.randn(bsz, 64, 256, generator=g) * 0.1).bfloat16()
    kbm = FusedKernel(descs.batch_matmul(bsz, 128, 64, 256), device=local, shard_rank=rank, shard_world=world)
    ok = ok and all(t.shard_kind == 1 for t in kbm.tensors) and kbm.inputs[1].shape == (2, 64, 256)
    obm = torch.empty(kbm.outputs[0].shape, dtype=torch.float32, device="cuda")
    comm.launch_sharded(kbm, [a_all[2 * rank:2 * rank + 2].contiguous().cuda(),
                              b_all[2 * rank:2 * rank + 2].contiguous().cuda(), obm])
    torch.cuda.synchronize()
    want_bm = torch.matmul(a_all.double(), b_all.double())[2 * rank:2 * rank + 2]
    ok = ok and bool(torch.allclose(obm.cpu().double(), want_bm, rtol=2e-3, atol=2e-3 * float(want_bm.abs().max())))
    # reductions over the split axis that feed later ops: the region runs as stages with the exchange between them.
    # Batch normalisation in training mode and its gradient over a batch split across the ranks, against the CPU oracle
    # on the whole batch (every rank evaluates it and checks its own slice and the per-channel results)
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tests"))
    from oracle import akg_oracle as O
    shape = [4 * world, 32, 14, 14]
    rows0 = 4 * world
    for build in (descs.batch_norm_training, descs.batch_norm_backward,
                  lambda _: descs.normalise_over_axis0(rows0, 1000), lambda _: descs.softmax_over_axis0(rows0, 520),
                  lambda _: descs.scale_by_global_max(rows0, 3000)):
        d = build(shape)
        rng = np.random.default_rng(11)
        full = [rng.standard_normal(t[0]["shape"], dtype=np.float32) for t in d["input_desc"]]
        if build is descs.batch_norm_backward:
            full[3] = np.abs(full[3]) + 0.5  # rstd
        want = O.evaluate(d, full)
        ks = FusedKernel(d, device=local, shard_rank=rank, shard_world=world)
        ok = ok and ks.op_class == "sharded_stages"
        lo, hi = 4 * rank, 4 * rank + 4
        ins = [torch.from_numpy(np.ascontiguousarray(a[lo:hi] if t.shard_kind == 1 else a)).cuda()
               for a, t in zip(full, ks.inputs)]
        outs = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in ks.outputs]
        for _ in range(2):
            comm.launch_sharded(ks, ins + outs)
        torch.cuda.synchronize()
        ok = ok and ks.check_device_error() == 0
        for o, w, t in zip(outs, want, ks.outputs):
            w = w[lo:hi] if t.shard_kind == 1 else w
            ok = ok and bool(np.allclose(o.cpu().numpy(), w, rtol=1e-4, atol=1e-4 * float(np.abs(w).max())))
        try:  # without a communicator the stages cannot exchange: refused, not run half-way
            ks.launch(ins + outs)
            ok = False
        except Exception:
            pass
    # random regions of the same kind: chains over [rows, cols] with one to three reductions over the split axis (or
    # over all elements) whose results, after small ops, flow back into the chain; against the oracle on the whole tensor
    for seed in range(10):
        d = random_staged_region(seed, 8 * world)
        frng = np.random.default_rng(100 + seed)
        full = [frng.standard_normal(t[0]["shape"], dtype=np.float32) for t in d["input_desc"]]
        want = O.evaluate(d, full)
        ks = FusedKernel(d, device=local, shard_rank=rank, shard_world=world)
        ok = ok and ks.op_class == "sharded_stages"
        lo, hi = 8 * rank, 8 * rank + 8
        ins = [torch.from_numpy(np.ascontiguousarray(a[lo:hi] if t.shard_kind == 1 else a)).cuda()
               for a, t in zip(full, ks.inputs)]
        outs = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in ks.outputs]
        comm.launch_sharded(ks, ins + outs)
        torch.cuda.synchronize()
        ok = ok and ks.check_device_error() == 0
        for o, w, t in zip(outs, want, ks.outputs):
            w = w[lo:hi] if t.shard_kind == 1 else w
            good = bool(np.allclose(o.cpu().numpy().reshape(w.shape), w, rtol=2e-4, atol=2e-4 * float(np.abs(w).max() + 1e-6)))
            if not good and rank == 0:
                print("FUZZ_STAGE_MISMATCH seed", seed, t.name, flush=True)
            ok = ok and good
    # the staged regions at the benchmark's reduction size, [65536 / world, 4096] float32 per rank, timed like the
    # reductions above (CUDA graph of 10 steps); checked through identities: the normalised columns have zero mean and
    # unit variance over ALL ranks' rows, the softmax columns sum to one
    staged_timings = {}
    if peer:
        for name, build in (("normalise_over_axis0", descs.normalise_over_axis0), ("softmax_over_axis0", descs.softmax_over_axis0)):
            kst = FusedKernel(build(65536, 4096), device=local, shard_rank=rank, shard_world=world)
            ok = ok and kst.op_class == "sharded_stages"
            ost = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in kst.outputs]
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(3):
                    comm.launch_sharded(kst, [big] + ost, s)
                s.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    for _ in range(10):
                        comm.launch_sharded(kst, [big] + ost, torch.cuda.current_stream())
                graph.replay()
                torch.cuda.synchronize()
                dist.barrier()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(s)
                graph.replay()
                t1.record(s)
                torch.cuda.synchronize()
            ok = ok and kst.check_device_error() == 0
            staged_timings[name] = (t0.elapsed_time(t1) / 10 * 1e3, kst.launch_count)
            y = ost[0].double()
            col_sum = y.sum(0)
            dist.all_reduce(col_sum)
            if name == "softmax_over_axis0":
                ok = ok and bool(torch.allclose(col_sum, torch.ones_like(col_sum), rtol=1e-4, atol=1e-4))
            else:
                col_sq = (y * y).sum(0)
                dist.all_reduce(col_sq)
                ok = ok and bool(col_sum.abs().max() < 1e-1) and bool(torch.allclose(col_sq / 65536, torch.ones_like(col_sq), rtol=1e-3))
    if rank == 0:
        print("PEER_EXCHANGE", "on" if peer else "off", flush=True)
        for name, (us, launches) in sorted(staged_timings.items()):
            print(f"TIMING staged {name} [65536/{world},4096] per rank, {launches} launches and the exchanges between the "
                  f"stages: {us:.1f} us per step", flush=True)
        for (name, label), us in sorted(timings.items()):
            print(f"TIMING {name} [65536/{world},4096] per rank, exchange by {label}: {us:.1f} us per step", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        print("COMM_OK" if int(flag.item()) == 1 else "COMM_MISMATCH", flush=True)
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
