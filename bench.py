#!/usr/bin/env python
"""Benchmark of the fused-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-classes]

A step is one launch of the headline fused op over one batch of synthetic input: the float16
bias + tanh-GELU * y -> float32 chain on [64,512,4096] (1.07 GB of algorithmic traffic, larger
than L2, so no flush is needed between steps).  Rank 0 prints ONE JSON line:

  value      algorithmic GB/s over all GPUs with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the host-pointer entry point akgb_run_host with pinned host
             buffers: H2D of the inputs and D2H of the output inside the timed region
  roofline   achieved GB/s of the dominant kernel against the measured copy bandwidth
  cpu_baseline  the C restatement of the reference CPU pipeline on a bounded slice of the workload
  classes    one row per fused-op class of the benchmark definition (same timing rules)

With N > 1 (under torchrun) every rank runs the same per-GPU workload on its own shard of a
leading axis that is N times longer (weak scaling); only the column-sum / global-max row of
`classes` has an exchange step (an NCCL all-reduce of the partials).

`--impl reference` times the reference arm instead: the CPU restatement with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "achieved HBM GB/s (algorithmic bytes / device time), fused elementwise-broadcast chain"
UNIT = "GB/s"
WORKLOAD = "bias+tanh-GELU*y->f32, f16 [64,512,4096] (configs[1])"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 1590.0, "fallback"


# ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, scaled to the full
# workload where the capture ran a smaller case; filled in from profiles/ (None = not captured yet)
NCU_TRAFFIC_BYTES = {"gelu": 537201152 + 483198720}  # profiles/gelu_chain_f16_64x512x4096.md, full-size capture


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            time.sleep(0.15)
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.1)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------------------- GPU arm
def torch_dtype(name):
    import torch
    return {"float16": torch.float16, "float32": torch.float32, "bfloat16": torch.bfloat16, "int8": torch.int8,
            "int32": torch.int32, "int64": torch.int64, "bool": torch.bool}[name]


def device_inputs(kernel, kinds, seed, device):
    """Synthetic inputs created on the device with the benchmark's distributions."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = []
    for t in kernel.inputs:
        kind = kinds.get(t.name, "normal")
        dt = torch_dtype(t.dtype)
        if kind == "normal":
            a = torch.randn(t.shape, generator=g, device=device, dtype=torch.float32).to(dt)
        elif kind == "normal_small":
            a = (torch.randn(t.shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dt)
        elif kind == "gamma":
            a = (torch.rand(t.shape, generator=g, device=device) + 0.5).to(dt)
        elif kind == "beta":
            a = (torch.rand(t.shape, generator=g, device=device) * 0.2 - 0.1).to(dt)
        elif kind == "causal":
            m = torch.ones(t.shape, device=device, dtype=torch.bool).tril()
            a = torch.where(m, 0.0, float("-inf")).to(dt)
        else:
            raise ValueError(kind)
        out.append(a.contiguous())
    return out


def device_outputs(kernel, device):
    import torch
    return [torch.empty(t.shape, dtype=torch_dtype(t.dtype), device=device) for t in kernel.outputs]


def time_launches(kernel, buffer_sets, steps, warmup, barrier=None, use_graph=True):
    """Average device time of one step in ms: CUDA events on the launch stream, sync on both sides.

    The `steps` launches are captured once into a CUDA graph and the graph is what gets timed, so that short
    kernels are not paced by the Python/ctypes call path; if capture is not possible (a collective in the step)
    the launches are issued directly.
    """
    import torch
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(warmup):
            kernel.launch(buffer_sets[i % len(buffer_sets)], stream)
        stream.synchronize()
        graph = None
        if use_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(steps):
                        kernel.launch(buffer_sets[i % len(buffer_sets)], torch.cuda.current_stream())
                graph.replay()  # one untimed replay
            except Exception:
                graph = None
        torch.cuda.synchronize()
        if barrier:
            barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        if graph is not None:
            graph.replay()
        else:
            for i in range(steps):
                kernel.launch(buffer_sets[i % len(buffer_sets)], stream)
        t1.record(stream)
        torch.cuda.synchronize()
        if barrier:
            barrier()
    return t0.elapsed_time(t1) / steps


def class_configs(world):
    """(key, description, input kinds) for every fused-op class; leading axes scale with the rank count."""
    from akg_b200 import descs
    w = world
    cfgs = [
        ("layernorm_f32_8192x1024", descs.layernorm(8192 * w, 1024), {"gamma": "gamma", "beta": "beta"}),
        ("gelu_chain_f16_64x512x4096", descs.gelu_chain([64 * w, 512, 4096]), {"bias": "normal_small"}),
        ("gelu_chain_f32math_64x512x4096", descs.gelu_chain([64 * w, 512, 4096], f32_math=True),
         {"bias": "normal_small"}),
        ("masked_softmax_f16_256x2048x2048", descs.masked_softmax(256 * w, 2048, 2048), {"mask": "causal"}),
        ("reduce_sum_axis0_f32_65536x4096", descs.reduce_sum_axis0(65536 * w, 4096), {}),
        ("reduce_max_all_f32_65536x4096", descs.reduce_max_all(65536 * w, 4096), {}),
        ("reduce_sum_and_max_f32_65536x4096", descs.reduce_sum_and_max(65536 * w, 4096), {}),
        ("transpose_f16_32x2048x32x128", descs.transpose([32 * w, 2048, 32, 128], [0, 2, 1, 3]), {}),
        ("matmul_bias_relu_bf16_8192x4096x8192", descs.matmul_bias_relu(8192 * w, 4096, 8192),
         {"a": "normal_small", "b": "normal_small", "bias": "normal_small"}),
    ]
    return cfgs


def run_classes(rank, world, device, steps, warmup, hbm_peak, tf_peak, barrier, comm):
    """One row per class: GB/s (or TFLOP/s) per GPU and aggregate, fraction of the measured peak."""
    import torch
    from akg_b200 import FusedKernel, UnsupportedError
    rows = {}
    for key, desc, kinds in class_configs(world):
        try:
            k = FusedKernel(desc, device=device.index, shard_rank=rank, shard_world=world)
        except UnsupportedError as e:
            rows[key] = {"unsupported": str(e)[:120]}
            continue
        per_set = sum(t.nbytes for t in k.tensors)
        nsets = 1 if per_set > 512 * 2**20 else max(2, int(np.ceil(512 * 2**20 / per_set)))
        sets = []
        for s in range(nsets):
            sets.append(device_inputs(k, kinds, 100 + s, device) + device_outputs(k, device))
        partial = [i for i, t in enumerate(k.tensors) if t.shard_kind >= 2]

        def step_launch(bufs, stream=None, k=k, partial=partial):
            if partial and comm is not None:
                comm.launch_sharded(k, bufs, stream)  # kernel + NCCL all-reduce of the partials, one stream
            else:
                k.launch(bufs, stream)

        class _K:  # adapter so that time_launches includes the exchange step
            launch = staticmethod(step_launch)
        # NCCL calls are not captured; the library's own exchange kernel is an ordinary kernel and is
        graphable = not (partial and world > 1) or (comm is not None and comm.peer_exchange)
        ms = time_launches(_K, sets, steps, warmup, barrier, use_graph=graphable)
        if partial and comm is not None and comm.peer_exchange:
            # a bounded wait of the exchange kernel that ran out on any rank: NCCL carries the exchange from here on
            try:
                bad = 1 if k.check_device_error() else 0
            except Exception:
                bad = 1
            if allreduce_max_scalar(float(bad), world) > 0:
                comm.disable_peer_exchange()
                ms = time_launches(_K, sets, steps, warmup, barrier, use_graph=False)
        ms_max = allreduce_max_scalar(ms, world)
        row = {"class": k.op_class, "ms": round(ms_max, 5), "launches_per_step": k.launch_count}
        if k.flops:
            tf = k.flops * world / (ms_max * 1e-3) / 1e12
            row.update({"tflops": round(tf, 2), "frac_of_peak": round(tf / world / tf_peak, 4), "bound": "tensor"})
        else:
            gbs = k.bytes * world / (ms_max * 1e-3) / 1e9
            row.update({"gbs": round(gbs, 1), "frac_of_peak": round(gbs / world / hbm_peak, 4), "bound": "hbm",
                        "frac_of_8TBs": round(gbs / world / 8000.0, 4), "buffer_sets": nsets})
        rows[key] = row
        del sets, k
        torch.cuda.empty_cache()
    return rows


_dist = {"on": False}


def allreduce_max_scalar(x, world):
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    from akg_b200 import FusedKernel, descs
    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    comm = None
    if world > 1:
        # NCCL may print its version banner on stdout when the communicator is created: keep stdout for the one
        # JSON line by pointing fd 1 at stderr until the first collective has run
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            warm = torch.zeros(1, device=device)
            dist.all_reduce(warm)
            torch.cuda.synchronize()
            # the library's own communicator carries the exchange step of the sharded reductions
            from akg_b200.sharding import Communicator
            comm = Communicator.from_process_group(device=local)
            if os.environ.get("AKGB_BENCH_NCCL_ONLY", "") != "1":
                comm.enable_peer_exchange()  # small partials: one kernel over the ranks' mapped buffers
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    hbm_peak, tf_peak, peak_src = measured_peaks()
    desc = descs.gelu_chain([64 * world, 512, 4096])
    k = FusedKernel(desc, device=local, shard_rank=rank, shard_world=world)
    kinds = {"bias": "normal_small"}
    bufs = device_inputs(k, kinds, 1 + rank, device) + device_outputs(k, device)

    # ---- device-resident throughput (value) + roofline of the dominant kernel
    with ClockSampler(local) as clk:
        ms = time_launches(k, [bufs], args.steps, args.warmup, barrier)
    ms = allreduce_max_scalar(ms, world)
    clocks = clk.summary()
    total_bytes = k.bytes * world
    value = total_bytes / (ms * 1e-3) / 1e9
    achieved = k.bytes / (ms * 1e-3) / 1e9

    # ---- end to end through the host-pointer entry point, pinned host buffers
    host = []
    for t, d in zip(bufs, k.tensors):
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        if not d.is_output:
            h.copy_(t)
        host.append(h)
    host_np = [h.view(torch.uint8).reshape(-1).numpy() for h in host]
    e2e_steps = max(2, min(args.steps, 5))
    k.run_host(host_np)  # warm-up: allocates the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        k.run_host(host_np)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = allreduce_max_scalar(e2e_s, world)
    h2d = sum(d.nbytes for d in k.inputs)
    d2h = sum(d.nbytes for d in k.outputs)
    # the e2e result must be the device result
    assert np.array_equal(host_np[-1][:4096], bufs[-1].view(torch.uint8).reshape(-1)[:4096].cpu().numpy())

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_shape": [64, 512, 4096], "shard": "axis 0 split over ranks",
                   "l2": "inputs larger than L2 (1.07 GB per step), no flush"},
        "clocks": clocks,
        "e2e": {"value": round(total_bytes / e2e_s / 1e9, 2), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world, "steps": e2e_steps, "ms_per_step": round(e2e_s * 1e3, 3)},
        "gpu_launches": k.launch_count * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4), "traffic": NCU_TRAFFIC_BYTES["gelu"],
                     "peak_source": peak_src, "kernel": "gelu_chain_f16_oneshot_kernel",
                     "frac_of_8TBs": round(achieved / 8000.0, 4)},
    }
    del bufs, host, host_np
    torch.cuda.empty_cache()
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline_sample()
    if not args.no_classes:
        line["classes"] = run_classes(rank, world, device, max(3, min(args.steps, 10)), max(3, min(args.warmup, 3)),
                                      hbm_peak, tf_peak, barrier, comm)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------- CPU arms
def cpu_workload(batches, seed=0):
    rng = np.random.default_rng(seed)
    shape = (batches, 512, 4096)
    x = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    y = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    bias = (rng.standard_normal(4096, dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    return x, bias, y


def cpu_time(batches, variant, reps):
    """GB/s of the CPU restatement on `batches` of the 64 leading slices of the workload."""
    from oracle import cpu_ref
    x, bias, y = cpu_workload(batches)
    nbytes = x.nbytes + y.nbytes + bias.nbytes + x.size * 4
    cpu_ref.gelu_chain(x, bias, y, variant=variant)  # warm-up, page-in
    best = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_ref.gelu_chain(x, bias, y, variant=variant)
        best.append(time.perf_counter() - t0)
    return nbytes / float(np.median(best)) / 1e9, float(np.median(best))


def cpu_baseline_sample():
    from oracle import cpu_ref
    cores = cpu_ref.num_threads()
    batches = 8
    gbs, sec = cpu_time(batches, "rp", 3)
    return {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{batches} of the 64 leading slices ([{batches},512,4096]), OpenMP over all host threads, "
                      f"median of 3, {sec:.2f} s each"}


def reference_arm(args):
    """The reference's CPU implementation of the path (C restatement: the MLIR toolchain cannot be built here)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import cpu_ref
    cores = cpu_ref.num_threads()
    batches = 8
    x, bias, y = cpu_workload(batches)
    nbytes = x.nbytes + y.nbytes + bias.nbytes + x.size * 4
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_ref.gelu_chain(x, bias, y, variant="rp")
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_ref.gelu_chain(x, bias, y, variant="rp")
    sec = (time.perf_counter() - t0) / steps
    gbs = nbytes / sec / 1e9
    sample = f"each step = {batches} of the 64 leading slices ([{batches},512,4096]); OpenMP over all host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_classes_table():
    """Times the C restatement of the reference CPU pipeline on a bounded slice of every benchmark config:
    R1 = the driver-default scalar single-thread loop nest, RP = OpenMP over all host threads.  Prints one JSON
    line; slices are stated per row (throughput is per algorithmic byte/FLOP of the slice)."""
    import ml_dtypes
    from oracle import cpu_ref as C
    rng = np.random.default_rng(0)
    cores = C.num_threads()

    def med(fn, reps=3):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return float(np.median(ts))

    rows = {}
    f32 = lambda *s: rng.standard_normal(s, dtype=np.float32)
    # C1 LayerNorm, full size
    x, g, b = f32(8192, 1024), rng.uniform(0.5, 1.5, 1024).astype(np.float32), rng.uniform(-.1, .1, 1024).astype(np.float32)
    nb = 67182592
    rows["layernorm_f32_8192x1024"] = {"slice": "full", "bytes": nb,
        "r1_gbs": nb / med(lambda: C.layernorm(x, g, b, variant="r1")) / 1e9,
        "rp_gbs": nb / med(lambda: C.layernorm(x, g, b, variant="rp")) / 1e9}
    # C2 GELU chain, 4 of 64 slices
    xh, bias, yh = cpu_workload(4)
    nb = xh.nbytes * 2 + bias.nbytes + xh.size * 4
    rows["gelu_chain_f16_64x512x4096"] = {"slice": "4 of 64 leading slices", "bytes": nb,
        "r1_gbs": nb / med(lambda: C.gelu_chain(xh, bias, yh, variant="r1"), 1) / 1e9,
        "rp_gbs": nb / med(lambda: C.gelu_chain(xh, bias, yh, variant="rp")) / 1e9}
    # C3 softmax, 4 of 256 batches
    s = f32(4, 2048, 2048).astype(np.float16)
    mask = np.where(np.tril(np.ones((2048, 2048), bool)), 0, -np.inf).astype(np.float16)
    nb = s.nbytes * 2 + mask.nbytes
    rows["masked_softmax_f16_256x2048x2048"] = {"slice": "4 of 256 batches", "bytes": nb,
        "r1_gbs": nb / med(lambda: C.softmax(s, mask, 1 / np.sqrt(128.0), variant="r1"), 1) / 1e9,
        "rp_gbs": nb / med(lambda: C.softmax(s, mask, 1 / np.sqrt(128.0), variant="rp")) / 1e9}
    # C4 reductions, 8192 of 65536 rows
    xr = f32(8192, 4096)
    nb = xr.nbytes + 16384
    rows["reduce_sum_axis0_f32_65536x4096"] = {"slice": "8192 of 65536 rows", "bytes": nb,
        "r1_gbs": nb / med(lambda: C.reduce_sum_axis0(xr, variant="r1")) / 1e9,
        "rp_gbs": nb / med(lambda: C.reduce_sum_axis0(xr, variant="rp")) / 1e9}
    rows["reduce_max_all_f32_65536x4096"] = {"slice": "8192 of 65536 rows", "bytes": xr.nbytes + 4,
        "r1_gbs": (xr.nbytes + 4) / med(lambda: C.reduce_max_all(xr, variant="r1")) / 1e9,
        "rp_gbs": (xr.nbytes + 4) / med(lambda: C.reduce_max_all(xr, variant="rp")) / 1e9}
    # C5b transpose, 4 of 32 batches
    xt = f32(4, 2048, 32, 128).astype(np.float16)
    rows["transpose_f16_32x2048x32x128"] = {"slice": "4 of 32 batches", "bytes": xt.nbytes * 2,
        "r1_gbs": xt.nbytes * 2 / med(lambda: C.transpose4(xt, [0, 2, 1, 3], variant="r1")) / 1e9,
        "rp_gbs": xt.nbytes * 2 / med(lambda: C.transpose4(xt, [0, 2, 1, 3], variant="rp")) / 1e9}
    # C5a matmul, 128 of 8192 rows of A (RP) / 16 rows (R1)
    A = (f32(128, 4096) * 0.02).astype(ml_dtypes.bfloat16)
    B = (f32(4096, 8192) * 0.02).astype(ml_dtypes.bfloat16)
    bi = (f32(8192) * 0.02).astype(ml_dtypes.bfloat16)
    fl = 2.0 * 128 * 4096 * 8192
    t_rp = med(lambda: C.matmul_bias_relu(A, B, bi, variant="rp"), 1)
    t_r1 = med(lambda: C.matmul_bias_relu(A[:16], B, bi, variant="r1"), 1)
    rows["matmul_bias_relu_bf16_8192x4096x8192"] = {"slice": "128 rows of A (RP), 16 rows (R1)",
        "r1_tflops": 2.0 * 16 * 4096 * 8192 / t_r1 / 1e12, "rp_tflops": fl / t_rp / 1e12}
    for r in rows.values():
        for k_, v in list(r.items()):
            if isinstance(v, float):
                r[k_] = float(f"{v:.4g}")
    print(json.dumps({"cpu_classes": rows, "cores": cores, "kind": "port",
                      "note": "C restatement of the reference CPU pipeline (oracle/cpu_ref.c); R1 scalar single "
                              "thread, RP OpenMP over all host threads"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-classes", action="store_true", help="skip the per-class table")
    ap.add_argument("--cpu-classes", action="store_true",
                    help="time the CPU restatement on a slice of every class (no GPU work) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.cpu_classes:
        cpu_classes_table()
        return
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
