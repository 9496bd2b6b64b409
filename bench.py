#!/usr/bin/env python
"""Benchmark of the fused-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-classes] [--scaling strong|weak]

A step is one launch of the headline fused op over one batch of synthetic input: the float16
bias + tanh-GELU * y -> float32 chain on [64,512,4096] (1.07 GB of algorithmic traffic).  Rank 0 prints ONE
JSON line:

  value      algorithmic GB/s of the whole job with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the host-pointer entry point akgb_run_host with pinned host buffers
             (H2D of the inputs and D2H of the output inside the timed region), next to `copy_only`: the bare
             pinned copies of the same bytes on all ranks at once, no kernel
  roofline   achieved GB/s of the dominant kernel against the measured copy bandwidth
  cpu_baseline  the C restatement of the reference CPU pipeline on a bounded slice of the workload
  classes    one row per fused-op class of the benchmark definition (same timing rules); every row carries
             "checked": a sample of its outputs compared with the CPU oracle after (outside) the timed region
             (tensor rows also "sustained": the same graph replayed for about a second with the SM clock sampled,
             step time x clock as "sm_mcycles_per_step")
  ceilings   plain copies of LayerNorm's 67 MB with the same buffer rotation and graph timing, and cuBLAS on the
             matmul class's own operands (measuring sticks: no class row runs them)

With N > 1 (under torchrun) the FIXED benchmark shapes are split along their leading axis over the N ranks
(strong scaling: per-GPU work shrinks with N); `value` is the full configuration's bytes over the slowest rank's
step time.  Only the reductions over the split axis have an exchange step; their rows say which way it went
("exchange").  The key "weak" repeats the headline and the reduction rows with every rank running the full
single-GPU shape (`--scaling weak` makes that the main mode).

`--impl reference` times the reference arm instead: the CPU restatement of the path with all host threads.
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
ROTATE_BELOW_BYTES = 512 * 2**20  # working sets smaller than this rotate through several buffer sets (L2 is 126 MB)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            global tf_sustained
            tf_sustained = float(d.get("bf16_tflops_sustained", 0.0))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 1590.0, "fallback"


tf_sustained = 1400.0  # the fallback's sustained figure; replaced by MEASURED_PEAKS.json's when present


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


def device_inputs(kernel, kinds, seed, device, rank=0):
    """Synthetic inputs created on the device with the benchmark's distributions.  Tensors every rank holds whole
    (bias, gamma, mask, the right matmul operand) get the same values on every rank, slices of the split axis differ."""
    import torch
    out = []
    for j, t in enumerate(kernel.inputs):
        g = torch.Generator(device=device)
        g.manual_seed(seed * 131 + j * 17 + (7919 * rank if t.shard_kind == 1 else 0))
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


def buffer_sets_for(kernel, kinds, device, rank, seed0=100):
    """Enough (inputs + outputs) sets that consecutive steps do not find their data in L2."""
    per_set = sum(t.nbytes for t in kernel.tensors)
    nsets = 1 if per_set >= ROTATE_BELOW_BYTES else max(2, int(np.ceil(ROTATE_BELOW_BYTES / per_set)))
    return [device_inputs(kernel, kinds, seed0 + s, device, rank) + device_outputs(kernel, device) for s in range(nsets)]


def time_launches(kernel, buffer_sets, steps, warmup, barrier=None, use_graph=True, sustain_s=0.0, sustained=None):
    """Average device time of one step in ms: CUDA events on the launch stream, sync on both sides.

    The `steps` launches are captured once into a CUDA graph and the graph is what gets timed, so that short
    kernels are not paced by the Python/ctypes call path; if capture is not possible (an NCCL call in the step)
    the launches are issued directly.
    """
    import torch
    stream = torch.cuda.Stream()
    if barrier:
        barrier()  # ranks start their warm-up together: a step with an exchange waits (bounded) for its peers
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
        if sustain_s > 0 and graph is not None and sustained is not None:
            # the same graph replayed back to back for `sustain_s` seconds: what the part sustains under its power cap
            one = t0.elapsed_time(t1)
            reps = max(2, int(sustain_s * 1e3 / max(one, 1e-3)))
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            for _ in range(reps):
                graph.replay()
            s1.record(stream)
            torch.cuda.synchronize()
            sustained["ms"] = s0.elapsed_time(s1) / (reps * steps)
            sustained["seconds"] = s0.elapsed_time(s1) / 1e3
        if barrier:
            barrier()
    return t0.elapsed_time(t1) / steps


def device_error_word(kernel):
    """Reads and clears the device error word through the C ABI without turning a non-zero word into an exception."""
    import ctypes
    word = ctypes.c_uint32(0)
    kernel._lib.akgb_check_device_error(kernel._handle, ctypes.byref(word))
    return int(word.value)


def allreduce_scalar(x, world, op="max"):
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op])
    return float(t.item())


# ----------------------------------------------------------------------------------------- classes and their checks
def class_table():
    """(key, make(lead) -> description, leading extent of the benchmark shape, input kinds, check, sample extent).

    `make(lead)` builds the class's description with `lead` as its leading extent, so the same table serves the
    benchmark shape, its split over ranks, the weak-scaling shape and the small slices the oracle evaluates."""
    from akg_b200 import descs
    ln = {"gamma": "gamma", "beta": "beta"}
    ge = {"bias": "normal_small"}
    mm = {"a": "normal_small", "b": "normal_small", "bias": "normal_small"}
    return [
        ("layernorm_f32_8192x1024", lambda r: descs.layernorm(r, 1024), 8192, ln, "f32", 64),
        ("gelu_chain_f16_64x512x4096", lambda b: descs.gelu_chain([b, 512, 4096]), 64, ge, "exact", 1),
        ("gelu_chain_f32math_64x512x4096", lambda b: descs.gelu_chain([b, 512, 4096], f32_math=True), 64, ge,
         "f32_rms", 1),
        ("masked_softmax_f16_256x2048x2048", lambda b: descs.masked_softmax(b, 2048, 2048), 256, {"mask": "causal"},
         "half", 1),
        ("reduce_sum_axis0_f32_65536x4096", lambda r: descs.reduce_sum_axis0(r, 4096), 65536, {}, "reduce", 0),
        ("reduce_max_all_f32_65536x4096", lambda r: descs.reduce_max_all(r, 4096), 65536, {}, "reduce", 0),
        ("reduce_sum_and_max_f32_65536x4096", lambda r: descs.reduce_sum_and_max(r, 4096), 65536, {}, "reduce", 0),
        ("transpose_f16_32x2048x32x128", lambda b: descs.transpose([b, 2048, 32, 128], [0, 2, 1, 3]), 32, {}, "exact", 1),
        ("matmul_bias_relu_bf16_8192x4096x8192", lambda m: descs.matmul_bias_relu(m, 4096, 8192), 8192, mm, "matmul", 16),
        # beyond the benchmark definition: transposes whose innermost output axis is strided in the input (tile mode)
        ("transpose_tile_f16_8192x8192", lambda r: descs.transpose([r, 8192], [1, 0]), 8192, {}, "exact_full", 0),
        ("transpose_tile_f32_64x1024x1024", lambda b: descs.transpose([b, 1024, 1024], [0, 2, 1], "float32"), 64, {},
         "exact", 1),
        # statistics over the split axis feed the normalisation: stages with the exchange between them at N > 1
        ("batchnorm_training_f32_64x256x56x56", lambda n: descs.batch_norm_training([n, 256, 56, 56]), 64,
         {"gamma": "gamma", "beta": "beta"}, "gathered", 0),
    ]


def to_numpy(t):
    """Device tensor -> numpy array of the same element type (bfloat16 through ml_dtypes)."""
    import torch
    if t.dtype == torch.bfloat16:
        import ml_dtypes
        return t.view(torch.int16).cpu().numpy().view(ml_dtypes.bfloat16)
    return t.cpu().numpy()


def check_sliced(make, kernel, bufs, how, sample):
    """Classes whose leading-axis slices are independent: the oracle evaluates the first and the last `sample`
    slices of this rank's tensors (a description of 2*sample slices), compared with the same slices of the output."""
    import torch
    from oracle import akg_oracle as O
    ins, outs = bufs[:kernel.num_inputs], bufs[kernel.num_inputs:]

    def ends(t):
        return torch.cat([t[:sample], t[-sample:]], dim=0)

    # at one rank nothing is marked as split: an input spans the leading axis when it has the first input's rank and
    # leading extent (bias, gamma, mask and the right matmul operand do not)
    lead = kernel.inputs[0]
    def spans(d):
        return d.shard_kind == 1 or (len(d.shape) == len(lead.shape) and d.shape[0] == lead.shape[0] and d.name != "b")
    host_in = [to_numpy(ends(t) if spans(d) else t) for t, d in zip(ins, kernel.inputs)]
    want = O.evaluate(make(2 * sample), host_in)
    for o, w, d in zip(outs, want, kernel.outputs):
        got = to_numpy(ends(o))
        w = np.ascontiguousarray(w)
        if how == "exact":
            if not np.array_equal(got.view(np.uint8), w.view(np.uint8)):
                return False
            continue
        g64, w64 = got.astype(np.float64), w.astype(np.float64)
        if how == "f32":  # 1e-5 relative (+1e-6 absolute, as the parity tests)
            ok = np.all(np.abs(g64 - w64) <= 1e-5 * np.abs(w64) + 1e-6)
        elif how == "f32_rms":  # the reference's comparison, np.allclose(rtol=atol), with atol scaled by the rms
            ok = np.all(np.abs(g64 - w64) <= 1e-5 * np.abs(w64) + 1e-5 * np.sqrt(np.mean(w64 * w64)))
        elif how == "half":  # 2e-3 for float16 / bfloat16 results; masked entries exactly zero
            ok = np.all(np.abs(g64 - w64) <= 2e-3 * np.abs(w64) + 1e-7) and np.array_equal(g64 == 0, w64 == 0)
        elif how == "matmul":  # the bfloat16 rounding of a value within 2e-3 of the oracle's float32 accumulate
            atol = 1e-3 * float(np.abs(w64).max() + 1e-30)
            ok = np.all(np.abs(g64 - w64) <= (2e-3 + 2.0 ** -8) * np.abs(w64) + atol)
        else:
            raise ValueError(how)
        if not ok:
            return False
    return True


def check_gathered(make, global_lead, kernel, bufs, rank, world):
    """Results that depend on the whole split axis (batch statistics): every rank gathers the split inputs, evaluates
    the oracle on the whole tensors and compares its own slice of the split results and the replicated results whole
    (1e-4 relative with an absolute term scaled by the largest expected value: float32 sums of 200 000 terms)."""
    import torch
    import torch.distributed as dist
    from oracle import akg_oracle as O
    ins, outs = bufs[:kernel.num_inputs], bufs[kernel.num_inputs:]
    full = []
    for t, d in zip(ins, kernel.inputs):
        if world > 1 and d.shard_kind == 1:
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            full.append(torch.cat(parts, dim=0).cpu().numpy())
        else:
            full.append(t.cpu().numpy())
    want = O.evaluate(make(global_lead), full)
    ok = True
    for o, w, d in zip(outs, want, kernel.outputs):
        if world > 1 and d.shard_kind == 1:
            n = d.shape[0]
            w = w[rank * n:(rank + 1) * n]
        got = o.cpu().numpy().reshape(w.shape).astype(np.float64)
        w = w.astype(np.float64)
        ok = ok and bool(np.all(np.abs(got - w) <= 1e-4 * np.abs(w) + 1e-4 * float(np.abs(w).max())))
    return ok


def check_reduction(make, kernel, bufs, rank, world):
    """Reductions over the split axis: every rank evaluates the oracle on ITS rows (float32, the oracle's own order) and
    a float64 sum; the per-rank results are combined over the ranks in float64 / by max and compared with what the
    library returned on every rank: column sums within 1e-5 * sum|x| of the float64 truth, the maximum bit for bit."""
    import torch
    import torch.distributed as dist
    from oracle import akg_oracle as O
    x = bufs[0]
    outs = bufs[kernel.num_inputs:]
    xh = x.cpu().numpy()
    want = O.evaluate(make(xh.shape[0]), [xh])
    dev = x.device
    ok = True
    for o, w, d in zip(outs, want, kernel.outputs):
        got = o.cpu().numpy().astype(np.float64).reshape(-1)
        if d.shard_kind == 3 or (world == 1 and got.size == 1):  # maximum of all elements
            m = torch.tensor([float(np.asarray(w).reshape(-1)[0])], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(m, op=dist.ReduceOp.MAX)
            ok = ok and got[0] == float(m.item())
            continue
        truth = np.zeros(xh.shape[1], np.float64)
        mag = np.zeros(xh.shape[1], np.float64)
        for r in range(0, xh.shape[0], 8192):
            blk = xh[r:r + 8192].astype(np.float64)
            truth += blk.sum(axis=0)
            mag += np.abs(blk).sum(axis=0)
        packed = torch.from_numpy(np.stack([truth, mag, np.asarray(w, np.float64).reshape(-1)])).to(dev)
        if world > 1:
            dist.all_reduce(packed, op=dist.ReduceOp.SUM)
        truth, mag, oracle_sum = packed.cpu().numpy()
        ok = ok and bool(np.all(np.abs(got - truth) <= 1e-5 * mag)) and bool(np.all(np.abs(oracle_sum - truth) <= 1e-5 * mag))
    if world > 1:  # the same bits on every rank
        for o in outs:
            parts = [torch.empty_like(o) for _ in range(world)]
            dist.all_gather(parts, o.contiguous())
            ok = ok and all(bool(torch.equal(p.view(torch.int32), parts[0].view(torch.int32))) for p in parts)
    return bool(ok)


def run_classes(rank, world, device, steps, warmup, hbm_peak, tf_peak, barrier, comm, scaling, only=None):
    """One row per class: GB/s (or TFLOP/s) of the whole job, fraction of the measured peak per GPU, oracle check."""
    import torch
    from akg_b200 import FusedKernel, UnsupportedError
    rows = {}
    for key, make, lead, kinds, how, sample in class_table():
        if only is not None and key not in only:
            continue
        global_lead = lead if scaling == "strong" else lead * world
        try:
            k = FusedKernel(make(global_lead), device=device.index, shard_rank=rank, shard_world=world)
        except UnsupportedError as e:
            rows[key] = {"unsupported": str(e)[:120]}
            continue
        sets = buffer_sets_for(k, kinds, device, rank)
        partial = [i for i, t in enumerate(k.tensors) if t.shard_kind >= 2] or (k.op_class == "sharded_stages")
        exchange = comm.exchange_kind(k) if (partial and comm is not None) else "none"

        def step_launch(bufs, stream=None, k=k, partial=partial):
            if partial and comm is not None:
                comm.launch_sharded(k, bufs, stream)  # the kernel and the exchange of its partials, one stream
            else:
                k.launch(bufs, stream)

        class _K:  # adapter so that time_launches includes the exchange step
            launch = staticmethod(step_launch)
        # NCCL calls are not captured into the graph; the library's own exchange runs inside ordinary kernels and is
        graphable = exchange in ("none", "peer-kernel", "in-reduction")
        sustained = {}
        if k.flops:  # tensor-core rows: also a second-long loop with the SM clock sampled, next to the short burst
            with ClockSampler(device.index) as clk_mm:
                ms = time_launches(_K, sets, steps, warmup, barrier, use_graph=graphable, sustain_s=1.0, sustained=sustained)
            sustained["clocks"] = clk_mm.summary()
        else:
            ms = time_launches(_K, sets, steps, warmup, barrier, use_graph=graphable)
        word = device_error_word(k)  # bounded device-side waits that gave up (0 = none); bit 8: a peer-memory exchange
        if exchange in ("peer-kernel", "in-reduction"):
            # a wait that ran out on any rank: NCCL carries the exchange from here on (on every rank)
            if allreduce_scalar(float(word != 0), world) > 0:
                comm.disable_peer_exchange()
                exchange = "nccl (after a peer-memory wait ran out)"
                ms = time_launches(_K, sets, steps, warmup, barrier, use_graph=False)
        ms_max = allreduce_scalar(ms, world)
        alone = None
        if partial and comm is not None and k.op_class != "sharded_stages":
            # the same shard on the same rank without the exchange step: what the exchange costs on top
            alone = allreduce_scalar(time_launches(k, sets, steps, warmup, barrier), world)
        bytes_job = k.bytes * world   # the ranks' shares add up to the global shape
        flops_job = k.flops * world
        row = {"class": k.op_class, "ms": round(ms_max, 5), "launches_per_step": k.launch_count,
               "per_gpu_lead": k.inputs[0].shape[0], "buffer_sets": len(sets)}
        if partial:
            row["exchange"] = exchange
        if alone is not None:
            row["ms_without_exchange"] = round(alone, 5)
            row["exchange_us"] = round((ms_max - alone) * 1e3, 2)
        if word:
            row["device_error_word"] = word
        if k.flops:
            tf = flops_job / (ms_max * 1e-3) / 1e12
            row.update({"tflops": round(tf, 2), "frac_of_peak": round(tf / world / tf_peak, 4), "bound": "tensor"})
            if "ms" in sustained:
                ms_s = allreduce_scalar(sustained["ms"], world)
                tf_s = flops_job / (ms_s * 1e-3) / 1e12
                mhz = sustained["clocks"].get("sm_mhz")
                row["sustained"] = {"tflops": round(tf_s, 2), "seconds": round(sustained["seconds"], 2), "sm_mhz": mhz,
                                    "reasons": sustained["clocks"].get("reasons"),
                                    "frac_of_sustained_peak": round(tf_s / world / tf_sustained, 4) if tf_sustained else None,
                                    # dense bf16 nominal 2 250 TFLOP/s at 1 965 MHz, scaled to the clock seen under load
                                    "frac_of_nominal_at_clock": round(tf_s / world / (2250.0 * mhz / 1965.0), 4) if mhz else None,
                                    # step time x median SM clock: runs at different clocks compare by this
                                    "sm_mcycles_per_step": round(ms_s * 1e-3 * mhz, 3) if mhz else None}
        else:
            gbs = bytes_job / (ms_max * 1e-3) / 1e9
            row.update({"gbs": round(gbs, 1), "frac_of_peak": round(gbs / world / hbm_peak, 4), "bound": "hbm",
                        "frac_of_8TBs": round(gbs / world / 8000.0, 4)})
        # ---- outside the timed region: a sample of the outputs against the CPU oracle
        try:
            step_launch(sets[0])
            torch.cuda.synchronize()
            if how == "reduce":
                good = check_reduction(make, k, sets[0], rank, world)
            elif how == "gathered":
                good = check_gathered(make, global_lead, k, sets[0], rank, world)
            elif how == "exact_full":  # the oracle on the whole tensors (no independent slices to sample)
                from oracle import akg_oracle as O
                want = O.evaluate(make(global_lead), [to_numpy(t) for t in sets[0][:k.num_inputs]])
                good = all(np.array_equal(to_numpy(o).view(np.uint8), np.ascontiguousarray(w).view(np.uint8))
                           for o, w in zip(sets[0][k.num_inputs:], want))
            else:
                good = check_sliced(make, k, sets[0], how, sample)
        except Exception as e:  # a check that cannot run is a failed check, not a crashed benchmark
            sys.stderr.write(f"[bench] check of {key} raised: {e!r}\n")
            good = False
        row["checked"] = bool(allreduce_scalar(1.0 if good else 0.0, world, "min") > 0)
        rows[key] = row
        del sets, k
        torch.cuda.empty_cache()
    return rows


def copy_ceilings(device, steps, warmup, hbm_peak):
    """What a plain copy of LayerNorm's bytes (33.5 MB in, 33.5 MB out) reaches with the same buffer rotation and graph
    timing: torch's copy kernel (the kernel the measured peak was taken with, at 2 GB) and this library's generated
    elementwise kernel on `Mul(x, 1)`.  A size-matched ceiling for the 67 MB row-wise classes."""
    import torch
    from akg_b200 import FusedKernel, descs
    n_sets = 8
    xs = [torch.randn(8192, 1024, device=device) for _ in range(n_sets)]
    ys = [torch.empty_like(x) for x in xs]
    nbytes = 2 * xs[0].numel() * 4

    class TorchCopy:
        @staticmethod
        def launch(b, stream=None):
            b[1].copy_(b[0])

    out = {}
    ms = time_launches(TorchCopy, [[x, y] for x, y in zip(xs, ys)], steps, warmup)
    out["torch_copy_67MB"] = {"ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1), "frac_of_peak": round(nbytes / ms / 1e6 / hbm_peak, 4)}
    try:
        k = FusedKernel(descs.scale_copy([8192, 1024]), device=device.index)
        ms = time_launches(k, [[x, y] for x, y in zip(xs, ys)], steps, warmup)
        out["library_copy_67MB"] = {"ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1),
                                    "frac_of_peak": round(nbytes / ms / 1e6 / hbm_peak, 4)}
    except Exception as e:
        out["library_copy_67MB"] = {"error": str(e)[:100]}
    return out


def matmul_ceiling(device, steps, warmup, tf_peak):
    """cuBLAS (torch.matmul) on the matmul class's own operands, 8192x4096 by 4096x8192 in bfloat16 without bias or
    ReLU, timed like the class row.  The measured tensor peak was taken on 8192^3, whose tiles run twice as many MMAs per
    result tile; this is the library's figure at the benchmark's shape.  A measuring stick only: no class row uses it."""
    import torch
    g = torch.Generator(device=device).manual_seed(5)
    a = (torch.randn(8192, 4096, device=device, generator=g) * 0.02).bfloat16()
    bs = [(torch.randn(4096, 8192, device=device, generator=g) * 0.02).bfloat16() for _ in range(2)]
    outs = [torch.empty(8192, 8192, dtype=torch.bfloat16, device=device) for _ in range(2)]

    class TorchMatmul:
        @staticmethod
        def launch(b, stream=None):
            torch.matmul(b[0], b[1], out=b[2])

    ms = time_launches(TorchMatmul, [[a, b, o] for b, o in zip(bs, outs)], steps, warmup)
    tf = 2.0 * 8192 * 4096 * 8192 / (ms * 1e-3) / 1e12
    return {"ms": round(ms, 5), "tflops": round(tf, 1), "frac_of_peak": round(tf / tf_peak, 4)}


def host_copy_only(bufs, kernel, device, steps, barrier, world):
    """Bare pinned copies of one step's bytes, no kernel: all inputs host->device on one stream while all outputs go
    device->host on another, on every rank at once.  Seconds per step (max over ranks)."""
    import torch
    ins = bufs[:kernel.num_inputs]
    outs = bufs[kernel.num_inputs:]
    h_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in ins]
    h_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def once():
        with torch.cuda.stream(s1):
            for d, h in zip(ins, h_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            for d, h in zip(outs, h_out):
                h.copy_(d, non_blocking=True)
    once()
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    torch.cuda.synchronize()
    barrier()
    sec = (time.perf_counter() - t0) / steps
    return allreduce_scalar(sec, world)


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
                comm.enable_peer_exchange()  # small partials travel inside the library's own kernels
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    hbm_peak, tf_peak, peak_src = measured_peaks()
    scaling = args.scaling
    lead = 64 if scaling == "strong" else 64 * world
    if lead % world:
        raise SystemExit(f"the leading extent {lead} does not split over {world} ranks")
    k = FusedKernel(descs.gelu_chain([lead, 512, 4096]), device=local, shard_rank=rank, shard_world=world)
    kinds = {"bias": "normal_small"}
    sets = buffer_sets_for(k, kinds, device, rank, seed0=1)
    bufs = sets[0]

    # ---- device-resident throughput (value) + roofline of the dominant kernel
    with ClockSampler(local) as clk:
        ms = time_launches(k, sets, args.steps, args.warmup, barrier)
    ms = allreduce_scalar(ms, world)
    clocks = clk.summary()
    total_bytes = k.bytes * world
    value = total_bytes / (ms * 1e-3) / 1e9
    achieved = k.bytes / (ms * 1e-3) / 1e9
    checked = check_sliced(lambda b: descs.gelu_chain([b, 512, 4096]), k, bufs, "exact", 1)
    checked = allreduce_scalar(1.0 if checked else 0.0, world, "min") > 0

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
    e2e_s = allreduce_scalar(e2e_s, world)
    h2d = sum(d.nbytes for d in k.inputs)
    d2h = sum(d.nbytes for d in k.outputs)
    # the end-to-end result must be the device result, bit for bit, on the whole output
    k.launch(bufs)
    torch.cuda.synchronize()
    e2e_same = bool(torch.equal(host[-1].view(torch.int32), bufs[-1].cpu().view(torch.int32)))
    e2e_same = allreduce_scalar(1.0 if e2e_same else 0.0, world, "min") > 0
    copy_s = host_copy_only(bufs, k, device, e2e_steps, barrier, world)

    per_gpu_shape = list(k.inputs[0].shape)
    nsets = len(sets)
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_shape": [lead, 512, 4096], "per_gpu_shape": per_gpu_shape,
                   "shard": "axis 0 split over ranks, no collective on this path",
                   "l2": ("inputs larger than L2 (1.07 GB per step), no flush" if nsets == 1 else
                          f"{nsets} buffer sets in rotation ({sum(t.nbytes for t in k.tensors) * nsets >> 20} MB), "
                          "every step reads and writes data last touched a full rotation ago")},
        "checked": bool(checked),
        "clocks": clocks,
        "e2e": {"value": round(total_bytes / e2e_s / 1e9, 2), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world, "steps": e2e_steps, "ms_per_step": round(e2e_s * 1e3, 3),
                "same_bits_as_device_launch": bool(e2e_same),
                "copy_only": {"value": round(total_bytes / copy_s / 1e9, 2), "unit": UNIT,
                              "ms_per_step": round(copy_s * 1e3, 3),
                              "what": "the same pinned H2D and D2H bytes on all ranks at once, no kernel"}},
        "gpu_launches": k.launch_count * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4),
                     "traffic": NCU_TRAFFIC_BYTES["gelu"] // world, "peak_source": peak_src,
                     "kernel": "gelu_chain_f16_oneshot_kernel", "frac_of_8TBs": round(achieved / 8000.0, 4)},
    }
    del bufs, sets, host, host_np
    torch.cuda.empty_cache()
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline_sample()
    csteps, cwarm = max(3, min(args.steps, 10)), max(3, min(args.warmup, 3))
    if not args.no_classes:
        only = set(args.only.split(",")) if args.only else None
        line["classes"] = run_classes(rank, world, device, csteps, cwarm, hbm_peak, tf_peak, barrier, comm, scaling, only)
        if world == 1:
            line["ceilings"] = copy_ceilings(device, csteps, cwarm, hbm_peak)
            if only is None or "matmul_bias_relu_bf16_8192x4096x8192" in only:
                try:
                    line["ceilings"]["cublas_bf16_8192x4096x8192"] = matmul_ceiling(device, csteps, cwarm, tf_peak)
                except Exception as e:
                    line["ceilings"]["cublas_bf16_8192x4096x8192"] = {"error": str(e)[:100]}
    if world > 1 and not args.no_classes:
        # the other scaling mode, for the headline and for the rows that have an exchange step
        other = "weak" if scaling == "strong" else "strong"
        ko = FusedKernel(descs.gelu_chain([64 * world if other == "weak" else 64, 512, 4096]), device=local,
                         shard_rank=rank, shard_world=world)
        so = buffer_sets_for(ko, kinds, device, rank, seed0=1)
        mo = allreduce_scalar(time_launches(ko, so, csteps, cwarm, barrier), world)
        del so
        torch.cuda.empty_cache()
        line[other] = {"value": round(ko.bytes * world / (mo * 1e-3) / 1e9, 1), "unit": UNIT,
                       "ms_per_step": round(mo, 5), "per_gpu_shape": list(ko.inputs[0].shape),
                       "classes": run_classes(rank, world, device, csteps, cwarm, hbm_peak, tf_peak, barrier, comm, other,
                                              only={"reduce_sum_axis0_f32_65536x4096", "reduce_max_all_f32_65536x4096",
                                                    "reduce_sum_and_max_f32_65536x4096"})}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        if comm is not None:
            comm.close()
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
    cores = cpu_ref.use_all_host_threads()  # not an OMP_NUM_THREADS inherited from a launcher
    batches = 8
    gbs, sec = cpu_time(batches, "rp", 3)
    return {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{batches} of the 64 leading slices ([{batches},512,4096]), OpenMP over {cores} host threads, "
                      f"median of 3, {sec:.2f} s each"}


def reference_arm(args):
    """The reference's CPU implementation of the path (C restatement: the MLIR toolchain cannot be built here), on all
    the host threads this process may use.  A step is the WHOLE workload ([64,512,4096]) when the run then ends within
    a few minutes, else a leading-axis slice of it (stated in the line); throughput is per algorithmic byte."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import cpu_ref
    cores = cpu_ref.use_all_host_threads()
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 3))
    # size the step from a probe on 4 slices
    px, pb, py = cpu_workload(4)
    cpu_ref.gelu_chain(px, pb, py, variant="rp")
    t0 = time.perf_counter()
    cpu_ref.gelu_chain(px, pb, py, variant="rp")
    per_slice = (time.perf_counter() - t0) / 4
    del px, py
    batches = 64
    while batches > 1 and per_slice * batches * (steps + warmup) > 150.0:
        batches //= 2
    x, bias, y = cpu_workload(batches)
    nbytes = x.nbytes + y.nbytes + bias.nbytes + x.size * 4
    for _ in range(warmup):
        cpu_ref.gelu_chain(x, bias, y, variant="rp")
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_ref.gelu_chain(x, bias, y, variant="rp")
    sec = (time.perf_counter() - t0) / steps
    gbs = nbytes / sec / 1e9
    whole = batches == 64
    sample = (f"each step = {'the whole workload' if whole else f'{batches} of the 64 leading slices'} "
              f"([{batches},512,4096]); OpenMP over {cores} host threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD + ("" if whole else f" -- CPU arm: {batches} of its 64 leading slices per step"),
                   "global_shape": [64, 512, 4096], "sample": sample},
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
    cores = C.use_all_host_threads()

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
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the fixed benchmark shapes over the ranks (strong) or give every rank the full "
                         "single-GPU shape (weak)")
    ap.add_argument("--no-classes", action="store_true", help="skip the per-class table")
    ap.add_argument("--only", default="", help="comma-separated class keys: restrict the per-class table to them")
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
