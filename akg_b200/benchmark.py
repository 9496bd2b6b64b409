"""Command-line harness in the spirit of the reference's ``akg_benchmark``
(``akg-mlir/python/akg_mlir/tools/benchmark.py:249-329``): take a fused-op
description, generate inputs, compile, run on the GPU and report timing.

    python -m akg_b200.benchmark -f Fused_xxx.info [--repeat 20]
    python -m akg_b200.benchmark --case softmax --shape 32,2048,2048 [--repeat 3]

``--case`` builds one of the benchmarked descriptions (``akg_b200.descs``)
instead of reading a file; small shapes make short, profiler-friendly runs.
Inputs follow the reference generator's convention (normal values, sigma 0.1,
``akg-mlir/python/akg_mlir/utils/gen_random.py:84-136``) unless the case names
its own distributions.  The numeric comparison the reference harness does
against its NumPy expectations lives in this repository's tests, not here.
"""
from __future__ import annotations

import argparse
import json
import sys

from . import descs
from .driver import FusedKernel

CASES = {
    "gelu": (lambda s: descs.gelu_chain(s), {"bias": "normal_small"}),
    "gelu_f32math": (lambda s: descs.gelu_chain(s, f32_math=True), {"bias": "normal_small"}),
    "layernorm": (lambda s: descs.layernorm(s[0], s[1]), {"gamma": "gamma", "beta": "beta"}),
    "softmax": (lambda s: descs.masked_softmax(s[0], s[1], s[2]), {"mask": "causal"}),
    "colsum": (lambda s: descs.reduce_sum_axis0(s[0], s[1]), {}),
    "gmax": (lambda s: descs.reduce_max_all(s[0], s[1]), {}),
    "transpose": (lambda s: descs.transpose(s, [0, 2, 1, 3]), {}),
    # the last two axes swapped (the innermost output axis is strided in the input); --dtype picks the element type
    "transpose_tile": (lambda s, dtype="float16": descs.transpose(s, list(range(len(s) - 2)) + [len(s) - 1, len(s) - 2],
                                                                  dtype), {}),
    "rmsnorm": (lambda s: descs.rmsnorm(s[0], s[1]), {"g": "gamma"}),
    # softmax with every op in the tensor's 16-bit type (--dtype float16 / bfloat16): a generated row kernel
    "softmax_typed": (lambda s, dtype="bfloat16": descs.softmax_rows_typed(s[0], s[1], dtype), {}),
    "mulsum_rows": (lambda s: descs.mul_reduce_sum(s[0], s[1], [0]), {}),
    "mulsum_all": (lambda s: descs.mul_reduce_sum(s[0], s[1], [0, 1]), {}),
    "layernorm_backward": (lambda s: descs.layer_norm_backward(s[0], s[1]), {"gamma": "gamma"}),
    "batchnorm_training": (lambda s: descs.batch_norm_training(s), {"gamma": "gamma", "beta": "beta"}),
    "batchnorm_backward": (lambda s: descs.batch_norm_backward(s), {"gamma": "gamma", "rstd": "gamma"}),
    "matmul": (lambda s, dtype="bfloat16": descs.matmul_bias_relu(s[0], s[1], s[2], dtype=dtype),
               {"a": "normal_small", "b": "normal_small", "bias": "normal_small"}),
}


def _torch_dtype(name):
    import torch
    return {"float16": torch.float16, "float32": torch.float32, "bfloat16": torch.bfloat16, "int8": torch.int8,
            "int16": torch.int16, "int32": torch.int32, "int64": torch.int64, "bool": torch.bool,
            "float64": torch.float64}[name]


def make_device_inputs(kernel: FusedKernel, kinds: dict, seed: int, device):
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = []
    for t in kernel.inputs:
        kind = kinds.get(t.name, "normal_0p1" if not kinds else "normal")
        dt = _torch_dtype(t.dtype)
        if not dt.is_floating_point:
            out.append(torch.randint(-100, 100, t.shape, generator=g, device=device).to(dt))
            continue
        r = torch.randn(t.shape, generator=g, device=device, dtype=torch.float32)
        if kind == "normal":
            a = r
        elif kind == "normal_0p1":
            a = r * 0.1
        elif kind == "normal_small":
            a = r * 0.02
        elif kind == "gamma":
            a = torch.rand(t.shape, generator=g, device=device) + 0.5
        elif kind == "beta":
            a = torch.rand(t.shape, generator=g, device=device) * 0.2 - 0.1
        elif kind == "causal":
            a = torch.where(torch.ones(t.shape, device=device, dtype=torch.bool).tril(), 0.0, float("-inf"))
        else:
            raise ValueError(kind)
        out.append(a.to(dt).contiguous())
    return out


def main(argv=None):
    import torch
    ap = argparse.ArgumentParser(prog="akg_b200.benchmark")
    ap.add_argument("-f", "--file", help="fused-op description (.info JSON)")
    ap.add_argument("--case", choices=sorted(CASES), help="build a benchmarked description instead")
    ap.add_argument("--shape", default="", help="comma-separated extents for --case")
    ap.add_argument("--dtype", default="", help="element type for --case matmul / transpose_tile")
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if bool(args.file) == bool(args.case):
        ap.error("give exactly one of -f/--file and --case")
    if args.file:
        with open(args.file, "r", encoding="utf-8") as f:
            desc = json.load(f)
        kinds = {}
    else:
        shape = [int(x) for x in args.shape.split(",") if x]
        build, kinds = CASES[args.case]
        desc = build(shape, args.dtype) if args.dtype and args.case in ("matmul", "transpose_tile", "softmax_typed") else build(shape)
    torch.cuda.set_device(args.device)
    device = torch.device("cuda", args.device)
    k = FusedKernel(desc, device=args.device)
    bufs = make_device_inputs(k, kinds, 0, device)
    bufs += [torch.empty(t.shape, dtype=_torch_dtype(t.dtype), device=device) for t in k.outputs]
    for _ in range(args.warmup):
        k.launch(bufs)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.repeat):
        k.launch(bufs)
    t1.record()
    torch.cuda.synchronize()
    us = t0.elapsed_time(t1) * 1e3 / max(1, args.repeat)
    row = {"op": desc["op"], "class": k.op_class, "avg_us": round(us, 3), "bytes": k.bytes, "flops": k.flops,
           "launches": k.launch_count, "device_error": k.check_device_error()}
    if k.flops:
        row["tflops"] = round(k.flops / us / 1e6, 2)
    else:
        row["gbs"] = round(k.bytes / us / 1e3, 1)
    row["meta"] = k.meta()
    print(json.dumps(row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
