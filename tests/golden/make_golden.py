"""Generates the golden fixtures in this directory from the reference's own
expected-value generator.

Run where a checkout of the reference is available; point ``AKG_REFERENCE`` at its root::

    AKG_REFERENCE=<checkout> python tests/golden/make_golden.py          # the benchmark classes
    python tests/golden/make_golden.py corpus   # the reference's own system-test descriptions -> corpus/
    python tests/golden/make_golden.py ops      # small regions over the whole op surface -> ops/

For every case it builds a fused-op description, draws seeded inputs, feeds
both through ``gen_json_data`` of
``akg-mlir/python/akg_mlir/utils/composite_op_helper.py`` (the generator the
reference's ``akg_benchmark`` compares every backend against) and stores
description + inputs + expected outputs in ``<case>.npz``.  Nothing of the
reference is copied: only its outputs are recorded.

bfloat16 tensors are stored as their uint16 bit patterns (key suffix
``__bf16``), because ``.npz`` cannot hold the ml_dtypes type portably.
"""
from __future__ import annotations

import json
import os
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from akg_b200 import descs  # noqa: E402
sys.path.insert(0, str(HERE.parent))
from helpers import corpus_inputs  # noqa: E402


def _reference_root() -> Path:
    root = os.environ.get("AKG_REFERENCE")
    if not root:
        raise SystemExit("set AKG_REFERENCE to the root of a checkout of the reference")
    return Path(root)


def _import_reference():
    ref = _reference_root() / "akg-mlir" / "python" / "akg_mlir"
    if not ref.exists():
        raise SystemExit(f"reference checkout not found at {ref}")
    import ml_dtypes
    shim = types.ModuleType("bfloat16")
    shim.bfloat16 = ml_dtypes.bfloat16
    sys.modules["bfloat16"] = shim
    pkg = types.ModuleType("akg")  # the wheel installs akg_mlir under this name
    pkg.__path__ = [str(ref)]
    sys.modules["akg"] = pkg
    os.environ["PROFILING_MODE"] = "true"  # keeps the input generator single-process
    from akg.utils import composite_op_helper  # type: ignore
    return composite_op_helper


def _inputs_for(desc: dict, seed: int, kinds: dict) -> list[np.ndarray]:
    import ml_dtypes
    rng = np.random.default_rng(seed)
    out = []
    for (d,) in desc["input_desc"]:
        shape, dt, name = d["shape"], d["data_type"], d["tensor_name"]
        kind = kinds.get(name, "normal")
        if kind == "all_f16":
            bits = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
            out.append(np.ascontiguousarray(bits[np.isfinite(bits)]))
            continue
        if kind == "normal":
            a = rng.standard_normal(shape)
        elif kind == "normal_small":
            a = rng.standard_normal(shape) * 0.02
        elif kind == "gamma":
            a = rng.uniform(0.5, 1.5, shape)
        elif kind == "beta":
            a = rng.uniform(-0.1, 0.1, shape)
        elif kind == "causal":
            a = np.where(np.tril(np.ones(shape, dtype=bool)), 0.0, -np.inf)
        else:
            raise ValueError(kind)
        npdt = ml_dtypes.bfloat16 if dt == "bfloat16" else np.dtype(dt)
        out.append(np.ascontiguousarray(a.astype(npdt)))
    return out


CASES = {
    # name: (description, input kinds, seed)
    "layernorm_64x256": (descs.layernorm(64, 256), {"gamma": "gamma", "beta": "beta"}, 0),
    "layernorm_7x100_nostats": (descs.layernorm(7, 100, with_stats=False), {"gamma": "gamma", "beta": "beta"}, 1),
    "gelu_4x16x128": (descs.gelu_chain([4, 16, 128]), {"bias": "normal_small"}, 0),
    "gelu_3x5x24_nobias": (descs.gelu_chain([3, 5, 24], with_bias=False), {}, 2),
    "softmax_2x64x128": (descs.masked_softmax(2, 64, 128), {"mask": "causal"}, 0),
    "softmax_f32_3x8x40_nomask": (descs.masked_softmax(3, 8, 40, dtype="float32", with_mask=False), {}, 3),
    "reduce_sum0_256x128": (descs.reduce_sum_axis0(256, 128), {}, 0),
    "reduce_max_all_256x128": (descs.reduce_max_all(256, 128), {}, 0),
    "reduce_both_100x52": (descs.reduce_sum_and_max(100, 52), {}, 4),
    "matmul_128x64x128": (descs.matmul_bias_relu(128, 64, 128),
                          {"a": "normal_small", "b": "normal_small", "bias": "normal_small"}, 0),
    "transpose_2x8x4x16": (descs.transpose([2, 8, 4, 16], [0, 2, 1, 3]), {}, 0),
    "tanh_f16_all": (descs.unary("Tanh", [63488], "float16"), {"x": "all_f16"}, 0),
    "transpose_6x10_true": (descs.transpose([6, 10], [1, 0], "float32"), {}, 5),
}


def main():
    helper = _import_reference()
    cwd = os.getcwd()
    os.chdir("/tmp")  # the generator writes a scratch .py next to the cwd
    try:
        for name, (desc, kinds, seed) in CASES.items():
            inputs = _inputs_for(desc, seed, kinds)
            text = json.dumps(desc)
            _, expect, _ = helper.gen_json_data(text, True, input_for_mod=[a.copy() for a in inputs])
            blob = {"desc": np.frombuffer(text.encode(), dtype=np.uint8)}
            for i, a in enumerate(inputs):
                _store(blob, f"in{i}", a)
            for i, e in enumerate(expect):
                e = np.ascontiguousarray(np.asarray(e)).reshape(desc["output_desc"][i]["shape"])
                _store(blob, f"out{i}", e)
            np.savez_compressed(HERE / f"{name}.npz", **blob)
            print(f"{name}: {len(inputs)} inputs, {len(expect)} outputs")
    finally:
        os.chdir(cwd)


def _op_cases():
    """Small regions that together touch the op surface of the JSON factory, for fixtures under ops/."""
    from akg_b200.descs import _Builder, _attr, _reduce_attr
    f, h = "float32", "float16"
    cases = {}

    def unary_chain(name, ops, shape=(6, 40), dtype=f):
        b = _Builder(f"Fused_{name}_1")
        t = b.input("x", list(shape), dtype)
        for op in ops:
            t = b.emit(op, [t], list(shape), dtype)
        b.output(t)
        cases[name] = b.build()

    unary_chain("abs_neg_floor", ["Abs", "Neg", "Floor"])
    unary_chain("exp_log_sqrt", ["Abs", "Exp", "Log", "Sqrt"])
    unary_chain("rsqrt_reciprocal", ["Abs", "Rsqrt", "Reciprocal"])
    unary_chain("sin_cos", ["Sin", "Cos"])
    unary_chain("asinh", ["Asinh"])
    unary_chain("tanh_f32", ["Tanh"])

    b = _Builder("Fused_binary_2")
    x, y = b.input("x", [5, 33], f), b.input("y", [33], f)
    t = b.emit("Add", [x, y], [5, 33], f)
    t = b.emit("Sub", [t, b.const(0.5, f)], [5, 33], f)
    t = b.emit("Mul", [t, y], [5, 33], f)
    t = b.emit("RealDiv", [t, b.const(3.0, f)], [5, 33], f)
    t = b.emit("Maximum", [t, x], [5, 33], f)
    t = b.emit("Minimum", [t, b.const(1.25, f)], [5, 33], f)
    b.output(t)
    cases["binary_broadcast"] = b.build()

    b = _Builder("Fused_pow_atan2_3")
    x, y = b.input("x", [4, 16], f), b.input("y", [4, 16], f)
    p = b.emit("Pow", [b.emit("Abs", [x], [4, 16], f), b.const(1.5, f)], [4, 16], f)
    b.output(b.emit("Atan2", [p, y], [4, 16], f))
    cases["pow_atan2"] = b.build()

    b = _Builder("Fused_compare_select_4")
    x, y = b.input("x", [7, 24], f), b.input("y", [7, 24], f)
    gt = b.emit("Greater", [x, y], [7, 24], "bool")
    le = b.emit("LessEqual", [x, b.const(0.0, f)], [7, 24], "bool")
    both = b.emit("LogicalOr", [b.emit("LogicalAnd", [gt, le], [7, 24], "bool"),
                                b.emit("LogicalNot", [gt], [7, 24], "bool")], [7, 24], "bool")
    b.output(b.emit("Select", [both, x, y], [7, 24], f))
    b.output(b.emit("Equal", [x, y], [7, 24], "bool"))
    b.output(b.emit("NotEqual", [x, b.const(0.0, f)], [7, 24], "bool"))
    b.output(b.emit("GreaterEqual", [x, y], [7, 24], "bool"))
    b.output(b.emit("Less", [x, y], [7, 24], "bool"))
    cases["compare_select"] = b.build()

    b = _Builder("Fused_isnan_5")
    x = b.input("x", [64], f)
    b.output(b.emit("IsNan", [x], [64], "bool"))
    b.output(b.emit("IsInf", [x], [64], "bool"))
    b.output(b.emit("IsFinite", [x], [64], "bool"))
    cases["isnan_isinf"] = b.build()

    b = _Builder("Fused_casts_6")
    i32, hx, bl = b.input("i", [3, 20], "int32"), b.input("hx", [3, 20], h), b.input("bl", [3, 20], "bool")
    a = b.emit("Cast", [i32], [3, 20], f, [_attr("dst_type", "str", f)])
    c = b.emit("Cast", [hx], [3, 20], f, [_attr("dst_type", "str", f)])
    d = b.emit("Cast", [bl], [3, 20], f, [_attr("dst_type", "str", f)])
    t = b.emit("Add", [b.emit("Mul", [a, c], [3, 20], f), d], [3, 20], f)
    b.output(b.emit("Cast", [t], [3, 20], h, [_attr("dst_type", "str", h)]))
    cases["casts"] = b.build()

    for name, op, axes, keep, oshape in (("reduce_min_x", "ReduceMin", [1], True, [9, 1]),
                                         ("reduce_prod_y", "ReduceProd", [0], False, [50]),
                                         ("reduce_max_all", "ReduceMax", [0, 1], False, [1])):
        b = _Builder(f"Fused_{name}_7")
        x = b.input("x", [9, 50], f)
        b.output(b.emit(op, [x], oshape, f, _reduce_attr(axes, keep)))
        cases[name] = b.build()

    b = _Builder("Fused_reduce_all_8")
    x = b.input("x", [12, 30], "bool")
    b.output(b.emit("ReduceAll", [x], [30], "bool", _reduce_attr([0], False)))
    cases["reduce_all_bool"] = b.build()

    b = _Builder("Fused_shapes_9")
    x, r = b.input("x", [4, 6, 10], f), b.input("r", [4, 1, 1], f)
    t = b.emit("Reshape", [x], [24, 10], f, [_attr("shape", "listInt", [24, 10])])
    t = b.emit("Transpose", [t], [10, 24], f, [_attr("perm", "listInt", [1, 0])])
    bc = b.emit("BroadcastTo", [r], [4, 6, 10], f, [_attr("shape", "listInt", [4, 6, 10])])
    b.output(t)
    b.output(b.emit("Add", [x, bc], [4, 6, 10], f))
    cases["reshape_transpose_broadcast"] = b.build()

    b = _Builder("Fused_tile_slice_10")
    x = b.input("x", [3, 8], f)
    t = b.emit("Tile", [x], [6, 16], f, [_attr("multiples", "listInt", [2, 2])])
    s1 = b.emit("Slice", [t], [4, 8], f, [_attr("begin", "listInt", [1, 4]), _attr("size", "listInt", [4, 8])])
    s2 = b.emit("StridedSlice", [t], [3, 8], f, [_attr("begin", "listInt", [0, 0]), _attr("end", "listInt", [6, 16]),
                                                 _attr("strides", "listInt", [2, 2])])
    b.output(s1)
    b.output(s2)
    cases["tile_slice_strided"] = b.build()

    b = _Builder("Fused_concat_addn_11")
    x, y, z = b.input("x", [4, 5], f), b.input("y", [4, 7], f), b.input("z", [4, 5], f)
    b._n += 1
    cat = {"tensor_name": "cat", "shape": [4, 12], "data_type": f, "format": "DefaultFormat"}
    b.ops.append({"name": "Concat", "attr": [_attr("axis", "int", 1)], "impl_path": "",
                  "input_desc": [[dict(x), dict(y)]], "output_desc": [dict(cat)]})
    add = {"tensor_name": "addn", "shape": [4, 5], "data_type": f, "format": "DefaultFormat"}
    b.ops.append({"name": "AddN", "attr": None, "impl_path": "",
                  "input_desc": [[dict(x), dict(z), dict(x)]], "output_desc": [dict(add)]})
    b.output(cat)
    b.output(add)
    cases["concat_addn"] = b.build()

    b = _Builder("Fused_gather_12")
    table, idx = b.input("table", [50, 16], f), b.input("idx", [3, 7], "int32")
    b.output(b.emit("Gather", [table, idx], [3, 7, 16], f, [_attr("axis", "int", 0), _attr("batch_dims", "int", 0)]))
    cases["gather_rows"] = b.build()

    b = _Builder("Fused_segsum_13")
    data, ids = b.input("data", [40, 8], f), b.input("ids", [40], "int32")
    b.output(b.emit("UnsortedSegmentSum", [data, ids], [6, 8], f, [_attr("num_segments", "int", 6)]))
    cases["unsorted_segment_sum"] = b.build()

    b = _Builder("Fused_batchmatmul_14")
    a, w = b.input("a", [3, 16, 24], h), b.input("w", [3, 24, 8], h)
    b.output(b.emit("BatchMatMul", [a, w], [3, 16, 8], f,
                    [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)]))
    cases["batch_matmul_f16"] = b.build()

    b = _Builder("Fused_assign_15")
    dst, val = b.input("dst", [5, 12], f), b.input("val", [5, 12], f)
    t = b.emit("Mul", [val, b.const(2.0, f)], [5, 12], f)
    a = b.emit("Assign", [dst, t], [5, 12], f)
    b.output(b.emit("Add", [a, b.const(1.0, f)], [5, 12], f))
    cases["assign"] = b.build()

    # reduce-X / reduce-Y regions that run as generated row and column kernels
    cases["rmsnorm_33x200"] = descs.rmsnorm(33, 200)
    cases["rmsnorm_f16_16x512"] = descs.rmsnorm(16, 512, "float16")
    cases["mul_reduce_rows_300x264"] = descs.mul_reduce_sum(300, 264, [0])
    cases["mul_reduce_all_300x264"] = descs.mul_reduce_sum(300, 264, [0, 1])
    b = _Builder("Fused_LogSoftmax_16")
    x = b.input("x", [5, 12, 96], f)
    m = b.emit("ReduceMax", [x], [5, 12, 1], f, _reduce_attr([2], True))
    d = b.emit("Sub", [x, m], [5, 12, 96], f)
    e = b.emit("ReduceSum", [b.emit("Exp", [d], [5, 12, 96], f)], [5, 12, 1], f, _reduce_attr([2], True))
    b.output(b.emit("Sub", [d, b.emit("Log", [e], [5, 12, 1], f)], [5, 12, 96], f))
    cases["log_softmax_5x12x96"] = b.build()

    # NCHW regions: BatchNorm statistics (chain + reduction over (0, 2, 3) + scaling), InstanceNorm with per-channel
    # scale and shift, a reduction over non-adjacent axes, a region that is a row region only in part
    nchw, stat = [8, 32, 16, 16], [1, 32, 1, 1]
    b = _Builder("Fused_BNStats_17")
    x = b.input("x", nchw, f)
    mean_in = b.input("mean", stat, f)
    dlt = b.emit("Sub", [x, mean_in], nchw, f)
    s2 = b.emit("ReduceSum", [b.emit("Mul", [dlt, dlt], nchw, f)], stat, f, _reduce_attr([0, 2, 3], True))
    b.output(b.emit("Mul", [s2, b.const(1.0 / (8 * 16 * 16), f)], stat, f))
    cases["bn_variance_nchw"] = b.build()

    b = _Builder("Fused_InstanceNorm_18")
    x, gamma, beta = b.input("x", nchw, f), b.input("gamma", stat, f), b.input("beta", stat, f)
    red = [8, 32, 1, 1]
    inv = b.const(1.0 / 256, f)
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], red, f, _reduce_attr([2, 3], True)), inv], red, f)
    dlt = b.emit("Sub", [x, mean], nchw, f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [dlt, dlt], nchw, f)], red, f, _reduce_attr([2, 3], True)), inv], red, f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], red, f)], red, f)
    b.output(b.emit("Add", [b.emit("Mul", [b.emit("Mul", [dlt, rstd], nchw, f), gamma], nchw, f), beta], nchw, f))
    cases["instance_norm_nchw"] = b.build()

    b = _Builder("Fused_ReduceNonAdjacent_19")
    x = b.input("x", [6, 40, 50], f)
    b.output(b.emit("ReduceSum", [x], [1, 40, 1], f, _reduce_attr([0, 2], True)))
    b.output(b.emit("ReduceMax", [x], [40], f, _reduce_attr([0, 2], False)))
    cases["reduce_non_adjacent"] = b.build()

    b = _Builder("Fused_Softmax_Transpose_20")
    x = b.input("x", [6, 10, 128], f)
    m = b.emit("ReduceMax", [x], [6, 10, 1], f, _reduce_attr([2], True))
    e = b.emit("Exp", [b.emit("Sub", [x, m], [6, 10, 128], f)], [6, 10, 128], f)
    p = b.emit("RealDiv", [e, b.emit("ReduceSum", [e], [6, 10, 1], f, _reduce_attr([2], True))], [6, 10, 128], f)
    t = b.emit("Transpose", [p], [10, 6, 128], f, [_attr("perm", "listInt", [1, 0, 2])])
    b.output(b.emit("Mul", [t, b.const(0.5, f)], [10, 6, 128], f))
    cases["softmax_transpose_scale"] = b.build()

    # batch normalisation in training mode: three reductions' worth of pieces, the centred values used twice
    b = _Builder("Fused_BatchNormTraining_21")
    x, gamma, beta = b.input("x", nchw, f), b.input("gamma", stat, f), b.input("beta", stat, f)
    inv = b.const(1.0 / (8 * 16 * 16), f)
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], stat, f, _reduce_attr([0, 2, 3], True)), inv], stat, f)
    dlt = b.emit("Sub", [x, mean], nchw, f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [dlt, dlt], nchw, f)], stat, f, _reduce_attr([0, 2, 3], True)), inv], stat, f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], stat, f)], stat, f)
    b.output(b.emit("Add", [b.emit("Mul", [b.emit("Mul", [dlt, rstd], nchw, f), gamma], nchw, f), beta], nchw, f))
    b.output(mean)
    b.output(rstd)
    cases["batch_norm_training_nchw"] = b.build()

    # rows too long for a thread group's registers
    b = _Builder("Fused_LogSoftmax_22")
    x = b.input("x", [3, 20000], f)
    m = b.emit("ReduceMax", [x], [3, 1], f, _reduce_attr([1], True))
    d = b.emit("Sub", [x, m], [3, 20000], f)
    e = b.emit("ReduceSum", [b.emit("Exp", [d], [3, 20000], f)], [3, 1], f, _reduce_attr([1], True))
    b.output(b.emit("Sub", [d, b.emit("Log", [e], [3, 1], f)], [3, 20000], f))
    cases["log_softmax_long_rows"] = b.build()

    b = _Builder("Fused_RMSNorm_23")
    x, g_ = b.input("x", [2, 16392], h), b.input("g", [16392], h)
    xf = b.emit("Cast", [x], [2, 16392], f, [_attr("dst_type", "str", f)])
    ms = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [xf, xf], [2, 16392], f)], [2, 1], f, _reduce_attr([1], True)),
                        b.const(1.0 / 16392, f)], [2, 1], f)
    y = b.emit("Mul", [xf, b.emit("Rsqrt", [b.emit("Add", [ms, b.const(1e-6, f)], [2, 1], f)], [2, 1], f)], [2, 16392], f)
    y = b.emit("Mul", [y, b.emit("Cast", [g_], [16392], f, [_attr("dst_type", "str", f)])], [2, 16392], f)
    b.output(b.emit("Cast", [y], [2, 16392], h, [_attr("dst_type", "str", h)]))
    cases["rmsnorm_long_rows_f16"] = b.build()
    return cases


def ops():
    """Golden vectors for `_op_cases()`, from the reference's expected-value generator, under ops/."""
    helper = _import_reference()
    outdir = HERE / "ops"
    outdir.mkdir(exist_ok=True)
    cwd = os.getcwd()
    os.chdir("/tmp")
    made = 0
    try:
        for k, (name, desc) in enumerate(sorted(_op_cases().items())):
            seed = 500 + k
            inputs = corpus_inputs(desc, seed)
            if name == "isnan_isinf":
                inputs[0][::7] = np.nan
                inputs[0][3::11] = np.inf
            text = json.dumps(desc)
            try:
                _, expect, _ = helper.gen_json_data(text, True, input_for_mod=[a.copy() for a in inputs])
            except Exception as e:
                print(f"skip {name}: expected-value generator raised {type(e).__name__}: {str(e)[:100]}")
                continue
            expect = expect if isinstance(expect, (list, tuple)) else [expect]
            blob = {"desc": np.frombuffer(text.encode(), dtype=np.uint8), "seed": np.asarray(seed)}
            try:
                for i, e in enumerate(expect):
                    shape = desc["output_desc"][i].get("shape") or [1]
                    _store(blob, f"out{i}", np.ascontiguousarray(np.asarray(e)).reshape(shape))
            except (ValueError, IndexError) as e:
                print(f"skip {name}: expected values do not fit the declared outputs ({e})")
                continue
            np.savez_compressed(outdir / f"{name}.npz", **blob)
            made += 1
            print(f"{name}: {len(inputs)} inputs, {len(expect)} outputs")
    finally:
        os.chdir(cwd)
    print(made, "op fixtures")


def _bind_by_position(desc: dict) -> dict:
    by_pos = {1: 24, 2: 10, 3: 12, 4: 32}

    def fix(t):
        if isinstance(t, dict):
            if isinstance(t.get("shape"), list):
                r = len(t["shape"])
                t["shape"] = [by_pos.get(r - i, 8) if e < 0 else e for i, e in enumerate(t["shape"])]
            for v in t.values():
                fix(v)
        elif isinstance(t, list):
            for v in t:
                fix(v)

    d = json.loads(json.dumps(desc))
    fix(d)
    return d


def corpus(max_bytes: int = 2 << 20):
    """Golden vectors for the fused-operator descriptions of the reference's own system tests
    (akg-mlir/tests/st/**/*.info*): static shapes, at most `max_bytes` of tensors, evaluated by the reference's
    expected-value generator on seeded inputs.  Stored under corpus/ as description + input seed + expected outputs."""
    helper = _import_reference()
    ref = _reference_root() / "akg-mlir" / "tests" / "st"
    outdir = HERE / "corpus"
    outdir.mkdir(exist_ok=True)
    cwd = os.getcwd()
    os.chdir("/tmp")
    made = 0
    try:
        for f in sorted(ref.rglob("*.info*")):
            desc = json.loads(f.read_text())
            tensors = [d for (d,) in desc["input_desc"] or []] + list(desc["output_desc"])
            shapes = [t.get("shape") or [1] for t in tensors]
            dynamic_text = None
            if any(e < 0 for s in shapes for e in s):
                # dynamic extents: the expected values are computed on a static copy in which an unknown extent
                # becomes 24 / 10 / 12 / 32 by its position from the end; the fixture keeps the dynamic description
                # too, for the launch-time binding path
                dynamic_text = json.dumps(desc)
                desc = _bind_by_position(desc)
                tensors = [d for (d,) in desc["input_desc"] or []] + list(desc["output_desc"])
                shapes = [t.get("shape") or [1] for t in tensors]
            itemsize = {"bool": 1, "int8": 1, "uint8": 1, "float16": 2, "bfloat16": 2, "int16": 2, "float64": 8,
                        "int64": 8}
            total = sum(int(np.prod(s)) * itemsize.get(t["data_type"], 4) for s, t in zip(shapes, tensors))
            if total > max_bytes:
                print(f"skip {f.name}: {total} bytes of tensors")
                continue
            seed = 100 + made
            inputs = corpus_inputs(desc, seed)
            text = json.dumps(desc)
            try:
                _, expect, _ = helper.gen_json_data(text, True, input_for_mod=[a.copy() for a in inputs])
            except Exception as e:  # the reference's generator itself fails on some of its disabled cases
                print(f"skip {f.name}: expected-value generator raised {type(e).__name__}: {str(e)[:80]}")
                continue
            expect = expect if isinstance(expect, (list, tuple)) else [expect]
            blob = {"desc": np.frombuffer(text.encode(), dtype=np.uint8)}
            if dynamic_text is not None:
                blob["desc_dynamic"] = np.frombuffer(dynamic_text.encode(), dtype=np.uint8)
            blob["seed"] = np.asarray(seed)  # the inputs are redrawn from it (tests/helpers.py::corpus_inputs)
            try:
                for i, e in enumerate(expect):
                    shape = desc["output_desc"][i].get("shape") or [1]
                    _store(blob, f"out{i}", np.ascontiguousarray(np.asarray(e)).reshape(shape))
            except ValueError as e:
                print(f"skip {f.name}: expected values do not have the declared shapes ({e})")
                continue
            name = f.name.split(".info")[0]
            np.savez_compressed(outdir / f"{name}.npz", **blob)
            made += 1
            print(f"{name}: {len(inputs)} inputs, {len(expect)} outputs, {total} bytes")
    finally:
        os.chdir(cwd)
    print(made, "corpus fixtures")


def _store(blob, key, a):
    if a.dtype.name == "bfloat16":
        blob[key + "__bf16"] = a.view(np.uint16)
    else:
        blob[key] = a


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "corpus":
        corpus()
    elif len(sys.argv) > 1 and sys.argv[1] == "ops":
        ops()
    else:
        main()
