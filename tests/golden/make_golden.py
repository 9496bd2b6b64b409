"""Generates the golden fixtures in this directory from the reference's own
expected-value generator.

Run in a container where the reference checkout is mounted (default
``/root/reference``, override with ``AKG_REFERENCE``)::

    python tests/golden/make_golden.py          # the benchmark classes
    python tests/golden/make_golden.py corpus   # the reference's own system-test descriptions -> corpus/

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


def _import_reference():
    ref = Path(os.environ.get("AKG_REFERENCE", "/root/reference")) / "akg-mlir" / "python" / "akg_mlir"
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
    ref = Path(os.environ.get("AKG_REFERENCE", "/root/reference")) / "akg-mlir" / "tests" / "st"
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
    else:
        main()
