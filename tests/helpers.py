"""Shared test helpers: golden fixtures, seeded inputs with the benchmark's distributions, tolerances."""
from __future__ import annotations

import json
from pathlib import Path

import ml_dtypes
import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"
BF16 = np.dtype(ml_dtypes.bfloat16)


def golden_cases():
    return sorted(p.stem for p in GOLDEN.glob("*.npz"))


def load_golden(name):
    z = np.load(GOLDEN / f"{name}.npz")
    desc = json.loads(bytes(z["desc"]).decode())

    def get(key):
        if key in z:
            return z[key]
        return z[key + "__bf16"].view(BF16)

    ins = [get(f"in{i}") for i in range(len(desc["input_desc"]))]
    outs = [get(f"out{i}") for i in range(len(desc["output_desc"]))]
    return desc, ins, outs


def make_inputs(desc, seed=0, kinds=None):
    """Seeded inputs: N(0,1) unless `kinds` says otherwise (names as in tests/golden/make_golden.py)."""
    kinds = kinds or {}
    rng = np.random.default_rng(seed)
    out = []
    for (d,) in desc["input_desc"]:
        shape, dt, name = d["shape"], d["data_type"], d["tensor_name"]
        kind = kinds.get(name, "normal")
        if kind == "normal":
            a = rng.standard_normal(shape, dtype=np.float32)
        elif kind == "normal_small":
            a = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        elif kind == "gamma":
            a = rng.uniform(0.5, 1.5, shape)
        elif kind == "beta":
            a = rng.uniform(-0.1, 0.1, shape)
        elif kind == "causal":
            a = np.where(np.tril(np.ones(shape, dtype=bool)), 0.0, -np.inf)
        else:
            raise ValueError(kind)
        npdt = BF16 if dt == "bfloat16" else np.dtype(dt)
        out.append(np.ascontiguousarray(a.astype(npdt)))
    return out


KINDS = {
    "layernorm": {"gamma": "gamma", "beta": "beta"},
    "gelu": {"bias": "normal_small"},
    "softmax": {"mask": "causal"},
    "matmul": {"a": "normal_small", "b": "normal_small", "bias": "normal_small"},
}


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.dtype == b.dtype and a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def ulp_diff_f16(a, b):
    """Distance in float16 steps between two float16 arrays (sign-magnitude aware)."""
    def key(x):
        i = x.view(np.int16).astype(np.int32)
        return np.where(i < 0, -(i & 0x7FFF), i)
    return np.abs(key(a) - key(b))
