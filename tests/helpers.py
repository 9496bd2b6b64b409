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


def corpus_inputs(desc: dict, seed: int) -> list[np.ndarray]:
    """Seeded inputs for a description of the reference's system-test corpus, by type; indices of
    UnsortedSegmentSum / Gather stay inside their axis."""
    rng = np.random.default_rng(seed)
    index_limit = {}
    for op in desc["op_desc"]:
        if op["name"] == "UnsortedSegmentSum":
            ids = op["input_desc"][1][0]["tensor_name"]
            index_limit[ids] = op["output_desc"][0]["shape"][0]
        if op["name"] == "Gather":
            axis = next((a["value"] for a in (op.get("attr") or []) if a["name"] == "axis"), 0)
            index_limit[op["input_desc"][1][0]["tensor_name"]] = op["input_desc"][0][0]["shape"][axis]
    positive = any(op["name"] in ("Sqrt", "Rsqrt", "Log") for op in desc["op_desc"])
    out = []
    for (d,) in desc["input_desc"]:
        shape, dt, name = d.get("shape") or [1], d["data_type"], d["tensor_name"]
        if name in index_limit:
            a = rng.integers(0, index_limit[name], shape)
        elif dt == "bool":
            a = rng.integers(0, 2, shape)
        elif dt.startswith("int") or dt.startswith("uint"):
            a = rng.integers(-5, 6, shape)
        else:
            a = rng.uniform(0.25, 1.75, shape)  # away from 0: the corpus divides
            if not positive:
                a = a * rng.choice([-1.0, 1.0], shape)
        npdt = BF16 if dt == "bfloat16" else np.dtype(dt)
        out.append(np.ascontiguousarray(a.astype(npdt)))
    return out


def ops_cases():
    return sorted(p.stem for p in (GOLDEN / "ops").glob("*.npz"))


def load_ops(name):
    """(description, inputs, expected outputs) of one op-surface fixture (tests/golden/make_golden.py ops)."""
    z = np.load(GOLDEN / "ops" / f"{name}.npz")
    desc = json.loads(bytes(z["desc"]).decode())
    ins = corpus_inputs(desc, int(z["seed"]))
    if name == "isnan_isinf":
        ins[0][::7] = np.nan
        ins[0][3::11] = np.inf
    outs = [z[f"out{i}"] if f"out{i}" in z else z[f"out{i}__bf16"].view(BF16) for i in range(len(desc["output_desc"]))]
    return desc, ins, outs


def corpus_cases():
    return sorted(p.stem for p in (GOLDEN / "corpus").glob("*.npz"))


def load_corpus(name):
    """(static description, dynamic description or None, inputs, expected outputs) of one corpus fixture."""
    z = np.load(GOLDEN / "corpus" / f"{name}.npz")
    desc = json.loads(bytes(z["desc"]).decode())
    dyn = json.loads(bytes(z["desc_dynamic"]).decode()) if "desc_dynamic" in z else None
    ins = corpus_inputs(desc, int(z["seed"]))
    outs = [z[f"out{i}"] if f"out{i}" in z else z[f"out{i}__bf16"].view(BF16) for i in range(len(desc["output_desc"]))]
    return desc, dyn, ins, outs


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


GUARD_BYTES = 4096
GUARD_PATTERN = 0xA5


def guarded_launch(desc, ins, flags=0):
    """One device launch with every tensor (inputs, outputs, workspace) placed between two guard zones.

    The sanitizer tools are not available on every machine these tests run on, so the tests carry their own evidence
    that kernels stay inside their buffers: each tensor sits at `GUARD_BYTES` inside a larger device allocation whose
    first and last `GUARD_BYTES` hold a known pattern (the zone behind a tensor starts at its last byte + 1, not at
    an aligned boundary, so a vector store that overshoots a ragged tail is caught too).  After the launch every guard
    zone must be intact and every input that the region does not store into unchanged.  Returns (outputs as numpy
    arrays, kernel)."""
    import torch
    from akg_b200 import FusedKernel
    k = FusedKernel(desc, flags=flags)
    dev = torch.device("cuda", torch.cuda.current_device())
    bufs, ptrs = [], []

    def alloc(nbytes, fill):
        b = torch.full((GUARD_BYTES + nbytes + GUARD_BYTES,), GUARD_PATTERN, dtype=torch.uint8, device=dev)
        if nbytes:
            b[GUARD_BYTES:GUARD_BYTES + nbytes] = fill
        assert b.data_ptr() % 256 == 0
        return b

    host_in = []
    for a, t in zip(ins, k.inputs):
        raw = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
        assert raw.size == t.nbytes, (t.name, raw.size, t.nbytes)
        b = alloc(t.nbytes, 0)
        if t.nbytes:
            b[GUARD_BYTES:GUARD_BYTES + t.nbytes] = torch.from_numpy(raw.copy()).to(dev)
        bufs.append(b)
        host_in.append(raw)
    for t in k.outputs:
        bufs.append(alloc(t.nbytes, 0xCD))
    ws = alloc(k.workspace_size, 0xCD)
    k.launch_ptrs([b.data_ptr() + GUARD_BYTES for b in bufs], ws.data_ptr() + GUARD_BYTES if k.workspace_size else 0,
                  k.workspace_size, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert k.check_device_error() == 0
    for b, t in zip(bufs + [ws], list(k.tensors) + [None]):
        name = t.name if t is not None else "workspace"
        n = t.nbytes if t is not None else k.workspace_size
        front, back = b[:GUARD_BYTES], b[GUARD_BYTES + n:]
        assert bool((front == GUARD_PATTERN).all()), f"bytes in front of '{name}' were overwritten"
        assert bool((back == GUARD_PATTERN).all()), f"bytes behind '{name}' were overwritten"
    for b, raw, t in zip(bufs, host_in, k.inputs):
        if not t.written_in_place and t.nbytes:
            assert np.array_equal(b[GUARD_BYTES:GUARD_BYTES + t.nbytes].cpu().numpy(), raw), f"input '{t.name}' was modified"
    outs = []
    for b, t in zip(bufs[k.num_inputs:], k.outputs):
        dt = BF16 if t.dtype == "bfloat16" else np.dtype(t.dtype)
        outs.append(b[GUARD_BYTES:GUARD_BYTES + t.nbytes].cpu().numpy().view(dt).reshape(t.shape))
    return outs, k
