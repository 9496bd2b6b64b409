"""Seeded random regions of elementwise ops, broadcasts and row reductions: the library (generated kernels and, with
run-time compilation off, the separate launches) against the NumPy restatement."""
import numpy as np
import pytest

from akg_b200 import FusedKernel
from akg_b200.descs import _Builder, _attr, _reduce_attr
from oracle import akg_oracle as O

pytestmark = pytest.mark.gpu

F = "float32"


def random_region(seed, long_rows=False):
    rng = np.random.default_rng(seed)
    lead = [int(v) for v in rng.choice([1, 2, 3, 5, 16, 33], size=int(rng.integers(1, 4)))]
    cols = int(rng.choice([8, 24, 40, 96, 257, 1024]))
    if long_rows:  # rows that do not fit a thread group's registers
        lead = [int(v) for v in rng.choice([1, 2, 3, 7], size=int(rng.integers(1, 3)))]
        cols = int(rng.choice([9000, 12288, 16392, 20000, 33000, 40001, 65536]))
    shape, red = lead + [cols], lead + [1]
    io_dtype = str(rng.choice([F, F, "float16"]))
    b = _Builder(f"Fused_Fuzz_{seed}")
    x = b.input("x", shape, io_dtype)
    full = [x if io_dtype == F else b.emit("Cast", [x], shape, F, [_attr("dst_type", "str", F)])]
    if rng.random() < 0.6:
        y = b.input("y", shape, io_dtype)
        full.append(y if io_dtype == F else b.emit("Cast", [y], shape, F, [_attr("dst_type", "str", F)]))
    cols_in = [b.input("g", [cols], F)] if rng.random() < 0.5 else []
    rows_in = [b.input("r", red, F)] if rng.random() < 0.4 else []
    rowvals = list(rows_in)
    # every declared input takes part at least once
    if len(full) > 1:
        full.append(b.emit(str(rng.choice(["Add", "Mul", "Maximum"])), [full[0], full[1]], shape, F))
    for extra_in in cols_in + rows_in:
        full.append(b.emit(str(rng.choice(["Add", "Mul", "Sub"])), [full[-1], extra_in], shape, F))
    n_ops = int(rng.integers(2, 11))
    for _ in range(n_ops):
        kind = rng.random()
        a = full[int(rng.integers(len(full)))]
        if kind < 0.25:
            op = str(rng.choice(["Abs", "Neg", "Tanh", "Floor", "Sqrt", "Exp"]))
            if op == "Sqrt":
                a = b.emit("Abs", [a], shape, F)
            if op == "Exp":
                a = b.emit("Minimum", [a, b.const(3.0, F)], shape, F)
            full.append(b.emit(op, [a], shape, F))
        elif kind < 0.7:
            op = str(rng.choice(["Add", "Sub", "Mul", "Maximum", "Minimum", "RealDiv"]))
            pool = full + cols_in + rowvals
            other = pool[int(rng.integers(len(pool)))] if rng.random() < 0.8 else b.const(float(rng.uniform(-2, 2)), F)
            if op == "RealDiv":
                oshape = other.get("shape", [1])
                other = b.emit("Add", [b.emit("Abs", [other], oshape, F), b.const(1.0, F)], oshape, F)
            full.append(b.emit(op, [a, other], shape, F))
        elif kind < 0.9:
            op = str(rng.choice(["ReduceSum", "ReduceMax", "ReduceMin"]))
            rv = b.emit(op, [a], red, F, _reduce_attr([len(shape) - 1], True))
            if op == "ReduceSum":
                rv = b.emit("Mul", [rv, b.const(1.0 / cols, F)], red, F)
            rowvals.append(rv)
            comb = str(rng.choice(["Sub", "Mul", "Add"]))
            full.append(b.emit(comb, [a, rv], shape, F))
        else:
            c = b.emit("Greater", [a, full[int(rng.integers(len(full)))]], shape, "bool")
            full.append(b.emit("Select", [c, a, b.const(0.25, F)], shape, F))
    out = full[-1]
    if io_dtype != F:
        out = b.emit("Cast", [out], shape, io_dtype, [_attr("dst_type", "str", io_dtype)])
    b.output(out)
    extra = [v for v in rowvals if v not in rows_in]
    if extra and rng.random() < 0.5:
        b.output(extra[-1])
    if rng.random() < 0.3:  # a sum over all rows beside the row-wise work (a weight gradient)
        src = full[int(rng.integers(len(full)))]
        b.output(b.emit("ReduceSum", [src], [cols], F, _reduce_attr(list(range(len(shape) - 1)), False)))
    desc = b.build()
    ins = []
    for (t,) in desc["input_desc"]:
        a = rng.standard_normal(t["shape"]).astype(np.float32)
        ins.append(a.astype(np.dtype(t["data_type"])))
    return desc, ins, io_dtype


@pytest.mark.parametrize("seed", range(40))
@pytest.mark.parametrize("flags", [0, 1, 8], ids=["generated", "separate", "generated-checked"])
def test_random_region(seed, flags):
    desc, ins, io_dtype = random_region(seed)
    k = FusedKernel(desc, flags=flags)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    want = O.evaluate(desc, ins, accum="float64")
    for g, w in zip(outs, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        g64, w64 = g.astype(np.float64), w.astype(np.float64)
        fin = np.isfinite(w64)
        assert np.array_equal(np.isfinite(g64), fin)
        scale = float(np.abs(w64[fin]).max()) if fin.any() else 1.0
        tol = 5e-3 if w.dtype == np.float16 else 2e-5
        # Floor / Greater / Select are discontinuous: a last-bit difference upstream may flip a few elements
        bad = np.abs(g64 - w64)[fin] > tol * max(scale, 1.0) + tol * np.abs(w64[fin])
        assert bad.mean() <= 2e-3, (seed, float(bad.mean()))


@pytest.mark.parametrize("seed", range(100, 130))
def test_random_long_row_region(seed):
    """The same random regions on rows of 16K-64K elements: the generated kernel walks the row once per reduction."""
    desc, ins, io_dtype = random_region(seed, long_rows=True)
    # odd seeds run the checked build: every global access of the generated kernels range-tested, error word 0 below
    k = FusedKernel(desc, flags=8 if seed % 2 else 0)
    has_reduce = any(op["name"].startswith("Reduce") for op in desc["op_desc"])
    sums_rows = any(op["name"] == "ReduceSum" and len(op["output_desc"][0]["shape"]) == 1 for op in desc["op_desc"])
    cols = desc["input_desc"][0][0]["shape"][-1]
    if has_reduce and not sums_rows and k.meta()["template"] == "akgb_row_jit":
        # (9000 or 12288 columns still fit the registers when few values are live at once)
        assert k.launch_count == 1 and (cols < 16392 or "c += (i64)T * VW" in k.jit_source(cols % 8 == 0))
    outs = k.empty_outputs()
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    want = O.evaluate(desc, ins, accum="float64")
    for g, w in zip(outs, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        g64, w64 = g.astype(np.float64), w.astype(np.float64)
        fin = np.isfinite(w64)
        assert np.array_equal(np.isfinite(g64), fin)
        scale = float(np.abs(w64[fin]).max()) if fin.any() else 1.0
        tol = 5e-3 if w.dtype == np.float16 else 2e-5
        bad = np.abs(g64 - w64)[fin] > tol * max(scale, 1.0) + tol * np.abs(w64[fin])
        assert bad.mean() <= 2e-3, (seed, float(bad.mean()))


def random_reduction_tail(seed):
    """An elementwise chain over [rows..., cols] that ends in a reduction over the leading axes or over all axes."""
    rng = np.random.default_rng(1000 + seed)
    lead = [int(v) for v in rng.choice([3, 16, 40, 130], size=int(rng.integers(1, 3)))]
    cols = int(rng.choice([8, 100, 256, 1030]))
    while int(np.prod(lead)) * cols < (1 << 16):
        lead[0] *= 4
    shape = lead + [cols]
    over_all = bool(rng.random() < 0.4)
    b = _Builder(f"Fused_FuzzTail_{seed}")
    vals = [b.input("x", shape, F), b.input("y", shape, F)]
    extras = []
    if not over_all and rng.random() < 0.6:
        extras.append(b.input("g", [cols], F))
    if not over_all and rng.random() < 0.4:
        extras.append(b.input("r", lead + [1], F))
    cur = b.emit(str(rng.choice(["Mul", "Add", "Sub"])), vals, shape, F)
    for e in extras:
        cur = b.emit(str(rng.choice(["Mul", "Add"])), [cur, e], shape, F)
    for _ in range(int(rng.integers(0, 4))):
        if rng.random() < 0.5:
            cur = b.emit(str(rng.choice(["Abs", "Tanh", "Neg"])), [cur], shape, F)
        else:
            cur = b.emit(str(rng.choice(["Mul", "Maximum", "Add"])), [cur, vals[int(rng.integers(2))]], shape, F)
    op = str(rng.choice(["ReduceSum", "ReduceSum", "ReduceMax", "ReduceMin"]))
    axes = list(range(len(shape))) if over_all else list(range(len(lead)))
    b.output(b.emit(op, [cur], [1] if over_all else [cols], F, _reduce_attr(axes, False)))
    n_out = 1
    if not over_all and rng.random() < 0.5:  # a second reduction over the same rows
        b.output(b.emit("ReduceSum", [vals[1]], [cols], F, _reduce_attr(axes, False)))
        n_out = 2
    desc = b.build()
    ins = [rng.standard_normal(t["shape"]).astype(np.float32) for (t,) in desc["input_desc"]]
    return desc, ins, axes, n_out


@pytest.mark.parametrize("seed", range(24))
@pytest.mark.parametrize("flags", [0, 1], ids=["generated", "separate"])
def test_random_reduction_tail(seed, flags):
    desc, ins, axes, n_out = random_reduction_tail(seed)
    k = FusedKernel(desc, flags=flags)
    outs = k.empty_outputs()
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    want = O.evaluate(desc, ins, accum="float64")
    count = int(np.prod([ins[0].shape[a] for a in axes]))
    for g, w in zip(outs, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        # a sum of `count` terms of magnitude O(1..10): float32 accumulation error well below 1e-5 * count * 10
        bound = 1e-4 * count if desc["op_desc"][-n_out]["name"] == "ReduceSum" or g is not outs[0] else 1e-5
        assert np.all(np.abs(g.astype(np.float64) - w.astype(np.float64)) <= bound + 1e-5 * np.abs(w))
    if flags == 0:
        assert k.meta()["template"] in ("akgb_col_jit", "akgb_row_jit")


def random_cut_region(seed):
    """Two row regions with a change of layout between them: a transpose of the leading axes, or a re-view of the rows."""
    rng = np.random.default_rng(5000 + seed)
    lead = [int(v) for v in rng.choice([2, 3, 5, 12], size=2)]
    cols = int(rng.choice([8, 40, 128, 264]))
    shape, red = lead + [cols], lead + [1]
    b = _Builder(f"Fused_FuzzCut_{seed}")
    x = b.input("x", shape, F)
    g_ = b.input("g", [cols], F)

    def row_block(cur, shp, rd):
        kind = int(rng.integers(3))
        ax = [len(shp) - 1]
        if kind == 0:  # centre
            m = b.emit("Mul", [b.emit("ReduceSum", [cur], rd, F, _reduce_attr(ax, True)), b.const(1.0 / shp[-1], F)], rd, F)
            return b.emit("Sub", [cur, m], shp, F)
        if kind == 1:  # softmax-like
            m = b.emit("ReduceMax", [cur], rd, F, _reduce_attr(ax, True))
            e = b.emit("Exp", [b.emit("Sub", [cur, m], shp, F)], shp, F)
            return b.emit("RealDiv", [e, b.emit("ReduceSum", [e], rd, F, _reduce_attr(ax, True))], shp, F)
        s_ = b.emit("ReduceSum", [b.emit("Mul", [cur, cur], shp, F)], rd, F, _reduce_attr(ax, True))
        return b.emit("Mul", [cur, b.emit("Rsqrt", [b.emit("Add", [s_, b.const(1.0, F)], rd, F)], rd, F)], shp, F)

    cur = b.emit("Mul", [row_block(x, shape, red), g_], shape, F)
    outs = []
    if rng.random() < 0.5:
        outs.append(cur)
    if rng.random() < 0.5:
        shape2 = [lead[1], lead[0], cols]
        cur = b.emit("Transpose", [cur], shape2, F, [_attr("perm", "listInt", [1, 0, 2])])
    else:
        shape2 = [lead[0] * lead[1], cols]
        cur = b.emit("Reshape", [cur], shape2, F, [_attr("shape", "listInt", shape2)])
    red2 = shape2[:-1] + [1]
    cur = b.emit("Add", [cur, g_], shape2, F)
    if rng.random() < 0.7:
        cur = row_block(cur, shape2, red2)
    outs.append(b.emit("Tanh", [cur], shape2, F))
    for o in outs:
        b.output(o)
    desc = b.build()
    ins = [rng.standard_normal(shape).astype(np.float32), rng.uniform(0.5, 1.5, [cols]).astype(np.float32)]
    return desc, ins


@pytest.mark.parametrize("seed", range(24))
@pytest.mark.parametrize("flags", [0, 1], ids=["generated", "separate"])
def test_random_cut_region(seed, flags):
    desc, ins = random_cut_region(seed)
    k = FusedKernel(desc, flags=flags)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    want = O.evaluate(desc, ins, accum="float64")
    for g, w in zip(outs, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=2e-5, atol=2e-5)


def random_statistics_region(seed):
    """Normalisation-like regions on [n, c, h, w]: one to three stages of (elementwise chain -> reduction over a random
    axis set -> ops on the reduced values), then a full-size result that uses the statistics and earlier full-size
    values. Statistics over (n, h, w), (h, w), (c, h, w), n or w."""
    rng = np.random.default_rng(9000 + seed)
    shape = [int(rng.choice([4, 8, 16])), int(rng.choice([16, 24, 32])), int(rng.choice([12, 20, 28])), int(rng.choice([24, 40, 56]))]
    axes = [[0, 2, 3], [2, 3], [1, 2, 3], [0], [3]][int(rng.integers(5))]
    stat = [1 if i in axes else s for i, s in enumerate(shape)]
    count = int(np.prod([shape[i] for i in axes]))
    b = _Builder(f"Fused_FuzzStat_{seed}")
    x = b.input("x", shape, F)
    per = b.input("p", stat, F)
    full, stats = [x], [per]
    if rng.random() < 0.5:
        full.append(b.emit("Mul", [x, b.input("y", shape, F)], shape, F))
    else:
        full.append(b.emit("Add", [x, per], shape, F))
    for _ in range(int(rng.integers(1, 4))):
        cur = full[int(rng.integers(len(full)))]
        for _ in range(int(rng.integers(0, 3))):
            kind = int(rng.integers(4))
            if kind == 0:
                cur = b.emit(str(rng.choice(["Sub", "Mul", "Add"])), [cur, stats[int(rng.integers(len(stats)))]], shape, F)
            elif kind == 1:
                cur = b.emit("Mul", [cur, cur], shape, F)
            elif kind == 2:
                cur = b.emit(str(rng.choice(["Abs", "Tanh", "Neg"])), [cur], shape, F)
            else:
                cur = b.emit(str(rng.choice(["Sub", "Maximum"])), [cur, full[int(rng.integers(len(full)))]], shape, F)
            full.append(cur)
        op = str(rng.choice(["ReduceSum", "ReduceSum", "ReduceMax", "ReduceMin"]))
        r = b.emit(op, [cur], stat, F, _reduce_attr(axes, True))
        if op == "ReduceSum":
            r = b.emit("Mul", [r, b.const(1.0 / count, F)], stat, F)
        if rng.random() < 0.5:
            r = b.emit("Rsqrt", [b.emit("Add", [b.emit("Abs", [r], stat, F), b.const(0.5, F)], stat, F)], stat, F)
        stats.append(r)
    y = full[int(rng.integers(len(full)))]
    y = b.emit(str(rng.choice(["Sub", "Mul"])), [y, stats[-1]], shape, F)
    y = b.emit("Add", [b.emit("Mul", [y, stats[int(rng.integers(1, len(stats)))]], shape, F), per], shape, F)
    b.output(y)
    if rng.random() < 0.6:
        b.output(stats[-1])
    desc = b.build()
    ins = [rng.standard_normal(t[0]["shape"]).astype(np.float32) for t in desc["input_desc"]]
    return desc, ins


@pytest.mark.parametrize("seed", range(40))
@pytest.mark.parametrize("flags", [0, 1], ids=["generated", "separate"])
def test_random_statistics_region(seed, flags):
    desc, ins = random_statistics_region(seed)
    k = FusedKernel(desc, flags=flags)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    want = O.evaluate(desc, ins, accum="float64")
    for g, w in zip(outs, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        scale = max(1.0, float(np.abs(w).max()))
        np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=5e-5, atol=5e-5 * scale)
