"""Regions that no specialised template claims run through the generic plan (elementwise interpreter + reduction /
transpose / matmul launches).  The shapes and op mixes follow the kinds of fused regions in the reference's own
system-test corpus (akg-mlir/tests/st/**: add chains, Cast+Mul, Sub+RealDiv with a broadcast operand, Mul+RealDiv+Exp,
LessEqual, Select, Mul->ReduceSum over X/ALL, ReduceSum over Y with keep_dims, [1,1]->[1,N] broadcasts)."""
import os

import numpy as np
import pytest

from akg_b200 import FusedKernel, descs
from akg_b200.descs import _Builder, _attr, _reduce_attr, batch_norm_training as _batch_norm_training, batch_norm_backward as _batch_norm_backward
from oracle import akg_oracle as O
from helpers import BF16, bits_equal, guarded_launch, make_inputs

pytestmark = pytest.mark.gpu


FLAGS = [0]  # set by the fixture below: 0 = run-time instantiated elementwise kernels, 1 = interpreter only
CHECKED = [0]  # 8 = generated kernels built with every global access range-tested (AKGB_FLAG_CHECKED)


def _flags():
    return FLAGS[0] | CHECKED[0]


@pytest.fixture(autouse=True, params=[(0, 0), (1, 0), (0, 8)], ids=["jit", "interp", "jit-checked"])
def _both_elementwise_paths(request):
    """Every test of this file runs three times: generated kernels, the interpreting kernel, and generated kernels in
    the checked build -- there every load and store is tested against the ranges of the launch's tensors, and `run`
    requires the device error word to stay 0 (bit 9 would report an access outside them)."""
    FLAGS[0], CHECKED[0] = request.param
    yield
    FLAGS[0], CHECKED[0] = 0, 0


def run(desc, ins):
    k = FusedKernel(desc, flags=_flags())
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    k.run_host(list(ins) + outs)
    assert k.check_device_error() == 0
    # the same region as a device launch between guard zones: same bits, nothing written outside the tensors
    guarded, _ = guarded_launch(desc, ins, flags=_flags())
    atomics = any(op["name"] == "UnsortedSegmentSum" for op in desc["op_desc"])  # float atomics: order varies
    for a, b in zip(outs, guarded):
        assert atomics or np.array_equal(np.ascontiguousarray(a).view(np.uint8).reshape(-1), b.view(np.uint8).reshape(-1))
    return outs, k


def check(desc, ins, rtol=0.0, atol=0.0, exact=False):
    got, k = run(desc, ins)
    want = O.evaluate(desc, ins)
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        if exact:
            assert bits_equal(g, w)
        else:
            np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=rtol, atol=atol)
    return k


def test_add_chain_f32_exact(lib):
    b = _Builder("Fused_AddChain_1")
    f = "float32"
    xs = [b.input(f"x{i}", [37, 129], f) for i in range(5)]
    t = xs[0]
    for x in xs[1:]:
        t = b.emit("Add", [t, x], [37, 129], f)
    b.output(t)
    d = b.build()
    k = check(d, make_inputs(d, 1), exact=True)
    assert k.meta()["template"] == "ew_generic" and k.launch_count == 1


def test_cast_mul_int_to_float_and_bf16(lib):
    b = _Builder("Fused_Cast_Mul_2")
    x = b.input("x", [64, 100], "int32")
    y = b.input("y", [64, 100], "float32")
    c = b.emit("Cast", [x], [64, 100], "float32", [_attr("dst_type", "str", "float32")])
    m = b.emit("Mul", [c, y], [64, 100], "float32")
    h = b.emit("Cast", [m], [64, 100], "bfloat16", [_attr("dst_type", "str", "bfloat16")])
    b.output(m)
    b.output(h)
    d = b.build()
    rng = np.random.default_rng(2)
    ins = [rng.integers(-1000, 1000, (64, 100)).astype(np.int32), rng.standard_normal((64, 100)).astype(np.float32)]
    check(d, ins, exact=True)


def test_sub_realdiv_with_broadcast_operands(lib):
    b = _Builder("Fused_Sub_RealDiv_3")
    f = "float32"
    x = b.input("x", [8, 33, 70], f)
    m = b.input("m", [8, 33, 1], f)   # broadcast over the last axis
    s = b.input("s", [70], f)         # broadcast over the leading axes
    c = b.input("c", [1, 1], f)       # scalar-like
    t = b.emit("Sub", [x, m], [8, 33, 70], f)
    t = b.emit("RealDiv", [t, s], [8, 33, 70], f)
    t = b.emit("Add", [t, c], [8, 33, 70], f)
    b.output(t)
    d = b.build()
    ins = make_inputs(d, 3)
    ins[2] = np.abs(ins[2]) + np.float32(0.5)
    check(d, ins, exact=True)


def test_mul_realdiv_exp_f16(lib):
    b = _Builder("Fused_Mul_RealDiv_Exp_4")
    h = "float16"
    x = b.input("x", [1000, 40], h)
    y = b.input("y", [1000, 40], h)
    t = b.emit("Mul", [x, b.const(0.5, h)], [1000, 40], h)
    t = b.emit("RealDiv", [t, y], [1000, 40], h)
    t = b.emit("Exp", [t], [1000, 40], h)
    b.output(t)
    d = b.build()
    ins = make_inputs(d, 4)
    ins[1] = (np.abs(ins[1]) + np.float16(1.0)).astype(np.float16)
    # Mul and RealDiv are exact per op; Exp is a transcendental: 2e-3
    check(d, ins, rtol=2e-3, atol=1e-6)


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_every_16_bit_pattern_through_add_mul_cast_with_shared_operands(lib, dt):
    """x runs over all 65 536 bit patterns of the type (NaNs, infinities, subnormals, both zeros), y is shared along
    the rows and z along the columns: the generated kernel keeps 16-bit granules packed until their turn and rounds
    results two per instruction, and every result bit must still be the oracle's (NaNs compared as NaNs)."""
    b = _Builder("Fused_Add_Mul_Cast_patterns_" + dt + "_3")
    npdt = BF16 if dt == "bfloat16" else np.dtype(dt)
    x = b.input("x", [256, 256], dt)
    y = b.input("y", [256], dt)
    z = b.input("z", [256, 1], dt)
    t = b.emit("Add", [x, y], [256, 256], dt)
    m = b.emit("Mul", [t, z], [256, 256], dt)
    w = b.emit("Cast", [m], [256, 256], "float32", [_attr("dst_type", "str", "float32")])
    n = b.emit("Cast", [b.emit("Mul", [w, b.const(0.333251953125, "float32")], [256, 256], "float32")], [256, 256], dt,
               [_attr("dst_type", "str", dt)])
    b.output(t)
    b.output(m)
    b.output(n)
    d = b.build()
    rng = np.random.default_rng(11)
    xs = np.arange(65536, dtype=np.uint16).reshape(256, 256).view(npdt)
    ys = rng.standard_normal(256).astype(np.float32).astype(npdt)
    zs = (rng.standard_normal((256, 1)) * 3).astype(np.float32).astype(npdt)
    got, k = run(d, [xs, ys, zs])
    want = O.evaluate(d, [xs, ys, zs])
    for g, w_ in zip(got, want):
        g32, w32 = g.astype(np.float32), w_.astype(np.float32)
        nan = np.isnan(w32)
        assert np.array_equal(np.isnan(g32), nan)
        assert np.array_equal(g.view(np.uint16)[~nan], w_.view(np.uint16)[~nan])
    assert k.meta()["template"] == "ew_generic"


def test_compare_select_maximum_bool_outputs(lib):
    b = _Builder("Fused_LessEqual_Select_5")
    f = "float32"
    x = b.input("x", [17, 300], f)
    y = b.input("y", [17, 300], f)
    le = b.emit("LessEqual", [x, y], [17, 300], "bool")
    mx = b.emit("Maximum", [x, b.const(0.0, f)], [17, 300], f)
    sel = b.emit("Select", [le, mx, y], [17, 300], f)
    ne = b.emit("NotEqual", [sel, y], [17, 300], "bool")
    b.output(le)
    b.output(sel)
    b.output(ne)
    d = b.build()
    check(d, make_inputs(d, 5), exact=True)


def test_int32_arithmetic(lib):
    b = _Builder("Fused_IntOps_6")
    i = "int32"
    x = b.input("x", [4096], i)
    y = b.input("y", [4096], i)
    t = b.emit("Add", [x, y], [4096], i)
    t = b.emit("Mul", [t, b.const(3, i)], [4096], i)
    t = b.emit("Sub", [t, x], [4096], i)
    a = b.emit("Abs", [t], [4096], i)
    b.output(a)
    d = b.build()
    rng = np.random.default_rng(6)
    check(d, [rng.integers(-9999, 9999, 4096).astype(np.int32) for _ in range(2)], exact=True)


def test_mul_reduce_sum_x_and_all(lib):
    # Square -> ReduceSum over all axes ([768,512] -> [1]) and over the last axis
    for axes, oshape in (([0, 1], [1]), ([1], [768])):
        b = _Builder("Fused_Mul_ReduceSum_7")
        f = "float32"
        x = b.input("x", [768, 512], f)
        sq = b.emit("Mul", [x, x], [768, 512], f)
        r = b.emit("ReduceSum", [sq], oshape, f, _reduce_attr(axes, False))
        b.output(r)
        d = b.build()
        ins = make_inputs(d, 7)
        got, k = run(d, ins)
        truth = (ins[0].astype(np.float64) ** 2).sum(axis=tuple(axes)).reshape(oshape)
        assert np.all(np.abs(got[0] - truth) <= 1e-5 * truth)
        assert k.launch_count >= (1 if FLAGS[0] == 0 and axes == [1] else 2)  # the row reduction: one generated kernel
        if FLAGS[0] == 0:  # the square is folded into the reduction's pass in both cases
            assert k.meta()["template"] == "akgb_row_jit"


def test_reduce_sum_y_keep_dims_and_batched(lib):
    b = _Builder("Fused_ReduceSum_8")
    f = "float32"
    x = b.input("x", [1, 510, 3072], f)
    r = b.emit("ReduceSum", [x], [1, 1, 3072], f, _reduce_attr([1], True))
    b.output(r)
    d = b.build()
    ins = make_inputs(d, 8)
    got, _ = run(d, ins)
    truth = ins[0].astype(np.float64).sum(axis=1, keepdims=True)
    assert np.all(np.abs(got[0] - truth) <= 1e-5 * np.abs(ins[0]).sum(axis=1, keepdims=True))
    # batched: reduce the middle axis of [6, 200, 96]
    b = _Builder("Fused_ReduceMax_9")
    x = b.input("x", [6, 200, 96], f)
    b.output(b.emit("ReduceMax", [x], [6, 96], f, _reduce_attr([1], False)))
    d = b.build()
    ins = make_inputs(d, 9)
    got, _ = run(d, ins)
    assert np.array_equal(got[0], ins[0].max(axis=1))


def test_broadcast_to_and_reshape_views(lib):
    b = _Builder("Fused_BroadcastTo_10")
    f = "float32"
    x = b.input("x", [1, 1], f)
    y = b.input("y", [1, 5000], f)
    bx = b.emit("BroadcastTo", [x], [1, 5000], f, [_attr("shape", "listInt", [1, 5000])])
    t = b.emit("Mul", [bx, y], [1, 5000], f)
    r = b.emit("Reshape", [t], [50, 100], f, [_attr("shape", "listInt", [50, 100])])
    u = b.emit("Add", [r, b.const(1.0, f)], [50, 100], f)
    b.output(u)
    b.output(b.emit("Reshape", [u], [5000], f, [_attr("shape", "listInt", [5000])], out_name="u_flat"))
    d = b.build()
    check(d, make_inputs(d, 10), exact=True)


def test_layernorm_other_spelling_runs_as_generic_plan(lib):
    # variance via E[x^2] - mean^2 and division instead of multiplication: not the template's spelling
    rows, cols = 48, 200
    b = _Builder("Fused_LayerNormVariant_11")
    f = "float32"
    x = b.input("x", [rows, cols], f)
    s1 = b.emit("ReduceSum", [x], [rows, 1], f, _reduce_attr([1], True))
    mean = b.emit("RealDiv", [s1, b.const(float(cols), f)], [rows, 1], f)
    sq = b.emit("Mul", [x, x], [rows, cols], f)
    s2 = b.emit("ReduceSum", [sq], [rows, 1], f, _reduce_attr([1], True))
    ex2 = b.emit("RealDiv", [s2, b.const(float(cols), f)], [rows, 1], f)
    var = b.emit("Sub", [ex2, b.emit("Mul", [mean, mean], [rows, 1], f)], [rows, 1], f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], [rows, 1], f)], [rows, 1], f)
    y = b.emit("Mul", [b.emit("Sub", [x, mean], [rows, cols], f), rstd], [rows, cols], f)
    b.output(y)
    d = b.build()
    ins = make_inputs(d, 11)
    got, k = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=2e-4, atol=2e-5)  # E[x^2]-mean^2 cancels: looser than 1e-5
    # one generated row kernel, or the separate launches when run-time compilation is off
    assert k.op_class == "reduce_x" and (k.launch_count == 1 if FLAGS[0] == 0 else k.launch_count >= 5)


def test_matmul_with_unfused_epilogue(lib):
    # MatMul -> Mul by a constant -> Add bias: not the bias/ReLU/cast template, runs as matmul + elementwise
    m, k_, n = 256, 192, 264
    b = _Builder("Fused_MatMul_Mul_Add_12")
    h, f = "bfloat16", "float32"
    a = b.input("a", [m, k_], h)
    w = b.input("b", [k_, n], h)
    bias = b.input("bias", [n], f)
    c = b.emit("MatMul", [a, w], [m, n], f, [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)])
    c = b.emit("Mul", [c, b.const(0.125, f)], [m, n], f)
    c = b.emit("Add", [c, bias], [m, n], f)
    b.output(c)
    d = b.build()
    ins = make_inputs(d, 12, {"a": "normal_small", "b": "normal_small"})
    got, kern = run(d, ins)
    want = O.evaluate(d, ins)[0]
    np.testing.assert_allclose(got[0], want, rtol=2e-3, atol=1e-3 * float(np.abs(want).max()))
    assert kern.launch_count == 2 and kern.flops == 2 * m * k_ * n


def test_transpose_then_elementwise(lib):
    b = _Builder("Fused_Transpose_Add_13")
    h = "float16"
    x = b.input("x", [12, 34, 56], h)
    y = b.input("y", [56, 12, 34], h)
    t = b.emit("Transpose", [x], [56, 12, 34], h, [_attr("perm", "listInt", [2, 0, 1])])
    b.output(b.emit("Add", [t, y], [56, 12, 34], h))
    d = b.build()
    check(d, make_inputs(d, 13), exact=True)


def test_float_to_int_cast_rounds_to_nearest_even_and_clamps(lib):
    """The reference's compiled route (tosa.cast) rounds to nearest even and clamps to the result type; its NumPy
    generator would truncate.  The library and the restatement follow the compiled route; NaN gives 0."""
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49999997, 126.5, 127.5, 300.0, -129.0, 32767.5, 40000.0, -40000.0,
                  3e10, -3e10, np.inf, -np.inf, np.nan, 1e-30, -7.75, 8388607.5] + [0.0] * 10, dtype=np.float32)
    rng = np.random.default_rng(15)
    x = np.concatenate([x, (rng.standard_normal(4096 - x.size) * 100).astype(np.float32)])
    for dst, src in (("int32", "float32"), ("int16", "float32"), ("int8", "float32"), ("int32", "float16"),
                     ("int8", "bfloat16")):
        b = _Builder(f"Fused_CastToInt_{dst}_{src}_14")
        xin = b.input("x", [4096], src)
        b.output(b.emit("Cast", [xin], [4096], dst, [_attr("dst_type", "str", dst)]))
        d = b.build()
        xv = x.astype(BF16 if src == "bfloat16" else np.dtype(src))
        k = check(d, [xv], exact=True)
        assert k.launch_count == 1
    got, _ = run(_cast_desc("int32"), [x])
    assert got[0][:6].tolist() == [0, 2, 2, 0, -2, -2] and got[0][14] == 2**31 - 1 and got[0][15] == -2**31
    assert got[0][18] == 0  # NaN
    # to int64: a generated kernel (64-bit integer registers; the interpreting kernel has no such mode); saturates at
    # +-2^63, from float32 and from float64
    if FLAGS[0] == 0:
        x64 = np.concatenate([x.astype(np.float64), np.array([9.3e18, -9.3e18, 2.0 ** 63, -(2.0 ** 63), 2.0 ** 62 + 1024,
                                                              4503599627370497.5, 1e300, -1e300] + [0.0] * 8)])
        for src, xv in (("float32", x), ("float64", x64)):
            b = _Builder(f"Fused_CastToInt64_{src}_14")
            xin = b.input("x", [xv.size], src)
            b.output(b.emit("Cast", [xin], [xv.size], "int64", [_attr("dst_type", "str", "int64")]))
            got, _ = run(b.build(), [xv])
            want = O.evaluate(b.build(), [xv])[0]
            assert got[0].dtype == np.int64 and np.array_equal(got[0], want)
            assert got[0][16] == 2**63 - 1 and got[0][17] == -2**63 and got[0][18] == 0  # +inf, -inf, NaN


def test_int64_values_run_in_generated_kernels(lib):
    """64-bit integer arithmetic, compares, selects and casts (index computations of embedding / gather regions): the
    generated kernel keeps all its integer registers in 64 bits; the interpreting kernel has no such mode, so the same
    region is refused when the run-time compiler is switched off."""
    from akg_b200 import UnsupportedError
    b = _Builder("Fused_I64_Chain_16")
    i64, i32 = "int64", "int32"
    x, y, z = b.input("x", [64, 40], i64), b.input("y", [40], i64), b.input("z", [64, 40], i32)
    t = b.emit("Mul", [b.emit("Add", [x, y], [64, 40], i64), b.const(3, i64)], [64, 40], i64)
    zc = b.emit("Cast", [z], [64, 40], i64, [_attr("dst_type", "str", i64)])
    m = b.emit("Maximum", [t, zc], [64, 40], i64)
    gt = b.emit("Greater", [t, zc], [64, 40], "bool")
    sel = b.emit("Select", [gt, b.emit("Sub", [m, zc], [64, 40], i64), b.emit("Neg", [m], [64, 40], i64)], [64, 40], i64)
    sel = b.emit("Sub", [sel, b.const(1099511627779, i64)], [64, 40], i64)  # a constant beyond 32 bits (2^40 + 3)
    b.output(sel)
    b.output(b.emit("Cast", [m], [64, 40], i32, [_attr("dst_type", "str", i32)]))
    b.output(gt)
    b.output(b.emit("Cast", [sel], [64, 40], "float32", [_attr("dst_type", "str", "float32")]))
    d = b.build()
    rng = np.random.default_rng(16)
    ins = [rng.integers(-2**40, 2**40, (64, 40)).astype(np.int64), rng.integers(-2**33, 2**33, 40).astype(np.int64),
           rng.integers(-2**31, 2**31 - 1, (64, 40)).astype(np.int32)]
    if FLAGS[0] != 0:
        with pytest.raises(UnsupportedError):
            run(d, ins)
        return
    k = check(d, ins, exact=True)
    assert k.launch_count == 1
    # ragged extent (element-wise accesses) and a strided operand (Tile)
    b = _Builder("Fused_I64_Tile_17")
    p_ = b.input("p", [3, 7], i64)
    tl = b.emit("Tile", [p_], [6, 21], i64, [_attr("multiples", "listInt", [2, 3])])
    q_ = b.input("q", [6, 21], i64)
    b.output(b.emit("Minimum", [b.emit("Abs", [tl], [6, 21], i64), q_], [6, 21], i64))
    d = b.build()
    check(d, [rng.integers(-2**50, 2**50, (3, 7)).astype(np.int64), rng.integers(0, 2**50, (6, 21)).astype(np.int64)], exact=True)


def test_float64_values_run_in_generated_kernels(lib):
    """float64 arithmetic, compares and casts: the generated kernel keeps all its floating-point registers as doubles
    (an op of a narrower type rounds its double result once to that type); the interpreting kernel has no such mode.
    + - * / sqrt and every cast are bit-exact against the oracle, transcendentals to 1e-14."""
    from akg_b200 import UnsupportedError
    b = _Builder("Fused_F64_Chain_18")
    f64, f32 = "float64", "float32"
    x, y, z = b.input("x", [96, 200], f64), b.input("y", [200], f64), b.input("z", [96, 200], f32)
    t = b.emit("Mul", [b.emit("Add", [x, y], [96, 200], f64), b.const(0.3, f64)], [96, 200], f64)
    zc = b.emit("Cast", [z], [96, 200], f64, [_attr("dst_type", "str", f64)])
    q = b.emit("RealDiv", [t, b.emit("Sqrt", [b.emit("Abs", [zc], [96, 200], f64)], [96, 200], f64)], [96, 200], f64)
    gt = b.emit("Greater", [t, zc], [96, 200], "bool")
    sel = b.emit("Select", [gt, b.emit("Sub", [q, zc], [96, 200], f64), b.emit("Maximum", [q, zc], [96, 200], f64)], [96, 200], f64)
    b.output(sel)
    for dst in (f32, "float16", "bfloat16", "int32"):
        b.output(b.emit("Cast", [sel], [96, 200], dst, [_attr("dst_type", "str", dst)]))
    # a float32-typed op inside the float64 program: correctly rounded float32 arithmetic
    b.output(b.emit("Mul", [z, b.emit("Cast", [t], [96, 200], f32, [_attr("dst_type", "str", f32)])], [96, 200], f32))
    d = b.build()
    rng = np.random.default_rng(18)
    ins = [rng.standard_normal((96, 200)) * 100, rng.standard_normal(200), (rng.standard_normal((96, 200)) * 50).astype(np.float32)]
    ins[0][0, :6] = [np.inf, -np.inf, np.nan, 1e300, -1e-310, 0.0]
    ins[2][1, :3] = [np.inf, np.nan, 0.0]
    if FLAGS[0] != 0:
        with pytest.raises(UnsupportedError):
            run(d, ins)
        return
    got, k = run(d, ins)
    want = O.evaluate(d, ins)
    assert k.launch_count == 1 and k.meta()["template"] == "ew_generic"
    for g, w in zip(got, want):
        assert g.dtype == w.dtype
        nan = np.isnan(w.astype(np.float64)) if w.dtype.kind == "f" or w.dtype == BF16 else np.zeros(w.shape, bool)
        assert np.array_equal(np.isnan(g.astype(np.float64)) if nan.any() else nan, nan)
        gb, wb = g.view(np.uint8).reshape(g.shape + (-1,)), np.ascontiguousarray(w).view(np.uint8).reshape(w.shape + (-1,))
        assert np.array_equal(gb[~nan], wb[~nan])
    # transcendentals, a ragged extent (element-wise accesses) and a float64 constant that float32 cannot hold
    b = _Builder("Fused_F64_Tanh_19")
    p_ = b.input("p", [37, 13], f64)
    e = b.emit("Exp", [b.emit("Mul", [b.emit("Tanh", [p_], [37, 13], f64), b.const(0.1234567890123456, f64)], [37, 13], f64)], [37, 13], f64)
    b.output(b.emit("Log", [b.emit("Add", [e, b.const(1.0, f64)], [37, 13], f64)], [37, 13], f64))
    d = b.build()
    check(d, [rng.standard_normal((37, 13)) * 3], rtol=1e-14, atol=1e-15)


def test_checked_build_reports_and_skips_accesses_outside_the_ranges(lib):
    """The checker itself: with 16 bytes taken off the end of every tensor range (a test hook; the tensors themselves
    keep their size) a checked launch sets bit 9 of the error word, leaves the last 16 bytes of the output untouched
    (the last 16 bytes of every input read as zeros) and everything those bytes do not feed correct; with the hook off the same kernel runs clean.  No access leaves a real tensor."""
    import ctypes
    import torch
    from akg_b200 import _capi
    if FLAGS[0] != 0 or CHECKED[0] == 0:
        pytest.skip("one mode is enough")
    libc = _capi.load()
    # (region, output shape, rows and columns at the end that the zeros read from the shrunk INPUT ranges may change:
    # the copy's last 4 elements; RMSNorm's last row and, through the last 4 weights, the last 4 columns of every row)
    for build, shape, rows_off, cols_off in ((lambda: descs.scale_copy([1, 65536]), (1, 65536), 0, 4),
                                             (lambda: descs.rmsnorm(48, 1024), (48, 1024), 1, 4)):
        d = build()
        k = FusedKernel(d, flags=8)
        ins = [torch.from_numpy(a).cuda() for a in make_inputs(d, 5)]
        want = torch.empty(shape, dtype=torch.float32, device="cuda")
        k.launch(ins + [want])
        torch.cuda.synchronize()
        assert k.check_device_error() == 0
        got = torch.full(shape, -7.0, dtype=torch.float32, device="cuda")
        libc.akgb_checked_shrink_for_test(16)
        try:
            k.launch(ins + [got])
            torch.cuda.synchronize()
            word = ctypes.c_uint32(0)
            status = libc.akgb_check_device_error(k._handle, ctypes.byref(word))
        finally:
            libc.akgb_checked_shrink_for_test(0)
        assert status == 8 and word.value == 512  # AKGB_OUT_OF_RANGE
        g, w = got.flatten(), want.flatten()
        assert torch.equal(g[-4:], torch.full((4,), -7.0, device="cuda"))
        r_end = shape[0] - rows_off
        assert torch.equal(got[:r_end, :-cols_off], want[:r_end, :-cols_off])
        k.launch(ins + [got])
        torch.cuda.synchronize()
        assert k.check_device_error() == 0 and torch.equal(got, want)


def _cast_desc(dst):
    b = _Builder(f"Fused_CastTo_{dst}_14")
    x = b.input("x", [4096], "float32")
    b.output(b.emit("Cast", [x], [4096], dst, [_attr("dst_type", "str", dst)]))
    return b.build()


def test_tile_slice_strided_slice_concat_addn(lib):
    """Data-movement ops of the JSON factory (TranslateToMindsporeDialect.cpp:1037-1160): bit-exact copies."""
    f = "float32"
    # Tile then an elementwise op on the tiled value
    b = _Builder("Fused_Tile_Div_20")
    x = b.input("x", [3, 5], f)
    y = b.input("y", [6, 15], f)
    t = b.emit("Tile", [x], [6, 15], f, [_attr("multiples", "listInt", [2, 3])])
    b.output(b.emit("RealDiv", [y, t], [6, 15], f))
    d = b.build()
    ins = make_inputs(d, 20)
    ins[0] = np.abs(ins[0]) + np.float32(1)
    check(d, ins, exact=True)
    # Slice and StridedSlice of the same input, plus AddN of three tensors
    b = _Builder("Fused_Slice_StridedSlice_AddN_21")
    x = b.input("x", [8, 10, 12], "float16")
    s1 = b.emit("Slice", [x], [4, 5, 6], "float16",
                [_attr("begin", "listInt", [2, 1, 3]), _attr("size", "listInt", [4, 5, 6])])
    s2 = b.emit("StridedSlice", [x], [4, 5, 6], "float16",
                [_attr("begin", "listInt", [0, 0, 0]), _attr("end", "listInt", [8, 10, 12]),
                 _attr("strides", "listInt", [2, 2, 2])])
    s3 = b.emit("StridedSlice", [x], [4, 5, 6], "float16",
                [_attr("begin", "listInt", [4, 5, 0]), _attr("end", "listInt", [8, -1, 6]),
                 _attr("strides", "listInt", [1, 1, 1]), _attr("end_mask", "int", 2)])
    node = {"name": "AddN", "attr": None, "impl_path": "", "input_desc": [[dict(s1), dict(s2), dict(s3)]],
            "output_desc": [{"data_type": "float16", "format": "DefaultFormat", "shape": [4, 5, 6], "tensor_name": "sum3"}]}
    b.ops.append(node)
    b.outputs.append(dict(node["output_desc"][0]))
    b.output(s2)
    d = b.build()
    check(d, make_inputs(d, 21), exact=True)
    # Concat along the middle axis, then a cast
    b = _Builder("Fused_Concat_Cast_22")
    p_, q_, r_ = b.input("p", [4, 3, 16], f), b.input("q", [4, 5, 16], f), b.input("r", [4, 1, 16], f)
    node = {"name": "Concat", "attr": [_attr("axis", "int", 1)], "impl_path": "",
            "input_desc": [[dict(p_), dict(q_), dict(r_)]],
            "output_desc": [{"data_type": f, "format": "DefaultFormat", "shape": [4, 9, 16], "tensor_name": "cat"}]}
    b.ops.append(node)
    cat = dict(node["output_desc"][0])
    b.output(b.emit("Cast", [cat], [4, 9, 16], "float16", [_attr("dst_type", "str", "float16")]))
    d = b.build()
    check(d, make_inputs(d, 22), exact=True)


def test_batch_matmul(lib):
    bsz, m, k_, n = 3, 128, 64, 256
    b = _Builder("Fused_BatchMatMul_23")
    h = "bfloat16"
    a = b.input("a", [bsz, m, k_], h)
    w = b.input("w", [bsz, k_, n], h)
    c = b.emit("BatchMatMul", [a, w], [bsz, m, n], "float32",
               [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)])
    b.output(c)
    d = b.build()
    ins = make_inputs(d, 23, {"a": "normal_small", "w": "normal_small"})
    got, kern = run(d, ins)
    want = O.evaluate(d, ins)[0]
    np.testing.assert_allclose(got[0], want, rtol=2e-3, atol=1e-3 * float(np.abs(want).max()))
    assert kern.launch_count == 1  # the batch is a tile coordinate of one launch
    # ragged rows (not a multiple of the 128-row tile) in every batch entry, one shared right operand, K-major B
    rng = np.random.default_rng(24)
    for shared, tb in ((True, False), (False, True), (True, True)):
        bsz, m, k_, n = 7, 100, 72, 136
        b = _Builder("Fused_BatchMatMul_24")
        a = b.input("a", [bsz, m, k_], h)
        wshape = ([n, k_] if tb else [k_, n]) if shared else ([bsz, n, k_] if tb else [bsz, k_, n])
        w = b.input("w", wshape, h)
        c = b.emit("BatchMatMul", [a, w], [bsz, m, n], "float32",
                   [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", tb)])
        b.output(c)
        d = b.build()
        av = (rng.standard_normal((bsz, m, k_)) * 0.1).astype(BF16)
        wv = (rng.standard_normal(wshape) * 0.1).astype(BF16)
        got, kern = run(d, [av, wv])
        w64 = wv.astype(np.float64)
        if tb:
            w64 = np.swapaxes(w64, -1, -2)
        want = av.astype(np.float64) @ w64
        assert kern.launch_count == 1
        np.testing.assert_allclose(got[0], want, rtol=2e-3, atol=2e-3 * float(np.abs(want).max()))
    # larger rows: the CTA-pair kernel with a batch coordinate
    bsz, m, k_, n = 3, 300, 64, 256
    b = _Builder("Fused_BatchMatMul_25")
    a = b.input("a", [bsz, m, k_], h)
    w = b.input("w", [bsz, k_, n], h)
    b.output(b.emit("BatchMatMul", [a, w], [bsz, m, n], h,
                    [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)]))
    d = b.build()
    av = (rng.standard_normal((bsz, m, k_)) * 0.1).astype(BF16)
    wv = (rng.standard_normal((bsz, k_, n)) * 0.1).astype(BF16)
    got, kern = run(d, [av, wv])
    want = av.astype(np.float64) @ wv.astype(np.float64)
    np.testing.assert_allclose(got[0].astype(np.float64), want, rtol=1e-2, atol=1e-2 * float(np.abs(want).max()))


def test_dynamic_shapes_match_the_static_plan(lib):
    """A region described with -1 extents, launched with two different sets of extents, against the same region
    compiled statically for each."""
    import copy
    import torch
    from akg_b200.descs import _Builder, _attr

    def region(s2, s3):
        b = _Builder("Fused_Sub_Mul_Cast_dyn_40")
        f = "float32"
        x = b.input("input_0", [32, 16, s2, s3], f)
        m = b.input("input_1", [32, 16, s2, 1], f)
        y = b.input("input_2", [32, 16, s2, s3], f)
        t = b.emit("Sub", [x, m], [32, 16, s2, s3], f)
        t = b.emit("Mul", [y, t], [32, 16, s2, s3], f)
        b.output(b.emit("Cast", [t], [32, 16, s2, s3], "float16", [_attr("dst_type", "str", "float16")]))
        return b.build()

    kd = FusedKernel(region(-1, -1), flags=_flags())
    assert kd.is_dynamic
    for s2, s3 in ((40, 24), (7, 129)):
        static = region(s2, s3)
        ins = make_inputs(static, 40 + s2)
        want = O.evaluate(static, ins)[0]
        dev = [torch.from_numpy(a).cuda() for a in ins]
        out = torch.empty(want.shape, dtype=torch.float16, device="cuda")
        kd.launch(dev + [out])
        torch.cuda.synchronize()
        assert bits_equal(out.cpu().numpy(), want)
    # dynamic softmax and LayerNorm pick the row templates at launch
    for desc_dyn, desc_static, kinds in (
            (descs.masked_softmax(-1, -1, 256), descs.masked_softmax(6, 32, 256), {"mask": "causal"}),
            (descs.layernorm(-1, 512), descs.layernorm(96, 512), {"gamma": "gamma", "beta": "beta"})):
        k = FusedKernel(desc_dyn, flags=_flags())
        ins = make_inputs(desc_static, 41, kinds)
        want = O.evaluate(desc_static, ins)
        dev = [torch.from_numpy(a).cuda() for a in ins]
        outs = [torch.empty(w.shape, dtype=torch.float16 if w.dtype == np.float16 else torch.float32, device="cuda")
                for w in want]
        k.launch(dev + outs)
        torch.cuda.synchronize()
        for o, w in zip(outs, want):
            np.testing.assert_allclose(o.cpu().numpy().astype(np.float32), w.astype(np.float32), rtol=2e-3, atol=1e-5)


def test_assign_writes_the_input_in_place(lib):
    # x <- x + 1 (the reference's Fused_AssignAdd) and an optimizer-like update with Select
    b = _Builder("Fused_AssignAdd_50")
    i = "int32"
    x = b.input("input_0", [1], i)
    t = b.emit("Add", [x, b.const(1, i)], [1], i)
    b.output(b.emit("Assign", [x, t], [1], i))
    d = b.build()
    k = FusedKernel(d, flags=_flags())
    assert k.inputs[0].written_in_place
    xin = np.array([41], dtype=np.int32)
    out = np.zeros(1, np.int32)
    k.run_host([xin, out])
    assert xin[0] == 42 and out[0] == 42

    b = _Builder("Fused_Mul_Maximum_Select_Assign_51")
    f = "float32"
    w = b.input("w", [300, 40], f)
    g_ = b.input("g", [300, 40], f)
    m = b.input("m", [300, 40], "bool")
    t = b.emit("Mul", [g_, b.const(0.5, f)], [300, 40], f)
    t = b.emit("Maximum", [t, b.const(-0.25, f)], [300, 40], f)
    t = b.emit("Select", [m, b.emit("Sub", [w, t], [300, 40], f), w], [300, 40], f)
    b.output(b.emit("Assign", [w, t], [300, 40], f))
    d = b.build()
    rng = np.random.default_rng(51)
    ins = [rng.standard_normal((300, 40)).astype(np.float32), rng.standard_normal((300, 40)).astype(np.float32),
           rng.integers(0, 2, (300, 40)).astype(bool)]
    want_out, want_in = O.evaluate(d, [a.copy() for a in ins], return_inputs=True)
    k = FusedKernel(d, flags=_flags())
    host = [a.copy() for a in ins] + k.empty_outputs()
    k.run_host(host)
    assert bits_equal(host[3], want_out[0]) and bits_equal(host[0], want_in[0])
    assert bits_equal(host[1], ins[1])  # other inputs untouched


def test_narrow_and_bool_reductions(lib):
    """float16 / bfloat16 reductions accumulate in float32 and round once (the expected-value generator's rule,
    op_dsl.py:126-154); ReduceAll / ReduceAny over bool."""
    for dt, tol in (("float16", 2e-3), ("bfloat16", 1e-2)):
        b = _Builder("Fused_ReduceSum_f16_52")
        x = b.input("x", [64, 300], dt)
        b.output(b.emit("ReduceSum", [x], [64, 1], dt, _reduce_attr([1], True)))
        b.output(b.emit("ReduceMax", [x], [300], dt, _reduce_attr([0], False)))
        d = b.build()
        ins = make_inputs(d, 52)
        got, _ = run(d, ins)
        want = O.evaluate(d, ins)
        np.testing.assert_allclose(got[0].astype(np.float32), want[0].astype(np.float32), rtol=tol, atol=tol)
        assert bits_equal(got[1], want[1])
    b = _Builder("Fused_ReduceAll_53")
    x = b.input("x", [50, 70], "bool")
    b.output(b.emit("ReduceAll", [x], [50], "bool", _reduce_attr([1], False)))
    b.output(b.emit("ReduceAny", [x], [1], "bool", _reduce_attr([0, 1], False)))
    d = b.build()
    rng = np.random.default_rng(53)
    xb = rng.random((50, 70)) < 0.97
    xb[3, :] = True
    got, _ = run(d, [xb])
    assert np.array_equal(got[0], xb.all(axis=1)) and bool(got[1][0]) == bool(xb.any())


def test_gather_and_unsorted_segment_sum(lib):
    rng = np.random.default_rng(60)
    # embedding lookup (axis 0) followed by a scale, and a gather along a middle axis with int64 indices
    b = _Builder("Fused_Gather_Mul_60")
    table = b.input("table", [1000, 64], "float16")
    idx = b.input("idx", [7, 33], "int32")
    g_ = b.emit("Gather", [table, idx], [7, 33, 64], "float16", [_attr("axis", "int", 0), _attr("batch_dims", "int", 0)])
    b.output(b.emit("Mul", [g_, b.const(8.0, "float16")], [7, 33, 64], "float16"))
    d = b.build()
    ins = [rng.standard_normal((1000, 64)).astype(np.float16), rng.integers(0, 1000, (7, 33)).astype(np.int32)]
    check(d, ins, exact=True)
    b = _Builder("Fused_Gather_61")
    x = b.input("x", [5, 40, 3], "float32")
    idx = b.input("idx", [11], "int64")
    b.output(b.emit("Gather", [x, idx], [5, 11, 3], "float32", [_attr("axis", "int", 1), _attr("batch_dims", "int", 0)]))
    d = b.build()
    check(d, [rng.standard_normal((5, 40, 3)).astype(np.float32), rng.integers(0, 40, 11).astype(np.int64)], exact=True)
    # scatter-add by segment id
    b = _Builder("Fused_UnsortedSegmentSum_62")
    data = b.input("data", [4000, 48], "float32")
    ids = b.input("ids", [4000], "int32")
    b.output(b.emit("UnsortedSegmentSum", [data, ids], [37, 48], "float32", [_attr("num_segments", "int", 37)]))
    d = b.build()
    ins = [rng.standard_normal((4000, 48)).astype(np.float32), rng.integers(0, 37, 4000).astype(np.int32)]
    got, _ = run(d, ins)
    want = O.evaluate(d, ins)[0]
    absum = np.zeros((37, 48))
    np.add.at(absum, ins[1], np.abs(ins[0]).astype(np.float64))
    assert np.all(np.abs(got[0] - want) <= 1e-5 * absum + 1e-30)  # atomics: order-dependent last bits
    # the other element types: int32 exact; float16 / bfloat16 accumulate in their own type (as the reference's loop
    # nest does), so the bound is one rounding per addition of a segment (about 110 rows each here)
    for dt, npdt, tol in (("int32", np.int32, 0.0), ("float16", np.float16, 2.0 ** -10), ("bfloat16", BF16, 2.0 ** -7)):
        b = _Builder(f"Fused_UnsortedSegmentSum_{dt}_62")
        data = b.input("data", [4000, 48], dt)
        ids = b.input("ids", [4000], "int64")
        b.output(b.emit("UnsortedSegmentSum", [data, ids], [37, 48], dt, [_attr("num_segments", "int", 37)]))
        d = b.build()
        vals = rng.integers(-50, 50, (4000, 48)) if dt == "int32" else rng.standard_normal((4000, 48))
        ins = [vals.astype(np.float32).astype(npdt) if dt != "int32" else vals.astype(np.int32),
               rng.integers(0, 37, 4000).astype(np.int64)]
        got, _ = run(d, ins)
        want = O.evaluate(d, ins)[0]
        if dt == "int32":
            assert bits_equal(got[0], want)
        else:
            absum = np.zeros((37, 48))
            np.add.at(absum, ins[1], np.abs(ins[0].astype(np.float64)))
            counts = np.bincount(ins[1], minlength=37)[:, None]
            assert np.all(np.abs(got[0].astype(np.float64) - want.astype(np.float64)) <= tol * counts * absum / 8 + tol * absum)


def test_pad_split_argmax(lib):
    rng = np.random.default_rng(70)
    # Pad, both attribute spellings, followed by an elementwise op
    for spelling in ("padding", "head_tail"):
        b = _Builder("Fused_Pad_Add_70")
        x = b.input("x", [3, 5, 16], "float16")
        if spelling == "padding":  # pairs from the last dimension backwards
            attrs = [_attr("padding", "listInt", [8, 0, 1, 2]), _attr("value", "int", 0), _attr("mode", "str", "constant")]
        else:
            attrs = [_attr("head", "listInt", [0, 1, 8]), _attr("tail", "listInt", [0, 2, 0]), _attr("pad_val", "float", 0.0)]
        p = b.emit("Pad", [x], [3, 8, 24], "float16", attrs)
        b.output(b.emit("Add", [p, b.const(1.5, "float16")], [3, 8, 24], "float16"))
        check(b.build(), [rng.standard_normal((3, 5, 16)).astype(np.float16)], exact=True)
    # Split into three uneven pieces along axis 1, each used afterwards
    b = _Builder("Fused_Split_71")
    x = b.input("x", [4, 10, 8], "float32")
    pieces = b.emit_multi("Split", [x], [([4, 2, 8], "float32"), ([4, 5, 8], "float32"), ([4, 3, 8], "float32")],
                          [_attr("axis", "int", 1), _attr("split_size_or_sections", "listInt", [2, 5, 3])])
    b.output(b.emit("Neg", [pieces[0]], [4, 2, 8], "float32"))
    b.output(b.emit("Abs", [pieces[1]], [4, 5, 8], "float32"))
    b.output(pieces[2])
    check(b.build(), [rng.standard_normal((4, 10, 8)).astype(np.float32)], exact=True)
    # ArgMax along the last axis (ties and NaN resolve to the first index) and along a middle axis
    b = _Builder("Fused_ArgMax_72")
    x = b.input("x", [6, 7, 333], "float32")
    b.output(b.emit("ArgMax", [x], [6, 7], "int32", _reduce_attr([2], False)))
    xv = rng.integers(-4, 5, (6, 7, 333)).astype(np.float32)  # many ties
    xv[2, 3, 100] = np.nan
    xv[2, 3, 200] = np.nan
    check(b.build(), [xv], exact=True)
    b = _Builder("Fused_ArgMax_73")
    x = b.input("x", [5, 40, 9], "float16")
    b.output(b.emit("ArgMax", [x], [5, 1, 9], "int32", _reduce_attr([1], True)))
    check(b.build(), [rng.standard_normal((5, 40, 9)).astype(np.float16)], exact=True)


def test_matmul_float16_and_float32_operands(lib):
    rng = np.random.default_rng(80)
    mm_attr = [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)]
    # float16 operands on the tensor cores, f32 accumulation, fused bias + ReLU + cast back to float16
    m, k_, n = 300, 136, 264
    b = _Builder("Fused_MatMul_Add_Max_Cast_80")
    a = b.input("a", [m, k_], "float16")
    w = b.input("w", [k_, n], "float16")
    bias = b.input("bias", [n], "float32")
    c = b.emit("MatMul", [a, w], [m, n], "float32", mm_attr)
    c = b.emit("Add", [c, bias], [m, n], "float32")
    c = b.emit("Maximum", [c, b.const(0.0, "float32")], [m, n], "float32")
    b.output(b.emit("Cast", [c], [m, n], "float16", [_attr("dst_type", "str", "float16")]))
    d = b.build()
    ins = [(rng.standard_normal((m, k_)) * 0.1).astype(np.float16), (rng.standard_normal((k_, n)) * 0.1).astype(np.float16),
           rng.standard_normal(n).astype(np.float32) * 0.1]
    got, kern = run(d, ins)
    want = np.maximum(ins[0].astype(np.float64) @ ins[1].astype(np.float64) + ins[2], 0.0)
    assert kern.launch_count == 1 and got[0].dtype == np.float16
    np.testing.assert_allclose(got[0].astype(np.float64), want, rtol=2e-3, atol=2e-3)
    # float32 operands: one fused-multiply-add chain per element in k order -> bit-exact against that chain
    for tb in (False, True):
        m, k_, n = 150, 77, 203  # ragged in every extent, rows not 16-byte aligned
        b = _Builder("Fused_MatMul_81")
        a = b.input("a", [m, k_], "float32")
        w = b.input("w", [n, k_] if tb else [k_, n], "float32")
        b.output(b.emit("MatMul", [a, w], [m, n], "float32",
                        [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", tb)]))
        d = b.build()
        av = rng.standard_normal((m, k_)).astype(np.float32)
        wv = rng.standard_normal((k_, n)).astype(np.float32)
        got, kern = run(d, [av, np.ascontiguousarray(wv.T) if tb else wv])
        acc = np.zeros((m, n), dtype=np.float64)
        for kk in range(k_):  # fma in float32: exact product + accumulator, rounded once (float64 holds it exactly)
            acc = (av[:, kk:kk + 1].astype(np.float64) * wv[kk:kk + 1, :].astype(np.float64) + acc).astype(np.float32).astype(np.float64)
        assert bits_equal(got[0], acc.astype(np.float32))
        np.testing.assert_allclose(got[0], O.evaluate(d, [av, np.ascontiguousarray(wv.T) if tb else wv])[0], rtol=1e-4, atol=1e-4)
    # batched float32 with a shared right operand
    b = _Builder("Fused_BatchMatMul_82")
    a = b.input("a", [5, 64, 48], "float32")
    w = b.input("w", [48, 96], "float32")
    b.output(b.emit("BatchMatMul", [a, w], [5, 64, 96], "float32", mm_attr))
    d = b.build()
    ins = [rng.standard_normal((5, 64, 48)).astype(np.float32), rng.standard_normal((48, 96)).astype(np.float32)]
    got, kern = run(d, ins)
    assert kern.launch_count == 1
    np.testing.assert_allclose(got[0], O.evaluate(d, ins)[0], rtol=1e-4, atol=1e-4)


def test_generated_kernels_are_reused_from_disk(tmp_path):
    """Two processes in a row with the same cache directory: the first compiles and stores the kernel, the second
    loads the stored image and compiles nothing; both produce the same bits."""
    import subprocess
    import sys
    script = r'''
import sys, numpy as np
sys.path.insert(0, sys.argv[1])
from akg_b200.driver import FusedKernel, set_cache_dir, jit_cache_stats
from akg_b200.descs import _Builder
set_cache_dir(sys.argv[2])
b = _Builder("Fused_Mul_Add_Exp_90")
x = b.input("x", [64, 1000], "float32"); y = b.input("y", [1000], "float32")
t = b.emit("Mul", [x, y], [64, 1000], "float32")
t = b.emit("Add", [t, b.const(0.25, "float32")], [64, 1000], "float32")
b.output(b.emit("Exp", [t], [64, 1000], "float32"))
k = FusedKernel(b.build())
rng = np.random.default_rng(5)
ins = [rng.standard_normal((64, 1000)).astype(np.float32), rng.standard_normal(1000).astype(np.float32)]
out = k.empty_outputs()
k.run_host(ins + out)
compiled, from_disk = jit_cache_stats()
print(compiled, from_disk, out[0].view(np.uint32).sum(dtype=np.uint64))
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    runs = []
    for _ in range(2):
        r = subprocess.run([sys.executable, "-c", script, root, str(tmp_path)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        runs.append(r.stdout.split())
    assert runs[0][:2] == ["1", "0"], runs
    assert runs[1][:2] == ["0", "1"], runs
    assert runs[0][2] == runs[1][2]
    files = [f for f in os.listdir(tmp_path) if f.startswith("akgb_ew_") and f.endswith(".sm_100a.cubin")]
    assert len(files) == 1



def test_matmul_epilogue_is_folded_inside_a_larger_region(lib):
    """Two matmuls in one region: bias + ReLU + cast after the first run in its launch, the rest as planned."""
    rng = np.random.default_rng(95)
    m, k_, n, n2 = 256, 128, 192, 64
    mm = [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)]
    b = _Builder("Fused_MatMul_Add_Max_Cast_MatMul_ReduceSum_95")
    h, f = "bfloat16", "float32"
    a = b.input("a", [m, k_], h)
    w1 = b.input("w1", [k_, n], h)
    bias = b.input("bias", [n], h)
    w2 = b.input("w2", [n, n2], h)
    bf = b.emit("Cast", [bias], [n], f, [_attr("dst_type", "str", f)])
    c = b.emit("MatMul", [a, w1], [m, n], f, mm)
    c = b.emit("Add", [c, bf], [m, n], f)
    c = b.emit("Maximum", [c, b.const(0.0, f)], [m, n], f)
    hcast = b.emit("Cast", [c], [m, n], h, [_attr("dst_type", "str", h)])
    o = b.emit("MatMul", [hcast, w2], [m, n2], f, mm)
    b.output(o)
    b.output(b.emit("ReduceSum", [o], [n2], f, _reduce_attr([0], False)))
    d = b.build()
    ins = [(rng.standard_normal(s) * 0.1).astype(BF16) for s in ((m, k_), (k_, n), (n,), (n, n2))]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins)
    assert kern.launch_count == 2 + FusedKernel(descs.reduce_sum_axis0(m, n2)).launch_count  # no elementwise launch
    for g_, w_ in zip(got, want):
        np.testing.assert_allclose(g_, w_, rtol=2e-2, atol=2e-2 * float(np.abs(w_).max()))


def _rows_region(kind, rows_shape, cols, dtype="float32"):
    """Reduce-X regions in spellings no hand-written template claims."""
    f = "float32"
    shape = list(rows_shape) + [cols]
    red = list(rows_shape) + [1]
    ax = [len(shape) - 1]
    b = _Builder(f"Fused_{kind}_{cols}")
    x = b.input("x", shape, dtype)
    xf = x if dtype == f else b.emit("Cast", [x], shape, f, [_attr("dst_type", "str", f)])
    if kind == "rmsnorm":
        g_ = b.input("g", [cols], f)
        ss = b.emit("ReduceSum", [b.emit("Mul", [xf, xf], shape, f)], red, f, _reduce_attr(ax, True))
        ms = b.emit("RealDiv", [ss, b.const(float(cols), f)], red, f)
        r = b.emit("Rsqrt", [b.emit("Add", [ms, b.const(1e-6, f)], red, f)], red, f)
        y = b.emit("Mul", [b.emit("Mul", [xf, r], shape, f), g_], shape, f)
        outs = [y]
    elif kind == "log_softmax":
        m = b.emit("ReduceMax", [xf], red, f, _reduce_attr(ax, True))
        d = b.emit("Sub", [xf, m], shape, f)
        lse = b.emit("Log", [b.emit("ReduceSum", [b.emit("Exp", [d], shape, f)], red, f, _reduce_attr(ax, True))], red, f)
        y = b.emit("Sub", [d, lse], shape, f)
        outs = [y]
    elif kind == "select_softmax":  # safe softmax with a boolean mask shared by the leading batch dims
        keep = b.input("keep", [rows_shape[-1], cols], "bool")
        s_ = b.emit("Select", [keep, xf, b.const(-1e30, f)], shape, f)
        m = b.emit("ReduceMax", [s_], red, f, _reduce_attr(ax, True))
        e = b.emit("Exp", [b.emit("Sub", [s_, m], shape, f)], shape, f)
        y = b.emit("RealDiv", [e, b.emit("ReduceSum", [e], red, f, _reduce_attr(ax, True))], shape, f)
        outs = [y]
    elif kind == "l2norm_stats":  # a full result and two per-row results, one of them without keep_dims
        ss = b.emit("ReduceSum", [b.emit("Mul", [xf, xf], shape, f)], red, f, _reduce_attr(ax, True))
        nrm = b.emit("Sqrt", [ss], red, f)
        y = b.emit("RealDiv", [xf, b.emit("Maximum", [nrm, b.const(1e-12, f)], red, f)], shape, f)
        mx = b.emit("ReduceMax", [xf], list(rows_shape), f, _reduce_attr(ax, False))
        outs = [y, nrm, mx]
    else:
        raise ValueError(kind)
    for i, o in enumerate(outs):
        if i == 0 and dtype != f:
            o = b.emit("Cast", [o], shape, dtype, [_attr("dst_type", "str", dtype)])
        b.output(o)
    return b.build()


@pytest.mark.parametrize("kind,rows_shape,cols,dtype", [
    ("rmsnorm", [300], 1024, "float32"),
    ("rmsnorm", [7, 5], 40, "float32"),           # narrow rows: several rows per warp
    ("rmsnorm", [33], 100, "float16"),            # cols not a multiple of 8: element-wise accesses
    ("log_softmax", [130], 4096, "float32"),      # wide rows: several warps per row
    ("log_softmax", [4, 50], 512, "bfloat16"),
    ("select_softmax", [3, 64], 256, "float16"),
    ("l2norm_stats", [257], 768, "float32"),
    ("l2norm_stats", [2, 3, 5], 8192, "float32"),
    ("log_softmax", [70], 32000, "float32"),      # rows too long for registers: one pass per reduction, one for the result
    ("rmsnorm", [33], 20000, "float16"),
    ("select_softmax", [2, 9], 24576, "bfloat16"),
    ("l2norm_stats", [5], 50001, "float32"),      # and not a multiple of 8
])
def test_reduce_x_regions_as_one_generated_kernel(lib, kind, rows_shape, cols, dtype):
    rng = np.random.default_rng(hash((kind, cols)) % 1000)
    d = _rows_region(kind, rows_shape, cols, dtype)
    ins = []
    for (t,) in d["input_desc"]:
        if t["data_type"] == "bool":
            a = rng.random(t["shape"]) < 0.7
            a[:, 0] = True  # no fully masked row
            ins.append(a)
        elif t["tensor_name"] == "g":
            ins.append(rng.uniform(0.5, 1.5, t["shape"]).astype(np.float32))
        else:
            npdt = BF16 if t["data_type"] == "bfloat16" else np.dtype(t["data_type"])
            ins.append(rng.standard_normal(t["shape"]).astype(np.float32).astype(npdt))
    got, k = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    tol = 1e-5 if dtype == "float32" else 4e-3
    for g_, w_ in zip(got, want):
        assert g_.shape == w_.shape and g_.dtype == w_.dtype
        scale = float(np.abs(w_.astype(np.float64)).max())
        np.testing.assert_allclose(g_.astype(np.float64), w_.astype(np.float64), rtol=tol, atol=tol * max(scale, 1e-6))
    if FLAGS[0] == 0:
        assert k.launch_count == 1 and k.meta()["template"] == "akgb_row_jit"
        assert "akgb_row_jit" in k.jit_source(cols % 8 == 0)
    else:
        assert k.launch_count > 1


@pytest.mark.parametrize("kind,rows_shape,cols,dtype,cluster", [
    ("log_softmax", [70], 32000, "float32", 2),       # 125 KB per row: two CTAs share a row
    ("rmsnorm", [33], 20000, "float16", 1),           # 39 KB: one CTA keeps its row
    ("select_softmax", [2, 9], 24576, "bfloat16", 1),  # exactly 48 KB of dynamic shared memory
    ("log_softmax", [9], 131072, "float32", 8),       # 512 KB per row: a cluster of eight
    ("log_softmax", [5], 100008, "bfloat16", 4),      # chunks of different length (the last CTA's is shorter)
])
def test_long_rows_staged_in_shared_memory_across_a_cluster(lib, kind, rows_shape, cols, dtype, cluster):
    """AKGB_FLAG_STAGE_LONG_ROWS: the first pass keeps the row in shared memory, a thread-block cluster shares rows that
    exceed one CTA's part, per-row reductions are completed through distributed shared memory.  Same bits as the
    default schedule (which re-reads the row through L2) when one CTA holds the row; within the tolerance of the
    region otherwise (the fold over the CTAs of a cluster changes the order of the sums)."""
    from akg_b200 import _capi
    if FLAGS[0] != 0:
        pytest.skip("generated kernels only")
    rng = np.random.default_rng(cols % 1000)
    d = _rows_region(kind, rows_shape, cols, dtype)
    ins = []
    for (t,) in d["input_desc"]:
        if t["data_type"] == "bool":
            a = rng.random(t["shape"]) < 0.7
            a[:, 0] = True
            ins.append(a)
        elif t["tensor_name"] == "g":
            ins.append(rng.uniform(0.5, 1.5, t["shape"]).astype(np.float32))
        else:
            npdt = BF16 if t["data_type"] == "bfloat16" else np.dtype(t["data_type"])
            ins.append(rng.standard_normal(t["shape"]).astype(np.float32).astype(npdt))
    base, _ = guarded_launch(d, ins)
    got, k = guarded_launch(d, ins, flags=_capi.AKGB_FLAG_STAGE_LONG_ROWS)
    src = k.jit_source()
    assert "stage_mem" in src and f"K = {cluster}" in src and (cluster == 1 or f"__cluster_dims__({cluster}, 1, 1)" in src)
    want = O.evaluate(d, ins, accum="float64")
    tol = 1e-5 if dtype == "float32" else 4e-3
    for g_, b_, w_ in zip(got, base, want):
        if cluster == 1:
            assert bits_equal(g_, b_)
        scale = float(np.abs(w_.astype(np.float64)).max())
        np.testing.assert_allclose(g_.astype(np.float64), w_.astype(np.float64), rtol=tol, atol=tol * max(scale, 1e-6))


@pytest.mark.parametrize("shape,k,cols_kind", [
    ([4096, 1024], 1, "plain"),       # dgamma-like: sum over rows of dy * xhat
    ([8, 600, 768], 2, "with_col"),   # two leading axes folded, a [cols] operand in the chain
    ([3000, 100], 1, "with_row"),     # cols not a multiple of 8, a per-row operand
    ([70000, 8], 1, "max"),
])
def test_elementwise_chain_folded_into_a_reduction_over_leading_axes(lib, shape, k, cols_kind):
    rng = np.random.default_rng(len(shape) * 100 + shape[-1])
    f = "float32"
    out_shape = shape[k:]
    b = _Builder("Fused_Mul_ReduceSum_Y_97")
    x = b.input("x", shape, f)
    y = b.input("y", shape, f)
    t = b.emit("Mul", [x, y], shape, f)
    if cols_kind == "with_col":
        g_ = b.input("g", out_shape, f)
        t = b.emit("Add", [t, g_], shape, f)
    if cols_kind == "with_row":
        r_ = b.input("r", shape[:k] + [1] * (len(shape) - k), f)
        t = b.emit("Sub", [t, r_], shape, f)
    op = "ReduceMax" if cols_kind == "max" else "ReduceSum"
    b.output(b.emit(op, [t], out_shape, f, _reduce_attr(list(range(k)), False)))
    d = b.build()
    ins = [rng.standard_normal(t_["shape"]).astype(np.float32) for (t_,) in d["input_desc"]]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")[0]
    full = ins[0].astype(np.float64) * ins[1].astype(np.float64)
    if cols_kind == "max":
        assert bits_equal(got[0], want)
    else:
        bound = 1e-5 * np.abs(full).sum(axis=tuple(range(k))) + 1e-4 * (cols_kind != "plain") * np.prod(shape[:k])
        assert np.all(np.abs(got[0].astype(np.float64) - want.astype(np.float64)) <= bound + 1e-6)
    if FLAGS[0] == 0:
        assert kern.meta()["template"] == "akgb_col_jit" and kern.launch_count <= 3


def test_prepare_allows_capturing_the_first_launch(lib):
    """After prepare() the first launch of a region with generated kernels can be recorded into a CUDA graph."""
    import torch
    d = _rows_region("rmsnorm", [64], 512)
    k = FusedKernel(d, flags=_flags())
    k.prepare()
    x = torch.randn(64, 512, device="cuda")
    g_ = torch.rand(512, device="cuda") + 0.5
    out = torch.empty(64, 512, device="cuda")
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            k.launch([x, g_, out], torch.cuda.current_stream())
        graph.replay()
    torch.cuda.synchronize()
    want = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * g_
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)


def test_two_column_reductions_share_one_pass(lib):
    """dgamma = sum_rows(dy * xhat) and dbeta = sum_rows(dy) of one region: one generated kernel reads dy and xhat once."""
    rng = np.random.default_rng(98)
    f = "float32"
    shape = [4, 1500, 512]
    b = _Builder("Fused_Mul_ReduceSum_ReduceSum_98")
    dy = b.input("dy", shape, f)
    xhat = b.input("xhat", shape, f)
    t = b.emit("Mul", [dy, xhat], shape, f)
    b.output(b.emit("ReduceSum", [t], [512], f, _reduce_attr([0, 1], False)))
    b.output(b.emit("ReduceSum", [dy], [512], f, _reduce_attr([0, 1], False)))
    d = b.build()
    ins = [rng.standard_normal(shape).astype(np.float32) for _ in range(2)]
    got, kern = run(d, ins)
    a64, b64 = ins[0].astype(np.float64), ins[1].astype(np.float64)
    want = [(a64 * b64).sum(axis=(0, 1)), a64.sum(axis=(0, 1))]
    bound = [1e-5 * np.abs(a64 * b64).sum(axis=(0, 1)), 1e-5 * np.abs(a64).sum(axis=(0, 1))]
    for g_, w_, bd in zip(got, want, bound):
        assert np.all(np.abs(g_.astype(np.float64) - w_) <= bd + 1e-6)
    if FLAGS[0] == 0:
        assert kern.meta()["template"] == "akgb_col_jit"


def test_reduction_over_non_adjacent_axes(lib):
    rng = np.random.default_rng(99)
    f = "float32"
    for shape, axes, keep in (([6, 40, 50], [0, 2], True), ([3, 4, 5, 64], [1, 3], False), ([5, 7, 1, 9], [0, 3], False)):
        oshape = [1 if i in axes else e for i, e in enumerate(shape)] if keep else [e for i, e in enumerate(shape) if i not in axes]
        for op in ("ReduceSum", "ReduceMax"):
            b = _Builder("Fused_Reduce_non_adjacent_99")
            x = b.input("x", shape, f)
            b.output(b.emit(op, [x], oshape, f, _reduce_attr(axes, keep)))
            d = b.build()
            xv = rng.standard_normal(shape).astype(np.float32)
            got, _ = run(d, [xv])
            want = O.evaluate(d, [xv], accum="float64")[0]
            if op == "ReduceMax":
                assert bits_equal(got[0], want)
            else:
                assert np.all(np.abs(got[0].astype(np.float64) - want) <= 1e-5 * np.abs(xv).sum(axis=tuple(axes), keepdims=keep))


def test_chain_then_reduction_over_trailing_and_leading_axes(lib):
    """BatchNorm statistics on NCHW: Mul(x, x) -> ReduceSum over (0, 2, 3) -> Mul(1/n).  The square and the fold over
    (H, W) run as one generated row kernel, the fold over N and the scaling on the row results."""
    rng = np.random.default_rng(101)
    f = "float32"
    n_, c_, h_, w_ = 8, 32, 28, 28
    shape = [n_, c_, h_, w_]
    for keep in (True, False):
        oshape = [1, c_, 1, 1] if keep else [c_]
        b = _Builder("Fused_Mul_ReduceSum_Mul_101")
        x = b.input("x", shape, f)
        y = b.input("y", shape, f)
        t = b.emit("Mul", [b.emit("Sub", [x, y], shape, f), x], shape, f)
        s_ = b.emit("ReduceSum", [t], oshape, f, _reduce_attr([0, 2, 3], keep))
        b.output(b.emit("Mul", [s_, b.const(1.0 / (n_ * h_ * w_), f)], oshape, f))
        b.output(s_)
        d = b.build()
        ins = [rng.standard_normal(shape).astype(np.float32) for _ in range(2)]
        got, kern = run(d, ins)
        want = O.evaluate(d, ins, accum="float64")
        full = (ins[0].astype(np.float64) - ins[1]) * ins[0]
        bound = 1e-5 * np.abs(full).sum(axis=(0, 2, 3), keepdims=keep)
        assert np.all(np.abs(got[1].astype(np.float64) - want[1]) <= bound)
        assert np.all(np.abs(got[0].astype(np.float64) - want[0]) <= bound / (n_ * h_ * w_) + 1e-7)
        if FLAGS[0] == 0:
            assert kern.meta()["template"] == "akgb_row_jit"
    # trailing axes only, over a multi-dimensional run: max over (H, W) of a difference
    b = _Builder("Fused_Sub_ReduceMax_102")
    x = b.input("x", shape, f)
    y = b.input("y", shape, f)
    b.output(b.emit("ReduceMax", [b.emit("Sub", [x, y], shape, f)], [n_, c_], f, _reduce_attr([2, 3], False)))
    d = b.build()
    ins = [rng.standard_normal(shape).astype(np.float32) for _ in range(2)]
    got, kern = run(d, ins)
    assert bits_equal(got[0], O.evaluate(d, ins)[0])
    if FLAGS[0] == 0:
        assert kern.meta()["template"] == "akgb_row_jit" and kern.launch_count == 1


def test_per_channel_operands_in_front_of_a_batchnorm_style_reduction(lib):
    """dgamma = sum over (N, H, W) of dy * (x - mean) * rstd with mean, rstd of shape [1, C, 1, 1], and dbeta = sum of dy."""
    rng = np.random.default_rng(103)
    f = "float32"
    shape, stat = [6, 24, 20, 24], [1, 24, 1, 1]
    b = _Builder("Fused_Sub_Mul_Mul_ReduceSum_ReduceSum_103")
    dy, x = b.input("dy", shape, f), b.input("x", shape, f)
    mean, rstd = b.input("mean", stat, f), b.input("rstd", stat, f)
    xhat = b.emit("Mul", [b.emit("Sub", [x, mean], shape, f), rstd], shape, f)
    b.output(b.emit("ReduceSum", [b.emit("Mul", [dy, xhat], shape, f)], stat, f, _reduce_attr([0, 2, 3], True)))
    b.output(b.emit("ReduceSum", [dy], stat, f, _reduce_attr([0, 2, 3], True)))
    d = b.build()
    ins = [rng.standard_normal(shape).astype(np.float32), rng.standard_normal(shape).astype(np.float32),
           rng.standard_normal(stat).astype(np.float32), rng.uniform(0.5, 2.0, stat).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    dy64, x64 = ins[0].astype(np.float64), ins[1].astype(np.float64)
    terms = np.abs(dy64 * (x64 - ins[2]) * ins[3])
    assert np.all(np.abs(got[0] - want[0]) <= 1e-5 * terms.sum(axis=(0, 2, 3), keepdims=True))
    assert np.all(np.abs(got[1] - want[1]) <= 1e-5 * np.abs(dy64).sum(axis=(0, 2, 3), keepdims=True))
    if FLAGS[0] == 0:
        assert kern.meta()["template"] == "akgb_row_jit"
        assert "(r / 1LL) % 24LL" in kern.jit_source()


@pytest.mark.parametrize("io", ["float32", "float16"])
def test_batch_norm_training_region_is_cut_at_its_reductions(lib, io):
    """Three pieces (mean; centred squares folded into the variance pass; scale and shift with the centred values
    computed again): only per-channel values cross launches."""
    rng = np.random.default_rng(106)
    shape = [6, 40, 24, 24]
    d = _batch_norm_training(shape, io, 106)
    ins = [(rng.standard_normal(shape) * 2 + 0.5).astype(np.dtype(io)), rng.uniform(0.5, 1.5, [1, 40, 1, 1]).astype(np.float32),
           rng.standard_normal([1, 40, 1, 1]).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0].astype(np.float32), want[0].astype(np.float32), rtol=2e-3 if io == "float16" else 1e-5,
                               atol=2e-3 if io == "float16" else 1e-5)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got[2], want[2], rtol=1e-5, atol=1e-6)
    if FLAGS[0] == 0:
        meta = kern.meta()
        assert "akgb_row_jit" in meta["steps"] and meta["workspace"] < 4 * shape[0] * shape[1] * 64


def test_batch_norm_backward_folds_both_sums_in_one_pass(lib):
    rng = np.random.default_rng(107)
    shape, stat = [6, 40, 24, 24], [1, 40, 1, 1]
    d = _batch_norm_backward(shape, 107)
    ins = [rng.standard_normal(shape).astype(np.float32), (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32),
           rng.standard_normal(stat).astype(np.float32) * 0.1 + 0.5, rng.uniform(0.4, 0.6, stat).astype(np.float32),
           rng.uniform(0.5, 1.5, stat).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(got[2], want[2], rtol=1e-4, atol=1e-3)
    if FLAGS[0] == 0:
        meta = kern.meta()
        assert meta["steps"].count("akgb_row_jit") == 1 and meta["workspace"] < (1 << 20)
        assert "out1" in kern.jit_source()  # one generated kernel with both row results


@pytest.mark.parametrize("rows,cols", [(300, 1024), (77, 200), (2048, 4096), (5, 8192), (700, 8192), (33, 8190), (40, 16384)])
def test_layer_norm_backward_sums_over_rows_inside_the_row_kernel(lib, rows, cols):
    """dx row by row, and in the same pass the weight and bias gradients as per-CTA column sums that a column
    reduction folds afterwards."""
    rng = np.random.default_rng(108)
    d = descs.layer_norm_backward(rows, cols)
    ins = [rng.standard_normal((rows, cols)).astype(np.float32), (rng.standard_normal((rows, cols)) * 2 + 0.5).astype(np.float32),
           rng.uniform(0.5, 1.5, cols).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-4, atol=1e-4)
    scale = np.sqrt(rows)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-4, atol=1e-4 * scale)
    np.testing.assert_allclose(got[2], want[2], rtol=1e-4, atol=1e-4 * scale)
    if FLAGS[0] == 0:
        meta = kern.meta()
        assert meta["steps"] == ["akgb_row_jit", "reduce_col_f32", "reduce_col_f32"]
        # the register schedule walks row blocks, the multi-pass schedule (rows too long for registers) rows
        src = kern.jit_source(cols % 8 == 0)
        assert ("rb += gridDim.x" in src) == (cols <= 4096) and ("r += gridDim.x" in src) == (cols > 4096)


def test_ops_behind_sums_over_rows_run_after_the_fold(lib):
    rng = np.random.default_rng(109)
    rows, cols = 600, 512
    d = descs.layer_norm_backward(rows, cols, grads_dtype="float16")
    ins = [rng.standard_normal((rows, cols)).astype(np.float32), (rng.standard_normal((rows, cols)) + 0.5).astype(np.float32),
           rng.uniform(0.5, 1.5, cols).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-4, atol=1e-4)
    for i in (1, 2):
        assert got[i].dtype == np.float16
        np.testing.assert_allclose(got[i].astype(np.float32), want[i].astype(np.float32), rtol=2e-3, atol=5e-2)
    if FLAGS[0] == 0:
        assert kern.meta()["steps"] == ["akgb_row_jit", "reduce_col_f32", "reduce_col_f32", "ew_generic"]


def test_instance_norm_on_nchw_is_one_row_kernel(lib):
    """Mean / variance over (H, W) with keep_dims, per-channel scale and shift of shape [1, C, 1, 1]."""
    rng = np.random.default_rng(104)
    f = "float32"
    n_, c_, h_, w_ = 3, 20, 24, 16
    shape, red, stat = [n_, c_, h_, w_], [n_, c_, 1, 1], [1, c_, 1, 1]
    b = _Builder("Fused_InstanceNorm_104")
    x, gamma, beta = b.input("x", shape, f), b.input("gamma", stat, f), b.input("beta", stat, f)
    inv = b.const(1.0 / (h_ * w_), f)
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], red, f, _reduce_attr([2, 3], True)), inv], red, f)
    d_ = b.emit("Sub", [x, mean], shape, f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [d_, d_], shape, f)], red, f, _reduce_attr([2, 3], True)), inv], red, f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], red, f)], red, f)
    y = b.emit("Add", [b.emit("Mul", [b.emit("Mul", [d_, rstd], shape, f), gamma], shape, f), beta], shape, f)
    b.output(y)
    b.output(mean)
    d = b.build()
    ins = [rng.standard_normal(shape).astype(np.float32), rng.uniform(0.5, 1.5, stat).astype(np.float32),
           rng.standard_normal(stat).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-5, atol=1e-6)
    if FLAGS[0] == 0:
        assert kern.launch_count == 1 and kern.meta()["template"] == "akgb_row_jit"
        assert f"constexpr int C = {h_ * w_}" in kern.jit_source()


def test_regions_that_are_row_regions_only_in_part(lib):
    rng = np.random.default_rng(105)
    f = "float32"
    # centred rows, flattened: the row kernel writes through the view
    b = _Builder("Fused_Mul_ReduceSum_Sub_Reshape_105")
    x = b.input("x", [96, 200], f)
    r = b.emit("ReduceSum", [b.emit("Mul", [x, x], [96, 200], f)], [96, 1], f, _reduce_attr([1], True))
    u = b.emit("Sub", [x, r], [96, 200], f)
    b.output(b.emit("Reshape", [u], [19200], f, [_attr("shape", "listInt", [19200])]))
    d = b.build()
    ins = [rng.standard_normal((96, 200)).astype(np.float32)]
    got, kern = run(d, ins)
    np.testing.assert_allclose(got[0], O.evaluate(d, ins, accum="float64")[0], rtol=1e-5, atol=1e-4)
    if FLAGS[0] == 0:
        assert kern.launch_count == 1
    # softmax over the last axis, then a transpose of the leading axes and a scale: row kernel + the rest
    b = _Builder("Fused_Softmax_Transpose_Mul_106")
    x = b.input("x", [6, 10, 128], f)
    m = b.emit("ReduceMax", [x], [6, 10, 1], f, _reduce_attr([2], True))
    e = b.emit("Exp", [b.emit("Sub", [x, m], [6, 10, 128], f)], [6, 10, 128], f)
    p = b.emit("RealDiv", [e, b.emit("ReduceSum", [e], [6, 10, 1], f, _reduce_attr([2], True))], [6, 10, 128], f)
    t = b.emit("Transpose", [p], [10, 6, 128], f, [_attr("perm", "listInt", [1, 0, 2])])
    b.output(b.emit("Mul", [t, b.const(0.5, f)], [10, 6, 128], f))
    b.output(m)
    d = b.build()
    ins = [rng.standard_normal((6, 10, 128)).astype(np.float32)]
    got, kern = run(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-7)
    assert bits_equal(got[1], want[1])
    if FLAGS[0] == 0:
        assert kern.launch_count == 3  # row kernel, transpose, scale
    # two row regions over different views with elementwise ops in between (GroupNorm-like)
    b = _Builder("Fused_GroupStats_Affine_107")
    x = b.input("x", [4, 8, 6, 10], f)       # [n, c, h, w]
    w = b.input("w", [1, 8, 1, 1], f)
    g_ = b.emit("Reshape", [x], [4, 2, 240], f, [_attr("shape", "listInt", [4, 2, 240])])
    mean = b.emit("Mul", [b.emit("ReduceSum", [g_], [4, 2, 1], f, _reduce_attr([2], True)), b.const(1 / 240, f)], [4, 2, 1], f)
    dd = b.emit("Sub", [g_, mean], [4, 2, 240], f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [dd, dd], [4, 2, 240], f)], [4, 2, 1], f, _reduce_attr([2], True)),
                         b.const(1 / 240, f)], [4, 2, 1], f)
    y = b.emit("Mul", [dd, b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], [4, 2, 1], f)], [4, 2, 1], f)], [4, 2, 240], f)
    y4 = b.emit("Reshape", [y], [4, 8, 6, 10], f, [_attr("shape", "listInt", [4, 8, 6, 10])])
    b.output(b.emit("Mul", [y4, w], [4, 8, 6, 10], f))
    d = b.build()
    ins = [rng.standard_normal((4, 8, 6, 10)).astype(np.float32), rng.uniform(0.5, 1.5, (1, 8, 1, 1)).astype(np.float32)]
    got, kern = run(d, ins)
    np.testing.assert_allclose(got[0], O.evaluate(d, ins, accum="float64")[0], rtol=1e-5, atol=1e-5)
    if FLAGS[0] == 0:
        assert kern.launch_count == 2  # statistics + normalisation as a row kernel, then the per-channel scale


def test_exported_binary_runs_through_the_driver_api_alone(lib, tmp_path):
    """The exported <kernel>.cubin is launched the way a foreign runtime would: cuModuleLoadData, the entry point and
    launch dimensions from <kernel>.json, the tensors' bare device pointers as the only arguments -- and gives the
    bits akgb_launch gives."""
    import ctypes
    import json
    import torch
    b = _Builder("Fused_Add_Tanh_Mul_export_2")
    f = "float32"
    x, y = b.input("x", [384, 1000], f), b.input("y", [1000], f)
    t = b.emit("Tanh", [b.emit("Add", [x, y], [384, 1000], f)], [384, 1000], f)
    b.output(b.emit("Mul", [t, x], [384, 1000], f))
    for d in (b.build(), descs.rmsnorm(300, 1024)):
        k = FusedKernel(d)
        k.export(tmp_path)
        meta = json.loads((tmp_path / (d["op"] + ".json")).read_text())
        image = (tmp_path / meta["binary"]).read_bytes()
        ins = [torch.from_numpy(a).cuda() for a in make_inputs(d, 41)]
        want = [torch.empty(t_.shape, dtype=torch.float32, device="cuda") for t_ in k.outputs]
        k.launch(ins + want)
        got = [torch.full(t_.shape, float("nan"), dtype=torch.float32, device="cuda") for t_ in k.outputs]
        torch.cuda.synchronize()
        cu = ctypes.CDLL("libcuda.so.1")
        mod, fn = ctypes.c_void_p(), ctypes.c_void_p()
        assert cu.cuModuleLoadData(ctypes.byref(mod), image) == 0
        assert cu.cuModuleGetFunction(ctypes.byref(fn), mod, meta["kernelName"].encode()) == 0
        ptrs = [ctypes.c_void_p(t_.data_ptr()) for t_ in ins + got]
        assert all(p.value % meta["pointer_alignment"] == 0 for p in ptrs)
        args = (ctypes.c_void_p * len(ptrs))(*[ctypes.cast(ctypes.pointer(p), ctypes.c_void_p) for p in ptrs])
        rc = cu.cuLaunchKernel(fn, meta["blockIdx.x"], meta["blockIdx.y"], meta["blockIdx.z"], meta["threadIdx.x"],
                               meta["threadIdx.y"], meta["threadIdx.z"], meta["shared_mem_bytes"],
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), args, None)
        assert rc == 0
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g.view(torch.int32), w.view(torch.int32))
        assert cu.cuModuleUnload(mod) == 0
