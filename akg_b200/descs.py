"""Builders of fused-op descriptions (``.info`` JSON) for the benchmarked operator classes.

The schema is the one MindSpore's graph-kernel module emits and
``akg-mlir/lib/Target/MindsporeDialect/TranslateToMindsporeDialect.cpp:295-415``
reads: ``op``, ``process``, ``input_desc`` (list of one-element lists),
``op_desc`` (name, attr, input_desc, output_desc) and ``output_desc``.
LayerNorm, GELU and softmax are spelled with primitive ops because the JSON
factory has no entry for them (``:417-486``).  Constants are operands that carry
a ``value`` (``:650-658``).
"""
from __future__ import annotations

import math
from typing import Sequence


def _t(name: str, shape: Sequence[int], dtype: str, value=None) -> dict:
    d = {"data_type": dtype, "format": "DefaultFormat", "shape": list(shape), "tensor_name": name}
    if value is not None:
        d["value"] = value
    return d


def _attr(name: str, dtype: str, value) -> dict:
    return {"name": name, "data_type": dtype, "value": value}


class _Builder:
    def __init__(self, op: str):
        self.op = op
        self.inputs: list[dict] = []
        self.ops: list[dict] = []
        self.outputs: list[dict] = []
        self._n = 0

    def input(self, name, shape, dtype):
        t = _t(name, shape, dtype)
        self.inputs.append(t)
        return t

    def const(self, value, dtype):
        self._n += 1
        return _t(f"const_{self._n}", [1], dtype, value)

    def emit(self, name, ins, shape, dtype, attr=None, out_name=None):
        self._n += 1
        out = _t(out_name or f"t{self._n}_{name.lower()}", shape, dtype)
        self.ops.append({"name": name, "attr": attr, "impl_path": "",
                         "input_desc": [[dict(i)] for i in ins], "output_desc": [dict(out)]})
        return out

    def emit_multi(self, name, ins, outs, attr=None):
        """An op with several results (Split): `outs` is a list of (shape, dtype)."""
        self._n += 1
        res = [_t(f"t{self._n}_{name.lower()}_{k}", shape, dtype) for k, (shape, dtype) in enumerate(outs)]
        self.ops.append({"name": name, "attr": attr, "impl_path": "",
                         "input_desc": [[dict(i)] for i in ins], "output_desc": [dict(o) for o in res]})
        return res

    def output(self, t):
        self.outputs.append(dict(t))

    def build(self) -> dict:
        return {"composite": True, "op": self.op, "process": "cuda", "platform": "AKG", "version": 2,
                "target_info": {"compute_capability": "10.0", "sm_count": 148},
                "input_desc": [[dict(i)] for i in self.inputs], "op_desc": self.ops,
                "output_desc": self.outputs}


def _reduce_attr(axes, keep_dims):
    return [_attr("axis", "listInt", list(axes)), _attr("keep_dims", "bool", bool(keep_dims))]


def layernorm(rows: int, cols: int, eps: float = 1e-5, with_stats: bool = True) -> dict:
    """x f32[rows, cols], gamma/beta f32[cols] -> y, mean[rows], var[rows]."""
    b = _Builder(f"Fused_LayerNorm_{rows}x{cols}_1")
    f = "float32"
    x = b.input("x", [rows, cols], f)
    gamma = b.input("gamma", [cols], f)
    beta = b.input("beta", [cols], f)
    inv_n = 1.0 / cols
    s1 = b.emit("ReduceSum", [x], [rows, 1], f, _reduce_attr([1], True))
    mean = b.emit("Mul", [s1, b.const(inv_n, f)], [rows, 1], f)
    d = b.emit("Sub", [x, mean], [rows, cols], f)
    sq = b.emit("Mul", [d, d], [rows, cols], f)
    s2 = b.emit("ReduceSum", [sq], [rows, 1], f, _reduce_attr([1], True))
    var = b.emit("Mul", [s2, b.const(inv_n, f)], [rows, 1], f)
    ve = b.emit("Add", [var, b.const(eps, f)], [rows, 1], f)
    rstd = b.emit("Rsqrt", [ve], [rows, 1], f)
    n0 = b.emit("Mul", [d, rstd], [rows, cols], f)
    n1 = b.emit("Mul", [n0, gamma], [rows, cols], f)
    y = b.emit("Add", [n1, beta], [rows, cols], f, out_name="y")
    b.output(y)
    if with_stats:
        shp = [_attr("shape", "listInt", [rows])]
        b.output(b.emit("Reshape", [mean], [rows], f, shp, out_name="mean_out"))
        b.output(b.emit("Reshape", [var], [rows], f, shp, out_name="var_out"))
    return b.build()


GELU_C0 = 0.044715
GELU_C1 = 0.7978845608
GELU_C2 = 0.5


def gelu_chain(shape: Sequence[int], with_bias: bool = True, with_mul: bool = True, cast_f32: bool = True,
               f32_math: bool = False) -> dict:
    """x f16[shape] (+ bias f16[shape[-1]]) -> tanh-GELU (* y f16[shape]) (-> f32); all math in f16, or, with
    `f32_math`, the same tensors widened to float32 first and every op in float32 (same bytes moved)."""
    shape = list(shape)
    b = _Builder("Fused_BiasAdd_Gelu_Mul_Cast_" + "x".join(map(str, shape)) + ("_f32math_2" if f32_math else "_2"))
    h = "float16"
    x = b.input("x", shape, h)
    bias = b.input("bias", [shape[-1]], h) if with_bias else None
    y = b.input("y", shape, h) if with_mul else None
    if f32_math:
        h = "float32"
        widen = [_attr("dst_type", "str", h)]
        x = b.emit("Cast", [x], shape, h, widen)
        bias = b.emit("Cast", [bias], [shape[-1]], h, widen) if with_bias else None
        y = b.emit("Cast", [y], shape, h, widen) if with_mul else None
        cast_f32 = False
    t = x
    if with_bias:
        t = b.emit("Add", [x, bias], shape, h)
    a = b.emit("Mul", [t, t], shape, h)
    t3 = b.emit("Mul", [a, t], shape, h)
    bb = b.emit("Mul", [t3, b.const(GELU_C0, h)], shape, h)
    c = b.emit("Add", [t, bb], shape, h)
    d = b.emit("Mul", [c, b.const(GELU_C1, h)], shape, h)
    e = b.emit("Tanh", [d], shape, h)
    f = b.emit("Add", [e, b.const(1.0, h)], shape, h)
    g = b.emit("Mul", [t, b.const(GELU_C2, h)], shape, h)
    out = b.emit("Mul", [g, f], shape, h)
    if with_mul:
        out = b.emit("Mul", [out, y], shape, h)
    if cast_f32:
        out = b.emit("Cast", [out], shape, "float32", [_attr("dst_type", "str", "float32")])
    b.output(out)
    return b.build()


def masked_softmax(batch: int, rows: int, cols: int, scale: float = 1.0 / math.sqrt(128.0), dtype: str = "float16",
                   with_mask: bool = True) -> dict:
    """scores[batch, rows, cols] * scale + mask[rows, cols] -> softmax over the last axis, same dtype out."""
    b = _Builder(f"Fused_Cast_Mul_Add_Softmax_Cast_{batch}x{rows}x{cols}_3")
    f = "float32"
    full = [batch, rows, cols]
    red = [batch, rows, 1]
    x = b.input("scores", full, dtype)
    s = x
    if dtype != f:
        s = b.emit("Cast", [s], full, f, [_attr("dst_type", "str", f)])
    s = b.emit("Mul", [s, b.const(scale, f)], full, f)
    if with_mask:
        m = b.input("mask", [rows, cols], dtype)
        mf = m
        if dtype != f:
            mf = b.emit("Cast", [m], [rows, cols], f, [_attr("dst_type", "str", f)])
        s = b.emit("Add", [s, mf], full, f)
    mx = b.emit("ReduceMax", [s], red, f, _reduce_attr([2], True))
    sh = b.emit("Sub", [s, mx], full, f)
    e = b.emit("Exp", [sh], full, f)
    sm = b.emit("ReduceSum", [e], red, f, _reduce_attr([2], True))
    out = b.emit("RealDiv", [e, sm], full, f)
    if dtype != f:
        out = b.emit("Cast", [out], full, dtype, [_attr("dst_type", "str", dtype)])
    b.output(out)
    return b.build()


def reduce_sum_axis0(rows: int, cols: int) -> dict:
    """x f32[rows, cols] -> sum over axis 0 -> f32[cols] (reduce-Y class)."""
    b = _Builder(f"Fused_ReduceSum_axis0_{rows}x{cols}_4")
    x = b.input("x", [rows, cols], "float32")
    b.output(b.emit("ReduceSum", [x], [cols], "float32", _reduce_attr([0], False), out_name="colsum"))
    return b.build()


def reduce_max_all(rows: int, cols: int) -> dict:
    """x f32[rows, cols] -> global max -> f32[1] (reduce-ALL class)."""
    b = _Builder(f"Fused_ReduceMax_all_{rows}x{cols}_5")
    x = b.input("x", [rows, cols], "float32")
    b.output(b.emit("ReduceMax", [x], [1], "float32", _reduce_attr([0, 1], False), out_name="gmax"))
    return b.build()


def reduce_sum_and_max(rows: int, cols: int) -> dict:
    """Both reductions of the same input in one fused region."""
    b = _Builder(f"Fused_ReduceSum_ReduceMax_{rows}x{cols}_6")
    x = b.input("x", [rows, cols], "float32")
    b.output(b.emit("ReduceSum", [x], [cols], "float32", _reduce_attr([0], False), out_name="colsum"))
    b.output(b.emit("ReduceMax", [x], [1], "float32", _reduce_attr([0, 1], False), out_name="gmax"))
    return b.build()


def matmul_bias_relu(m: int, k: int, n: int, transpose_b: bool = False, with_bias: bool = True,
                     relu: bool = True, dtype: str = "bfloat16") -> dict:
    """A[m,k] x B[k,n] -> f32 accumulate (+ bias[n]) (ReLU) -> [m,n] in the operand type (bfloat16, float16, float32)."""
    b = _Builder(f"Fused_MatMul_BiasAdd_ReLU_Cast_{m}x{k}x{n}_7")
    h, f = dtype, "float32"
    a = b.input("a", [m, k], h)
    bm = b.input("b", [n, k] if transpose_b else [k, n], h)
    attr = [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", bool(transpose_b))]
    c = b.emit("MatMul", [a, bm], [m, n], f, attr)
    if with_bias:
        bias = b.input("bias", [n], h)
        bf = bias if h == f else b.emit("Cast", [bias], [n], f, [_attr("dst_type", "str", f)])
        c = b.emit("Add", [c, bf], [m, n], f)
    if relu:
        c = b.emit("Maximum", [c, b.const(0.0, f)], [m, n], f)
    out = c if h == f else b.emit("Cast", [c], [m, n], h, [_attr("dst_type", "str", h)], out_name="out")
    b.output(out)
    return b.build()


def batch_matmul(batch: int, m: int, k: int, n: int, shared_b: bool = False, transpose_b: bool = False,
                 dtype: str = "bfloat16", out_dtype: str = "float32") -> dict:
    """a[batch,m,k] x b[batch,k,n] (or one shared b[k,n]; [.., n, k] with transpose_b) -> [batch,m,n]."""
    b = _Builder(f"Fused_BatchMatMul_{batch}x{m}x{k}x{n}_9")
    a = b.input("a", [batch, m, k], dtype)
    inner = [n, k] if transpose_b else [k, n]
    w = b.input("b", inner if shared_b else [batch] + inner, dtype)
    attr = [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", bool(transpose_b))]
    b.output(b.emit("BatchMatMul", [a, w], [batch, m, n], out_dtype, attr))
    return b.build()


def rmsnorm(rows: int, cols: int, dtype: str = "float32", eps: float = 1e-6) -> dict:
    """x[rows, cols] * rsqrt(mean(x^2) + eps) * g[cols]; float32 math, `dtype` in and out."""
    f = "float32"
    b = _Builder(f"Fused_RMSNorm_{rows}x{cols}_9")
    x = b.input("x", [rows, cols], dtype)
    g = b.input("g", [cols], f)
    xf = x if dtype == f else b.emit("Cast", [x], [rows, cols], f, [_attr("dst_type", "str", f)])
    ss = b.emit("ReduceSum", [b.emit("Mul", [xf, xf], [rows, cols], f)], [rows, 1], f, _reduce_attr([1], True))
    ms = b.emit("RealDiv", [ss, b.const(float(cols), f)], [rows, 1], f)
    r = b.emit("Rsqrt", [b.emit("Add", [ms, b.const(eps, f)], [rows, 1], f)], [rows, 1], f)
    y = b.emit("Mul", [b.emit("Mul", [xf, r], [rows, cols], f), g], [rows, cols], f)
    if dtype != f:
        y = b.emit("Cast", [y], [rows, cols], dtype, [_attr("dst_type", "str", dtype)])
    b.output(y)
    return b.build()


def softmax_rows_typed(rows: int, cols: int, dtype: str = "bfloat16") -> dict:
    """Softmax over the last axis with EVERY op in the tensor's own type (no widening casts): max, subtract, exp, sum,
    divide each round to `dtype` -- a region of the reduce-X class that runs as a generated row kernel."""
    b = _Builder(f"Fused_SoftmaxTyped_{dtype}_{rows}x{cols}_6")
    x = b.input("x", [rows, cols], dtype)
    m = b.emit("ReduceMax", [x], [rows, 1], dtype, _reduce_attr([1], True))
    e = b.emit("Exp", [b.emit("Sub", [x, m], [rows, cols], dtype)], [rows, cols], dtype)
    s_ = b.emit("ReduceSum", [e], [rows, 1], dtype, _reduce_attr([1], True))
    b.output(b.emit("RealDiv", [e, s_], [rows, cols], dtype))
    return b.build()


def mul_reduce_sum(rows: int, cols: int, axes: Sequence[int]) -> dict:
    """sum over `axes` of x * y, both float32[rows, cols] (the shape of bias / scale gradients)."""
    f = "float32"
    axes = list(axes)
    b = _Builder(f"Fused_Mul_ReduceSum_{rows}x{cols}_" + "".join(map(str, axes)) + "_10")
    x = b.input("x", [rows, cols], f)
    y = b.input("y", [rows, cols], f)
    out = [1] if len(axes) == 2 else ([cols] if axes == [0] else [rows])
    b.output(b.emit("ReduceSum", [b.emit("Mul", [x, y], [rows, cols], f)], out, f, _reduce_attr(axes, False)))
    return b.build()


def transpose(shape: Sequence[int], perm: Sequence[int], dtype: str = "float16") -> dict:
    shape, perm = list(shape), list(perm)
    b = _Builder("Fused_Transpose_" + "x".join(map(str, shape)) + "_8")
    x = b.input("x", shape, dtype)
    oshape = [shape[p] for p in perm]
    b.output(b.emit("Transpose", [x], oshape, dtype, [_attr("perm", "listInt", perm)], out_name="xt"))
    return b.build()


def scale_copy(shape: Sequence[int], dtype: str = "float32") -> dict:
    """`Mul(x, 1)`: the smallest elementwise region -- every element read once and written once (a copy)."""
    b = _Builder("Fused_Mul_" + "x".join(map(str, shape)) + "_3")
    x = b.input("x", list(shape), dtype)
    b.output(b.emit("Mul", [x, b.const(1.0, dtype)], list(shape), dtype))
    return b.build()


def unary(op: str, shape: Sequence[int], dtype: str) -> dict:
    """A single unary operator over one tensor."""
    shape = list(shape)
    b = _Builder(f"Fused_{op}_" + "x".join(map(str, shape)) + "_9")
    x = b.input("x", shape, dtype)
    b.output(b.emit(op, [x], shape, dtype, out_name="out"))
    return b.build()


def batch_norm_training(shape: Sequence[int], io: str = "float32", seed: int = 0) -> dict:
    """Mean over (N, H, W), variance of the centred values, scale and shift; the centred values are used twice."""
    f = "float32"
    n_, c_, h_, w_ = shape
    stat = [1, c_, 1, 1]
    b = _Builder(f"Fused_BatchNormTraining_{seed}")
    x0, gamma, beta = b.input("x", shape, io), b.input("gamma", stat, f), b.input("beta", stat, f)
    x = x0 if io == f else b.emit("Cast", [x0], shape, f, [_attr("dst_type", "str", f)])
    inv = b.const(1.0 / (n_ * h_ * w_), f)
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], stat, f, _reduce_attr([0, 2, 3], True)), inv], stat, f)
    d_ = b.emit("Sub", [x, mean], shape, f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [d_, d_], shape, f)], stat, f, _reduce_attr([0, 2, 3], True)), inv], stat, f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(1e-5, f)], stat, f)], stat, f)
    y = b.emit("Add", [b.emit("Mul", [b.emit("Mul", [d_, rstd], shape, f), gamma], shape, f), beta], shape, f)
    b.output(y if io == f else b.emit("Cast", [y], shape, io, [_attr("dst_type", "str", io)]))
    b.output(mean)
    b.output(rstd)
    return b.build()


def batch_norm_backward(shape: Sequence[int], seed: int = 0) -> dict:
    """dbeta = sum dy, dgamma = sum dy * xhat over (N, H, W), dx = gamma * rstd * (dy - dbeta / m - xhat * dgamma / m)."""
    f = "float32"
    n_, c_, h_, w_ = shape
    stat = [1, c_, 1, 1]
    m_ = n_ * h_ * w_
    b = _Builder(f"Fused_BatchNormGrad_{seed}")
    dy, x = b.input("dy", shape, f), b.input("x", shape, f)
    mean, rstd, gamma = b.input("mean", stat, f), b.input("rstd", stat, f), b.input("gamma", stat, f)
    xhat = b.emit("Mul", [b.emit("Sub", [x, mean], shape, f), rstd], shape, f)
    dbeta = b.emit("ReduceSum", [dy], stat, f, _reduce_attr([0, 2, 3], True))
    dgamma = b.emit("ReduceSum", [b.emit("Mul", [dy, xhat], shape, f)], stat, f, _reduce_attr([0, 2, 3], True))
    inv = b.const(1.0 / m_, f)
    t = b.emit("Sub", [dy, b.emit("Mul", [dbeta, inv], stat, f)], shape, f)
    t = b.emit("Sub", [t, b.emit("Mul", [xhat, b.emit("Mul", [dgamma, inv], stat, f)], shape, f)], shape, f)
    b.output(b.emit("Mul", [t, b.emit("Mul", [gamma, rstd], stat, f)], shape, f))
    b.output(dgamma)
    b.output(dbeta)
    return b.build()


def normalise_over_axis0(rows: int, cols: int, eps: float = 1e-5) -> dict:
    """(x - mean) * rsqrt(var + eps) with the statistics over axis 0 (per column): the reductions fold the leading axis
    and feed the ops behind them."""
    f = "float32"
    b = _Builder(f"Fused_NormaliseAxis0_{rows}x{cols}_4")
    x = b.input("x", [rows, cols], f)
    stat = [1, cols]
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], stat, f, _reduce_attr([0], True)), b.const(1.0 / rows, f)], stat, f)
    d = b.emit("Sub", [x, mean], [rows, cols], f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [d, d], [rows, cols], f)], stat, f, _reduce_attr([0], True)),
                         b.const(1.0 / rows, f)], stat, f)
    r = b.emit("Rsqrt", [b.emit("Add", [var, b.const(eps, f)], stat, f)], stat, f)
    b.output(b.emit("Mul", [d, r], [rows, cols], f))
    return b.build()


def softmax_over_axis0(rows: int, cols: int) -> dict:
    """exp(x - max) / sum exp(x - max) with the maximum and the sum over axis 0 (per column)."""
    f = "float32"
    b = _Builder(f"Fused_SoftmaxAxis0_{rows}x{cols}_5")
    x = b.input("x", [rows, cols], f)
    stat = [1, cols]
    m = b.emit("ReduceMax", [x], stat, f, _reduce_attr([0], True))
    e = b.emit("Exp", [b.emit("Sub", [x, m], [rows, cols], f)], [rows, cols], f)
    b.output(b.emit("RealDiv", [e, b.emit("ReduceSum", [e], stat, f, _reduce_attr([0], True))], [rows, cols], f))
    return b.build()


def scale_by_global_max(rows: int, cols: int) -> dict:
    """x / max|x| over the whole tensor, and the maximum itself."""
    f = "float32"
    b = _Builder(f"Fused_ScaleByGlobalMax_{rows}x{cols}_6")
    x = b.input("x", [rows, cols], f)
    m = b.emit("ReduceMax", [b.emit("Abs", [x], [rows, cols], f)], [1], f, _reduce_attr([0, 1], False))
    b.output(b.emit("RealDiv", [x, m], [rows, cols], f))
    b.output(m)
    return b.build()


def layer_norm_backward(rows: int, cols: int, eps: float = 1e-5, grads_dtype: str = "float32") -> dict:
    """Statistics recomputed from x, then dx (row-wise) with dgamma = sum over rows of dy * xhat and dbeta = sum of dy
    (cast to `grads_dtype`, the parameters' type, when that is not float32)."""
    f = "float32"
    full, red = [rows, cols], [rows, 1]
    b = _Builder(f"Fused_LayerNormGrad_{rows}x{cols}")
    dy, x, gamma = b.input("dy", full, f), b.input("x", full, f), b.input("gamma", [cols], f)
    inv = b.const(1.0 / cols, f)
    mean = b.emit("Mul", [b.emit("ReduceSum", [x], red, f, _reduce_attr([1], True)), inv], red, f)
    d = b.emit("Sub", [x, mean], full, f)
    var = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [d, d], full, f)], red, f, _reduce_attr([1], True)), inv], red, f)
    rstd = b.emit("Rsqrt", [b.emit("Add", [var, b.const(eps, f)], red, f)], red, f)
    xhat = b.emit("Mul", [d, rstd], full, f)
    g_ = b.emit("Mul", [dy, gamma], full, f)
    m1 = b.emit("Mul", [b.emit("ReduceSum", [g_], red, f, _reduce_attr([1], True)), inv], red, f)
    m2 = b.emit("Mul", [b.emit("ReduceSum", [b.emit("Mul", [g_, xhat], full, f)], red, f, _reduce_attr([1], True)), inv], red, f)
    t = b.emit("Sub", [b.emit("Sub", [g_, m1], full, f), b.emit("Mul", [xhat, m2], full, f)], full, f)
    b.output(b.emit("Mul", [t, rstd], full, f))
    dgamma = b.emit("ReduceSum", [b.emit("Mul", [dy, xhat], full, f)], [cols], f, _reduce_attr([0], False))
    dbeta = b.emit("ReduceSum", [dy], [cols], f, _reduce_attr([0], False))
    for grad in (dgamma, dbeta):
        b.output(grad if grads_dtype == f else b.emit("Cast", [grad], [cols], grads_dtype, [_attr("dst_type", "str", grads_dtype)]))
    return b.build()
