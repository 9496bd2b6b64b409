"""Front door for PyTorch programs: clusters fusable aten ops and runs each cluster as one fused-operator description.

The reference reaches its kernel generator from PyTorch through an MLIR pipeline: torch dialect -> decomposition to
meta ops -> clustering of the ops the generator can take (``mfusion/lib/Dialect/Mfuse/Transforms/Cluster/AKGCluster.cc:30-118``:
static shapes only, no empty tensors, no complex types) -> outlining of every cluster -> one ``akg_call`` custom call
per cluster that carries the serialised subgraph (``mfusion/include/mfusion/Dialect/Mfuse/IR/MfuseOps.td:26-51``,
``mfusion/python/mfusion/torch/inductor.py:86-211``).  This module does the same steps on a ``torch.fx`` graph of aten
ops and hands every cluster to the library as the JSON description it compiles:

    trace (make_fx + decompositions)  ->  cluster  ->  one description per cluster  ->  graph with akg_call nodes

Differences from the reference's cluster list, both deliberate: reductions, matmuls, casts and shape ops are
clusterable too (the kernel library takes them), and a cluster must contain at least one op that computes something.

torch is used for tracing, device memory and streams.  All arithmetic of a cluster runs in the CUDA library; there
is no eager fallback for a cluster once it has been formed (a description the library refuses raises).
"""
from __future__ import annotations

import json
import math
import operator
from typing import Callable, Sequence

import torch
from torch import fx

from .descs import _attr, _Builder, _reduce_attr

aten = torch.ops.aten

_DTYPE_NAMES = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
                torch.int32: "int32", torch.int8: "int8", torch.int16: "int16", torch.bool: "bool"}
_FLOATS = (torch.float32, torch.float16, torch.bfloat16)


# --------------------------------------------------------------------------------------------------------------------
# aten op -> description ops.  Every lowering receives a _Lower context, the fx node and the already lowered operands
# (a tensor entry of the description, or a Python scalar) and returns the tensor entry of the result.
# --------------------------------------------------------------------------------------------------------------------
class _Lower:
    def __init__(self, name: str):
        self.b = _Builder(name)

    @staticmethod
    def shape(node) -> list[int]:
        return [int(s) for s in node.meta["val"].shape] or [1]

    @staticmethod
    def dtype(node) -> str:
        return _DTYPE_NAMES[node.meta["val"].dtype]

    def emit(self, name, ins, node, attr=None, shape=None, dtype=None):
        return self.b.emit(name, ins, shape if shape is not None else self.shape(node),
                           dtype or self.dtype(node), attr)

    def as_tensor(self, v, dtype: str):
        """Operand of a description op: tensors pass, scalars become typed constants."""
        if isinstance(v, dict):
            return v
        return self.b.const(float(v) if not isinstance(v, bool) else (1.0 if v else 0.0), dtype)

    def cast_to(self, t, dtype: str):
        if not isinstance(t, dict) or t["data_type"] == dtype:
            return t
        return self.b.emit("Cast", [t], t["shape"], dtype, [_attr("dst_type", "str", dtype)])


def _compute_dtype(node, operands) -> str:
    """The type torch computes a binary op in: the promoted type of its operands."""
    vals = []
    for a in node.args[:2]:
        if isinstance(a, fx.Node):
            vals.append(a.meta["val"])
        else:
            vals.append(a)
    return _DTYPE_NAMES[torch.result_type(*vals)]


def _unary(name):
    def lower(L: _Lower, node, x):
        return L.emit(name, [x], node)
    return lower


def _binary(name, alpha_arg=False):
    def lower(L: _Lower, node, a, b, **kw):
        dt = L.dtype(node)
        alpha = kw.get("alpha", 1)
        a, b = L.cast_to(a, dt), L.cast_to(b, dt)
        if alpha_arg and alpha != 1:
            b = (L.b.emit("Mul", [b, L.b.const(float(alpha), dt)], b["shape"], dt) if isinstance(b, dict)
                 else b * alpha)
        return L.emit(name, [L.as_tensor(a, dt), L.as_tensor(b, dt)], node)
    return lower


def _compare(name):
    def lower(L: _Lower, node, a, b):
        dt = _compute_dtype(node, (a, b))
        a, b = L.cast_to(a, dt), L.cast_to(b, dt)
        return L.emit(name, [L.as_tensor(a, dt), L.as_tensor(b, dt)], node)
    return lower


def _relu(L, node, x):
    return L.emit("Maximum", [x, L.b.const(0.0, L.dtype(node))], node)


def _sigmoid(L, node, x):
    dt = L.dtype(node)
    e = L.emit("Exp", [L.emit("Neg", [x], node)], node)
    return L.emit("Reciprocal", [L.emit("Add", [e, L.b.const(1.0, dt)], node)], node)


def _rsub(L, node, a, b, alpha=1):  # b - alpha * a
    dt = L.dtype(node)
    a = L.cast_to(a, dt)
    if alpha != 1:
        a = L.b.emit("Mul", [a, L.b.const(float(alpha), dt)], a["shape"], dt)
    return L.emit("Sub", [L.as_tensor(b, dt), L.as_tensor(a, dt)], node)


def _div(L, node, a, b, rounding_mode=None):
    return _binary("RealDiv")(L, node, a, b)


def _where(L, node, c, a, b):
    dt = L.dtype(node)
    return L.emit("Select", [c, L.as_tensor(L.cast_to(a, dt), dt), L.as_tensor(L.cast_to(b, dt), dt)], node)


def _to_copy(L, node, x, **kw):
    dt = L.dtype(node)
    if x["data_type"] == dt:
        return L.emit("Reshape", [x], node, [_attr("shape", "listInt", L.shape(node))])
    return L.emit("Cast", [x], node, [_attr("dst_type", "str", dt)])


def _reshape(L, node, x, *_, **__):
    return L.emit("Reshape", [x], node, [_attr("shape", "listInt", L.shape(node))])


def _expand(L, node, x, *_):
    shape = L.shape(node)
    if list(x["shape"]) == shape:
        return _reshape(L, node, x)
    # BroadcastTo keeps the rank of its operand's trailing dims; add leading 1s first when the rank grows
    if len(x["shape"]) < len(shape):
        lead = [1] * (len(shape) - len(x["shape"])) + list(x["shape"])
        x = L.b.emit("Reshape", [x], lead, x["data_type"], [_attr("shape", "listInt", lead)])
    return L.emit("BroadcastTo", [x], node, [_attr("shape", "listInt", shape)])


def _permute(L, node, x, perm):
    r = len(x["shape"])
    return L.emit("Transpose", [x], node, [_attr("perm", "listInt", [int(p) % r for p in perm])])


def _transpose_int(L, node, x, d0, d1):
    r = len(x["shape"])
    perm = list(range(r))
    perm[d0 % r], perm[d1 % r] = perm[d1 % r], perm[d0 % r]
    return _permute(L, node, x, perm)


def _t(L, node, x):
    return _permute(L, node, x, [1, 0]) if len(x["shape"]) == 2 else _reshape(L, node, x)


def _axes(x, dims):
    r = len(x["shape"])
    if dims is None or (isinstance(dims, (list, tuple)) and len(dims) == 0):
        return list(range(r))
    dims = [dims] if isinstance(dims, int) else list(dims)
    return sorted({int(d) % r for d in dims})


def _reduce(name):
    def lower(L: _Lower, node, x, dims=None, keepdim=False, **kw):
        dt = L.dtype(node)
        x = L.cast_to(x, dt)  # sum(dtype=...) converts first
        return L.emit(name, [x], node, _reduce_attr(_axes(x, dims), bool(keepdim)))
    return lower


def _mean(L, node, x, dims=None, keepdim=False, **kw):
    dt = L.dtype(node)
    x = L.cast_to(x, dt)
    axes = _axes(x, dims)
    count = math.prod(x["shape"][a] for a in axes)
    s = L.emit("ReduceSum", [x], node, _reduce_attr(axes, bool(keepdim)))
    return L.emit("RealDiv", [s, L.b.const(float(count), dt)], node)


def _untransposed(L: _Lower, b):
    """If `b` is the transpose of its last two dims inside this cluster, the tensor it was transposed from (the MatMul
    then reads it with transpose_b instead of materialising the transpose)."""
    for op in L.b.ops:
        if op["output_desc"][0]["tensor_name"] != b["tensor_name"] or op["name"] != "Transpose":
            continue
        perm = next(a["value"] for a in op["attr"] if a["name"] == "perm")
        r = len(perm)
        if r >= 2 and perm == list(range(r - 2)) + [r - 1, r - 2]:
            return op["input_desc"][0][0]
    return None


def _matmul(L, node, a, b, name, shape=None, dtype=None):
    src = _untransposed(L, b)
    attr = [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", src is not None)]
    return L.emit(name, [a, src if src is not None else b], node, attr, shape=shape, dtype=dtype)


def _mm(L, node, a, b):
    return _matmul(L, node, a, b, "MatMul")


def _bmm(L, node, a, b):
    return _matmul(L, node, a, b, "BatchMatMul")


def _addmm(L, node, bias, a, b, beta=1, alpha=1):
    dt = L.dtype(node)
    if dt == "float32":
        return L.emit("Add", [_mm(L, node, a, b), bias], node)
    # half types: accumulate and add the bias in float32, round once (what the library GEMM epilogues do)
    f = "float32"
    c = _matmul(L, node, a, b, "MatMul", dtype=f)
    c = L.emit("Add", [c, L.cast_to(bias, f)], node, dtype=f)
    return L.emit("Cast", [c], node, [_attr("dst_type", "str", dt)])


def _cat(L, node, tensors, dim=0):
    r = len(tensors[0]["shape"])
    L.b._n += 1
    out = {"tensor_name": f"t{L.b._n}_concat", "shape": L.shape(node), "data_type": L.dtype(node),
           "format": "DefaultFormat"}
    L.b.ops.append({"name": "Concat", "attr": [_attr("axis", "int", int(dim) % r)], "impl_path": "",
                    "input_desc": [[dict(t) for t in tensors]], "output_desc": [dict(out)]})
    return out


def _slice(L, node, x, dim=0, start=None, end=None, step=1):
    shape = list(x["shape"])
    r = len(shape)
    dim = int(dim) % r
    n = shape[dim]
    start = 0 if start is None else int(start)
    end = n if end is None else int(end)
    start = max(0, min(n, start + n if start < 0 else start))
    end = max(0, min(n, end + n if end < 0 else end))
    begin, stop, strides = [0] * r, list(shape), [1] * r
    begin[dim], stop[dim], strides[dim] = start, end, int(step)
    return L.emit("StridedSlice", [x], node, [_attr("begin", "listInt", begin), _attr("end", "listInt", stop),
                                              _attr("strides", "listInt", strides)])


def _pow_scalar(L, node, x, e):
    """Small whole exponents as products, like torch's own kernels (x * x is also the correctly rounded square)."""
    dt = L.dtype(node)
    x = L.cast_to(x, dt)
    if float(e) == 2.0:
        return L.emit("Mul", [x, x], node)
    if float(e) == 3.0:
        return L.emit("Mul", [L.emit("Mul", [x, x], node), x], node)
    if float(e) == 1.0:
        return L.emit("Mul", [x, L.b.const(1.0, dt)], node)
    return L.emit("Pow", [x, L.b.const(float(e), dt)], node)


_LOWERINGS: dict = {}


def _register():
    def put(ops, fn, compute=True):
        for op in ops if isinstance(ops, (list, tuple)) else [ops]:
            _LOWERINGS[op] = (fn, compute)
    for a, n in [(aten.abs.default, "Abs"), (aten.neg.default, "Neg"), (aten.exp.default, "Exp"),
                 (aten.log.default, "Log"), (aten.tanh.default, "Tanh"), (aten.sqrt.default, "Sqrt"),
                 (aten.rsqrt.default, "Rsqrt"), (aten.reciprocal.default, "Reciprocal"), (aten.floor.default, "Floor"),
                 (aten.sin.default, "Sin"), (aten.cos.default, "Cos"), (aten.asinh.default, "Asinh"),
                 (aten.acosh.default, "Acosh"), (aten.atan.default, "Atan"), (aten.asin.default, "ASin"),
                 (aten.acos.default, "ACos"), (aten.isinf.default, "IsInf"), (aten.isnan.default, "IsNan"),
                 (aten.isfinite.default, "IsFinite"), (aten.logical_not.default, "LogicalNot")]:
        put(a, _unary(n))
    put(aten.relu.default, _relu)
    put(aten.sigmoid.default, _sigmoid)
    put([aten.add.Tensor, aten.add.Scalar], _binary("Add", alpha_arg=True))
    put([aten.sub.Tensor, aten.sub.Scalar], _binary("Sub", alpha_arg=True))
    put([aten.rsub.Scalar, aten.rsub.Tensor], _rsub)
    put([aten.mul.Tensor, aten.mul.Scalar], _binary("Mul"))
    put([aten.div.Tensor, aten.div.Scalar], _div)
    put(aten.maximum.default, _binary("Maximum"))
    put(aten.minimum.default, _binary("Minimum"))
    put(aten.pow.Tensor_Scalar, _pow_scalar)
    put(aten.pow.Tensor_Tensor, _binary("Pow"))
    put(aten.atan2.default, _binary("Atan2"))
    for base, n in [("eq", "Equal"), ("ne", "NotEqual"), ("gt", "Greater"), ("ge", "GreaterEqual"), ("lt", "Less"),
                    ("le", "LessEqual")]:
        put([getattr(aten, base).Tensor, getattr(aten, base).Scalar], _compare(n))
    put(aten.logical_and.default, _binary("LogicalAnd"))
    put(aten.logical_or.default, _binary("LogicalOr"))
    put(aten.where.self, _where)
    put(aten._to_copy.default, _to_copy)
    put([aten.view.default, aten._unsafe_view.default, aten.reshape.default, aten.unsqueeze.default,
         aten.squeeze.dim, aten.squeeze.dims, aten.squeeze.default, aten.clone.default, aten.alias.default,
         aten.detach.default], _reshape, compute=False)
    put(aten.expand.default, _expand, compute=False)
    put(aten.permute.default, _permute)
    put(aten.transpose.int, _transpose_int)
    put(aten.t.default, _t)
    put(aten.sum.dim_IntList, _reduce("ReduceSum"))
    put(aten.sum.default, _reduce("ReduceSum"))
    put(aten.amax.default, _reduce("ReduceMax"))
    put(aten.amin.default, _reduce("ReduceMin"))
    put(aten.mean.dim, _mean)
    put(aten.mm.default, _mm)
    put(aten.bmm.default, _bmm)
    put(aten.addmm.default, _addmm)
    put(aten.cat.default, _cat)
    put(aten.slice.Tensor, _slice)


_register()


def _native_layer_norm(x, normalized_shape, weight, bias, eps):
    """LayerNorm as the op chain the fused row kernel recognises: mean, centred values, their mean square, rsqrt."""
    dims = list(range(x.dim() - len(normalized_shape), x.dim()))
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    mean = xf.mean(dims, keepdim=True)
    d = xf - mean
    var = (d * d).mean(dims, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = d * rstd
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y.to(x.dtype), mean, rstd


def _split(x, size, dim=0):
    n = x.shape[dim]
    return tuple(x.narrow(dim, s, min(size, n - s)) for s in range(0, n, size))


def _split_with_sizes(x, sizes, dim=0):
    out, s = [], 0
    for z in sizes:
        out.append(x.narrow(dim, s, z))
        s += z
    return tuple(out)


_MATMULS = (aten.mm.default, aten.bmm.default, aten.addmm.default)
_REDUCTIONS = (aten.sum.dim_IntList, aten.sum.default, aten.amax.default, aten.amin.default, aten.mean.dim)


def _dims_of(x, dim):
    if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0):
        return list(range(x.dim()))
    return [dim] if isinstance(dim, int) else list(dim)


def _var_correction(x, dim=None, *, correction=None, keepdim=False):
    dims = _dims_of(x, dim)
    n = math.prod(x.shape[d] for d in dims)
    c = 1 if correction is None else correction
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    d = xf - xf.mean(dims, keepdim=True)
    return ((d * d).sum(dims, keepdim=keepdim) / max(n - c, 0)).to(x.dtype)


def _std_correction(x, dim=None, *, correction=None, keepdim=False):
    return torch.sqrt(_var_correction(x, dim, correction=correction, keepdim=keepdim))


def _logsumexp(x, dim, keepdim=False):
    dims = _dims_of(x, dim)
    m = x.amax(dims, keepdim=True)
    out = torch.log(torch.exp(x - m).sum(dims, keepdim=True)) + m
    return out if keepdim else out.squeeze(dims)


def _vector_norm(x, ord=2, dim=None, keepdim=False, *, dtype=None):
    if ord != 2 or dtype is not None:
        return NotImplemented
    return torch.sqrt((x * x).sum(_dims_of(x, dim), keepdim=keepdim))


def _var_mean_correction(x, dim=None, *, correction=None, keepdim=False):
    dims = _dims_of(x, dim)
    return _var_correction(x, dim, correction=correction, keepdim=keepdim), x.mean(dims, keepdim=keepdim)


def _rms_norm(x, normalized_shape, weight=None, eps=None):
    dims = list(range(x.dim() - len(normalized_shape), x.dim()))
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    eps = torch.finfo(x.dtype).eps if eps is None else eps
    y = xf * torch.rsqrt((xf * xf).mean(dims, keepdim=True) + eps)
    if weight is not None:
        y = y * weight
    return y.to(x.dtype)


def _fused_rms_norm(x, normalized_shape, weight=None, eps=None):
    """The (result, reciprocal rms) pair rms_norm traces to on device tensors."""
    dims = list(range(x.dim() - len(normalized_shape), x.dim()))
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    eps = torch.finfo(x.dtype).eps if eps is None else eps
    rstd = torch.rsqrt((xf * xf).mean(dims, keepdim=True) + eps)
    y = xf * rstd
    if weight is not None:
        y = y * weight
    return y.to(x.dtype), rstd


def _native_group_norm(x, weight, bias, n, c, hxw, group, eps):
    """Statistics per (sample, group) on the [n, group, rest] view, then the per-channel scale and shift."""
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    g = xf.reshape(n, group, (c // group) * hxw)
    mean = g.mean(-1, keepdim=True)
    d = g - mean
    rstd = torch.rsqrt((d * d).mean(-1, keepdim=True) + eps)
    # scale and shift on x's own shape: what follows the normalisation (an activation) is then one elementwise group
    per_channel = [1, c] + [1] * (x.dim() - 2)
    y = (d * rstd).reshape(x.shape)
    if weight is not None:
        y = y * weight.reshape(per_channel)
    if bias is not None:
        y = y + bias.reshape(per_channel)
    return y.to(x.dtype), mean.reshape(n, group).to(x.dtype), rstd.reshape(n, group).to(x.dtype)


def _decompositions():
    from torch._decomp import get_decompositions
    table = _stock_decompositions()
    table[aten.native_group_norm.default] = _native_group_norm
    table[aten.var_mean.correction] = _var_mean_correction
    if hasattr(aten, "rms_norm"):
        table[aten.rms_norm.default] = _rms_norm
    if hasattr(aten, "_fused_rms_norm"):
        table[aten._fused_rms_norm.default] = _fused_rms_norm
    table[aten.var.correction] = _var_correction
    table[aten.std.correction] = _std_correction
    table[aten.logsumexp.default] = _logsumexp
    table[aten.linalg_vector_norm.default] = _vector_norm
    table[aten.native_layer_norm.default] = _native_layer_norm
    table[aten.split.Tensor] = _split                       # pieces become slices the library takes
    table[aten.split_with_sizes.default] = _split_with_sizes
    return table


def _stock_decompositions():
    from torch._decomp import get_decompositions
    return get_decompositions([
        aten.gelu, aten.native_layer_norm, aten.layer_norm, aten._softmax, aten._log_softmax, aten.var_mean,
        aten.var, aten.std, aten.silu, aten.addcmul, aten.addcdiv, aten.hardtanh, aten.leaky_relu, aten.elu,
        aten.softplus, aten.square, aten.rsub, aten.mse_loss, aten.masked_fill, aten.native_dropout,
        aten.clamp, aten.clamp_min, aten.clamp_max, aten.sigmoid_backward, aten.tanh_backward,
        aten.threshold_backward, aten.gelu_backward, aten.linear, aten.matmul, aten.expand_as, aten.ones_like,
        aten.zeros_like, aten.full_like, aten.log_sigmoid_forward, aten.hardswish, aten.hardsigmoid,
        aten.native_batch_norm, aten._native_batch_norm_legit, aten._native_batch_norm_legit_no_training,
        aten._native_batch_norm_legit_functional, aten.native_group_norm, aten.repeat,
        # what batch_norm / instance_norm dispatch to when traced on device tensors
        aten.cudnn_batch_norm, aten.miopen_batch_norm, aten._batch_norm_with_update, aten._batch_norm_no_update,
        aten._batch_norm_with_update_functional,
        # backward passes of the normalisations and softmaxes
        aten.native_batch_norm_backward, aten.cudnn_batch_norm_backward, aten.batch_norm_backward,
        aten.native_layer_norm_backward, aten.native_group_norm_backward, aten._softmax_backward_data,
        aten._log_softmax_backward_data,
    ])


# --------------------------------------------------------------------------------------------------------------------
# clustering
# --------------------------------------------------------------------------------------------------------------------
def _tensor_ok(val) -> bool:
    if not isinstance(val, torch.Tensor):
        return False
    if val.dtype not in _DTYPE_NAMES:
        return False
    for s in val.shape:
        if not isinstance(s, int) or s == 0:  # static, non-empty extents only (AKGCluster.cc:78-110)
            return False
    return True


def _float_to_int_cast(node) -> bool:
    if node.target is not aten._to_copy.default:
        return False
    src, dst = node.args[0].meta["val"].dtype, node.meta["val"].dtype
    return src in _FLOATS and dst not in _FLOATS and dst != torch.bool


def is_clusterable(node: fx.Node) -> bool:
    """The op has a lowering, every tensor it touches is static, non-empty and of a supported type."""
    if node.op != "call_function" or node.target not in _LOWERINGS:
        return False
    if not _tensor_ok(node.meta.get("val")):
        return False
    for a in node.all_input_nodes:
        if not _tensor_ok(a.meta.get("val")):
            return False
    if _float_to_int_cast(node):
        return False
    if node.target is aten._to_copy.default and any(k in node.kwargs and node.kwargs[k] is not None
                                                    for k in ("device", "layout", "memory_format")):
        return False
    if node.target in (aten.div.Tensor, aten.div.Scalar) and node.meta["val"].dtype not in _FLOATS:
        return False
    if node.target in (aten.mm.default, aten.bmm.default, aten.addmm.default) and \
            node.meta["val"].dtype not in _FLOATS:
        return False
    if node.target is aten.addmm.default and (node.kwargs.get("beta", 1) != 1 or node.kwargs.get("alpha", 1) != 1):
        return False
    return True


def cluster_nodes(graph: fx.Graph) -> list[list[fx.Node]]:
    """Groups clusterable nodes into maximal convex clusters (merging along producer->consumer edges whenever the
    merged cluster would not have a path that leaves it and comes back)."""
    nodes = list(graph.nodes)
    cid = {n: i for i, n in enumerate(nodes)}          # cluster id of every node (singletons at first)
    members = {i: [n] for i, n in enumerate(nodes)}
    ok = {n: is_clusterable(n) for n in nodes}

    def successors(c):
        out = set()
        for n in members[c]:
            for u in n.users:
                if cid[u] != c:
                    out.add(cid[u])
        return out

    def reaches_around(a, b):
        """Is there a path a -> x -> ... -> b with x outside {a, b}?"""
        stack = [s for s in successors(a) if s != b]
        seen = set(stack)
        while stack:
            c = stack.pop()
            for s in successors(c):
                if s == b:
                    return True
                if s not in seen:
                    seen.add(s)
                    stack.append(s)
        return False

    # The counterpart of the reference's split stage (inductor.py "Mfuse Split"): a cluster holds at most one matmul
    # (its bias / activation / cast run in the matmul's launch) and no reduction beside a matmul, so that LayerNorm-,
    # softmax- and GELU-like parts stay regions of their own, each of which the library runs as one kernel.
    def kind_counts(c):
        mm = sum(1 for m in members[c] if m.target in _MATMULS)
        red = sum(1 for m in members[c] if m.target in _REDUCTIONS)
        return mm, red

    for n in nodes:
        if not ok[n]:
            continue
        for p in n.all_input_nodes:
            if not ok[p] or cid[p] == cid[n]:
                continue
            a, b = cid[p], cid[n]
            (mm_a, red_a), (mm_b, red_b) = kind_counts(a), kind_counts(b)
            if mm_a + mm_b > 1 or (mm_a + mm_b >= 1 and red_a + red_b >= 1):
                continue
            if reaches_around(a, b):
                continue
            for m in members[b]:
                cid[m] = a
            members[a].extend(members.pop(b))
    order = {n: i for i, n in enumerate(nodes)}
    clusters = []
    for c, ms in members.items():
        if not ok[ms[0]]:
            continue
        if not any(_LOWERINGS[m.target][1] for m in ms):
            continue  # views only: nothing to compute
        clusters.append(sorted(ms, key=order.__getitem__))
    return clusters


# --------------------------------------------------------------------------------------------------------------------
# cluster -> description
# --------------------------------------------------------------------------------------------------------------------
class FusedSubgraph:
    """One cluster: its description, the fx nodes that feed it and the fx nodes it produces."""

    def __init__(self, name: str, desc: dict, inputs: list[fx.Node], outputs: list[fx.Node]):
        self.name, self.desc, self.inputs, self.outputs = name, desc, inputs, outputs
        self.out_meta = [(tuple(int(s) for s in o.meta["val"].shape), o.meta["val"].dtype) for o in outputs]
        self.desc_json = json.dumps(desc)


def lower_cluster(cluster: Sequence[fx.Node], index: int) -> FusedSubgraph:
    inside = set(cluster)
    names = "_".join(dict.fromkeys(str(n.target).split(".")[1].capitalize() for n in cluster
                                   if _LOWERINGS[n.target][1]))
    L = _Lower(f"Fused_{names[:80]}_{index}")
    env: dict[fx.Node, dict] = {}
    inputs: list[fx.Node] = []

    def operand(a):
        if isinstance(a, fx.Node):
            if a not in env:
                env[a] = L.b.input(f"in{len(inputs)}_{a.name}", _Lower.shape(a), _Lower.dtype(a))
                inputs.append(a)
            return env[a]
        if isinstance(a, (list, tuple)) and a and isinstance(a[0], fx.Node):
            return [operand(x) for x in a]
        return a

    for n in cluster:
        fn, _ = _LOWERINGS[n.target]
        env[n] = fn(L, n, *[operand(a) for a in n.args], **{k: operand(v) for k, v in n.kwargs.items()})
    outputs = [n for n in cluster if any(u not in inside for u in n.users)]
    seen = set()
    for n in outputs:
        t = env[n]
        if t["tensor_name"] in seen or t["tensor_name"] in {env[i]["tensor_name"] for i in inputs}:
            # a result listed twice, or an input passed straight through: give it a node of its own
            t = L.b.emit("Reshape", [t], t["shape"], t["data_type"], [_attr("shape", "listInt", list(t["shape"]))])
        seen.add(t["tensor_name"])
        L.b.output(t)
    # drop ops nothing reads any more (a transpose folded into its MatMul) and the inputs only they read
    live = {o["tensor_name"] for o in L.b.outputs}
    kept = []
    for op in reversed(L.b.ops):
        if any(o["tensor_name"] in live for o in op["output_desc"]):
            kept.append(op)
            for group in op["input_desc"]:
                live.update(t["tensor_name"] for t in group)
    L.b.ops = kept[::-1]
    keep_in = [i for i, t in enumerate(L.b.inputs) if t["tensor_name"] in live]
    L.b.inputs = [L.b.inputs[i] for i in keep_in]
    inputs = [inputs[i] for i in keep_in]
    return FusedSubgraph(L.b.op, L.b.build(), inputs, outputs)


# --------------------------------------------------------------------------------------------------------------------
# execution of one cluster
# --------------------------------------------------------------------------------------------------------------------
class AkgExecutor:
    """Compiles a cluster's description with the CUDA library on first use and launches it on torch's current stream."""

    def __init__(self):
        self._kernels: dict[str, object] = {}

    def kernel(self, sub: FusedSubgraph, device: torch.device):
        from .driver import FusedKernel
        key = (sub.desc_json, device.index)  # the description itself: names repeat across programs
        k = self._kernels.get(key)
        if k is None:
            k = self._kernels[key] = FusedKernel(sub.desc_json, device=device.index if device.index is not None else -1)
        return k

    def __call__(self, sub: FusedSubgraph, *tensors: torch.Tensor):
        dev = tensors[0].device
        if dev.type != "cuda":
            raise RuntimeError("akg_call runs on CUDA tensors only; there is no host path")
        k = self.kernel(sub, dev)
        ins = [t.contiguous() for t in tensors]
        outs = [torch.empty(shape, dtype=dt, device=dev) for shape, dt in sub.out_meta]
        k.launch(ins + outs)
        return tuple(outs)


_default_executor = AkgExecutor()


def akg_call(sub: FusedSubgraph, *tensors: torch.Tensor, executor: Callable | None = None):
    """The custom call a fused cluster is replaced by (the counterpart of ``mfuse.akg_call``): runs the cluster's
    description on the given tensors and returns its results as a tuple."""
    return (executor or _default_executor)(sub, *tensors)


def _bound_call(sub: FusedSubgraph, executor, index: int):
    def call(*tensors):
        return akg_call(sub, *tensors, executor=executor)
    call.__name__ = call.__qualname__ = f"akg_call_{index}"
    return call


# --------------------------------------------------------------------------------------------------------------------
# whole-graph rewrite
# --------------------------------------------------------------------------------------------------------------------
class FusedModule(torch.nn.Module):
    """Result of `fuse_and_optimize`: call it like the original function."""

    def __init__(self, gm: fx.GraphModule, subgraphs: list[FusedSubgraph], n_clustered: int, n_total: int):
        super().__init__()
        self.gm = gm
        self.subgraphs = subgraphs
        self.clustered_ops = n_clustered
        self.total_ops = n_total

    def forward(self, *args):
        return self.gm(*args)

    def descriptions(self) -> list[dict]:
        return [s.desc for s in self.subgraphs]


def trace(fn: Callable, example_inputs: Sequence[torch.Tensor]) -> fx.GraphModule:
    """aten-level graph of `fn` with shapes and types recorded on every node (no kernels run: fake tensors)."""
    from torch.fx.experimental.proxy_tensor import make_fx
    # in-place ops (x.add_(1)) become their out-of-place forms first, so that they can sit inside a cluster
    gm = make_fx(torch.func.functionalize(fn), decomposition_table=_decompositions(),
                 tracing_mode="fake")(*example_inputs)
    _functionalize_leftovers(gm.graph)
    _merge_repeated_ops(gm.graph)
    gm.recompile()
    return gm


def _merge_repeated_ops(graph: fx.Graph) -> None:
    """Common subexpressions: decompositions often compute the same value twice (the mean of batch normalisation, once
    for the variance and once for the result); the later op is replaced by the earlier one.  Only ops with a lowering
    are merged: all of them are pure functions of their arguments."""
    def freeze(a):
        if isinstance(a, (list, tuple)):
            return tuple(freeze(v) for v in a)
        if isinstance(a, dict):
            return tuple(sorted((k, freeze(v)) for k, v in a.items()))
        if isinstance(a, fx.Node):
            return ("node", id(a))
        return (type(a).__name__, a) if a.__hash__ is not None else ("obj", id(a))

    seen = {}
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target not in _LOWERINGS:
            continue
        if any(isinstance(u, fx.Node) and u.op == "call_function" and u.target in _INPLACE for u in node.users):
            continue  # mutated later by an op that stayed in place
        key = (node.target, freeze(node.args), freeze(node.kwargs))
        first = seen.setdefault(key, node)
        if first is not node:
            node.replace_all_uses_with(first)
            graph.erase_node(node)


_INPLACE = {}


def _functionalize_leftovers(graph: fx.Graph) -> None:
    """Decompositions run after functionalization and may leave in-place ops on their own temporaries
    (``t.add_(eps)``): each becomes its out-of-place form, and later readers of the temporary read the result."""
    if not _INPLACE:
        for name in ("add", "sub", "mul", "div", "clamp_min", "clamp_max", "clamp", "relu", "neg", "exp", "sqrt",
                     "rsqrt", "tanh", "sigmoid", "pow", "abs"):
            packet, inplace = getattr(aten, name, None), getattr(aten, name + "_", None)
            if packet is None or inplace is None:
                continue
            for overload in inplace.overloads():
                if hasattr(packet, overload):
                    _INPLACE[getattr(inplace, overload)] = getattr(packet, overload)
    order = {n: i for i, n in enumerate(graph.nodes)}
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target not in _INPLACE:
            continue
        target = node.args[0]
        if not isinstance(target, fx.Node) or target.op != "call_function":
            continue  # a mutation of an argument of the program is visible to the caller: left alone
        node.target = _INPLACE[node.target]
        for user in list(target.users):
            if user is not node and order[user] > order[node]:
                user.replace_input_with(target, node)


def fuse_and_optimize(fn: Callable, example_inputs: Sequence[torch.Tensor],
                      executor: Callable | None = None) -> FusedModule:
    """Traces `fn`, clusters what the kernel library can run and returns a module in which every cluster is one
    ``akg_call``.  Shapes are those of `example_inputs` (static, like the reference's clustering)."""
    gm = trace(fn, example_inputs)
    gm.graph.eliminate_dead_code()
    clusters = cluster_nodes(gm.graph)
    subs = [lower_cluster(c, i) for i, c in enumerate(clusters)]
    owner = {n: i for i, c in enumerate(clusters) for n in c}

    # Rebuild the graph in dependency order with one call per cluster (a cluster's first outside user may sit before
    # the cluster's last node in the traced order).
    new = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    emitted: set[int] = set()
    old_nodes = list(gm.graph.nodes)

    def emit_cluster(i):
        if i in emitted:
            return
        emitted.add(i)
        sub = subs[i]
        for a in sub.inputs:
            ensure(a)
        call = new.call_function(_bound_call(sub, executor, i), tuple(env[a] for a in sub.inputs))
        for k, o in enumerate(sub.outputs):
            env[o] = new.call_function(operator.getitem, (call, k))

    def ensure(n):
        if n in env:
            return
        if n in owner:
            emit_cluster(owner[n])
            return
        for a in n.all_input_nodes:
            ensure(a)
        env[n] = new.node_copy(n, lambda x: env[x])

    for n in old_nodes:
        if n.op == "placeholder":
            ensure(n)
    for n in old_nodes:
        if n.op == "output":
            for a in n.all_input_nodes:
                ensure(a)
            new.output(fx.node.map_arg(n.args[0], lambda x: env[x]))
        elif n not in owner:
            ensure(n)
    new.lint()
    out = fx.GraphModule(gm, new)
    n_total = sum(1 for n in old_nodes if n.op == "call_function")
    return FusedModule(out, subs, sum(len(c) for c in clusters), n_total)
