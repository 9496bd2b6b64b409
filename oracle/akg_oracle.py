"""CPU oracle for fused-op descriptions — TEST INFRASTRUCTURE, not a product path.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module; the library itself never does.

It restates, in NumPy, what the reference computes for a ``.info`` JSON: the op
list is walked in order and every op is evaluated **in its declared element
type** (one rounding per op), which is what both of the reference's CPU-side
evaluators do:

* the MLIR CPU pipeline lowers each op to arithmetic in the op's element type
  (``akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:377-483``,
  ``akg-mlir/lib/Conversion/MindSporeToTosa/MindSporeToTosa.cpp:475-504``);
* the expected-value generator of ``akg_benchmark`` emits one NumPy statement
  per op (``akg-mlir/python/akg_mlir/utils/op_dsl.py:1154-1244``,
  ``composite_op_helper.py:757-775``).

Pinning: ``tests/test_oracle_golden.py`` checks this module against fixtures
recorded from the reference's generator itself (``tests/golden/``).

Where the two reference evaluators differ, or where last bits depend on a
math library that is not part of the reference checkout (upstream MLIR
TOSA->Linalg and libm/libdevice), this oracle fixes one documented choice:

* transcendental ops (Exp, Log, Tanh, ...) are evaluated in float64 and rounded
  once to the op's type.  For float16/bfloat16 this is the correctly rounded
  result; NumPy's own float16 loop goes through float32 and agrees except on
  double-rounding ties.  Parity at the last bit of float32 transcendentals is
  unpinned (no golden vectors exist in the reference).
* Rsqrt is ``1/sqrt(x)`` with two roundings (``op_dsl.py:792-794``).
* reductions of float16/bfloat16 accumulate in float32 and cast back
  (``op_dsl.py:126-154``); float32 reductions use NumPy's pairwise sum.  With
  ``accum="float64"`` sums run in float64 and are rounded once — the "truth"
  that bounds compare against.  ``accum="sequential"`` reproduces the MLIR CPU
  loop order (``MindSporeToLinalg.cpp:1401-1426``) for small cases.
* ReduceMax/Min ignore NaN like ``arith.maxnumf`` (``:878-879``); inputs in the
  tests are NaN-free.
* MatMul upcasts float16/bfloat16 operands to float32 and accumulates in
  float32 (``op_dsl.py:295-327``); descriptions give MatMul a float32 result.
* float -> int Cast: the reference's NumPy generator truncates (``astype``), its compiled route rounds to nearest
  even and clamps (upstream ``tosa.cast``).  This restatement follows the compiled route, the one the results must
  match; no fixture of the reference pins it (parity unpinned for this op).
"""
from __future__ import annotations

import json
from typing import Sequence

import numpy as np

try:  # bfloat16 support
    import ml_dtypes

    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    BF16 = None


def np_dtype(name: str) -> np.dtype:
    if name == "uint8":  # read as int8, TranslateToMindsporeDialect.cpp:331-333
        name = "int8"
    if name == "bfloat16":
        if BF16 is None:
            raise RuntimeError("bfloat16 needs ml_dtypes")
        return BF16
    return np.dtype(name)


def _is_low_float(dt: np.dtype) -> bool:
    return dt == np.float16 or (BF16 is not None and dt == BF16)


def _round_to(a64: np.ndarray, dt: np.dtype) -> np.ndarray:
    """One rounding from float64 to dt."""
    if BF16 is not None and dt == BF16:
        # float64 -> bf16 in one step: round the float64 to 8 significant bits
        a64 = np.asarray(a64, dtype=np.float64)
        out = np.empty(a64.shape, dtype=np.float32)
        finite = np.isfinite(a64) & (a64 != 0)
        m, e = np.frexp(np.where(finite, a64, 1.0))
        r = np.ldexp(np.rint(np.ldexp(m, 8)), e - 8)
        out[...] = np.where(finite, r, a64)
        return out.astype(BF16)
    return np.asarray(a64, dtype=np.float64).astype(dt)


def _transcendental(fn, x: np.ndarray, dt: np.dtype) -> np.ndarray:
    with np.errstate(all="ignore"):
        return _round_to(fn(x.astype(np.float64)), dt)


_UNARY = {
    "Exp": np.exp, "Log": np.log, "Tanh": np.tanh, "Sin": np.sin, "Cos": np.cos, "Asinh": np.arcsinh,
    "Acosh": np.arccosh, "Atan": np.arctan, "ASin": np.arcsin, "ACos": np.arccos,
}
_BINARY = {
    "Add": np.add, "TensorAdd": np.add, "Sub": np.subtract, "Mul": np.multiply, "RealDiv": np.divide,
    "Div": np.divide, "Maximum": np.maximum, "Minimum": np.minimum,
}
_COMPARE = {
    "Equal": np.equal, "NotEqual": np.not_equal, "Greater": np.greater, "GreaterEqual": np.greater_equal,
    "Less": np.less, "LessEqual": np.less_equal,
}
_REDUCE = {"ReduceSum": "sum", "ReduceMax": "max", "ReduceMin": "min", "ReducePrd": "prod", "ReduceProd": "prod"}


def _attr(attrs, name, default=None):
    for a in attrs or []:
        if a.get("name") == name:
            return a.get("value")
    return default


def _reduce(kind: str, x: np.ndarray, axes: tuple, keep: bool, accum: str) -> np.ndarray:
    dt = x.dtype
    if kind in ("max", "min"):
        fn = np.nanmax if kind == "max" else np.nanmin  # maxnumf/minnumf skip NaN
        with np.errstate(all="ignore"):
            return fn(x.astype(np.float32) if _is_low_float(dt) else x, axis=axes, keepdims=keep).astype(dt)
    if accum == "float64":
        r = getattr(np, kind)(x.astype(np.float64), axis=axes, keepdims=keep)
        return _round_to(r, dt)
    if accum == "sequential":
        # the MLIR CPU loop nest: accumulate in the result type, walking the
        # reduced axes in row-major order
        moved = np.moveaxis(x, axes, range(len(axes)))
        flat = moved.reshape((-1,) + moved.shape[len(axes):])
        acc = np.zeros(flat.shape[1:], dtype=dt) if kind == "sum" else np.ones(flat.shape[1:], dtype=dt)
        for i in range(flat.shape[0]):
            acc = (acc + flat[i]).astype(dt) if kind == "sum" else (acc * flat[i]).astype(dt)
        if keep:
            shape = list(x.shape)
            for a in axes:
                shape[a] = 1
            acc = acc.reshape(shape)
        return acc
    src = x.astype(np.float32) if _is_low_float(dt) else x
    return getattr(np, kind)(src, axis=axes, keepdims=keep).astype(dt)


def evaluate(desc: dict | str, inputs: Sequence[np.ndarray], accum: str = "numpy", return_inputs: bool = False):
    """Evaluates the description on `inputs` (input_desc order); returns outputs in output_desc order (and, with
    `return_inputs`, the inputs as they stand afterwards: Assign/InplaceAssign store into them)."""
    if isinstance(desc, (str, bytes)):
        desc = json.loads(desc)
    env: dict[str, np.ndarray] = {}
    for (d,), a in zip(desc["input_desc"] or [], inputs):
        dt = np_dtype(d["data_type"])
        a = np.asarray(a)
        if a.dtype != dt:
            raise TypeError(f"input {d['tensor_name']}: expected {dt}, got {a.dtype}")
        env[d["tensor_name"]] = a.reshape(d.get("shape") or [1])

    def operand(d):
        name = d["tensor_name"]
        if name in env and d.get("value") is None:
            return env[name]
        if d.get("value") is None:
            raise KeyError(f"operand {name} is undefined")
        # a literal is a typed constant: one rounding from the JSON double
        return _round_to(np.asarray(d["value"], dtype=np.float64), np_dtype(d["data_type"])) \
            if np_dtype(d["data_type"]).kind == "f" or np_dtype(d["data_type"]) == BF16 \
            else np.asarray(d["value"]).astype(np_dtype(d["data_type"]))

    for op in desc["op_desc"]:
        name = op["name"]
        ins = [i[0] for i in op["input_desc"]]
        if name in ("Concat", "AddN"):  # all tensors sit in the first input entry (op_dsl.py:197-207, :901-907)
            ins = list(op["input_desc"][0])
        if name == "Split":  # several results: pieces of the declared extents along the axis (op_dsl.py:416-425)
            axis = _attr(op.get("attr"), "axis", 0)
            x = operand(ins[0])
            cuts = np.cumsum([(o.get("shape") or [1])[axis] for o in op["output_desc"]])[:-1]
            for o, piece in zip(op["output_desc"], np.split(x, cuts, axis)):
                env[o["tensor_name"]] = np.ascontiguousarray(piece)
            continue
        out = op["output_desc"][0]
        odt = np_dtype(out["data_type"])
        oshape = out.get("shape") or [1]
        attrs = op.get("attr")
        with np.errstate(all="ignore"):
            if name in _BINARY:
                a, b = operand(ins[0]), operand(ins[1])
                r = _BINARY[name](a, b).astype(odt)
            elif name in _COMPARE:
                r = _COMPARE[name](operand(ins[0]), operand(ins[1]))
            elif name in _UNARY:
                r = _transcendental(_UNARY[name], operand(ins[0]), odt)
            elif name == "Rsqrt":
                x = operand(ins[0])
                r = (np.asarray(1.0, dtype=x.dtype) / np.sqrt(x)).astype(odt)
            elif name == "Sqrt":
                r = np.sqrt(operand(ins[0])).astype(odt)
            elif name == "Reciprocal":
                x = operand(ins[0])
                r = (np.asarray(1.0, dtype=x.dtype) / x).astype(odt)
            elif name == "Abs":
                r = np.abs(operand(ins[0]))
            elif name == "Neg":
                r = np.negative(operand(ins[0]))
            elif name == "Floor":
                r = np.floor(operand(ins[0]))
            elif name == "Square":
                x = operand(ins[0])
                r = np.multiply(x, x)
            elif name == "Pow":
                r = np.power(operand(ins[0]), operand(ins[1])).astype(odt)
            elif name == "Atan2":  # op_dsl.py:1052-1055
                a, b = operand(ins[0]), operand(ins[1])
                r = _round_to(np.arctan2(a.astype(np.float64), b.astype(np.float64)), odt)
            elif name in ("IsNan", "IsInf", "IsFinite"):  # op_dsl.py:717-744
                x = operand(ins[0])
                x = x.astype(np.float32) if _is_low_float(x.dtype) else x
                r = {"IsNan": np.isnan, "IsInf": np.isinf, "IsFinite": np.isfinite}[name](x)
            elif name == "LogicalNot":
                r = np.logical_not(operand(ins[0]))
            elif name in ("LogicalAnd", "LogicalOr"):
                fn = np.logical_and if name == "LogicalAnd" else np.logical_or
                r = fn(operand(ins[0]), operand(ins[1]))
            elif name == "Cast":
                x = operand(ins[0])
                if x.dtype.kind == "f" or (BF16 is not None and x.dtype == BF16):
                    if odt.kind in "iu":
                        # the MLIR route (upstream tosa.cast): round to nearest even, clamp to the result type; the
                        # reference's NumPy generator would truncate instead.  NaN gives 0.
                        x64 = np.nan_to_num(x.astype(np.float64), nan=0.0, posinf=np.inf, neginf=-np.inf)
                        info = np.iinfo(odt)
                        if odt.itemsize > 4:
                            # 2^63 - 1 is no float64: saturate by comparison, convert only what is in range
                            rr = np.rint(x64)
                            hi, lo = rr >= 2.0 ** 63, rr <= -(2.0 ** 63)
                            r = np.where(hi | lo, 0.0, rr).astype(odt)
                            r[hi] = info.max
                            r[lo] = info.min
                        else:
                            r = np.clip(np.rint(x64), info.min, info.max).astype(odt)
                    # widening is exact; narrowing rounds to nearest even (arith.truncf)
                    elif _is_low_float(x.dtype):
                        r = x.astype(np.float32).astype(odt)
                    else:
                        r = x.astype(odt)
                else:
                    r = x.astype(odt)
            elif name == "Select":
                r = np.where(operand(ins[0]), operand(ins[1]), operand(ins[2])).astype(odt)
            elif name in _REDUCE:
                x = operand(ins[0])
                axes = _attr(attrs, "axis")
                if (axes is None or axes == []) and len(ins) == 2:
                    axes = ins[1]["value"]
                if axes is None or axes == []:
                    axes = list(range(x.ndim))
                if not isinstance(axes, (list, tuple)):
                    axes = [axes]
                axes = tuple(sorted({a + x.ndim if a < 0 else a for a in axes}))
                keep = bool(_attr(attrs, "keep_dims", False))
                r = _reduce(_REDUCE[name], x, axes, keep, accum)
            elif name in ("Assign", "InplaceAssign"):
                # the value lands in the caller's first operand; the result is the value (Assign) or the third
                # operand (InplaceAssign) — op_dsl.py:956-961, 1032-1037
                val = operand(ins[1])
                env[ins[0]["tensor_name"]] = np.array(val, dtype=val.dtype).reshape(env[ins[0]["tensor_name"]].shape)
                r = val if name == "Assign" or len(ins) < 3 else operand(ins[2])
            elif name in ("ReduceAll", "ReduceAny", "ElemAny"):
                x = operand(ins[0])
                axes = _attr(attrs, "axis")
                if (axes is None or axes == []) and len(ins) == 2:
                    axes = ins[1]["value"]
                if axes is None or axes == [] or name == "ElemAny":
                    axes = list(range(x.ndim))
                if not isinstance(axes, (list, tuple)):
                    axes = [axes]
                axes = tuple(sorted({a + x.ndim if a < 0 else a for a in axes}))
                fn = np.all if name == "ReduceAll" else np.any
                r = fn(x, axis=axes, keepdims=bool(_attr(attrs, "keep_dims", False)) or name == "ElemAny")
            elif name == "ArgMax":
                axis = _attr(attrs, "axis")
                if len(op["input_desc"]) > 1:
                    axis = op["input_desc"][1][0]["value"]
                axis = axis[0] if isinstance(axis, (list, tuple)) else axis
                x = operand(ins[0])
                x = x.astype(np.float32) if x.dtype.itemsize == 2 else x
                r = np.argmax(x, axis=axis)  # op_dsl.py:1345 spells the index the same way
                if _attr(attrs, "keep_dims", False):
                    r = np.expand_dims(r, axis)
                r = r.astype(odt)
            elif name == "Pad":
                x = operand(ins[0])
                padding = _attr(attrs, "padding")
                if padding is not None:  # MindSporeToTosa.cpp:339-357: pairs from the last dimension backwards
                    width = [(0, 0)] * x.ndim
                    for i in range(len(padding) // 2):
                        width[x.ndim - 1 - i] = (padding[2 * i], padding[2 * i + 1])
                    value = _attr(attrs, "value", 0)
                else:  # op_dsl.py:623-634
                    width = list(zip(_attr(attrs, "head"), _attr(attrs, "tail")))
                    value = _attr(attrs, "pad_val", 0)
                r = np.pad(x, width, mode="constant", constant_values=np.asarray(value).astype(x.dtype))
            elif name == "Gather":
                axis = _attr(attrs, "axis", 0)
                if len(op["input_desc"]) > 2:
                    axis = op["input_desc"][2][0]["value"]
                r = np.take(operand(ins[0]), operand(ins[1]), axis)  # op_dsl.py:101-104, 1119-1125
            elif name == "UnsortedSegmentSum":
                data, ids = operand(ins[0]), operand(ins[1])
                nseg = _attr(attrs, "num_segments") or _attr(attrs, "numSegments")
                if nseg is None and len(op["input_desc"]) > 2:
                    nseg = op["input_desc"][2][0]["value"]
                r = np.zeros([nseg] + list(data.shape[ids.ndim:]), dtype=np.float64)
                np.add.at(r, ids, data.astype(np.float64))  # op_dsl.py:1109-1116, accumulated in float64 here
                r = r.astype(odt)
            elif name == "AddN":
                r = operand(ins[0])
                for other in ins[1:]:
                    r = np.add(r, operand(other)).astype(odt)  # "a + b + c", left to right (op_dsl.py:901-907)
            elif name == "Tile":
                mult = _attr(attrs, "multiples")
                if mult is None and len(op["input_desc"]) == 2:
                    mult = op["input_desc"][1][0]["value"]
                r = np.tile(operand(ins[0]), mult)  # op_dsl.py:910-915
            elif name == "Slice":
                begin, size = _attr(attrs, "begin"), _attr(attrs, "size")
                r = operand(ins[0])[tuple(slice(b, b + s) for b, s in zip(begin, size))]  # op_dsl.py:397-413
            elif name == "StridedSlice":
                # masks other than begin/end are not evaluated here (the library rejects them)
                def val(key, idx):
                    v = _attr(attrs, key)
                    if v:
                        return list(v)
                    v = op["input_desc"][idx][0]["value"]
                    return list(v) if isinstance(v, (list, tuple)) else [v]
                x = operand(ins[0])
                begin, end, strides = val("begin", 1), val("end", 2), val("strides", 3)
                bm = _attr(attrs, "begin_mask", 0) or 0
                em = _attr(attrs, "end_mask", 0) or 0
                sl = []
                for i in range(len(begin)):
                    b = None if (bm >> i) & 1 else begin[i]
                    e = None if (em >> i) & 1 else end[i]
                    sl.append(slice(b, e, strides[i]))  # op_dsl.py:340-394
                r = x[tuple(sl)]
            elif name == "Concat":
                r = np.concatenate([operand(i) for i in ins], axis=_attr(attrs, "axis", 0))  # op_dsl.py:197-207
            elif name == "Reshape":
                r = operand(ins[0])
            elif name == "BroadcastTo":
                r = np.broadcast_to(operand(ins[0]), oshape)
            elif name == "Transpose":
                perm = _attr(attrs, "perm")
                if perm is None and len(ins) == 2:
                    perm = ins[1]["value"]
                r = np.ascontiguousarray(np.transpose(operand(ins[0]), axes=perm))
            elif name in ("MatMul", "BatchMatMul"):
                a, b = operand(ins[0]), operand(ins[1])
                if _attr(attrs, "transpose_a", False):
                    raise NotImplementedError("transpose_a is rejected by the reference lowering "
                                              "(MindSporeToLinalg.cpp:1508-1510)")
                if _attr(attrs, "transpose_b", False):
                    b = np.swapaxes(b, -1, -2)
                r = np.matmul(a.astype(np.float32), b.astype(np.float32)).astype(odt)
            else:
                raise NotImplementedError(f"op {name}")
        env[out["tensor_name"]] = np.ascontiguousarray(np.asarray(r, dtype=odt if name not in _COMPARE else None)
                                                       ).reshape(oshape)
    outs = [env[o["tensor_name"]].reshape(o.get("shape") or [1]) for o in desc["output_desc"]]
    if return_inputs:
        return outs, [env[d["tensor_name"]] for (d,) in desc["input_desc"] or []]
    return outs
