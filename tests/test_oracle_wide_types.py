"""The oracle on 64-bit element types (no GPU): float -> int64 casts follow the compiled route of the reference
(tosa.cast: round to nearest even, clamp to the result type, NaN gives 0; upstream TOSA lowering behind
akg-mlir/lib/Conversion/MindSporeToTosa/MindSporeToTosa.cpp:489), float64 arithmetic is NumPy's own
(akg-mlir/python/akg_mlir/utils/op_dsl.py:752-825).  No fixture of the reference pins these types: parity unpinned for
them, as for the narrower float -> integer casts."""
import numpy as np

from akg_b200.descs import _Builder, _attr
from oracle import akg_oracle as O


def _cast(src, dst, n):
    b = _Builder(f"Fused_Cast_{src}_{dst}_1")
    x = b.input("x", [n], src)
    b.output(b.emit("Cast", [x], [n], dst, [_attr("dst_type", "str", dst)]))
    return b.build()


def test_float_to_int64_rounds_to_even_and_saturates():
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 4503599627370497.5, 2.0 ** 62 + 1024, 9.3e18, -9.3e18, 2.0 ** 63,
                  -(2.0 ** 63), 1e300, -1e300, np.inf, -np.inf, np.nan, -0.0], dtype=np.float64)
    got = O.evaluate(_cast("float64", "int64", x.size), [x])[0]
    hi, lo = 2 ** 63 - 1, -2 ** 63
    assert got.dtype == np.int64
    assert got.tolist() == [0, 2, 2, 0, -2, -2, 4503599627370498, 2 ** 62 + 1024, hi, lo, hi, lo, hi, lo, hi, lo, 0, 0]
    x32 = np.array([3e10, -3e10, 1e20, -1e20, np.nan, 8388607.5], dtype=np.float32)
    got32 = O.evaluate(_cast("float32", "int64", x32.size), [x32])[0]
    assert got32.tolist() == [30000001024, -30000001024, hi, lo, 0, 8388608]


def test_float64_chain_is_numpy_float64():
    rng = np.random.default_rng(3)
    x, y = rng.standard_normal((17, 33)) * 1e3, rng.standard_normal(33)
    f = "float64"
    b = _Builder("Fused_F64_oracle_2")
    xi, yi = b.input("x", [17, 33], f), b.input("y", [33], f)
    t = b.emit("RealDiv", [b.emit("Mul", [b.emit("Add", [xi, yi], [17, 33], f), b.const(0.1234567890123456, f)], [17, 33], f),
                           b.emit("Sqrt", [b.emit("Abs", [xi], [17, 33], f)], [17, 33], f)], [17, 33], f)
    b.output(t)
    b.output(b.emit("Cast", [t], [17, 33], "float16", [_attr("dst_type", "str", "float16")]))
    got = O.evaluate(b.build(), [x, y])
    want = (x + y) * 0.1234567890123456 / np.sqrt(np.abs(x))
    assert got[0].dtype == np.float64 and np.array_equal(got[0], want)
    # one rounding from float64 to float16, not two through float32
    assert got[1].dtype == np.float16 and np.array_equal(got[1], want.astype(np.float16))
