"""The C restatement of the reference CPU pipeline (oracle/cpu_ref.c) against the NumPy oracle."""
import numpy as np
import pytest

from akg_b200 import descs
from oracle import akg_oracle as O
from oracle import cpu_ref as C
from helpers import BF16, KINDS, bits_equal, make_inputs


@pytest.mark.parametrize("variant", ["r1", "rp"])
def test_layernorm(variant):
    d = descs.layernorm(33, 200)
    x, g, b = make_inputs(d, 1, KINDS["layernorm"])
    y, m, v = C.layernorm(x, g, b, variant=variant)
    oy, om, ov = O.evaluate(d, [x, g, b])
    np.testing.assert_allclose(y, oy, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(m, om, rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(v, ov, rtol=1e-5)


@pytest.mark.parametrize("variant", ["r1", "rp"])
def test_gelu_chain_is_bit_exact(variant):
    d = descs.gelu_chain([3, 7, 64])
    x, bias, y = make_inputs(d, 2, KINDS["gelu"])
    assert bits_equal(C.gelu_chain(x, bias, y, variant=variant), O.evaluate(d, [x, bias, y])[0])


@pytest.mark.parametrize("variant", ["r1", "rp"])
def test_softmax(variant):
    d = descs.masked_softmax(2, 48, 96)
    s, mask = make_inputs(d, 3, KINDS["softmax"])
    got = C.softmax(s, mask, 1.0 / np.sqrt(128.0), variant=variant)
    want = O.evaluate(d, [s, mask])[0]
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=2e-3, atol=1e-7)
    assert np.array_equal(got == 0, want == 0)


@pytest.mark.parametrize("variant", ["r1", "rp"])
def test_reductions(variant):
    x = make_inputs(descs.reduce_sum_axis0(300, 70), 4)[0]
    truth = x.astype(np.float64).sum(axis=0)
    got = C.reduce_sum_axis0(x, variant=variant)
    assert np.all(np.abs(got - truth) <= 1e-5 * np.abs(x).sum(axis=0))
    # the sequential order is the oracle's "sequential" accumulator, bit for bit
    assert bits_equal(got, O.evaluate(descs.reduce_sum_axis0(300, 70), [x], accum="sequential")[0])
    assert C.reduce_max_all(x, variant=variant)[0] == x.max()


@pytest.mark.parametrize("variant", ["r1", "rp"])
def test_matmul_and_transpose(variant):
    d = descs.matmul_bias_relu(32, 48, 64)
    a, b, bias = make_inputs(d, 5, KINDS["matmul"])
    got = C.matmul_bias_relu(a, b, bias, variant=variant).view(BF16)
    want = O.evaluate(d, [a, b, bias])[0]
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=2e-3, atol=1e-6)
    x = make_inputs(descs.transpose([2, 6, 3, 8], [0, 2, 1, 3]), 6)[0]
    assert bits_equal(C.transpose4(x, [0, 2, 1, 3], variant=variant), np.ascontiguousarray(x.transpose(0, 2, 1, 3)))
