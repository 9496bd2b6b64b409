"""Pins the CPU oracle against fixtures recorded from the reference's own expected-value generator
(akg-mlir/python/akg_mlir/utils/composite_op_helper.py:833-902), see tests/golden/make_golden.py."""
import numpy as np
import pytest

from oracle import akg_oracle as O
from helpers import bits_equal, golden_cases, load_golden, ulp_diff_f16

# fixtures whose ops are add/mul/div/sqrt/compare/reduce/matmul/transpose only: the oracle must
# reproduce the reference generator bit for bit
EXACT = [c for c in golden_cases() if not c.startswith(("gelu", "softmax", "tanh"))]


@pytest.mark.parametrize("case", EXACT)
def test_bit_exact_cases(case):
    desc, ins, outs = load_golden(case)
    got = O.evaluate(desc, ins)
    assert len(got) == len(outs)
    for g, e in zip(got, outs):
        assert bits_equal(g, e), case


@pytest.mark.parametrize("case", [c for c in golden_cases() if c.startswith("softmax")])
def test_softmax_cases(case):
    # Exp is evaluated in float64 and rounded once here; the fixture used NumPy's float32 exp.
    desc, ins, outs = load_golden(case)
    got = O.evaluate(desc, ins)[0]
    e = outs[0]
    if e.dtype == np.float16:
        assert ulp_diff_f16(got, e).max() <= 1
        assert (got != e).mean() < 1e-3
    else:
        np.testing.assert_allclose(got, e, rtol=1e-6, atol=1e-9)
    # masked positions are exactly zero in both
    assert np.array_equal(got == 0, e == 0)


@pytest.mark.parametrize("case", [c for c in golden_cases() if c.startswith("gelu")])
def test_gelu_cases(case):
    # The fixture was recorded on a CPU where NumPy's float16 tanh loop is up to 3 float16 steps off
    # (see test_tanh_f16_all); every other op of the chain is exact, so the two agree to the
    # reference's own comparison tolerance for float16-derived results (result_analysis.py:439-459).
    desc, ins, outs = load_golden(case)
    got = O.evaluate(desc, ins)[0]
    e = outs[0]
    close = np.isclose(got, e, rtol=1e-3, atol=1e-3)
    assert close.mean() > 0.99
    assert np.allclose(got, e, rtol=1e-2, atol=1e-2)


def test_tanh_f16_all():
    """All finite float16 inputs: the oracle's Tanh is the correctly rounded value, which is also what
    extend-to-float32 + tanhf + truncate gives (the MLIR CPU route); the recorded NumPy float16 loop is
    within 3 steps of it."""
    desc, ins, outs = load_golden("tanh_f16_all")
    got = O.evaluate(desc, ins)[0]
    x = ins[0]
    via_f32 = np.tanh(x.astype(np.float32)).astype(np.float16)
    assert bits_equal(got, via_f32)
    assert ulp_diff_f16(got, outs[0]).max() <= 3


def test_sequential_and_float64_accumulators_bound_the_pairwise_sum():
    desc, ins, outs = load_golden("reduce_sum0_256x128")
    pair = O.evaluate(desc, ins)[0]
    seq = O.evaluate(desc, ins, accum="sequential")[0]
    truth = O.evaluate(desc, ins, accum="float64")[0]
    scale = np.abs(ins[0]).sum(axis=0)
    assert np.all(np.abs(pair - truth) <= 1e-6 * scale)
    assert np.all(np.abs(seq - truth) <= 1e-5 * scale)
