"""Small regions over the op surface of the JSON factory, with expected values recorded from the reference's
expected-value generator (tests/golden/make_golden.py ops): the NumPy restatement on the CPU, the CUDA library through
the C ABI on the GPU.  (The reference's generator raises on its own Gather and UnsortedSegmentSum handlers and returns
no value for an Assign result, so those three have no fixture; they are covered against the restatement elsewhere.)"""
import numpy as np
import pytest

from helpers import bits_equal, load_ops, ops_cases
from oracle import akg_oracle as O

CASES = ops_cases()
# results that involve only exactly rounded arithmetic, comparisons, selections, type changes and data movement
EXACT = {"abs_neg_floor", "binary_broadcast", "compare_select", "isnan_isinf", "casts", "reduce_min_x", "reduce_max_all",
         "reduce_all_bool", "reshape_transpose_broadcast", "tile_slice_strided", "concat_addn"}


def _check(got, want, name, loose):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        g = np.asarray(g).reshape(w.shape)
        assert g.dtype == w.dtype, (name, g.dtype, w.dtype)
        if w.dtype.kind in "biu" or (name in EXACT and not loose):
            assert bits_equal(np.ascontiguousarray(g), np.ascontiguousarray(w)), name
            continue
        tol = 2e-3 if (w.dtype.itemsize == 2 or name.startswith("batch_matmul")) else (1e-5 if loose else 2e-6)
        w64, g64 = w.astype(np.float64), g.astype(np.float64)
        fin = np.isfinite(w64)
        scale = float(np.abs(w64[fin]).max()) if fin.any() else 1.0
        np.testing.assert_allclose(g64, w64, rtol=tol, atol=tol * max(scale, 1e-30), equal_nan=True)


def test_fixtures_present():
    assert len(CASES) >= 28


@pytest.mark.parametrize("name", CASES)
def test_restatement_against_the_reference_values(name):
    desc, ins, want = load_ops(name)
    _check(O.evaluate(desc, ins), want, name, loose=False)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_library_against_the_reference_values(name):
    from akg_b200 import FusedKernel
    desc, ins, want = load_ops(name)
    k = FusedKernel(desc)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    k.run_host([a.copy() for a in ins] + outs)
    assert k.check_device_error() == 0
    _check(outs, want, name, loose=name not in EXACT)
