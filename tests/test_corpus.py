"""The fused-operator descriptions of the reference's own system tests (akg-mlir/tests/st/**/*.info*), with expected
values recorded from the reference's expected-value generator (tests/golden/make_golden.py corpus).

CPU: the NumPy restatement against those values.  GPU: the CUDA library through the C ABI against the same values, the
dynamic-shape descriptions additionally through the launch-time binding path with their original -1 extents.
"""
import numpy as np
import pytest

from helpers import bits_equal, corpus_cases, load_corpus
from oracle import akg_oracle as O

CASES = corpus_cases()
# float32 -> int32 Cast: the recorded values come from the reference's expected-value generator, which truncates like
# NumPy; the reference's compiled pipeline (tosa.cast) rounds to nearest even and clamps, and that is the route the
# restatement and the library follow.  For this description the two evaluations are compared with each other and the
# recorded values only where truncation and rounding agree.
ROUNDS_NOT_TRUNCATES = {"Fused_Cast_fusion_9232082611397577167"}


def _compare(got, want, desc):
    assert len(got) == len(want)
    for g, w, od in zip(got, want, desc["output_desc"]):
        g = np.asarray(g).reshape(w.shape)
        assert g.dtype == w.dtype, (g.dtype, w.dtype)
        if w.dtype.kind in "biu":
            assert bits_equal(np.ascontiguousarray(g), np.ascontiguousarray(w))
            continue
        tol = 2e-3 if w.dtype.itemsize == 2 else 2e-5
        w64, g64 = w.astype(np.float64), g.astype(np.float64)
        scale = float(np.nanmax(np.abs(w64[np.isfinite(w64)]))) if np.isfinite(w64).any() else 1.0
        np.testing.assert_allclose(g64, w64, rtol=tol, atol=tol * max(scale, 1e-30), equal_nan=True)


def test_corpus_is_present():
    assert len(CASES) >= 25


@pytest.mark.parametrize("name", CASES)
def test_restatement_against_the_reference_values(name):
    desc, _, ins, want = load_corpus(name)
    got = O.evaluate(desc, ins)
    if name in ROUNDS_NOT_TRUNCATES:
        for g, w in zip(got, want):
            assert g.dtype == w.dtype and int(np.abs(g.astype(np.int64) - w.astype(np.int64)).max()) <= 1
            assert (g == w).mean() > 0.3  # truncation and rounding agree below .5
        return
    _compare(got, want, desc)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_library_against_the_reference_values(name):
    from akg_b200 import FusedKernel, UnsupportedError
    desc, dyn, ins, want = load_corpus(name)
    if name in ROUNDS_NOT_TRUNCATES:
        want = O.evaluate(desc, ins)  # the compiled route's rounding, see above
    k = FusedKernel(desc)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD
    args = [a.copy() for a in ins] + outs
    k.run_host(args)
    assert k.check_device_error() == 0
    _compare(outs, want, desc)
    if dyn is None:
        return
    import torch
    kd = FusedKernel(dyn)
    assert kd.is_dynamic
    dev_in = [torch.from_numpy(a.copy()).cuda() for a in ins]
    dev_out = [torch.empty(o.shape, dtype=torch.from_numpy(o).dtype, device="cuda") for o in outs]
    kd.launch(dev_in + dev_out)
    torch.cuda.synchronize()
    _compare([t.cpu().numpy() for t in dev_out], want, desc)


@pytest.mark.gpu
def test_driver_runs_a_dynamic_shape_description_from_a_file(tmp_path):
    """The host-side mirror of the reference driver on one of the reference's dynamic-shape descriptions: compile()
    from the .info file, run() with host arrays whose extents bind the -1 dimensions."""
    import json
    from akg_b200 import MlirDriver
    name = next(n for n in CASES if load_corpus(n)[1] is not None and n.startswith("Fused_Sub_Mul_Mul_Add_Softmax"))
    desc, dyn, ins, want = load_corpus(name)
    info = tmp_path / (dyn["op"] + ".info")
    info.write_text(json.dumps(dyn))
    drv = MlirDriver(dyn["op"], str(info), output_dir=str(tmp_path), dynamic_shape=True, backend="gpu")
    drv.compile()
    outs = [np.full(o.shape, np.nan, dtype=o.dtype) for o in want]
    drv.run([a.copy() for a in ins] + outs)
    _compare(outs, want, desc)
    meta = json.loads((tmp_path / (dyn["op"] + ".json")).read_text())
    assert meta["is_dynamic"] is True and meta["kernelName"] == dyn["op"] + "_kernel"
