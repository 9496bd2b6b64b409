"""Parity of the CUDA path with the CPU oracle, through the C ABI.  Needs a B200.

Tolerances (stated by the benchmark definition): bit-exact for transpose and for the float16 GELU chain
(every op of the chain is reproduced with its own rounding); 1e-5 relative for float32 results; 2e-3 for
float16/bfloat16 results of reductions and transcendentals.
"""
import numpy as np
import pytest

from akg_b200 import FusedKernel, descs
from oracle import akg_oracle as O
from helpers import BF16, KINDS, bits_equal, golden_cases, guarded_launch, load_golden, make_inputs, ulp_diff_f16

pytestmark = pytest.mark.gpu


def run_host(desc, ins, **kw):
    """The host-pointer entry point (what the reference's launcher does), and the same region once more as a device
    launch between guard zones: same bits, nothing written outside the tensors."""
    k = FusedKernel(desc, **kw)
    outs = k.empty_outputs()
    for o in outs:
        o.view(np.uint8)[...] = 0xCD  # poison
    k.run_host(list(ins) + outs)
    if not kw:
        guarded, _ = guarded_launch(desc, ins)
        for a, b in zip(outs, guarded):
            assert np.array_equal(np.ascontiguousarray(a).view(np.uint8).reshape(-1), b.view(np.uint8).reshape(-1))
    return outs, k


# ------------------------------------------------------------------ golden fixtures
GPU_GOLDEN = [c for c in golden_cases() if not c.startswith("tanh")]


@pytest.mark.parametrize("case", GPU_GOLDEN)
def test_golden_fixtures(lib, case):
    desc, ins, want = load_golden(case)
    got, _ = run_host(desc, ins)
    for g, e in zip(got, want):
        if case.startswith("transpose") or case.startswith("reduce_max"):
            assert bits_equal(g, e)
        elif case.startswith("gelu"):
            # the fixture's float16 tanh is up to 3 steps off (see test_oracle_golden.py); the oracle is exact
            assert bits_equal(g, O.evaluate(desc, ins)[0])
            assert np.allclose(g, e, rtol=1e-2, atol=1e-2)
        elif case.startswith("softmax") or case.startswith("matmul"):
            np.testing.assert_allclose(g.astype(np.float32), e.astype(np.float32), rtol=2e-3, atol=1e-6)
        elif case.startswith("reduce"):
            x = ins[0]
            if g.size == 1:
                assert bits_equal(g, e)
            else:
                assert np.all(np.abs(g - e) <= 1e-5 * np.abs(x).sum(axis=0))
        else:  # layernorm
            np.testing.assert_allclose(g, e, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ elementwise chain
@pytest.mark.parametrize("shape,bias,mul,f32", [
    ([64, 4096], True, True, True), ([5, 7, 24], True, True, True), ([3, 50], True, True, True),
    ([1, 8], True, True, True), ([1000], False, True, True), ([17, 128], True, False, False),
    ([2, 3, 4, 40], False, False, True), ([1], False, False, False),
])
def test_gelu_chain_bit_exact(lib, shape, bias, mul, f32):
    d = descs.gelu_chain(shape, with_bias=bias, with_mul=mul, cast_f32=f32)
    ins = make_inputs(d, 11, KINDS["gelu"])
    got, _ = run_host(d, ins)
    assert bits_equal(got[0], O.evaluate(d, ins)[0])


def test_gelu_chain_covers_every_float16_value(lib):
    # d = c*c1 sweeps all float16 magnitudes when x does (no bias): the tanh table and its two cut-offs
    # are exercised on every input, including subnormals, infinities and NaN
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    x = np.tile(bits, 2).view(np.float16)
    d = descs.gelu_chain([x.size], with_bias=False, with_mul=False, cast_f32=False)
    got, _ = run_host(d, [x])
    want = O.evaluate(d, [x])[0]
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got[0]), nan)
    assert bits_equal(got[0][~nan], want[~nan])


# ------------------------------------------------------------------ LayerNorm
@pytest.mark.parametrize("rows,cols,stats", [(256, 1024, True), (7, 100, False), (33, 2048, True), (5, 3000, True),
                                             (1, 4, True), (64, 129, False),
                                             # many rows (several waves of CTAs), widths on either side of the vector-per-lane steps
                                             (8192, 256, True), (5000, 1000, False), (4736, 132, True), (10001, 8, True),
                                             (6000, 1024, True), (4800, 2048, True), (4096, 1024, True), (3700, 1024, False)])
def test_layernorm(lib, rows, cols, stats):
    d = descs.layernorm(rows, cols, with_stats=stats)
    ins = make_inputs(d, 12, KINDS["layernorm"])
    got, _ = run_host(d, ins)
    want = O.evaluate(d, ins, accum="float64")
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-6)
    for g, e in zip(got[1:], want[1:]):
        np.testing.assert_allclose(g, e, rtol=1e-5, atol=1e-7)


# ------------------------------------------------------------------ softmax
@pytest.mark.parametrize("b,r,c,dt,mask", [(2, 64, 128, "float16", True), (1, 2048, 2048, "float16", True),
                                           (3, 8, 40, "float32", False), (2, 16, 24, "bfloat16", True),
                                           (1, 5, 5000, "float16", True), (2, 3, 7, "float16", True),
                                           (4, 32, 256, "bfloat16", True), (3, 100, 1000, "float16", False),
                                           (5, 77, 2048, "float16", True), (1, 300, 8, "bfloat16", False)])
def test_softmax(lib, b, r, c, dt, mask):
    d = descs.masked_softmax(b, r, c, dtype=dt, with_mask=mask)
    ins = make_inputs(d, 13, KINDS["softmax"])
    got, _ = run_host(d, ins)
    want = O.evaluate(d, ins)[0]
    tol = 1e-5 if dt == "float32" else 2e-3
    np.testing.assert_allclose(got[0].astype(np.float32), want.astype(np.float32), rtol=tol, atol=1e-7)
    assert np.array_equal(got[0].astype(np.float32) == 0, want.astype(np.float32) == 0)  # masked entries


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1000, 52), (3, 7), (1, 1), (70000, 16), (513, 1030)])
def test_column_sum_and_global_max(lib, rows, cols):
    d = descs.reduce_sum_and_max(rows, cols)
    x = make_inputs(d, 14)[0]
    got, k = run_host(d, [x])
    assert k.op_class == ("reduce_y" if rows > 1 and cols > 1 else k.op_class)
    truth = x.astype(np.float64).sum(axis=0)
    assert np.all(np.abs(got[0] - truth) <= 1e-5 * np.abs(x).sum(axis=0) + 1e-30)
    assert got[1][0] == x.max()


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1000, 52), (70000, 16), (513, 1030), (20000, 3000)])
def test_fold_by_the_last_cta_gives_the_bits_of_the_fold_in_a_second_launch(lib, rows, cols):
    """AKGB_FLAG_FOLD_IN_LAUNCH: the CTA that arrives last folds the row splits (arrival counters that every launch
    leaves at zero, so launches repeat); same order of operations, same bits, one launch less per fold."""
    from akg_b200 import _capi
    x = make_inputs(descs.reduce_sum_axis0(rows, cols), 19)[0]
    for build in (descs.reduce_sum_axis0, descs.reduce_max_all, descs.reduce_sum_and_max):
        want, k0 = run_host(build(rows, cols), [x])
        k1 = FusedKernel(build(rows, cols), flags=_capi.AKGB_FLAG_FOLD_IN_LAUNCH)
        assert k1.launch_count < k0.launch_count or k0.launch_count == 1
        for _ in range(3):  # the counters are back at zero after every launch
            got = k1.empty_outputs()
            for o in got:
                o.view(np.uint8)[...] = 0xCD
            k1.run_host([x] + got)
            for g, w in zip(got, want):
                assert bits_equal(g, w)


def test_row_reductions_and_other_combiners(lib):
    import json
    x = make_inputs(descs.reduce_sum_axis0(300, 260), 15)[0]
    for op, ref in (("ReduceSum", np.sum), ("ReduceMax", np.max), ("ReduceMin", np.min)):
        d = descs.reduce_sum_axis0(300, 260)
        d["op_desc"][0]["name"] = op
        d["op_desc"][0]["attr"][0]["value"] = [1]
        d["op_desc"][0]["output_desc"][0]["shape"] = [300]
        d["output_desc"][0]["shape"] = [300]
        got, k = run_host(json.loads(json.dumps(d)), [x])
        assert k.op_class == "reduce_x"
        want = ref(x.astype(np.float64), axis=1)
        if op == "ReduceSum":
            assert np.all(np.abs(got[0] - want) <= 1e-5 * np.abs(x).sum(axis=1))
        else:
            assert np.array_equal(got[0], want.astype(np.float32))


# ------------------------------------------------------------------ transpose
@pytest.mark.parametrize("shape,perm,dt", [
    ([2, 64, 4, 128], [0, 2, 1, 3], "float16"), ([6, 10], [1, 0], "float32"), ([3, 5, 7], [2, 0, 1], "float16"),
    ([2, 3, 4, 5, 6], [4, 2, 0, 3, 1], "int8"), ([1, 9, 1, 8], [3, 1, 2, 0], "float32"), ([130, 70], [1, 0], "float16"),
    ([4, 8, 16], [0, 1, 2], "float32"), ([2, 33, 65], [0, 2, 1], "int64"),
    # tile mode with 16-byte loads and 128-byte stores (2- and 4-byte elements), whole and ragged tiles, batches
    ([256, 192], [1, 0], "float16"), ([100, 64], [1, 0], "float32"), ([3, 72, 40], [0, 2, 1], "float16"),
    ([2, 3, 64, 48], [0, 1, 3, 2], "float32"), ([5, 128, 8], [2, 0, 1], "int16"), ([1000, 1016], [1, 0], "float16"),
    ([7, 36, 260], [0, 2, 1], "int32"), ([4, 6, 8, 24], [2, 0, 3, 1], "float16"), ([2, 130, 72], [0, 2, 1], "float16"),
])
def test_transpose_bit_exact(lib, shape, perm, dt):
    d = descs.transpose(shape, perm, dt)
    rng = np.random.default_rng(16)
    x = rng.integers(-100, 100, size=shape).astype(np.dtype(dt))
    got, _ = run_host(d, [x])
    assert bits_equal(got[0], np.ascontiguousarray(np.transpose(x, perm)))


# ------------------------------------------------------------------ empty tensors
def test_empty_leading_extent(lib):
    """A region over zero rows is legal: nothing is read or written, reductions over the empty axis return the
    reference's init values (sum 0, max -FLT_MAX: MindSporeToLinalg.cpp:791-843), launches with nothing to do are
    skipped rather than rejected by the driver."""
    import torch
    flt_max = np.finfo(np.float32).max
    for d in (descs.gelu_chain([0, 8, 64]), descs.layernorm(0, 128), descs.masked_softmax(0, 16, 64),
              descs.transpose([0, 4, 8, 16], [0, 2, 1, 3]), descs.transpose([0, 6], [1, 0], "float32"),
              descs.rmsnorm(0, 256)):
        ins = make_inputs(d, 3, {"mask": "causal"})
        got, k = guarded_launch(d, ins)
        assert all(g.size == 0 for g in got) and k.check_device_error() == 0
    for d, want in ((descs.reduce_sum_axis0(0, 48), [np.zeros(48, np.float32)]),
                    (descs.reduce_max_all(0, 48), [np.full(1, -flt_max, np.float32)]),
                    (descs.reduce_sum_and_max(0, 48), [np.zeros(48, np.float32), np.full(1, -flt_max, np.float32)])):
        got, k = guarded_launch(d, make_inputs(d, 3))
        for g, w in zip(got, want):
            assert bits_equal(g.reshape(w.shape), w)
    torch.cuda.synchronize()


# ------------------------------------------------------------------ launch path + metadata
def test_device_launch_matches_host_run_and_reports_dims(lib):
    import torch
    d = descs.layernorm(512, 1024)
    ins = make_inputs(d, 17, KINDS["layernorm"])
    want, k = run_host(d, ins)
    dev = [torch.from_numpy(a).cuda() for a in ins]
    outs = [torch.empty(t.shape, dtype=torch.float32, device="cuda") for t in k.outputs]
    k.launch(dev + outs)
    torch.cuda.synchronize()
    for o, w in zip(outs, want):
        assert bits_equal(o.cpu().numpy(), w)
    meta = k.meta()
    assert meta["blockIdx.x"] >= 1 and meta["threadIdx.x"] in (128, 256)
    us = k.profile_host(list(ins) + [w.copy() for w in want], number=5, repeat=2)
    assert 0 < us < 1e5


# ------------------------------------------------------------------ matmul + epilogue
@pytest.mark.parametrize("m,k,n,tb,bias,relu", [
    (128, 64, 256, False, True, True), (128, 64, 256, True, True, True), (256, 512, 512, False, True, True),
    (100, 72, 136, False, True, True), (100, 72, 136, True, False, False), (1, 8, 8, False, True, True),
    (300, 1000, 520, False, True, False), (1024, 4096, 1024, False, True, True),
])
def test_matmul_epilogue(lib, m, k, n, tb, bias, relu):
    """The 2e-3 bound applies to the value BEFORE the final Cast: the bfloat16 rounding itself moves a
    value by up to 2^-8 relative, so two correct f32 accumulations that differ in summation order may
    land on neighbouring bfloat16 values.  Checked: (1) every output is the bfloat16 rounding of a value
    within 2e-3 of the oracle's f32 result; (2) outputs that differ from the rounded oracle do so by one
    bfloat16 step and are rare."""
    d = descs.matmul_bias_relu(m, k, n, transpose_b=tb, with_bias=bias, relu=relu)
    ins = make_inputs(d, 18, KINDS["matmul"])
    got, kern = run_host(d, ins)
    assert kern.check_device_error() == 0
    want = O.evaluate(d, ins)[0]
    # the same description without its final Cast: the f32 value the epilogue rounds
    import copy
    d32 = copy.deepcopy(d)
    d32["op_desc"].pop()
    last = d32["op_desc"][-1]["output_desc"][0]
    d32["output_desc"] = [dict(last)]
    ref32 = O.evaluate(d32, ins)[0].astype(np.float64)
    g = got[0].astype(np.float64)
    atol = 1e-3 * float(np.abs(ref32).max() + 1e-30)
    half_step = 2.0 ** -8
    assert np.all(np.abs(g - ref32) <= (2e-3 + half_step) * np.abs(ref32) + atol)
    gi = got[0].view(np.uint16).astype(np.int32)
    wi = want.view(np.uint16).astype(np.int32)
    diff = np.abs(gi - wi)
    assert diff.max() <= 1 or np.all(np.abs(g - want.astype(np.float64))[diff > 1] <= atol)
    assert (diff > 0).mean() < 2e-3
    # the f32-output variant of the same template meets the f32 bound directly
    k32, outs32 = FusedKernel(d32), None
    outs32 = k32.empty_outputs()
    k32.run_host(list(ins) + outs32)
    np.testing.assert_allclose(outs32[0], ref32, rtol=2e-3, atol=atol)


@pytest.mark.parametrize("name,desc,kinds", [
    ("gelu", descs.gelu_chain([16, 512, 4096]), KINDS["gelu"]),
    ("softmax", descs.masked_softmax(32, 512, 2048), KINDS["softmax"]),
    ("transpose", descs.transpose([16, 1024, 32, 128], [0, 2, 1, 3]), {}),
    ("layernorm", descs.layernorm(16384, 1024), KINDS["layernorm"]),
])
def test_chunked_host_entry_point_matches_device_launch(lib, name, desc, kinds):
    """Above 64 MB akgb_run_host cuts axis 0 into (at most 16) chunks and overlaps copies with kernels; the bytes it returns
    must be those of one launch over the whole tensors."""
    import torch
    ins = make_inputs(desc, 21, kinds)
    got, k = run_host(desc, ins)
    dev = [torch.from_numpy(a).cuda() for a in ins]
    outs = [torch.empty(t.nbytes, dtype=torch.uint8, device="cuda") for t in k.outputs]
    k.launch(dev + outs)
    torch.cuda.synchronize()
    for g, o in zip(got, outs):
        assert np.array_equal(np.ascontiguousarray(g).view(np.uint8).reshape(-1), o.cpu().numpy())
    # and a second call reuses the staging buffers
    got2 = k.empty_outputs()
    k.run_host(list(ins) + got2)
    for a, b in zip(got, got2):
        assert bits_equal(a, b)
