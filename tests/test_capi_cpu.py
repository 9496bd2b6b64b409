"""Host-side checks that need no GPU: the library loads, exports every symbol the header declares,
parses the reference's JSON schema, tags operator classes by the reference's rules and plans."""
import ctypes
import json
import re
from pathlib import Path

import pytest

from akg_b200 import FusedKernel, UnsupportedError, AkgbError, descs, _capi

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "akgb.h").read_text()
    declared = set(re.findall(r"\b(akgb_[a-z_0-9]+)\s*\(", header))
    assert declared, "no prototypes found in include/akgb.h"
    bound = {name for name, _, _ in _capi._SIGNATURES}
    assert declared <= bound, declared - bound
    for name in declared:
        assert getattr(lib, name) is not None


def test_version_and_error_text(lib):
    assert b"sm_100a" in lib.akgb_version()
    h = ctypes.c_void_p()
    st = lib.akgb_compile(b"{not json", 9, None, ctypes.byref(h))
    assert st == _capi.AKGB_INVALID_JSON
    assert lib.akgb_last_error()


CONFIGS = {
    "layernorm": (descs.layernorm(8192, 1024), "layernorm", 67182592),
    "gelu": (descs.gelu_chain([64, 512, 4096]), "broadcast", 1073750016),
    "softmax": (descs.masked_softmax(256, 2048, 2048), "softmax", 4303355904),
    "colsum": (descs.reduce_sum_axis0(65536, 4096), "reduce_y", 1073758208),
    "gmax": (descs.reduce_max_all(65536, 4096), "reduce_all", 1073741828),
    "transpose": (descs.transpose([32, 2048, 32, 128], [0, 2, 1, 3]), "transpose", 1073741824),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_benchmark_configs_plan_without_a_gpu(lib, name):
    desc, klass, nbytes = CONFIGS[name]
    k = FusedKernel(desc)
    assert k.op_class == klass
    assert k.bytes == nbytes  # the algorithmic bytes the roofline is computed from
    assert k.num_inputs == len(desc["input_desc"])
    assert [t.name for t in k.outputs] == [o["tensor_name"] for o in desc["output_desc"]]
    meta = k.meta()
    for key in ("kernelName", "blockIdx.x", "threadIdx.x", "is_dynamic", "sha256", "class", "bytes"):
        assert key in meta
    assert meta["kernelName"] == desc["op"] + "_kernel"
    assert len(meta["sha256"]) == 64
    k.close()


def test_sha256_matches_hashlib(lib):
    import hashlib
    text = json.dumps(descs.reduce_max_all(4, 8))
    k = FusedKernel(text)
    assert k.meta()["sha256"] == hashlib.sha256(text.encode()).hexdigest()


def test_schema_defaults_and_variants(lib):
    d = descs.reduce_sum_axis0(16, 8)
    # axis as a constant second operand instead of an attribute (TranslateToMindsporeDialect.cpp:1282-1300)
    op = d["op_desc"][0]
    op["attr"] = [{"name": "keep_dims", "data_type": "bool", "value": False}]
    op["input_desc"].append([{"data_type": "int64", "format": "DefaultFormat", "shape": [1],
                              "tensor_name": "axis_c", "value": [0]}])
    k = FusedKernel(d)
    assert k.op_class == "reduce_y"
    # negative axis wraps
    d2 = descs.reduce_sum_axis0(16, 8)
    d2["op_desc"][0]["attr"][0]["value"] = [-2]
    assert FusedKernel(d2).op_class == "reduce_y"
    # uint8 is read as int8 (:331-333): a transpose of bytes plans
    d3 = descs.transpose([4, 6], [1, 0], "uint8")
    assert FusedKernel(d3).tensors[0].dtype == "int8"


def test_commutative_spellings_match_and_reassociation_does_not(lib):
    d = descs.gelu_chain([2, 64])
    for op in d["op_desc"]:
        if op["name"] in ("Mul", "Add"):
            op["input_desc"].reverse()
    assert FusedKernel(d).op_class == "broadcast"
    # dropping the rounding step of t3*c0 changes results: the GELU template must not claim this graph;
    # it runs through the generic elementwise kernel, op by op, instead
    d = descs.gelu_chain([2, 64])
    del d["op_desc"][3]  # remove Mul(t3, c0) and rewire
    d["op_desc"][3]["input_desc"][1][0]["tensor_name"] = d["op_desc"][2]["output_desc"][0]["tensor_name"]
    k = FusedKernel(d)
    assert k.meta()["template"] == "ew_generic" and k.op_class == "broadcast"
    assert FusedKernel(descs.gelu_chain([2, 64])).meta()["template"] == "gelu_chain_f16"


def test_unsupported_and_malformed(lib):
    d = descs.unary("Erf", [8], "float32")  # not in the JSON factory: UnknownOp in the reference
    with pytest.raises(UnsupportedError):
        FusedKernel(d)
    d = descs.reduce_max_all(4, 4)
    del d["op_desc"][0]["output_desc"]
    with pytest.raises(AkgbError) as e:
        FusedKernel(d)
    assert e.value.status == _capi.AKGB_INVALID_JSON
    d = descs.matmul_bias_relu(128, 64, 128)
    d["op_desc"][0]["attr"][0]["value"] = True  # transpose_a is rejected like MindSporeToLinalg.cpp:1508-1510
    with pytest.raises(UnsupportedError):
        FusedKernel(d)


def test_leading_axis_sharding_plans(lib):
    k = FusedKernel(descs.gelu_chain([64, 512, 4096]), shard_rank=1, shard_world=4)
    by = {t.name: t for t in k.tensors}
    assert by["x"].shape == (16, 512, 4096) and by["x"].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert by["bias"].shape == (4096,) and by["bias"].shard_kind == _capi.SHARD_REPLICATED
    assert k.outputs[0].shape == (16, 512, 4096)
    k = FusedKernel(descs.reduce_sum_axis0(65536, 4096), shard_rank=0, shard_world=8)
    assert k.inputs[0].shape == (8192, 4096)
    assert k.outputs[0].shape == (4096,) and k.outputs[0].shard_kind == _capi.SHARD_PARTIAL_SUM
    k = FusedKernel(descs.reduce_max_all(65536, 4096), shard_rank=0, shard_world=2)
    assert k.outputs[0].shard_kind == _capi.SHARD_PARTIAL_MAX
    k = FusedKernel(descs.masked_softmax(256, 2048, 2048), shard_rank=3, shard_world=8)
    assert k.inputs[0].shape == (32, 2048, 2048) and k.inputs[1].shard_kind == _capi.SHARD_REPLICATED
    k = FusedKernel(descs.layernorm(8192, 1024), shard_rank=0, shard_world=8)
    assert [t.shape for t in k.outputs] == [(1024, 1024), (1024,), (1024,)]
    k = FusedKernel(descs.transpose([32, 2048, 32, 128], [0, 2, 1, 3]), shard_rank=0, shard_world=8)
    assert k.outputs[0].shape == (4, 32, 2048, 128)
    with pytest.raises(UnsupportedError):  # the split axis moves
        FusedKernel(descs.transpose([8, 16], [1, 0]), shard_rank=0, shard_world=2)
    with pytest.raises(UnsupportedError):  # 7 rows over 2 ranks
        FusedKernel(descs.layernorm(7, 100), shard_rank=0, shard_world=2)


def test_mlir_driver_writes_kernel_meta_like_the_reference(lib, tmp_path, monkeypatch):
    from akg_b200 import MlirDriver
    from akg_b200.driver import get_kernel_meta_path
    d = descs.reduce_sum_axis0(64, 32)
    info = tmp_path / (d["op"] + ".info")
    info.write_text(json.dumps(d))
    monkeypatch.setenv("KERNEL_META_DIR", "akg_meta")
    monkeypatch.setenv("MS_COMPILER_CACHE_PATH", str(tmp_path))
    assert get_kernel_meta_path() == str(tmp_path / "akg_meta")
    drv = MlirDriver(d["op"], str(info), backend="gpu")
    drv.compile()
    meta = json.loads((tmp_path / "akg_meta" / (d["op"] + ".json")).read_text())
    assert meta["kernelName"] == d["op"] + "_kernel" and meta["is_dynamic"] is False and len(meta["sha256"]) == 64
    with pytest.raises(RuntimeError):
        MlirDriver(d["op"], str(info), backend="ascend")


def test_generated_kernels_export_a_loadable_binary(lib, tmp_path):
    """<kernel>.cubin + <kernel>.json for regions that run as one generated kernel (the pair the reference leaves in
    the kernel meta directory, mlir_driver.py:776-815); template regions have no stand-alone binary.  Compiling needs
    the run-time compiler but no device."""
    import hashlib
    from akg_b200.descs import _Builder
    b = _Builder("Fused_Add_Mul_export_1")
    f = "float32"
    x, y = b.input("x", [64, 256], f), b.input("y", [256], f)
    b.output(b.emit("Mul", [b.emit("Add", [x, y], [64, 256], f), b.const(0.5, f)], [64, 256], f))
    d = b.build()
    for desc in (d, descs.rmsnorm(128, 512)):
        k = FusedKernel(desc)
        try:
            k.export(tmp_path)
        except UnsupportedError as e:
            if "could not be generated or compiled" in str(e):
                pytest.skip("no run-time compiler on this host")
            raise
        image = (tmp_path / (desc["op"] + ".cubin")).read_bytes()
        meta = json.loads((tmp_path / (desc["op"] + ".json")).read_text())
        assert image[:4] == b"\x7fELF" and meta["sha256"] == hashlib.sha256(image).hexdigest()
        assert meta["kernelName"] == desc["op"] + "_kernel" and meta["kernelName"].encode() in image
        assert meta["blockIdx.x"] >= 1 and meta["threadIdx.x"] >= 32 and meta["is_dynamic"] is False
        assert meta["binary"] == desc["op"] + ".cubin" and meta["pointer_alignment"] in (1, 16)
    with pytest.raises(UnsupportedError, match="no stand-alone binary"):
        FusedKernel(descs.layernorm(64, 1024)).export(tmp_path)
    with pytest.raises(UnsupportedError):
        FusedKernel(descs.reduce_sum_axis0(4096, 512)).export(tmp_path)


def test_generic_plan_splits_at_shape_changes(lib):
    """Elementwise groups, reductions and data-movement ops become separate launches; Reshape is a view."""
    from akg_b200.descs import _Builder, _attr, _reduce_attr
    b = _Builder("Fused_Generic_30")
    f = "float32"
    x = b.input("x", [32, 64], f)
    t = b.emit("Mul", [x, x], [32, 64], f)
    r = b.emit("ReduceSum", [t], [32, 1], f, _reduce_attr([1], True))
    u = b.emit("Sub", [x, r], [32, 64], f)
    v = b.emit("Reshape", [u], [2048], f, [_attr("shape", "listInt", [2048])])
    b.output(v)
    k = FusedKernel(b.build(), flags=1)  # run-time compilation off: the separate launches
    assert k.launch_count == 3 and k.workspace_size > 0 and k.op_class == "reduce_x"
    assert k.meta()["template"] == "ew_generic"
    # with it on, the ops in front of the Reshape are a row region of their own and write through the view
    k = FusedKernel(b.build())
    assert k.launch_count == 1 and k.workspace_size == 0 and k.meta()["template"] == "akgb_row_jit"


def _dynamic_sub_mul_cast():
    """The shape of region the reference's gpu_dynamic_shape test holds: Sub with a broadcast operand, Mul, Cast,
    extents [32,16,-1,-1] and [32,16,-1,1]."""
    from akg_b200.descs import _Builder, _attr
    b = _Builder("Fused_Sub_Mul_Cast_dyn_40")
    f = "float32"
    x = b.input("input_0", [32, 16, -1, -1], f)
    m = b.input("input_1", [32, 16, -1, 1], f)
    y = b.input("input_2", [32, 16, -1, -1], f)
    t = b.emit("Sub", [x, m], [32, 16, -1, -1], f)
    t = b.emit("Mul", [y, t], [32, 16, -1, -1], f)
    b.output(b.emit("Cast", [t], [32, 16, -1, -1], "float16", [_attr("dst_type", "str", "float16")]))
    return b.build()


def test_dynamic_shape_region_plans_per_extent_set(lib):
    d = _dynamic_sub_mul_cast()
    k = FusedKernel(d)
    assert k.is_dynamic and k.meta()["is_dynamic"] is True
    assert k.tensors[0].shape == (32, 16, -1, -1) and k.tensors[0].nbytes == -1
    shapes = [[32, 16, 40, 24], [32, 16, 40, 1], [32, 16, 40, 24], [32, 16, 40, 24]]
    assert k.bind_shapes(shapes) == 0            # one elementwise group: no workspace
    assert k.bind_shapes(shapes) == 0            # cached
    with pytest.raises(AkgbError):               # a static extent contradicted
        k.bind_shapes([[31, 16, 40, 24], [32, 16, 40, 1], [32, 16, 40, 24], [32, 16, 40, 24]])
    with pytest.raises(AkgbError):               # operands that do not broadcast
        k.bind_shapes([[32, 16, 40, 24], [32, 16, 39, 1], [32, 16, 40, 24], [32, 16, 40, 24]])
    with pytest.raises(AkgbError):               # wrong number of extents
        k.bind_shapes([[32, 16, 40, 24]])
    # a dynamic softmax: the row templates are chosen once the extents are known
    s = descs.masked_softmax(-1, -1, 256)
    ks = FusedKernel(s)
    assert ks.is_dynamic
    ks.bind_shapes([[4, 8, 256], [8, 256], [4, 8, 256]])


def test_fake_output_takes_shape_and_type_of_the_first_operand(lib):
    """An op marked fake_output declares a placeholder result; its real shape and type are those of its first operand
    (the reference's parser substitutes them)."""
    from akg_b200 import FusedKernel
    from akg_b200.descs import _Builder, _attr
    b = _Builder("Fused_Assign_fake_1")
    dst = b.input("dst", [6, 10], "float32")
    val = b.input("val", [6, 10], "float32")
    t = b.emit("Add", [val, b.const(1.0, "float32")], [6, 10], "float32")
    a = b.emit("Assign", [dst, t], [1], "float16", [_attr("fake_output", "bool", True)])  # placeholder shape / type
    b.output(b.emit("Mul", [a, b.const(2.0, "float32")], [6, 10], "float32"))
    k = FusedKernel(b.build())
    assert k.inputs[0].written_in_place and k.outputs[0].shape == (6, 10) and k.outputs[0].dtype == "float32"


def test_planning_of_generated_kernels_needs_no_device(lib):
    """Which plan a region gets is decided at compile time on the host: reduce-X regions become one row program,
    elementwise chains ending in a reduction over leading / all axes a column / row program plus the fold of the
    partials, and with run-time compilation off the same regions are planned as separate launches."""
    from akg_b200 import FusedKernel, descs
    from akg_b200.descs import _Builder, _attr, _reduce_attr
    k = FusedKernel(descs.rmsnorm(300, 1024))
    assert k.meta()["template"] == "akgb_row_jit" and k.launch_count == 1
    src = k.jit_source()
    assert "akgb_row_jit" in src and "constexpr int C = 1024, T = 32" in src and "row_reduce<0>" in src
    assert FusedKernel(descs.rmsnorm(300, 1024), flags=1).launch_count > 1
    # threads per row follow the row length: several warps for long rows, a few lanes for short ones
    assert "T = 128" in FusedKernel(descs.rmsnorm(64, 4096)).jit_source()
    assert "T = 8," in FusedKernel(descs.rmsnorm(64, 64)).jit_source()
    assert "VW = 1" in FusedKernel(descs.rmsnorm(64, 100)).jit_source(False)
    # rows too long for registers: still one launch, a 512-thread block per row that walks the row once per reduction
    kl = FusedKernel(descs.rmsnorm(64, 40000))
    assert kl.launch_count == 1 and "T = 512" in kl.jit_source() and "c += (i64)T * VW" in kl.jit_source()
    kc = FusedKernel(descs.mul_reduce_sum(4096, 512, [0]))
    assert kc.meta()["template"] == "akgb_col_jit" and "akgb_col_jit" in kc.jit_source()
    ka = FusedKernel(descs.mul_reduce_sum(4096, 512, [0, 1]))
    assert ka.meta()["template"] == "akgb_row_jit" and "C = 4096" in ka.jit_source() and ka.launch_count == 3
    # small tensors are not worth a generated reduction kernel
    assert FusedKernel(descs.mul_reduce_sum(64, 64, [0])).meta()["template"] != "akgb_col_jit"


def test_batch_norm_training_is_planned_without_full_size_intermediates(lib):
    """Cut at the reductions: the centred squares are folded into the variance pass, the centred values are computed
    again by the scale-and-shift launch, so only per-channel values live in the workspace."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from test_gpu_generic import _batch_norm_training
    from akg_b200 import FusedKernel
    k = FusedKernel(_batch_norm_training([64, 256, 56, 56]))
    meta = k.meta()
    assert meta["steps"].count("akgb_row_jit") == 1 and meta["steps"][-1] == "ew_generic"
    assert meta["workspace"] < (1 << 20) and len(meta["steps"]) == 7
    assert FusedKernel(_batch_norm_training([64, 256, 56, 56]), flags=1).meta()["workspace"] > (100 << 20)


def test_layer_norm_backward_is_one_row_kernel_with_column_sums(lib):
    from akg_b200 import FusedKernel, descs
    k = FusedKernel(descs.layer_norm_backward(16384, 4096))
    assert k.meta()["steps"] == ["akgb_row_jit", "reduce_col_f32", "reduce_col_f32"]
    src = k.jit_source()
    assert "rb += gridDim.x" in src and "cs1[k][j] = __fadd_rn" in src
    # ops behind the sums (a cast to the parameters' type) are split off and run after the partial sums are folded
    kb = FusedKernel(descs.layer_norm_backward(16384, 4096, grads_dtype="bfloat16"))
    assert kb.meta()["steps"] == ["akgb_row_jit", "reduce_col_f32", "reduce_col_f32", "ew_generic"]
    # rows too long for registers keep the separate column reductions
    assert "akgb_row_jit" in FusedKernel(descs.layer_norm_backward(64, 40000)).meta()["steps"]
    assert "rb += gridDim.x" not in FusedKernel(descs.layer_norm_backward(64, 40000)).jit_source()


def test_planning_of_the_wider_op_surface(lib):
    from akg_b200 import FusedKernel, descs
    from akg_b200.descs import _Builder, _attr, _reduce_attr
    f = "float32"
    # matmul epilogue inside a larger region: bias, ReLU and the narrowing cast ride in the matmul launch
    b = _Builder("Fused_MatMul_Add_Max_Cast_Neg_1")
    a, w, bias = b.input("a", [256, 128], "bfloat16"), b.input("w", [128, 192], "bfloat16"), b.input("bias", [192], f)
    c = b.emit("MatMul", [a, w], [256, 192], f, [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)])
    c = b.emit("Maximum", [b.emit("Add", [c, bias], [256, 192], f), b.const(0.0, f)], [256, 192], f)
    c = b.emit("Cast", [c], [256, 192], "bfloat16", [_attr("dst_type", "str", "bfloat16")])
    b.output(b.emit("Neg", [c], [256, 192], "bfloat16"))
    assert FusedKernel(b.build()).launch_count == 2
    # float32 and float16 operands, batches in one launch
    assert FusedKernel(descs.matmul_bias_relu(256, 64, 128, dtype="float32")).meta()["template"] == "sgemm_f32"
    assert FusedKernel(descs.matmul_bias_relu(256, 64, 128, dtype="float16")).launch_count == 1
    b = _Builder("Fused_BatchMatMul_2")
    a, w = b.input("a", [12, 128, 64], "float16"), b.input("w", [12, 64, 128], "float16")
    b.output(b.emit("BatchMatMul", [a, w], [12, 128, 128], f,
                    [_attr("transpose_a", "bool", False), _attr("transpose_b", "bool", False)]))
    assert FusedKernel(b.build()).launch_count == 1
    # Pad, Split, ArgMax, Gather, UnsortedSegmentSum are accepted
    b = _Builder("Fused_Pad_Split_ArgMax_3")
    x = b.input("x", [6, 10], f)
    p = b.emit("Pad", [x], [8, 12], f, [_attr("head", "listInt", [1, 0]), _attr("tail", "listInt", [1, 2]),
                                        _attr("pad_val", "float", 0.0)])
    halves = b.emit_multi("Split", [p], [([8, 6], f), ([8, 6], f)], [_attr("axis", "int", 1)])
    b.output(b.emit("ArgMax", [halves[0]], [8], "int32", _reduce_attr([1], False)))
    b.output(halves[1])
    k = FusedKernel(b.build())
    assert [o.dtype for o in k.outputs] == ["int32", "float32"] and k.launch_count >= 3
    b = _Builder("Fused_Gather_SegSum_4")
    table, idx = b.input("table", [100, 16], f), b.input("idx", [40], "int32")
    g = b.emit("Gather", [table, idx], [40, 16], f, [_attr("axis", "int", 0), _attr("batch_dims", "int", 0)])
    b.output(b.emit("UnsortedSegmentSum", [g, idx], [7, 16], f, [_attr("num_segments", "int", 7)]))
    assert FusedKernel(b.build()).launch_count == 2


def test_batch_matmul_shards_on_the_batch_of_both_operands(lib):
    """The split axis of a BatchMatMul is the batch of its LEFT operand; a right operand that carries the same batch is
    split with it, a 2-D shared one stays whole -- whichever of the two inputs is larger."""
    # batch == world, right operand larger than the left one
    k = FusedKernel(descs.batch_matmul(2, 64, 64, 256), shard_rank=1, shard_world=2)
    by = {t.name: t for t in k.tensors}
    assert by["a"].shape == (1, 64, 64) and by["a"].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert by["b"].shape == (1, 64, 256) and by["b"].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert k.outputs[0].shape == (1, 64, 256) and k.outputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert k.flops == 2 * 64 * 64 * 256  # one batch entry per rank
    # batch > world
    k = FusedKernel(descs.batch_matmul(8, 128, 64, 256, transpose_b=True), shard_rank=0, shard_world=4)
    assert [t.shape for t in k.tensors] == [(2, 128, 64), (2, 256, 64), (2, 128, 256)]
    assert all(t.shard_kind == _capi.SHARD_SPLIT_AXIS0 for t in k.tensors) and k.flops == 2 * 2 * 128 * 64 * 256
    # one shared 2-D right operand, even when its leading extent equals the batch
    k = FusedKernel(descs.batch_matmul(64, 128, 64, 256, shared_b=True), shard_rank=0, shard_world=4)
    by = {t.name: t for t in k.tensors}
    assert by["a"].shape == (16, 128, 64) and by["b"].shape == (64, 256) and by["b"].shard_kind == _capi.SHARD_REPLICATED
    # a square MatMul: the weight has as many rows as the left operand and must not be cut
    k = FusedKernel(descs.matmul_bias_relu(256, 256, 256), shard_rank=1, shard_world=2)
    by = {t.name: t for t in k.tensors}
    assert by["a"].shape == (128, 256) and by["b"].shape == (256, 256) and by["b"].shard_kind == _capi.SHARD_REPLICATED
    assert k.outputs[0].shape == (128, 256)
    with pytest.raises(UnsupportedError):  # the batch does not divide
        FusedKernel(descs.batch_matmul(3, 64, 64, 256), shard_rank=0, shard_world=2)


def test_reductions_over_the_split_axis_that_feed_later_ops_run_as_stages(lib):
    """Batch-norm statistics over a batch that is split across ranks: the region is cut at the reductions over the
    split axis; the caller sees one kernel whose per-channel results arrive completed (the exchange runs between the
    stages inside akgb_launch_sharded)."""
    k = FusedKernel(descs.batch_norm_training([8, 16, 4, 4]), shard_rank=1, shard_world=2)
    assert k.op_class == "sharded_stages" and k.workspace_size > 0
    by = {t.name: t for t in k.tensors}
    assert by["x"].shape == (4, 16, 4, 4) and by["x"].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert by["gamma"].shard_kind == _capi.SHARD_REPLICATED
    assert k.outputs[0].shape == (4, 16, 4, 4) and k.outputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert all(o.shape == (1, 16, 1, 1) and o.shard_kind == _capi.SHARD_REPLICATED for o in k.outputs[1:])
    # three stages (sum; centred squares; normalisation), each at least one launch
    assert k.launch_count >= 3
    kb = FusedKernel(descs.batch_norm_backward([8, 16, 4, 4]), shard_rank=0, shard_world=4)
    assert kb.op_class == "sharded_stages" and kb.inputs[0].shape == (2, 16, 4, 4)
    # the same descriptions unsplit are ordinary kernels
    assert FusedKernel(descs.batch_norm_training([8, 16, 4, 4])).op_class != "sharded_stages"
    # statistics per column over the split rows; a softmax over the split axis (max, then sum: two exchanges); a scale
    # taken from the whole tensor, which is also a result (it lives in the caller's output, not in the workspace)
    for d, stages in ((descs.normalise_over_axis0(4096, 512), 3), (descs.softmax_over_axis0(4096, 512), 3),
                      (descs.scale_by_global_max(4096, 512), 2)):
        ks = FusedKernel(d, shard_rank=1, shard_world=4)
        assert ks.op_class == "sharded_stages" and ks.inputs[0].shape == (1024, 512)
        assert sum(1 for s_ in ks.meta()["steps"] if s_.startswith("| ")) == stages - 1
        assert ks.outputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert FusedKernel(descs.scale_by_global_max(4096, 512), shard_rank=0, shard_world=4).outputs[1].shard_kind == _capi.SHARD_REPLICATED
    # a stage is planned like a region of its own: the centred squares and their column sum are ONE generated kernel
    # (no full-size value crosses memory), and the small per-channel ops of a stage come before its full-size ops
    kn = FusedKernel(descs.normalise_over_axis0(8192, 512), shard_rank=0, shard_world=2)
    assert "| akgb_col_jit" in kn.meta()["steps"] and kn.workspace_size < (1 << 20)
    kt = FusedKernel(descs.batch_norm_training([64, 256, 56, 56]), shard_rank=0, shard_world=2)
    assert kt.meta()["steps"][-2:] == ["| ew_generic", "ew_generic"] and kt.launch_count == 7


def test_symbolic_shapes_bind_consistently(lib):
    """symbolic_shape / symbol_calc_expr (TranslateToMindsporeDialect.cpp:55-75): a symbol names one extent; the
    inputs define the symbols, the expressions derive further ones, every argument dim that carries a symbol must
    agree when the launch-time extents are bound."""
    from akg_b200.descs import _Builder, _attr
    b = _Builder("Fused_Concat_Mul_sym_5")
    f = "float32"
    x, y = b.input("x", [-1, 8], f), b.input("y", [-1, 8], f)
    x["symbolic_shape"], y["symbolic_shape"] = ["s0", "8"], ["s1", 8]
    node = {"name": "Concat", "attr": [_attr("axis", "int", 0)], "impl_path": "",
            "input_desc": [[dict(x), dict(y)]],
            "output_desc": [{"data_type": f, "format": "DefaultFormat", "shape": [-1, 8], "tensor_name": "cat"}]}
    b.ops.append(node)
    out = b.emit("Mul", [dict(node["output_desc"][0]), b.const(2.0, f)], [-1, 8], f)
    out["symbolic_shape"] = ["s2", "8"]
    b.output(out)
    d = b.build()
    d["symbol_calc_expr"] = {"s2": "s0 + s1"}
    k = FusedKernel(d)
    assert k.is_dynamic
    k.bind_shapes([[5, 8], [7, 8], [12, 8]])
    with pytest.raises(AkgbError, match="symbol 's2'"):
        k.bind_shapes([[5, 8], [7, 8], [13, 8]])  # the result must have s0 + s1 rows
    # one symbol on two inputs: both must be bound to the same extent
    b = _Builder("Fused_Add_sym_6")
    p_, q_ = b.input("p", [-1, 16], f), b.input("q", [-1, 16], f)
    p_["symbolic_shape"], q_["symbolic_shape"] = ["n", "16"], ["n", "16"]
    b.output(b.emit("Add", [p_, q_], [-1, 16], f))
    k = FusedKernel(b.build())
    k.bind_shapes([[9, 16], [9, 16], [9, 16]])
    with pytest.raises(AkgbError, match="symbol 'n'"):
        k.bind_shapes([[9, 16], [1, 16], [9, 16]])  # would broadcast, but the description says the extents are equal
    # products, quotients and parentheses; a numeric entry must match the extent
    b = _Builder("Fused_Reshape_sym_7")
    r_ = b.input("r", [-1, -1, 4], f)
    r_["symbolic_shape"] = ["a", "b", "4"]
    o_ = b.emit("Reshape", [r_], [-1, 2], f, [_attr("shape", "listInt", [-1, 2])])
    o_["symbolic_shape"] = ["m", "2"]
    b.output(o_)
    d = b.build()
    d["symbol_calc_expr"] = {"m": "(a * b * 4) / 2"}
    k = FusedKernel(d)
    k.bind_shapes([[3, 5, 4], [30, 2]])
    with pytest.raises(AkgbError):
        k.bind_shapes([[3, 5, 4], [15, 4]])


def test_generated_kernels_shard_like_the_templates(lib):
    from akg_b200 import FusedKernel, _capi, descs
    k = FusedKernel(descs.rmsnorm(4096, 1024), shard_rank=1, shard_world=4)
    assert k.meta()["template"] == "akgb_row_jit"
    assert k.inputs[0].shape == (1024, 1024) and k.inputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
    assert k.inputs[1].shard_kind == _capi.SHARD_REPLICATED and k.outputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
    kc = FusedKernel(descs.mul_reduce_sum(8192, 512, [0]), shard_rank=0, shard_world=2)
    assert kc.meta()["template"] == "akgb_col_jit" and kc.inputs[0].shape == (4096, 512)
    assert kc.outputs[0].shard_kind == _capi.SHARD_PARTIAL_SUM
    # LayerNorm backward over a slice of the rows: dx stays split, the weight and bias gradients are partial sums
    kl = FusedKernel(descs.layer_norm_backward(16384, 4096), shard_rank=1, shard_world=4)
    assert kl.meta()["steps"] == ["akgb_row_jit", "reduce_col_f32", "reduce_col_f32"] and kl.inputs[0].shape == (4096, 4096)
    assert [t.shard_kind for t in kl.outputs] == [_capi.SHARD_SPLIT_AXIS0, _capi.SHARD_PARTIAL_SUM, _capi.SHARD_PARTIAL_SUM]


def test_float64_regions_plan_as_generated_kernels_only(lib):
    """float64 elementwise chains are one generated kernel whose registers are doubles; reductions or row programs over
    float64 are refused (no float64 reduction template)."""
    from akg_b200 import FusedKernel, UnsupportedError
    from akg_b200.descs import _Builder, _attr, _reduce_attr
    f = "float64"
    b = _Builder("Fused_F64_plan_1")
    x, y = b.input("x", [64, 256], f), b.input("y", [256], f)
    b.output(b.emit("Mul", [b.emit("Add", [x, y], [64, 256], f), b.const(0.1, f)], [64, 256], f))
    d = b.build()
    k = FusedKernel(d)
    assert k.meta()["template"] == "ew_generic" and k.launch_count == 1
    src = k.jit_source()
    assert "double a0[U][E]" in src and "__dadd_rn" in src and "__longlong_as_double(0x" in src
    b = _Builder("Fused_F64_reduce_2")
    x = b.input("x", [64, 256], f)
    b.output(b.emit("ReduceSum", [x], [64, 1], f, _reduce_attr([1], True)))
    with pytest.raises(UnsupportedError):
        FusedKernel(b.build())


def test_random_regions_with_reductions_over_the_split_axis_plan_as_stages(lib):
    """Random chains with one to three reductions over axis 0 (or over all elements) that flow back into the chain:
    unsplit they are ordinary kernels, split over 2 / 4 / 8 ranks they plan as stages with at least one exchange, and
    the kernel the caller sees keeps the region's arguments.  (The same regions run against the oracle on 2+ GPUs in
    tests/comm_worker.py.)"""
    import importlib.util
    import os
    from akg_b200 import FusedKernel, _capi
    spec = importlib.util.spec_from_file_location("comm_worker", os.path.join(os.path.dirname(__file__), "comm_worker.py"))
    cw = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cw)
    for seed in range(60):
        d = cw.random_staged_region(seed, 64)
        assert FusedKernel(d).op_class != "sharded_stages"
        for world in (2, 4, 8):
            k = FusedKernel(d, shard_rank=world - 1, shard_world=world)
            assert k.op_class == "sharded_stages", seed
            assert sum(1 for s in k.meta()["steps"] if s.startswith("| ")) >= 1
            assert k.inputs[0].shape[0] == 64 // world and k.inputs[0].shard_kind == _capi.SHARD_SPLIT_AXIS0
            assert len(k.outputs) == len(d["output_desc"])
            assert k.outputs[-1].shape[0] == 64 // world and k.outputs[-1].shard_kind == _capi.SHARD_SPLIT_AXIS0


def test_descriptions_that_cannot_be_real_are_refused_not_planned(lib):
    """Extents whose product would overflow the 64-bit element counts used throughout, and malformed texts: a status
    and a message, never a crash (the reference exits the process on such input, code_template.py:47-56)."""
    import copy
    from akg_b200 import AkgbError, FusedKernel, UnsupportedError, descs
    d = copy.deepcopy(descs.layernorm(64, 256))
    d["input_desc"][0][0]["shape"] = [2 ** 40, 2 ** 30]
    with pytest.raises(UnsupportedError):
        FusedKernel(d)
    for text in (b"", b"{", b"[]", b"null", b'{"op":1}', b"\xff\xfe\x00", b'{"a":' * 5000):
        with pytest.raises(AkgbError):
            FusedKernel(text)
