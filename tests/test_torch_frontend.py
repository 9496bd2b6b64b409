"""The PyTorch front door: tracing, clustering and the descriptions it emits.

CPU tests run every cluster through the NumPy restatement (the checker) in place of the CUDA library and compare the
whole program with torch eager; GPU tests run the clusters on the device through the library.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from akg_b200 import torch_frontend as TF  # noqa: E402
from oracle import akg_oracle as O  # noqa: E402

_NP = {torch.float32: np.float32, torch.float16: np.float16, torch.int32: np.int32, torch.bool: np.bool_,
       torch.int8: np.int8}


def oracle_executor(sub, *tensors):
    ins = [t.detach().cpu().contiguous().numpy() for t in tensors]
    ins = [a.reshape(d[0]["shape"]) for a, d in zip(ins, sub.desc["input_desc"])]
    outs = O.evaluate(sub.desc, ins)
    return tuple(torch.from_numpy(np.ascontiguousarray(o)).reshape(shape).to(tensors[0].device)
                 for o, (shape, _) in zip(outs, sub.out_meta))


def gelu_bias(x, bias, y):
    return torch.nn.functional.gelu(x + bias, approximate="tanh") * y


def layer_norm(x, g, b):
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), g, b, 1e-5)


def masked_softmax(s, mask):
    return torch.softmax(s * 0.125 + mask, dim=-1)


def mlp(x, w1, b1, w2):
    h = torch.relu(x @ w1 + b1)
    return (h @ w2).sum(dim=0)


def mixed(x, idx, y):
    # an op the library does not take (index_select) between two fusable regions
    a = torch.tanh(x) * 2.0
    g = torch.index_select(a, 0, idx)
    return torch.where(g > 0.5, g, y) - 1.0, a.amax(dim=1)


def transformer_block(x, ln1w, ln1b, wqkv, bqkv, wo, bo, ln2w, ln2b, w1, b1, w2, b2):
    """Pre-norm attention + MLP block, 4 heads."""
    import math
    bsz, seq, dim = x.shape
    heads = 4
    h = torch.nn.functional.layer_norm(x, (dim,), ln1w, ln1b, 1e-5)
    q, k, v = torch.nn.functional.linear(h, wqkv, bqkv).split(dim, dim=-1)
    q, k, v = (t.reshape(bsz, seq, heads, dim // heads).permute(0, 2, 1, 3) for t in (q, k, v))
    att = torch.softmax((q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(dim // heads)), dim=-1)
    o = (att @ v).permute(0, 2, 1, 3).reshape(bsz, seq, dim)
    x = x + torch.nn.functional.linear(o, wo, bo)
    h = torch.nn.functional.layer_norm(x, (dim,), ln2w, ln2b, 1e-5)
    m = torch.nn.functional.gelu(torch.nn.functional.linear(h, w1, b1), approximate="tanh")
    return x + torch.nn.functional.linear(m, w2, b2)


def transformer_inputs(dtype, gen, bsz=2, seq=128, dim=256):
    shapes = [(bsz, seq, dim), (dim,), (dim,), (3 * dim, dim), (3 * dim,), (dim, dim), (dim,), (dim,), (dim,),
              (4 * dim, dim), (4 * dim,), (dim, 4 * dim), (dim,)]
    ins = []
    for i, s in enumerate(shapes):
        t = torch.randn(s, generator=gen) * (1.0 if i == 0 else 0.05)
        if i in (1, 7):
            t = t + 1.0
        ins.append(t.to(dtype))
    return ins


def _g(seed=0):
    return torch.Generator().manual_seed(seed)


def _pull(fn, primals, dy):
    out, pull = torch.func.vjp(fn, *primals)
    return pull(dy)


MORE = {
    "softmax_dim1": (lambda x: torch.softmax(x, dim=1), lambda g: [torch.randn(4, 16, 32, generator=g)]),
    "center_over_axes_0_2": (lambda x: (x - x.mean(dim=(0, 2), keepdim=True)) * 2,
                             lambda g: [torch.randn(4, 16, 32, generator=g)]),
    "var_unbiased": (lambda x: x.var(dim=-1), lambda g: [torch.randn(8, 64, generator=g)]),
    "std_keepdim": (lambda x: x / (x.std(dim=-1, keepdim=True) + 1e-3), lambda g: [torch.randn(8, 64, generator=g)]),
    "silu_mul": (lambda x, y: torch.nn.functional.silu(x) * y,
                 lambda g: [torch.randn(8, 64, generator=g), torch.randn(8, 64, generator=g)]),
    "logsumexp": (lambda x: torch.logsumexp(x, dim=-1), lambda g: [torch.randn(8, 64, generator=g)]),
    "cat_slice": (lambda x, y: torch.cat([x, y], dim=1)[:, 3:50:2] + 1,
                  lambda g: [torch.randn(8, 30, generator=g), torch.randn(8, 40, generator=g)]),
    "int_ops": (lambda i: (i * 3 + 1).float() / 2, lambda g: [torch.randint(-5, 5, (8, 16), generator=g, dtype=torch.int32)]),
    "bmm_transposed": (lambda a, b: torch.relu(a @ b.transpose(1, 2)),
                       lambda g: [torch.randn(3, 16, 24, generator=g), torch.randn(3, 8, 24, generator=g)]),
    "l2_normalise": (lambda x: x / x.norm(dim=-1, keepdim=True), lambda g: [torch.randn(8, 64, generator=g)]),
    "rms_norm": (lambda x, w: torch.nn.functional.rms_norm(x, (64,), w, 1e-6),
                 lambda g: [torch.randn(8, 64, generator=g), torch.rand(64, generator=g) + 0.5]),
    "log_softmax": (lambda x: torch.nn.functional.log_softmax(x, dim=-1), lambda g: [torch.randn(8, 64, generator=g)]),
    "instance_norm": (lambda x, w, b: torch.nn.functional.instance_norm(x, weight=w, bias=b),
                      lambda g: [torch.randn(2, 8, 12, 16, generator=g), torch.rand(8, generator=g) + 0.5,
                                 torch.randn(8, generator=g)]),
    "batch_norm_training": (lambda x, w, b: torch.nn.functional.batch_norm(x, None, None, w, b, training=True),
                            lambda g: [torch.randn(4, 8, 12, 16, generator=g), torch.rand(8, generator=g) + 0.5,
                                       torch.randn(8, generator=g)]),
    "group_norm": (lambda x, w, b: torch.nn.functional.group_norm(x, 4, w, b),
                   lambda g: [torch.randn(2, 8, 12, 16, generator=g), torch.rand(8, generator=g) + 0.5,
                              torch.randn(8, generator=g)]),
    # forward and backward in one trace: the backward ops of normalisations and softmaxes are decomposed too
    "layer_norm_backward": (lambda x, w, b, dy: _pull(lambda x, w, b: torch.nn.functional.layer_norm(x, (64,), w, b), (x, w, b), dy),
                            lambda g: [torch.randn(24, 64, generator=g), torch.rand(64, generator=g) + 0.5,
                                       torch.randn(64, generator=g), torch.randn(24, 64, generator=g)]),
    "rms_norm_backward": (lambda x, w, dy: _pull(lambda x, w: torch.nn.functional.rms_norm(x, (64,), w, 1e-6), (x, w), dy),
                          lambda g: [torch.randn(24, 64, generator=g), torch.rand(64, generator=g) + 0.5,
                                     torch.randn(24, 64, generator=g)]),
    "softmax_backward": (lambda x, dy: _pull(lambda x: torch.softmax(x, -1), (x,), dy),
                         lambda g: [torch.randn(24, 64, generator=g), torch.randn(24, 64, generator=g)]),
    "log_softmax_backward": (lambda x, dy: _pull(lambda x: torch.log_softmax(x, -1), (x,), dy),
                             lambda g: [torch.randn(24, 64, generator=g), torch.randn(24, 64, generator=g)]),
    "batch_norm_backward": (lambda x, w, b, dy: _pull(lambda x, w, b: torch.nn.functional.batch_norm(x, None, None, w, b, training=True),
                                                      (x, w, b), dy),
                            lambda g: [torch.randn(4, 8, 12, 16, generator=g), torch.rand(8, generator=g) + 0.5,
                                       torch.randn(8, generator=g), torch.randn(4, 8, 12, 16, generator=g)]),
    "gelu_erf_stays_with_torch": (lambda x: torch.nn.functional.gelu(x) * 2, lambda g: [torch.randn(8, 64, generator=g)]),
}


CASES = {
    "gelu_bias": (gelu_bias, lambda g: [torch.randn(4, 64, 128, generator=g), torch.randn(128, generator=g) * 0.02,
                                       torch.randn(4, 64, 128, generator=g)], 1e-5),
    "layer_norm": (layer_norm, lambda g: [torch.randn(64, 256, generator=g), torch.rand(256, generator=g) + 0.5,
                                         torch.randn(256, generator=g) * 0.1], 1e-5),
    "masked_softmax": (masked_softmax, lambda g: [torch.randn(3, 32, 32, generator=g),
                                                 torch.triu(torch.full((32, 32), float("-inf")), 1)], 1e-6),
    "mlp": (mlp, lambda g: [torch.randn(48, 64, generator=g), torch.randn(64, 96, generator=g) * 0.1,
                            torch.randn(96, generator=g), torch.randn(96, 32, generator=g) * 0.1], 1e-4),
    "mixed": (mixed, lambda g: [torch.randn(16, 40, generator=g), torch.tensor([3, 1, 7, 7, 0, 15]),
                                torch.randn(6, 40, generator=g)], 1e-6),
}


def _close(got, want, tol):
    got = got if isinstance(got, (tuple, list)) else [got]
    want = want if isinstance(want, (tuple, list)) else [want]
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert a.shape == b.shape and a.dtype == b.dtype
        torch.testing.assert_close(a.cpu(), b.cpu(), rtol=tol, atol=tol)


@pytest.mark.parametrize("name", list(CASES))
def test_clusters_reproduce_eager_on_the_checker(name):
    fn, make, tol = CASES[name]
    ins = make(torch.Generator().manual_seed(0))
    fused = TF.fuse_and_optimize(fn, ins, executor=oracle_executor)
    assert fused.subgraphs, "nothing was clustered"
    _close(fused(*ins), fn(*ins), tol)
    # fresh values through the same module
    ins2 = make(torch.Generator().manual_seed(1))
    _close(fused(*ins2), fn(*ins2), tol)


def test_cluster_structure():
    g = torch.Generator().manual_seed(0)
    # one cluster for a pure elementwise/broadcast chain, with exactly the external tensors as inputs
    fn, make, _ = CASES["gelu_bias"]
    fused = TF.fuse_and_optimize(fn, make(g), executor=oracle_executor)
    assert len(fused.subgraphs) == 1 and fused.clustered_ops == fused.total_ops
    d = fused.subgraphs[0].desc
    assert len(d["input_desc"]) == 3 and len(d["output_desc"]) == 1
    assert {o["name"] for o in d["op_desc"]} >= {"Add", "Mul", "Tanh"}
    # the unsupported op splits the program in two clusters and stays a torch call
    fn, make, _ = CASES["mixed"]
    fused = TF.fuse_and_optimize(fn, make(g), executor=oracle_executor)
    assert len(fused.subgraphs) == 2
    targets = [n.target for n in fused.gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.aten.index_select.default in targets
    assert sum(1 for t in targets if getattr(t, "__name__", "").startswith("akg_call_")) == 2


def test_what_is_not_clustered():
    g = torch.Generator().manual_seed(0)

    def f(x):  # float -> int conversion: its rounding is not pinned, so it stays with torch
        return (x * 3.0).to(torch.int32) + 1

    fused = TF.fuse_and_optimize(f, [torch.randn(8, 8, generator=g)], executor=oracle_executor)
    kept = [n.target for n in fused.gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.aten._to_copy.default in kept
    x = torch.randn(8, 8, generator=g)
    _close(fused(x), f(x), 0)

    def views_only(x):
        return x.reshape(4, 16).unsqueeze(0)

    fused = TF.fuse_and_optimize(views_only, [torch.randn(8, 8, generator=g)], executor=oracle_executor)
    assert not fused.subgraphs


def test_default_executor_has_no_host_path():
    fn, make, _ = CASES["gelu_bias"]
    ins = make(torch.Generator().manual_seed(0))
    fused = TF.fuse_and_optimize(fn, ins)
    with pytest.raises(RuntimeError, match="CUDA"):
        fused(*ins)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_fused_module_on_the_device(name):
    fn, make, tol = CASES[name]
    ins = [t.cuda() for t in make(torch.Generator().manual_seed(2))]
    fused = TF.fuse_and_optimize(fn, ins)
    assert fused.subgraphs
    _close(fused(*ins), fn(*ins), max(tol, 2e-5))


@pytest.mark.gpu
def test_bfloat16_linear_layers_on_the_device():
    """F.linear in bfloat16: the transposes fold into the matmuls, bias and ReLU into their launches."""
    g = torch.Generator().manual_seed(4)

    def net(x, w1, b1, w2, b2):
        h = torch.relu(torch.nn.functional.linear(x, w1, b1))
        return torch.nn.functional.linear(h, w2, b2)

    ins = [(torch.randn(s, generator=g) * 0.1).bfloat16().cuda() for s in ((256, 128), (192, 128), (192,), (64, 192), (64,))]
    fused = TF.fuse_and_optimize(net, ins)
    assert len(fused.subgraphs) == 2  # one matmul per cluster
    from akg_b200.driver import FusedKernel
    for sub in fused.subgraphs:
        names = [o["name"] for o in sub.desc["op_desc"]]
        assert "Transpose" not in names and names.count("MatMul") == 1
        assert FusedKernel(sub.desc_json).launch_count == 1
    got, want = fused(*ins), net(*ins)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_fused_half_precision_chain_on_the_device():
    g = torch.Generator().manual_seed(3)
    ins = [torch.randn(8, 256, 512, generator=g).half().cuda(), (torch.randn(512, generator=g) * 0.02).half().cuda(),
           torch.randn(8, 256, 512, generator=g).half().cuda()]
    fused = TF.fuse_and_optimize(gelu_bias, ins)
    got, want = fused(*ins), gelu_bias(*ins)
    assert got.dtype == torch.float16
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-3, atol=2e-3)


def test_transformer_block_clusters():
    """Every op of the block lands in a cluster; matmuls, LayerNorms, the softmax and the GELU get regions of their own."""
    ins = transformer_inputs(torch.float32, torch.Generator().manual_seed(0))
    fused = TF.fuse_and_optimize(transformer_block, ins, executor=oracle_executor)
    assert fused.clustered_ops == fused.total_ops and len(fused.subgraphs) == 9
    for sub in fused.subgraphs:
        names = [o["name"] for o in sub.desc["op_desc"]]
        n_mm = sum(n in ("MatMul", "BatchMatMul") for n in names)
        n_red = sum(n.startswith("Reduce") for n in names)
        assert n_mm <= 1 and not (n_mm and n_red)
    _close(fused(*ins), transformer_block(*ins), 2e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_transformer_block_on_the_device(dtype, tol):
    ins = [t.cuda() for t in transformer_inputs(dtype, torch.Generator().manual_seed(5))]
    fused = TF.fuse_and_optimize(transformer_block, ins)
    assert fused.clustered_ops == fused.total_ops
    got, want = fused(*ins), transformer_block(*ins)
    assert got.dtype == dtype and got.shape == want.shape
    torch.testing.assert_close(got.float(), want.float(), rtol=tol, atol=tol)
    from akg_b200.driver import FusedKernel
    launches = sum(FusedKernel(s.desc_json).launch_count for s in fused.subgraphs)
    assert launches <= 22


@pytest.mark.parametrize("name", list(MORE))
def test_more_programs_on_the_checker(name):
    fn, make = MORE[name]
    ins = make(_g(0))
    fused = TF.fuse_and_optimize(fn, ins, executor=oracle_executor)
    assert fused.subgraphs
    _close(fused(*ins), fn(*ins), 5e-6)
    from akg_b200.driver import FusedKernel
    for sub in fused.subgraphs:  # every cluster is something the library plans
        assert FusedKernel(sub.desc_json).launch_count >= 1


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(MORE))
def test_more_programs_on_the_device(name):
    fn, make = MORE[name]
    ins = [t.cuda() for t in make(_g(1))]
    fused = TF.fuse_and_optimize(fn, ins)
    _close(fused(*ins), fn(*ins), 2e-5)


def test_batch_norm_as_traced_on_device_tensors():
    """On device tensors batch_norm / instance_norm trace to the vendor-library op; it is decomposed like the native one."""
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(4, 8, 12, 16, generator=g), torch.rand(8, generator=g) + 0.5, torch.randn(8, generator=g)
    fn = lambda x, w, b: torch.ops.aten.cudnn_batch_norm(x, w, b, None, None, True, 0.1, 1e-5)[0]
    fused = TF.fuse_and_optimize(fn, [x, w, b], executor=oracle_executor)
    assert len(fused.subgraphs) == 1
    kept = [n.target for n in fused.gm.graph.nodes if n.op == "call_function" and n.target is torch.ops.aten.cudnn_batch_norm.default]
    assert not kept
    _close(fused(x, w, b), torch.nn.functional.batch_norm(x, None, None, w, b, training=True), 1e-5)


@pytest.mark.skipif(not hasattr(torch.ops.aten, "_fused_rms_norm"), reason="this torch has no fused rms norm op")
def test_rms_norm_as_traced_on_device_tensors():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(8, 64, generator=g), torch.rand(64, generator=g) + 0.5
    fn = lambda x, w: torch.ops.aten._fused_rms_norm(x, [64], w, 1e-6)[0] * 2
    fused = TF.fuse_and_optimize(fn, [x, w], executor=oracle_executor)
    assert len(fused.subgraphs) == 1
    assert not [n for n in fused.gm.graph.nodes if n.op == "call_function" and n.target is torch.ops.aten._fused_rms_norm.default]
    _close(fused(x, w), torch.nn.functional.rms_norm(x, (64,), w, 1e-6) * 2, 1e-5)
