"""The torch.compile routing pass on hand-built ATen graphs with fake CUDA tensors (no GPU needed):
which nodes are rewritten to torch.ops.b200k.*, and which are left alone."""

import operator

import pytest
import torch
from torch import fx
from torch._subclasses.fake_tensor import FakeTensorMode

import iree_turbine_b200 as tb  # noqa: F401
from iree_turbine_b200 import dynamo_backend as db

aten = torch.ops.aten


def _fake(shape, dtype=torch.float16, device="cuda"):
    with FakeTensorMode():
        return torch.empty(shape, dtype=dtype, device=device)


def _graph(build):
    g = fx.Graph()
    out = build(g)
    g.output(out)
    return fx.GraphModule(torch.nn.Module(), g)


def _ph(g, name, val):
    n = g.placeholder(name)
    n.meta["val"] = val
    return n


def _targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


@pytest.mark.parametrize("transpose", ["t", "transpose", "permute"])
def test_mm_nt_is_routed(transpose):
    def build(g):
        a = _ph(g, "a", _fake((64, 256)))
        w = _ph(g, "w", _fake((512, 256)))
        if transpose == "t":
            wt = g.call_function(aten.t.default, (w,))
        elif transpose == "transpose":
            wt = g.call_function(aten.transpose.int, (w, 0, 1))
        else:
            wt = g.call_function(aten.permute.default, (w, [1, 0]))
        wt.meta["val"] = _fake((256, 512))
        mm = g.call_function(aten.mm.default, (a, wt))
        mm.meta["val"] = _fake((64, 512))
        return mm

    gm = _graph(build)
    assert db.apply_replacements(gm) == 1
    assert torch.ops.b200k.gemm_nt.default in _targets(gm) and aten.mm.default not in _targets(gm)
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.gemm_nt.default)
    assert node.args[2] == torch.float16 and [a.name for a in node.args[:2]] == ["a", "w"]


def test_bmm_is_routed_and_float32_bmm_left_alone():
    def build(dtype):
        def f(g):
            a = _ph(g, "a", _fake((4, 64, 128), dtype))
            b = _ph(g, "b", _fake((4, 128, 32), dtype))
            out = g.call_function(aten.bmm.default, (a, b))
            out.meta["val"] = _fake((4, 64, 32), dtype)
            return out
        return f

    gm = _graph(build(torch.bfloat16))
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.bmm.default)
    assert [a.name for a in node.args[:2]] == ["a", "b"] and node.args[2] == torch.bfloat16
    gm = _graph(build(torch.float32))
    assert db.apply_replacements(gm) == 0 and aten.bmm.default in _targets(gm)


def test_addmm_becomes_fused_linear():
    def build(g):
        bias = _ph(g, "bias", _fake((512,)))
        a = _ph(g, "a", _fake((64, 256)))
        w = _ph(g, "w", _fake((512, 256)))
        wt = g.call_function(aten.t.default, (w,))
        wt.meta["val"] = _fake((256, 512))
        out = g.call_function(aten.addmm.default, (bias, a, wt))
        out.meta["val"] = _fake((64, 512))
        return out

    gm = _graph(build)
    assert db.apply_replacements(gm) == 1
    t = _targets(gm)
    assert torch.ops.b200k.linear_act.default in t and aten.addmm.default not in t
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.linear_act.default)
    assert [a.name for a in node.args[:3]] == ["a", "w", "bias"] and node.args[3] == "none"


def test_mm_nn_form_is_routed_to_the_general_op():
    def build(g):
        a = _ph(g, "a", _fake((64, 256)))
        b = _ph(g, "b", _fake((256, 512)))
        mm = g.call_function(aten.mm.default, (a, b))
        mm.meta["val"] = _fake((64, 512))
        return mm

    gm = _graph(build)
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.gemm.default)
    assert node.args[2] is False and node.args[3] is False


@pytest.mark.parametrize("case", ["odd_rows", "float32", "cpu", "three_d"])
def test_mm_left_alone(case):
    def build(g):
        dtype = torch.float32 if case == "float32" else torch.float16
        dev = "cpu" if case == "cpu" else "cuda"
        a = _ph(g, "a", _fake((4, 64, 256) if case == "three_d" else (64, 256), dtype, dev))
        if case == "odd_rows":
            b = _ph(g, "b", _fake((256, 516), dtype, dev))   # rows of 516 halves are not 16-byte multiples
        else:
            w = _ph(g, "w", _fake((512, 256), dtype, dev))
            b = g.call_function(aten.t.default, (w,))
            b.meta["val"] = _fake((256, 512), dtype, dev)
        mm = g.call_function(aten.mm.default, (a, b))
        mm.meta["val"] = _fake((64, 512), dtype, dev)
        return mm

    gm = _graph(build)
    assert db.apply_replacements(gm) == 0
    assert aten.mm.default in _targets(gm)


def _flash_graph(aux_used=False, causal=False, sq=256, skv=256, d=128, dropout=0.0, hq=8, hkv=8):
    def build(g):
        q = _ph(g, "q", _fake((2, hq, sq, d), torch.bfloat16))
        k = _ph(g, "k", _fake((2, hkv, skv, d), torch.bfloat16))
        v = _ph(g, "v", _fake((2, hkv, skv, d), torch.bfloat16))
        n = g.call_function(aten._scaled_dot_product_flash_attention.default, (q, k, v, dropout, causal, False),
                            {"scale": 0.125})
        o = g.call_function(operator.getitem, (n, 0))
        o.meta["val"] = _fake((2, hq, sq, d), torch.bfloat16)
        lse = g.call_function(operator.getitem, (n, 1))
        lse.meta["val"] = _fake((2, hq, sq), torch.float32)
        if aux_used:
            return (o, lse)
        return o

    return _graph(build)


def test_flash_sdpa_is_routed_with_scale_and_causal_flag():
    gm = _flash_graph(causal=True)
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.attention.default)
    assert node.args[3] == 0.125 and node.args[4] is True
    assert aten._scaled_dot_product_flash_attention.default not in _targets(gm)
    assert operator.getitem not in _targets(gm)


def test_flash_sdpa_with_its_statistic_in_use_becomes_attention_lse():
    gm = _flash_graph(aux_used=True)
    assert db.apply_replacements(gm) == 1
    assert torch.ops.b200k.attention_lse.default in _targets(gm)


@pytest.mark.parametrize("kw", [dict(causal=True, sq=128, skv=256), dict(d=96), dict(dropout=0.1), dict(hq=8, hkv=3),
                                dict(aux_used=True, d=96)])
def test_flash_sdpa_left_alone(kw):
    gm = _flash_graph(**kw)
    assert db.apply_replacements(gm) == 0
    assert aten._scaled_dot_product_flash_attention.default in _targets(gm)


def _flash_training_graph(d=128, causal=True):
    """Forward graph of a training step: output, log-sum-exp and the random-number state are graph outputs."""
    def build(g):
        q = _ph(g, "q", _fake((2, 8, 256, d), torch.bfloat16))
        k = _ph(g, "k", _fake((2, 4, 256, d), torch.bfloat16))
        v = _ph(g, "v", _fake((2, 4, 256, d), torch.bfloat16))
        n = g.call_function(aten._scaled_dot_product_flash_attention.default, (q, k, v, 0.0, causal, False),
                            {"scale": 0.1})
        outs = []
        for idx, val in ((0, _fake((2, 8, 256, d), torch.bfloat16)), (1, _fake((2, 8, 256), torch.float32)),
                         (6, _fake((2,), torch.uint64)), (7, _fake((), torch.uint64))):
            u = g.call_function(operator.getitem, (n, idx))
            u.meta["val"] = val
            outs.append(u)
        mq = g.call_function(operator.getitem, (n, 4))
        mq.meta["val"] = 256
        outs.append(mq)
        return tuple(outs)

    return _graph(build)


@pytest.mark.parametrize("d", [128, 64])
def test_flash_sdpa_of_a_training_graph_becomes_attention_lse(d):
    gm = _flash_training_graph(d)
    assert db.apply_replacements(gm) == 1
    t = _targets(gm)
    assert torch.ops.b200k.attention_lse.default in t and aten._scaled_dot_product_flash_attention.default not in t
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.attention_lse.default)
    assert node.args[3] == 0.1 and node.args[4] is True
    out = next(n for n in gm.graph.nodes if n.op == "output").args[0]
    assert out[0].target is operator.getitem and out[0].args == (node, 0)
    assert out[1].target is operator.getitem and out[1].args == (node, 1)
    assert out[2].target is aten.empty.memory_format and out[2].kwargs["dtype"] == torch.uint64
    assert out[4] == 256


def test_flash_sdpa_backward_is_routed_and_unsupported_left_alone():
    def build(dropout, d=128):
        def f(g):
            names = ("grad", "q", "k", "v", "out")
            shapes = ((2, 8, 256, d), (2, 8, 256, d), (2, 4, 256, d), (2, 4, 256, d), (2, 8, 256, d))
            grad, q, k, v, out = (_ph(g, n, _fake(s, torch.bfloat16)) for n, s in zip(names, shapes))
            lse = _ph(g, "lse", _fake((2, 8, 256), torch.float32))
            seed = _ph(g, "seed", _fake((2,), torch.uint64))
            off = _ph(g, "off", _fake((), torch.uint64))
            n = g.call_function(aten._scaled_dot_product_flash_attention_backward.default,
                                (grad, q, k, v, out, lse, None, None, 256, 256, dropout, True, seed, off), {"scale": 0.1})
            pieces = []
            for i, shp in enumerate(((2, 8, 256, d), (2, 4, 256, d), (2, 4, 256, d))):
                u = g.call_function(operator.getitem, (n, i))
                u.meta["val"] = _fake(shp, torch.bfloat16)
                pieces.append(u)
            return tuple(pieces)
        return f

    gm = _graph(build(0.0))
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.attention_bwd.default)
    assert [a.name for a in node.args[:5]] == ["q", "k", "v", "out", "grad"]
    assert node.args[5] == 0.1 and node.args[6] is True and node.args[7].name == "lse"
    out = next(n for n in gm.graph.nodes if n.op == "output").args[0]
    assert all(o.args[0] is node and o.args[1] == i for i, o in enumerate(out))
    for kw in (dict(dropout=0.1), dict(dropout=0.0, d=96)):
        gm = _graph(build(**kw))
        assert db.apply_replacements(gm) == 0


def test_cudnn_sdpa_of_a_training_graph_and_its_backward_are_routed():
    """The cuDNN form keeps its statistic as [B, H, Sq, 1]: the forward rewrite appends that axis, the backward
    rewrite drops it again."""
    def fwd(g):
        q = _ph(g, "q", _fake((2, 8, 256, 128), torch.bfloat16))
        k = _ph(g, "k", _fake((2, 8, 256, 128), torch.bfloat16))
        v = _ph(g, "v", _fake((2, 8, 256, 128), torch.bfloat16))
        n = g.call_function(aten._scaled_dot_product_cudnn_attention.default, (q, k, v, None, True, 0.0, True, False),
                            {"scale": 0.1})
        o = g.call_function(operator.getitem, (n, 0))
        o.meta["val"] = _fake((2, 8, 256, 128), torch.bfloat16)
        lse = g.call_function(operator.getitem, (n, 1))
        lse.meta["val"] = _fake((2, 8, 256, 1), torch.float32)
        return (o, lse)

    gm = _graph(fwd)
    assert db.apply_replacements(gm) == 1
    out = next(n for n in gm.graph.nodes if n.op == "output").args[0]
    assert out[1].target is aten.unsqueeze.default
    assert out[1].args[0].args[0].target is torch.ops.b200k.attention_lse.default

    def bwd(g):
        names = ("grad", "q", "k", "v", "out")
        grad, q, k, v, out = (_ph(g, n, _fake((2, 8, 256, 128), torch.bfloat16)) for n in names)
        lse = _ph(g, "lse", _fake((2, 8, 256, 1), torch.float32))
        seed = _ph(g, "seed", _fake((), torch.int64))
        n = g.call_function(aten._scaled_dot_product_cudnn_attention_backward.default,
                            (grad, q, k, v, out, lse, seed, seed, None, None, None, 256, 256, 0.0, True), {"scale": 0.1})
        u = g.call_function(operator.getitem, (n, 0))
        u.meta["val"] = _fake((2, 8, 256, 128), torch.bfloat16)
        return u

    gm = _graph(bwd)
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.attention_bwd.default)
    assert node.args[7].target is aten.squeeze.dim and node.args[4].name == "grad"


def test_flash_sdpa_head_dim_64_is_routed():
    gm = _flash_graph(d=64)
    assert db.apply_replacements(gm) == 1
    assert torch.ops.b200k.attention.default in _targets(gm)


def test_efficient_sdpa_with_bias_left_alone_and_without_routed():
    def build_with(bias):
        def build(g):
            q = _ph(g, "q", _fake((1, 4, 128, 128)))
            k = _ph(g, "k", _fake((1, 4, 128, 128)))
            v = _ph(g, "v", _fake((1, 4, 128, 128)))
            b = _ph(g, "b", _fake((1, 4, 128, 128))) if bias else None
            n = g.call_function(aten._scaled_dot_product_efficient_attention.default, (q, k, v, b, False, 0.0, False))
            o = g.call_function(operator.getitem, (n, 0))
            o.meta["val"] = _fake((1, 4, 128, 128))
            return o
        return build

    gm = _graph(build_with(True))
    assert db.apply_replacements(gm) == 0
    gm = _graph(build_with(False))
    assert db.apply_replacements(gm) == 1
    node = next(n for n in gm.graph.nodes if n.target is torch.ops.b200k.attention.default)
    assert abs(node.args[3] - 128 ** -0.5) < 1e-12 and node.args[4] is False


def test_backend_is_registered():
    assert "b200k" in torch._dynamo.list_backends(exclude_tags=())
