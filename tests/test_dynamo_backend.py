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


@pytest.mark.parametrize("kw", [dict(aux_used=True), dict(causal=True, sq=128, skv=256), dict(d=96),
                                dict(dropout=0.1), dict(hq=8, hkv=3)])
def test_flash_sdpa_left_alone(kw):
    gm = _flash_graph(**kw)
    assert db.apply_replacements(gm) == 0
    assert aten._scaled_dot_product_flash_attention.default in _targets(gm)


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
