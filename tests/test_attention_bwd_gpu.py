"""Attention backward on the GPU: the CUDA kernels (through torch.ops.b200k -> C ABI) against the
CPU oracle's written-out formulas.  Tolerance: the path's rtol = atol = 1e-2, taken relative to the
largest reference gradient (gradients of a 16-bit attention are sums of many rounded products)."""

import pytest
import torch

import iree_turbine_b200 as tb
from iree_turbine_b200 import ops
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCALE = 1.0 / 128 ** 0.5


def _d_o(shape, dtype, seed=9):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def _run(q, k, v, d_o, causal, scale=SCALE):
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, d_o))
    o = torch.ops.b200k.attention(qd, kd, vd, scale, causal)
    out = torch.ops.b200k.attention_bwd(qd, kd, vd, o, dod, scale, causal)
    torch.cuda.synchronize()
    assert tb.device_status() == 0, "a kernel reported a timed-out wait"
    return out


def _assert_close(got, ref, tol=1e-2):
    got = got.float().cpu()
    assert not torch.isnan(got).any()
    bound = tol * max(ref.abs().max().item(), 1.0)
    assert (got - ref).abs().max().item() <= bound


CASES = [
    (1, 1, 1, 128, 128, False), (1, 1, 1, 128, 128, True),      # one tile
    (1, 2, 1, 256, 256, False), (2, 4, 2, 256, 384, True),      # grouped heads, Skv > Sq
    (1, 2, 2, 200, 300, False), (1, 2, 1, 200, 300, True),      # ragged tiles
    (1, 1, 1, 300, 200, True),                                  # Sq > Skv: the first 100 queries see no key
    (1, 8, 2, 8, 8, True), (1, 1, 1, 1, 1, False),              # tiny
    (1, 2, 2, 1024, 1024, True),
]


@pytest.mark.parametrize("b,hq,hkv,sq,skv,causal", CASES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_matches_oracle(b, hq, hkv, sq, skv, causal, dtype):
    q, k, v = oracle.make_attention_inputs(b, hq, hkv, sq, skv, dtype=dtype, seed=5)
    d_o = _d_o((b, hq, sq, 128), dtype)
    got = _run(q, k, v, d_o, causal)
    ref = oracle.attention_bwd(q, k, v, d_o, SCALE, causal)
    for g, r in zip(got, ref):
        _assert_close(g, r)


@pytest.mark.parametrize("b,hq,hkv,sq,skv,causal", CASES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64_matches_oracle(b, hq, hkv, sq, skv, causal, dtype):
    scale = 0.125
    q, k, v = oracle.make_attention_inputs(b, hq, hkv, sq, skv, head_dim=64, dtype=dtype, seed=6)
    d_o = _d_o((b, hq, sq, 64), dtype)
    got = _run(q, k, v, d_o, causal, scale)
    ref = oracle.attention_bwd(q, k, v, d_o, scale, causal)
    for g, r in zip(got, ref):
        assert g.shape[-1] == 64
        _assert_close(g, r)


def test_head_dim_64_autograd_wrapper_with_forward_lse():
    """ops.sdpa at head dim 64 (forward LSE handed to the backward) against torch's own autograd in fp32."""
    from iree_turbine_b200 import ops

    g = torch.Generator().manual_seed(15)
    q, k, v = (torch.randn(2, h, 320, 64, generator=g).to(torch.bfloat16) for h in (4, 2, 2))
    d_o = _d_o((2, 4, 320, 64), torch.bfloat16)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    o = ops.sdpa(qd, kd, vd, None, True)
    o.backward(d_o.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, is_causal=True, enable_gqa=True)
    ref.backward(d_o.float())
    _assert_close(o.detach(), ref.detach())
    for got, want in ((qd.grad, qr.grad), (kd.grad, kr.grad), (vd.grad, vr.grad)):
        _assert_close(got, want)


def test_rows_without_a_visible_key_get_zero_gradient():
    q, k, v = oracle.make_attention_inputs(1, 1, 1, 300, 200, dtype=torch.float16, seed=6)
    d_q, _, _ = _run(q, k, v, _d_o(q.shape, torch.float16), True)
    assert torch.count_nonzero(d_q[0, 0, :100]).item() == 0


def test_results_do_not_depend_on_batching_or_head_sharding():
    """Every output element is accumulated by one CTA in a fixed order: the gradients of a
    (batch, kv head) slice computed alone are bitwise those of the full call."""
    q, k, v = oracle.make_attention_inputs(2, 4, 2, 384, 384, dtype=torch.bfloat16, seed=7)
    d_o = _d_o(q.shape, torch.bfloat16)
    full = _run(q, k, v, d_o, True)
    again = _run(q, k, v, d_o, True)
    for a, b_ in zip(full, again):
        assert torch.equal(a, b_)
    part = _run(q[1:, 2:], k[1:, 1:], v[1:, 1:], d_o[1:, 2:], True)
    assert torch.equal(part[0], full[0][1:, 2:])
    assert torch.equal(part[1], full[1][1:, 1:])
    assert torch.equal(part[2], full[2][1:, 1:])


def test_strided_inputs_and_autograd_wrapper():
    """[B, S, H, D] memory viewed as [B, H, S, D] (rows contiguous) goes to the kernel as it is;
    ops.sdpa routes autograd to the backward kernels."""
    b, h, s = 2, 4, 256
    g = torch.Generator().manual_seed(11)
    base = [torch.randn(b, s, h, 128, generator=g).to(torch.bfloat16) for _ in range(3)]
    q, k, v = (t.to(DEV).transpose(1, 2).requires_grad_() for t in base)
    d_o = _d_o((b, h, s, 128), torch.bfloat16)
    out = ops.sdpa(q, k, v, is_causal=True)
    out.backward(d_o.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    qc, kc, vc = (t.transpose(1, 2) for t in base)
    ref = oracle.attention_bwd(qc, kc, vc, d_o, SCALE, True)
    for t, r in zip((q, k, v), ref):
        _assert_close(t.grad, r)


def test_gradient_against_torch_sdpa_autograd_on_the_same_device():
    b, h, s = 1, 2, 512
    q, k, v = (t.to(DEV) for t in oracle.make_attention_inputs(b, h, h, s, s, dtype=torch.float16, seed=12))
    d_o = _d_o((b, h, s, 128), torch.float16).to(DEV)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, is_causal=True).backward(d_o.float())
    o = torch.ops.b200k.attention(q, k, v, SCALE, True)
    got = torch.ops.b200k.attention_bwd(q, k, v, o, d_o, SCALE, True)
    for g, r in zip(got, (qr.grad, kr.grad, vr.grad)):
        _assert_close(g, r.cpu())


@pytest.mark.parametrize("b,hq,hkv,sq,skv,causal", [(1, 2, 1, 200, 300, True), (1, 1, 1, 300, 200, True),
                                                    (2, 4, 2, 256, 384, False)])
def test_forward_lse_and_backward_from_it(b, hq, hkv, sq, skv, causal):
    """The forward's optional row statistic is ln sum exp(scale * s) (-inf where a row sees no key);
    given to the backward it replaces the statistics sweep: same gradients within tolerance of
    the oracle, and the forward output is bitwise the one of the plain op."""
    q, k, v = oracle.make_attention_inputs(b, hq, hkv, sq, skv, dtype=torch.bfloat16, seed=15)
    d_o = _d_o((b, hq, sq, 128), torch.bfloat16)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, d_o))
    o, lse = torch.ops.b200k.attention_lse(qd, kd, vd, SCALE, causal)
    assert torch.equal(o, torch.ops.b200k.attention(qd, kd, vd, SCALE, causal))
    s = torch.matmul(q.float(), k.float().repeat_interleave(hq // hkv, 1).transpose(-1, -2)) * SCALE
    if causal:
        i, j = torch.arange(sq).unsqueeze(1), torch.arange(skv).unsqueeze(0)
        s = s.masked_fill(j > i + (skv - sq), float("-inf"))
    ref_lse = torch.logsumexp(s, dim=-1)
    dead = torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(lse.cpu()), dead) and (lse.cpu()[dead] < 0).all()
    assert (lse.cpu()[~dead] - ref_lse[~dead]).abs().max().item() < 1e-3
    got = torch.ops.b200k.attention_bwd(qd, kd, vd, o, dod, SCALE, causal, lse)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    for g, r in zip(got, oracle.attention_bwd(q, k, v, d_o, SCALE, causal)):
        _assert_close(g, r)
    again = torch.ops.b200k.attention_bwd(qd, kd, vd, o, dod, SCALE, causal, lse)
    for a, b_ in zip(got, again):
        assert torch.equal(a, b_)


def test_golden_fixture():
    """Inputs and torch-autograd gradients committed under tests/golden/ (generated by make_golden.py)."""
    import os

    import numpy as np

    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_bwd_bf16_causal_gqa.npz"))
    q, k, v, d_o = (torch.from_numpy(z[n].copy()).view(torch.bfloat16) for n in ("q", "k", "v", "d_o"))
    got = _run(q, k, v, d_o, True, float(z["scale"]))
    for g, name in zip(got, ("dq", "dk", "dv")):
        _assert_close(g, torch.from_numpy(z[name]))


def test_bad_arguments_are_rejected():
    q = torch.zeros(1, 2, 128, 128, dtype=torch.float16, device=DEV)
    k = torch.zeros(1, 2, 128, 64, dtype=torch.float16, device=DEV)
    with pytest.raises((RuntimeError, ValueError)):
        torch.ops.b200k.attention_bwd(q, k, k, q, q, SCALE, False)
    with pytest.raises((RuntimeError, ValueError)):
        torch.ops.b200k.attention_bwd(q, q.float(), q, q, q, SCALE, False)
