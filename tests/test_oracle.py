"""Pins the CPU oracle: against torch's own operators, against itself (blockwise vs. full,
paged vs. contiguous) and against the committed fixtures in tests/golden/."""

import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _from_bits(arr, bf16=False):
    t = torch.from_numpy(arr.copy())
    return t.view(torch.bfloat16 if bf16 else torch.float16)


def test_gemm_matches_torch_mm_and_fixture():
    z = np.load(os.path.join(GOLDEN, "gemm_f16_96x80x64.npz"))
    a, b = _from_bits(z["a"]), _from_bits(z["b"])
    a2, b2 = oracle.make_gemm_inputs(96, 80, 64, torch.float16, seed=10)
    assert torch.equal(a, a2) and torch.equal(b, b2), "seeded input generator drifted from the fixture"
    c = oracle.gemm_nt(a, b)
    torch.testing.assert_close(c, torch.from_numpy(z["c"]), rtol=1e-6, atol=1e-5)
    torch.testing.assert_close(c, torch.mm(a.float(), b.float().t()), rtol=1e-6, atol=1e-5)
    # float64 cross-check: fp32 accumulation error is far inside the 1e-2 tolerance of the path
    c64 = a.double() @ b.double().t()
    assert float((c.double() - c64).abs().max()) < 1e-4


@pytest.mark.parametrize("name", ["attn_f16_noncausal", "attn_bf16_causal_gqa", "attn_f16_causal_offset"])
def test_attention_matches_fixture(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    bf16 = bool(z["bf16"])
    q, k, v = (_from_bits(z[n], bf16) for n in ("q", "k", "v"))
    o = oracle.attention(q, k, v, float(z["scale"]), bool(z["causal"]))
    torch.testing.assert_close(o, torch.from_numpy(z["o"]), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_matches_sdpa(causal):
    q, k, v = oracle.make_attention_inputs(2, 4, 4, 96, 96, 128, torch.float16, seed=3)
    scale = 128 ** -0.5
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal, scale=scale)
    torch.testing.assert_close(oracle.attention(q, k, v, scale, causal), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("causal,sq,skv", [(False, 200, 328), (True, 256, 256), (True, 100, 300)])
def test_blockwise_online_softmax_equals_full(causal, sq, skv):
    q, k, v = oracle.make_attention_inputs(1, 2, 1, sq, skv, 128, torch.float16, seed=4)
    scale = 128 ** -0.5
    full = oracle.attention(q, k, v, scale, causal)
    blk = oracle.attention_blockwise(q, k, v, scale, causal, 128, 128)
    torch.testing.assert_close(blk, full, rtol=2e-5, atol=2e-5)
    # rounding P to 16 bits before P V (what the kernels do) stays far inside the 1e-2 tolerance
    blk16 = oracle.attention_blockwise(q, k, v, scale, causal, 128, 128, p_dtype=torch.float16)
    assert float((blk16 - full).abs().max()) < 2e-3


def test_quantize_e4m3_range_and_roundtrip():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 96, generator=g)
    y, s = oracle.quantize_e4m3(x)
    assert y.dtype == torch.float8_e4m3fn and s.shape == (1,)
    assert float(y.float().abs().max()) == 448.0
    rel = float(((y.float() * s) - x).norm() / x.norm())
    assert rel < 0.04  # e4m3 has 3 mantissa bits: relative rounding error <= 2^-4 per element
    yz, sz = oracle.quantize_e4m3(torch.zeros(4, 4))
    assert float(sz) == 1.0 and float(yz.float().abs().max()) == 0.0


def test_fp8_gemm_oracle_is_dequantised_product():
    a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(48, 40, 64, seed=6)
    c = oracle.gemm_fp8_nt(a8, b8, sa, sb)
    ref = (a8.float() * sa) @ (b8.float() * sb).t()
    torch.testing.assert_close(c, ref, rtol=1e-5, atol=1e-5)


def test_paged_fixture_and_index_math():
    z = np.load(os.path.join(GOLDEN, "paged_decode_f16.npz"))
    q, kc, vc = _from_bits(z["q"]), _from_bits(z["k_cache"]), _from_bits(z["v_cache"])
    bt, sl = torch.from_numpy(z["block_table"]), torch.from_numpy(z["seq_lens"])
    scale = float(z["scale"])
    o = oracle.paged_decode_attention(q, kc, vc, bt, sl, scale)
    torch.testing.assert_close(o, torch.from_numpy(z["o"]), rtol=1e-5, atol=1e-5)
    # gather: bit-exact against the per-token loop stored in the fixture
    gk = oracle.paged_gather(kc, bt, sl, int(sl.max()))
    assert torch.equal(gk.view(torch.int16), torch.from_numpy(z["gathered_k"]))
    # index function: every offset addresses the element the 4-D index names
    pages, hkv, page, d = kc.shape
    flat = kc.reshape(-1)
    for s in range(bt.shape[0]):
        n = int(sl[s])
        for h in range(hkv):
            off = oracle.paged_row_offsets(bt.numpy(), s, h, n, page, hkv, d)
            assert off.dtype == np.int64
            for t in (0, n // 2, n - 1) if n else ():
                assert torch.equal(flat[off[t]:off[t] + d], kc[int(bt[s, t // page]), h, t % page])


def test_paged_inputs_block_table_is_a_permutation():
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=8, min_len=5, max_len=200, seed=7)
    used = bt[bt >= 0]
    assert used.numel() == kc.shape[0]
    assert torch.equal(torch.sort(used).values, torch.arange(kc.shape[0], dtype=torch.int32))
    pages = (sl + 15) // 16
    assert int(pages.sum()) == kc.shape[0]
    for s in range(8):
        assert (bt[s, : int(pages[s])] >= 0).all() and (bt[s, int(pages[s]):] == -1).all()


def test_decode_equals_attention_with_one_query():
    q, k, v = oracle.make_attention_inputs(3, 8, 2, 1, 77, 128, torch.float16, seed=8)
    lens = torch.tensor([77, 1, 40], dtype=torch.int32)
    o = oracle.decode_attention(q[:, :, 0], k, v, lens, 0.1)
    for s in range(3):
        n = int(lens[s])
        ref = oracle.attention(q[s:s + 1], k[s:s + 1, :, :n], v[s:s + 1, :, :n], 0.1, False)
        torch.testing.assert_close(o[s], ref[0, :, 0], rtol=1e-6, atol=1e-6)


def test_kv_append_then_gather_round_trip():
    """Appended rows come back through the gather at their token positions; nothing else moves."""
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(lens=[20, 33], seed=1)
    kn = torch.randn(2, 3, 8, 128).half()
    vn = torch.randn(2, 3, 8, 128).half()
    pos = torch.tensor([17, 30], dtype=torch.int32)
    k2, v2 = oracle.kv_append(kn, vn, kc, vc, bt, pos)
    gk, gv = oracle.paged_gather(k2, bt, sl, 48), oracle.paged_gather(v2, bt, sl, 48)
    assert torch.equal(gk[0, :, 17:20], kn[0].transpose(0, 1)) and torch.equal(gk[1, :, 30:33], kn[1].transpose(0, 1))
    assert torch.equal(gv[0, :, 17:20], vn[0].transpose(0, 1)) and torch.equal(gv[1, :, 30:33], vn[1].transpose(0, 1))
    g0 = oracle.paged_gather(kc, bt, sl, 48)
    assert torch.equal(gk[0, :, :17], g0[0, :, :17]) and torch.equal(gk[1, :, :30], g0[1, :, :30])
    assert int((k2 != kc).any(dim=-1).sum()) <= 2 * 3 * 8


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_forms_match_torch_mm(trans_a, trans_b):
    g = torch.Generator().manual_seed(2)
    m, n, k = 24, 40, 16
    a = torch.randn((k, m) if trans_a else (m, k), generator=g, dtype=torch.float64)
    b = torch.randn((n, k) if trans_b else (k, n), generator=g, dtype=torch.float64)
    ref = torch.mm(a.t() if trans_a else a, b.t() if trans_b else b)
    torch.testing.assert_close(oracle.gemm(a, b, trans_a, trans_b).double(), ref, rtol=1e-5, atol=1e-5)
    # the backward products of the NT form are two of these forms (gemm.py:233-270 of the reference)
    if not trans_a and trans_b:
        x = a.clone().requires_grad_()
        w = b.clone().requires_grad_()
        dy = torch.randn(m, n, generator=g, dtype=torch.float64)
        (torch.mm(x, w.t()) * dy).sum().backward()
        torch.testing.assert_close(oracle.gemm(dy, b, False, False).double(), x.grad, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(oracle.gemm(dy, a, True, False).double(), w.grad, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("activation", ["none", "relu", "gelu", "silu"])
def test_linear_act_matches_torch_functional(activation):
    g = torch.Generator().manual_seed(3)
    a = torch.randn(12, 32, generator=g)
    w = torch.randn(20, 32, generator=g)
    bias = torch.randn(20, generator=g)
    y = torch.nn.functional.linear(a, w, bias)
    ref = {"none": lambda t: t, "relu": torch.relu, "gelu": torch.nn.functional.gelu,
           "silu": torch.nn.functional.silu}[activation](y)
    torch.testing.assert_close(oracle.linear_act(a, w, bias, activation), ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(oracle.linear_act(a, w, None, "none"), torch.mm(a, w.t()), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
def test_paged_attention_matches_sdpa_per_sequence(causal):
    lens, sq = [40, 23, 0], 8
    q0, kc, vc, bt, sl = oracle.make_paged_decode_inputs(q_heads=4, kv_heads=2, lens=lens, seed=4)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(3, 4, sq, 128, generator=g).half()
    out = oracle.paged_attention(q, kc, vc, bt, sl, 128 ** -0.5, causal)
    for i, n in enumerate(lens):
        if n == 0:
            assert bool((out[i] == 0).all())
            continue
        # explicit per-token gather, independent of oracle.paged_gather
        rows_k = torch.stack([kc[int(bt[i, t // 16]), :, t % 16] for t in range(n)], dim=1)   # [Hkv, n, D]
        rows_v = torch.stack([vc[int(bt[i, t // 16]), :, t % 16] for t in range(n)], dim=1)
        kk = rows_k.float().repeat_interleave(2, dim=0).unsqueeze(0)
        vv = rows_v.float().repeat_interleave(2, dim=0).unsqueeze(0)
        mask = None
        if causal:
            ii = torch.arange(sq).unsqueeze(1)
            jj = torch.arange(n).unsqueeze(0)
            mask = jj <= ii + (n - sq)
        ref = torch.nn.functional.scaled_dot_product_attention(q[i:i + 1].float(), kk, vv, attn_mask=mask,
                                                               scale=128 ** -0.5)
        torch.testing.assert_close(out[i:i + 1], ref, rtol=1e-4, atol=1e-5)


def test_linear_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "linear_f16_72x88x64.npz"))
    h = lambda n: torch.from_numpy(z[n].copy()).view(torch.float16)  # noqa: E731
    x, w, bias, dy = h("x"), h("w"), h("bias"), h("dy")
    for act, key in (("none", "y"), ("gelu", "y_gelu"), ("silu", "y_silu")):
        torch.testing.assert_close(oracle.linear_act(x, w, bias, act), torch.from_numpy(z[key]), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(oracle.gemm(dy, w, False, False), torch.from_numpy(z["dx"]), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(oracle.gemm(dy, x, True, False), torch.from_numpy(z["dw"]), rtol=1e-5, atol=1e-5)


def test_paged_prefill_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "paged_prefill_bf16.npz"))
    h = lambda n: torch.from_numpy(z[n].copy()).view(torch.bfloat16)  # noqa: E731
    bt, sl, pos = (torch.from_numpy(z[n]) for n in ("block_table", "seq_lens", "positions"))
    k2, v2 = oracle.kv_append(h("k_new"), h("v_new"), h("k_cache"), h("v_cache"), bt, pos)
    assert torch.equal(k2.view(torch.int16), torch.from_numpy(z["k_after"]))
    assert torch.equal(v2.view(torch.int16), torch.from_numpy(z["v_after"]))
    out = oracle.paged_attention(h("q"), k2, v2, bt, sl, float(z["scale"]), True)
    torch.testing.assert_close(out, torch.from_numpy(z["o"]), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("shape", [(1, 2, 1, 40, 56, True), (2, 4, 2, 33, 33, False), (1, 2, 2, 24, 16, True)])
def test_attention_bwd_matches_torch_autograd(shape):
    """Pins the written-out backward formulas against autograd through the same expression
    (float64), including grouped heads and query rows that see no key (causal, Sq > Skv)."""
    b, hq, hkv, sq, skv, causal = shape
    q, k, v = oracle.make_attention_inputs(b, hq, hkv, sq, skv, dtype=torch.float32, seed=3)
    q, k, v = (x.double().requires_grad_() for x in (q, k, v))
    d_o = torch.randn(b, hq, sq, 128, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    kk, vv = k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1)
    s = q @ kk.transpose(-1, -2) * 0.1
    if causal:
        i, j = torch.arange(sq).unsqueeze(1), torch.arange(skv).unsqueeze(0)
        s = s.masked_fill(j > i + (skv - sq), float("-inf"))
    dead = torch.isinf(s.max(-1, keepdim=True).values)
    p = torch.softmax(torch.where(dead, torch.zeros_like(s), s), -1)
    p = torch.where(dead, torch.zeros_like(p), p)
    (p @ vv).backward(d_o)
    got = oracle.attention_bwd(q.detach().float(), k.detach().float(), v.detach().float(), d_o.float(), 0.1, causal)
    for g, ref in zip(got, (q.grad, k.grad, v.grad)):
        assert (g.double() - ref).abs().max().item() < 1e-4


def _load_bwd_fixture():
    z = np.load(os.path.join(GOLDEN, "attn_bwd_bf16_causal_gqa.npz"))
    ins = [torch.from_numpy(z[n].copy()).view(torch.bfloat16) for n in ("q", "k", "v", "d_o")]
    refs = [torch.from_numpy(z[n]) for n in ("dq", "dk", "dv")]
    return ins, refs, float(z["scale"])


def test_attention_bwd_golden_fixture():
    """Expected gradients in the fixture come from torch autograd through
    scaled_dot_product_attention, not from the oracle."""
    (q, k, v, d_o), refs, scale = _load_bwd_fixture()
    got = oracle.attention_bwd(q, k, v, d_o, scale, True)
    for g, r in zip(got, refs):
        assert g.shape == r.shape
        assert (g - r).abs().max().item() < 1e-4


def test_bmm_oracle_is_aten_bmm_in_fp32():
    g = torch.Generator().manual_seed(5)
    a = torch.randn(3, 17, 24, generator=g).half()
    b = torch.randn(3, 24, 9, generator=g).half()
    ref = torch.stack([a[i].float() @ b[i].float() for i in range(3)])
    assert torch.equal(oracle.bmm(a, b), torch.bmm(a.float(), b.float()))
    assert torch.allclose(oracle.bmm(a, b), ref, rtol=1e-6, atol=1e-6)
