"""GEMM parity on the GPU: CUDA kernel (through torch.ops.b200k -> C ABI) vs. the CPU oracle.

Tolerances are the path's: rtol = atol = 1e-2 for f16/bf16 operands against the fp32 oracle,
3e-2 relative for fp8 (against the fp32 product of the dequantised operands)."""

import os

import numpy as np
import pytest
import torch

import iree_turbine_b200 as tb
from iree_turbine_b200 import ops
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _run(a, b, out_dtype=None, tile_n=0, tile_m=0):
    a, b = a.to(DEV), b.to(DEV)
    if tile_n == 0 and tile_m == 0:
        c = torch.ops.b200k.gemm_nt(a, b, out_dtype)
    else:
        c = torch.empty(a.size(0), b.size(0), dtype=out_dtype or torch.float32, device=DEV)
        ops._launch_gemm(a, b, c, None, None, tile_n=tile_n, tile_m=tile_m)
    torch.cuda.synchronize()
    assert tb.device_status() == 0, "a kernel reported a timed-out wait"
    return c


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 64), (128, 128, 256), (256, 512, 512)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_small_exact_tiles(m, n, k, tile_n):
    a, b = oracle.make_gemm_inputs(m, n, k, torch.float16, seed=1)
    oracle.assert_close_half(_run(a, b, tile_n=tile_n), oracle.gemm_nt(a, b))


def test_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "gemm_f16_96x80x64.npz"))
    a = torch.from_numpy(z["a"].copy()).view(torch.float16)
    b = torch.from_numpy(z["b"].copy()).view(torch.float16)
    oracle.assert_close_half(_run(a, b), torch.from_numpy(z["c"]))


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 768, 320), (300, 300, 136), (1, 8, 8), (1280, 2304, 512)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_256x256_tiles(m, n, k, dtype):
    """Forced 256 x 256 tiles (two 128-row halves sharing each B stage), exact and ragged shapes;
    1280 x 2304 gives 45 tiles so several CTAs run more than one tile through the single accumulator set."""
    a, b = oracle.make_gemm_inputs(m, n, k, dtype, seed=8)
    c = _run(a, b, tile_m=256)
    oracle.assert_close_half(c, oracle.gemm_nt(a, b))
    assert torch.equal(c, _run(a, b, tile_m=256))


@pytest.mark.parametrize("m,n,k", [(200, 136, 72), (1, 8, 8), (130, 260, 1032), (1000, 24, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_ragged_shapes(m, n, k, dtype):
    a, b = oracle.make_gemm_inputs(m, n, k, dtype, seed=2)
    oracle.assert_close_half(_run(a, b), oracle.gemm_nt(a, b))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_output(dtype):
    a, b = oracle.make_gemm_inputs(384, 200, 320, dtype, seed=3)
    c = _run(a, b, out_dtype=dtype)
    assert c.dtype == dtype
    # the only extra error is the final rounding of the output (2^-11 / 2^-8 relative)
    rt = 1e-2 if dtype == torch.float16 else 2e-2
    oracle.assert_close_half(c, oracle.gemm_nt(a, b), rtol=rt, atol=rt)


def test_config_2048_cubed_f16_fp32_out():
    a, b = oracle.make_gemm_inputs(2048, 2048, 2048, torch.float16, seed=10)
    c = _run(a, b)
    assert c.dtype == torch.float32 and c.shape == (2048, 2048)
    oracle.assert_close_half(c, oracle.gemm_nt(a, b))
    # repeat-run determinism (catches races): bitwise equal
    c2 = _run(a, b)
    assert torch.equal(c, c2)
    # every tile shape gives the same math
    oracle.assert_close_half(_run(a, b, tile_n=128), oracle.gemm_nt(a, b))
    oracle.assert_close_half(_run(a, b, tile_m=256), oracle.gemm_nt(a, b))


def test_block_of_ones_lands_where_it_should():
    """Structured indexing check (cf. the reference's block-of-ones numerics test,
    iree/turbine/kernel/boo/driver/numerics.py:319-355)."""
    m, n, k = 512, 768, 256
    a = torch.zeros(m, k, dtype=torch.float16)
    b = torch.zeros(n, k, dtype=torch.float16)
    a[130:190, 64:128] = 1
    b[300:517, 100:164] = 1
    c = _run(a, b).cpu()
    exp = torch.zeros(m, n)
    exp[130:190, 300:517] = 28  # overlap of k ranges: 100..127
    assert torch.equal(c, exp)


def test_non_contiguous_inputs_are_handled():
    a, b = oracle.make_gemm_inputs(256, 128, 192, torch.float16, seed=4)
    a_wide = torch.zeros(256, 256, dtype=torch.float16)
    a_wide[:, :192] = a
    av = a_wide.to(DEV)[:, :192]  # row stride 256 elements: used in place
    bt = b.t().contiguous().to(DEV).t()  # column-major: copied to row-major by the op
    c = torch.ops.b200k.gemm_nt(av, bt)
    torch.cuda.synchronize()
    oracle.assert_close_half(c, oracle.gemm_nt(a, b))


def test_template_constructor_runs():
    shape = tb.GemmShape(256, 384, 128)
    kern = tb.get_gemm_kernel(shape, torch.bfloat16, out_dtype=torch.bfloat16)
    a, b = oracle.make_gemm_inputs(256, 384, 128, torch.bfloat16, seed=5)
    c = kern(a.to(DEV), b.to(DEV))
    oracle.assert_close_half(c, oracle.gemm_nt(a, b), rtol=2e-2, atol=2e-2)


# ---- fp8 ----
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (200, 72, 1040)])
def test_fp8_small(m, n, k):
    a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(m, n, k, seed=6)
    c = torch.ops.b200k.gemm_fp8_nt(a8.to(DEV), b8.to(DEV), sa.to(DEV), sb.to(DEV))
    torch.cuda.synchronize()
    assert c.dtype == torch.bfloat16
    fro, mx = oracle.fp8_errors(c, oracle.gemm_fp8_nt(a8, b8, sa, sb))
    assert fro <= 3e-2 and mx <= 3e-2, (fro, mx)
    c32 = torch.ops.b200k.gemm_fp8_nt(a8.to(DEV), b8.to(DEV), sa.to(DEV), sb.to(DEV), torch.float32)
    fro32, _ = oracle.fp8_errors(c32, oracle.gemm_fp8_nt(a8, b8, sa, sb))
    assert fro32 <= 2e-3, fro32  # products of e4m3 values are exact in fp32; only the accumulation differs


def test_fp8_config_8192_slices():
    """Full 8192^3 problem on the GPU; the oracle checks row/column slices (the CPU fp32 product of
    the whole problem takes minutes) and linearity covers the rest: C(A, [B1;B2]) = [C(A,B1), C(A,B2)]."""
    m = n = k = 8192
    g = torch.Generator(device=DEV).manual_seed(10)
    a = torch.randn(m, k, generator=g, device=DEV)
    b = torch.randn(n, k, generator=g, device=DEV)
    a8, sa = torch.ops.b200k.quantize_e4m3(a)
    b8, sb = torch.ops.b200k.quantize_e4m3(b)
    c = torch.ops.b200k.gemm_fp8_nt(a8, b8, sa, sb)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191])
    cols = torch.tensor([0, 255, 256, 4097, 8191])
    a8c, b8c, sac, sbc = a8.cpu(), b8.cpu(), sa.cpu(), sb.cpu()
    ref_rows = oracle.gemm_fp8_nt(a8c[rows], b8c, sac, sbc)
    fro, mx = oracle.fp8_errors(c[rows.to(DEV)], ref_rows)
    assert fro <= 3e-2 and mx <= 3e-2, (fro, mx)
    ref_cols = oracle.gemm_fp8_nt(a8c, b8c[cols], sac, sbc)
    fro, mx = oracle.fp8_errors(c[:, cols.to(DEV)], ref_cols)
    assert fro <= 3e-2 and mx <= 3e-2, (fro, mx)
    # column-parallel decomposition (what sharding over N computes) is bitwise the same
    c_lo = torch.ops.b200k.gemm_fp8_nt(a8, b8[:4096], sa, sb)
    c_hi = torch.ops.b200k.gemm_fp8_nt(a8, b8[4096:], sa, sb)
    assert torch.equal(torch.cat([c_lo, c_hi], dim=1), c)


def test_quantize_matches_oracle_bitwise():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(513, 257, generator=g)
    y, s = torch.ops.b200k.quantize_e4m3(x.to(DEV))
    yo, so = oracle.quantize_e4m3(x)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(y.cpu().view(torch.uint8), yo.view(torch.uint8))


# ---- fused bias / activation epilogue ----
@pytest.mark.parametrize("activation", ["none", "relu", "gelu", "silu"])
@pytest.mark.parametrize("bias_dtype", [None, torch.float32, torch.float16])
def test_linear_act_matches_oracle(activation, bias_dtype):
    m, n, k = 300, 520, 256   # ragged M and N: edge tiles take the bias guard
    a, w = oracle.make_gemm_inputs(m, n, k, torch.float16, seed=7)
    a, w = a * 0.25, w * 0.25
    bias = None if bias_dtype is None else torch.randn(n, generator=torch.Generator().manual_seed(8)).to(bias_dtype)
    ref = oracle.linear_act(a, w, bias, activation)
    for out_dtype in (None, torch.float16):
        y = torch.ops.b200k.linear_act(a.to(DEV), w.to(DEV), None if bias is None else bias.to(DEV), activation, out_dtype)
        torch.cuda.synchronize()
        assert tb.device_status() == 0
        assert y.dtype == (torch.float32 if out_dtype is None else torch.float16)
        oracle.assert_close_half(y, ref)


@pytest.mark.parametrize("tile", [(128, 128), (128, 256), (256, 256)])
def test_linear_act_all_tile_shapes_and_unaligned_output(tile):
    m, n, k = 512, 512, 128
    a, w = oracle.make_gemm_inputs(m, n, k, torch.bfloat16, seed=9)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(10))
    ref = oracle.linear_act(a, w, bias, "silu")
    # TMA-store epilogue
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops._launch_gemm(a.to(DEV), w.to(DEV), out, None, None, tile_n=tile[1], tile_m=tile[0], bias=bias.to(DEV), activation="silu")
    # predicated-store epilogue: a view whose rows are not 16-byte aligned
    wide = torch.empty(m, n + 3, dtype=torch.bfloat16, device=DEV)
    out2 = wide[:, 1:n + 1]
    ops._launch_gemm(a.to(DEV), w.to(DEV), out2, None, None, tile_n=tile[1], tile_m=tile[0], bias=bias.to(DEV), activation="silu")
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(out, ref)
    assert torch.equal(out, out2)


def test_linear_act_rejects_unknown_activation():
    a, w = oracle.make_gemm_inputs(128, 128, 64, torch.float16, seed=1)
    with pytest.raises((RuntimeError, ValueError)):
        torch.ops.b200k.linear_act(a.to(DEV), w.to(DEV), None, "tanh", None)


# ---- operand storage orders (the four BLAS forms) and the backward products ----
@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("mnk", [(256, 256, 128), (296, 200, 136), (512, 768, 1024)])
def test_gemm_all_forms(trans_a, trans_b, mnk):
    m, n, k = mnk
    g = torch.Generator().manual_seed(12)
    a = torch.randn((k, m) if trans_a else (m, k), generator=g).half()
    b = torch.randn((n, k) if trans_b else (k, n), generator=g).half()
    c = torch.ops.b200k.gemm(a.to(DEV), b.to(DEV), trans_a, trans_b, None)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(c, oracle.gemm(a, b, trans_a, trans_b))


@pytest.mark.parametrize("tile", [(128, 128), (128, 256), (256, 256)])
def test_gemm_mn_major_operands_every_tile_shape(tile):
    m, n, k = 512, 512, 320
    g = torch.Generator().manual_seed(13)
    a = torch.randn(k, m, generator=g).bfloat16()   # stored [K, M]
    b = torch.randn(k, n, generator=g).bfloat16()   # stored [K, N]
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops._launch_gemm(a.to(DEV), b.to(DEV), out, None, None, tile_n=tile[1], tile_m=tile[0], a_km=True, b_kn=True)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(out, oracle.gemm(a, b, True, False))


def test_linear_autograd_matches_torch():
    g = torch.Generator().manual_seed(14)
    x = (torch.randn(384, 256, generator=g) * 0.5).half()
    w = (torch.randn(512, 256, generator=g) * 0.5).half()
    bias = torch.randn(512, generator=g).half()
    dy = (torch.randn(384, 512, generator=g) * 0.5).half()
    xr, wr, br = (t.float().requires_grad_() for t in (x, w, bias))
    (torch.nn.functional.linear(xr, wr, br) * dy.float()).sum().backward()
    xd, wd, bd = (t.to(DEV).requires_grad_() for t in (x, w, bias))
    y = ops.linear(xd, wd, bd)
    (y.float() * dy.to(DEV).float()).sum().backward()
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(y.detach(), torch.nn.functional.linear(x.float(), w.float(), bias.float()))
    for got, ref in ((xd.grad, xr.grad), (wd.grad, wr.grad), (bd.grad, br.grad)):
        scale = ref.abs().max().item()
        assert (got.float().cpu() - ref).abs().max().item() <= 1e-2 * max(scale, 1.0)


def test_gemm_rejects_rows_that_are_not_16_byte_multiples():
    a = torch.zeros(136, 300, dtype=torch.float16, device=DEV)   # stored [K, M] with M = 300
    b = torch.zeros(136, 200, dtype=torch.float16, device=DEV)
    with pytest.raises((RuntimeError, ValueError)):
        torch.ops.b200k.gemm(a, b, True, False, None)


def test_linear_golden_fixture_forward_and_backward_products():
    z = np.load(os.path.join(GOLDEN, "linear_f16_72x88x64.npz"))
    h = lambda n: torch.from_numpy(z[n].copy()).view(torch.float16).to(DEV)  # noqa: E731
    x, w, bias, dy = h("x"), h("w"), h("bias"), h("dy")
    for act, key in (("none", "y"), ("gelu", "y_gelu"), ("silu", "y_silu")):
        oracle.assert_close_half(torch.ops.b200k.linear_act(x, w, bias, act, None), torch.from_numpy(z[key]))
    oracle.assert_close_half(torch.ops.b200k.gemm(dy, w, False, False, None), torch.from_numpy(z["dx"]))
    oracle.assert_close_half(torch.ops.b200k.gemm(dy, x, True, False, None), torch.from_numpy(z["dw"]))
    assert tb.device_status() == 0


# ---- batched product (aten::bmm) ----
@pytest.mark.parametrize("bsz,m,n,k", [(1, 128, 128, 64), (3, 200, 136, 72), (16, 128, 64, 128), (5, 300, 520, 136),
                                        (32, 64, 64, 64)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bmm_against_oracle_and_per_problem_calls(bsz, m, n, k, dtype):
    g = torch.Generator().manual_seed(13)
    a = torch.randn(bsz, m, k, generator=g).to(dtype)
    b = torch.randn(bsz, k, n, generator=g).to(dtype)
    ad, bd = a.to(DEV), b.to(DEV)
    c = torch.ops.b200k.bmm(ad, bd)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert c.shape == (bsz, m, n) and c.dtype == torch.float32
    oracle.assert_close_half(c, oracle.bmm(a, b))
    # the batched launch gives each problem the bits of its own call
    for i in (0, bsz - 1):
        assert torch.equal(c[i], torch.ops.b200k.gemm(ad[i], bd[i], False, False))
    # a transposed view of [B, N, K] storage (the attention-style q @ k^T) is read in place
    bt = b.transpose(1, 2).contiguous().to(DEV)  # [B, N, K]
    c2 = torch.ops.b200k.bmm(ad, bt.transpose(1, 2), dtype)
    oracle.assert_close_half(c2, oracle.bmm(a, b))
    # aten.bmm itself, in fp32, for reference
    assert torch.allclose(c.cpu(), torch.bmm(a.float(), b.float()), rtol=1e-2, atol=1e-2)


def test_bmm_block_of_ones_lands_in_the_right_problem():
    """Structured indexing check (the reference's block-of-ones idea, kernel/boo/driver/numerics.py:319-355):
    zeros everywhere except one block of ones in one problem of the batch."""
    bsz, m, n, k = 7, 256, 384, 128
    a = torch.zeros(bsz, m, k, dtype=torch.float16)
    b = torch.zeros(bsz, k, n, dtype=torch.float16)
    a[4, 130:140, 16:48] = 1
    b[4, 16:48, 300:310] = 1
    c = torch.ops.b200k.bmm(a.to(DEV), b.to(DEV)).cpu()
    ref = torch.zeros(bsz, m, n)
    ref[4, 130:140, 300:310] = 32
    assert torch.equal(c, ref)


# ---- split-K over a thread-block cluster ----
def _run_split(a, b, out_dtype, tile_n, split_k, **kw):
    m = a.size(1) if kw.get("a_km") else a.size(0)
    n = b.size(1) if kw.get("b_kn") else b.size(0)
    c = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    ops._launch_gemm(a.to(DEV), b.to(DEV), c, None, None, tile_n=tile_n, split_k=split_k, **kw)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    return c


@pytest.mark.parametrize("split_k", [2, 4, 8])
@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("m,n,k,dtype,out_dtype", [
    (128, 128, 512, torch.float16, torch.float32),
    (256, 512, 4096, torch.float16, torch.float16),
    (200, 300, 1000, torch.bfloat16, torch.bfloat16),     # ragged M, N and a K tail
    (384, 136, 2056, torch.bfloat16, torch.float32),
    (1, 8, 640, torch.float16, torch.float32),
])
def test_split_k_matches_oracle_and_is_reproducible(m, n, k, dtype, out_dtype, tile_n, split_k):
    a, b = oracle.make_gemm_inputs(m, n, k, dtype, seed=21)
    c = _run_split(a, b, out_dtype, tile_n, split_k)
    oracle.assert_close_half(c, oracle.gemm_nt(a, b))
    assert torch.equal(c, _run_split(a, b, out_dtype, tile_n, split_k)), "split-K result depends on timing"


def test_split_k_slices_that_do_not_divide_the_k_blocks():
    """9 k-blocks over 4 and 8 CTAs: the library lowers the split until every slice has work."""
    a, b = oracle.make_gemm_inputs(128, 256, 9 * 64, torch.float16, seed=22)
    for s in (2, 4, 8):
        oracle.assert_close_half(_run_split(a, b, torch.float32, 128, s), oracle.gemm_nt(a, b))


@pytest.mark.parametrize("activation", ["none", "relu", "gelu", "silu"])
@pytest.mark.parametrize("bias_dtype", [None, torch.float32, torch.bfloat16])
def test_split_k_fused_bias_and_activation(activation, bias_dtype):
    m, n, k = 200, 262, 2048      # N tail: the last chunk of a row is partly outside the matrix
    a, w = oracle.make_gemm_inputs(m, n + 2, k, torch.bfloat16, seed=23)
    a, w = a * 0.25, w[:n] * 0.25
    bias = None if bias_dtype is None else torch.randn(n, generator=torch.Generator().manual_seed(24)).to(bias_dtype)
    ref = oracle.linear_act(a, w, bias, activation)
    for split_k, pitch in ((2, n + 2), (4, n + 1)):   # 16-byte-multiple pitch: vector stores + a ragged last chunk; odd pitch: scalar stores
        c = torch.full((m, pitch), float("nan"), dtype=torch.float32, device=DEV)[:, :n]
        ops._launch_gemm(a.to(DEV), w.to(DEV), c, None, None, tile_n=128, split_k=split_k,
                         bias=None if bias is None else bias.to(DEV), activation=activation)
        torch.cuda.synchronize()
        assert tb.device_status() == 0
        oracle.assert_close_half(c, ref)


def test_split_k_fp8():
    a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(256, 384, 4096, seed=25)
    ref = oracle.gemm_fp8_nt(a8, b8, sa, sb)
    for split_k, tile_n in ((2, 128), (4, 256), (8, 128)):
        c = torch.full((256, 384), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops._launch_gemm(a8.to(DEV), b8.to(DEV), c, sa.to(DEV), sb.to(DEV), tile_n=tile_n, split_k=split_k)
        torch.cuda.synchronize()
        assert tb.device_status() == 0
        fro, mx = oracle.fp8_errors(c, ref)
        assert fro < 3e-2, (split_k, fro, mx)


@pytest.mark.parametrize("a_km,b_kn", [(True, False), (False, True), (True, True)])
def test_split_k_with_transposed_storage(a_km, b_kn):
    """The weight-gradient shape: few output tiles, K = the token count."""
    m, n, k = 256, 384, 4096
    g = torch.Generator().manual_seed(26)
    a = (torch.randn((k, m) if a_km else (m, k), generator=g) * 0.5).half()
    b = (torch.randn((k, n) if b_kn else (n, k), generator=g) * 0.5).half()
    ref = oracle.gemm(a, b, a_km, not b_kn)
    for split_k in (2, 8):
        c = _run_split(a, b, torch.float32, 128, split_k, a_km=a_km, b_kn=b_kn)
        oracle.assert_close_half(c, ref)


def test_split_k_chosen_by_the_library_on_few_tiles_long_k():
    """1024 x 1024 x 4096 has 64 tiles of 128 x 128 for 148 SMs; whatever the library picks, the result is the oracle's,
    and the same bits on every call."""
    a, b = oracle.make_gemm_inputs(1024, 1024, 4096, torch.float16, seed=27)
    c = _run(a, b, torch.float16)
    oracle.assert_close_half(c, oracle.gemm_nt(a, b))
    assert torch.equal(c, _run(a, b, torch.float16))
    # a batch of two narrow problems: four tiles in all
    ab = torch.randn(2, 128, 8192, generator=torch.Generator().manual_seed(28)).half()
    bb = torch.randn(2, 8192, 256, generator=torch.Generator().manual_seed(29)).half()
    cb = torch.ops.b200k.bmm(ab.to(DEV), bb.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(cb, oracle.bmm(ab, bb))


def test_split_k_argument_errors():
    a = torch.zeros(128, 256, dtype=torch.float16, device=DEV)
    c = torch.empty(128, 128, dtype=torch.float32, device=DEV)
    with pytest.raises(ValueError, match="split_k must be"):
        ops._launch_gemm(a, a, c, None, None, split_k=3)
    with pytest.raises(ValueError, match="128-row tiles"):
        ops._launch_gemm(a, a, c, None, None, tile_m=256, split_k=2)
    with pytest.raises(ValueError, match="exceeds the number of k-blocks"):
        ops._launch_gemm(a, a, c, None, None, split_k=8)
