"""Attention forward parity on the GPU vs. the CPU oracle (rtol = atol = 1e-2, f16 / bf16).

Two kernels implement the forward (one 128-row query tile per work item, or a pair of tiles; see
include/b200k.h): every test in this file runs once with each of them forced, so both are checked
on every shape whatever the library would pick by itself; head dim 64 exists in the pair kernel only."""

import os

import numpy as np
import pytest
import torch

import iree_turbine_b200 as tb
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SCALE = 128 ** -0.5


@pytest.fixture(autouse=True, params=["one_tile", "tile_pair"])
def forced_kernel(request):
    from iree_turbine_b200 import _launcher as L

    old = tb.ops.ATTENTION_KERNEL
    tb.ops.ATTENTION_KERNEL = L.ATTN_ONE_TILE if request.param == "one_tile" else L.ATTN_TILE_PAIR
    yield request.param
    tb.ops.ATTENTION_KERNEL = old


def _run(q, k, v, scale, causal):
    o = torch.ops.b200k.attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, causal)
    torch.cuda.synchronize()
    assert tb.device_status() == 0, "a kernel reported a timed-out wait"
    return o


@pytest.mark.parametrize("sq,skv", [(128, 128), (256, 256), (256, 128), (512, 384), (128, 1024)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_noncausal_exact_tiles(sq, skv, dtype):
    q, k, v = oracle.make_attention_inputs(1, 2, 2, sq, skv, 128, dtype, seed=1)
    oracle.assert_close_half(_run(q, k, v, SCALE, False), oracle.attention(q, k, v, SCALE, False))


@pytest.mark.parametrize("sq,skv", [(72, 200), (1, 17), (300, 300), (257, 129), (130, 1000)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_lengths(sq, skv, causal):
    if causal and sq > skv:
        pytest.skip("rows with no visible key are undefined in the oracle (NaN)")
    q, k, v = oracle.make_attention_inputs(2, 2, 1, sq, skv, 128, torch.float16, seed=2, std=0.5)
    oracle.assert_close_half(_run(q, k, v, SCALE, causal), oracle.attention(q, k, v, SCALE, causal))


@pytest.mark.parametrize("s", [128, 256, 640, 1024])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_causal_square(s, dtype):
    q, k, v = oracle.make_attention_inputs(1, 4, 2, s, s, 128, dtype, seed=3, std=0.5)
    oracle.assert_close_half(_run(q, k, v, SCALE, True), oracle.attention(q, k, v, SCALE, True))


@pytest.mark.parametrize("name", ["attn_f16_noncausal", "attn_bf16_causal_gqa", "attn_f16_causal_offset"])
def test_golden_fixtures(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = torch.bfloat16 if bool(z["bf16"]) else torch.float16
    q, k, v = (torch.from_numpy(z[n].copy()).view(dt) for n in ("q", "k", "v"))
    o = _run(q, k, v, float(z["scale"]), bool(z["causal"]))
    oracle.assert_close_half(o, torch.from_numpy(z["o"]))


def test_large_scores_and_rescaling():
    """Scores with a wide dynamic range force the running max to grow across KV tiles."""
    q, k, v = oracle.make_attention_inputs(1, 2, 2, 256, 1024, 128, torch.float16, seed=4, std=1.0)
    k[:, :, 700:] *= 3.0  # later tiles hold much larger scores than earlier ones
    scale = 0.35
    oracle.assert_close_half(_run(q, k, v, scale, False), oracle.attention(q, k, v, scale, False))


def test_strided_views_and_determinism():
    q, k, v = oracle.make_attention_inputs(2, 4, 4, 384, 384, 128, torch.float16, seed=5)
    # [B, S, H, D] storage viewed as [B, H, S, D]: head stride 128, row stride H*128
    qd = q.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    kd = k.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    vd = v.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    o1 = torch.ops.b200k.attention(qd, kd, vd, SCALE, True)
    o2 = torch.ops.b200k.attention(q.to(DEV), k.to(DEV), v.to(DEV), SCALE, True)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)
    oracle.assert_close_half(o1, oracle.attention(q, k, v, SCALE, True))
    for _ in range(5):
        assert torch.equal(torch.ops.b200k.attention(qd, kd, vd, SCALE, True), o1)


@pytest.mark.parametrize("sq,skv,causal", [(128, 128, False), (256, 256, True), (300, 333, True), (1, 17, False),
                                           (640, 1024, True), (1024, 1024, False), (700, 200, False)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64(sq, skv, causal, dtype, forced_kernel):
    """Head dim 64 (the reference's own SDPA sample, kernel/boo/driver/sample_commands.txt:26, and its
    in-tree attention statement, tests/kernel/fused_attention_test.py:79-90, use it)."""
    if forced_kernel == "one_tile":
        pytest.skip("head dim 64 always takes the pair kernel")
    q, k, v = oracle.make_attention_inputs(2, 4, 2, sq, skv, 64, dtype, seed=6, std=0.7)
    oracle.assert_close_half(_run(q, k, v, 0.125, causal), oracle.attention(q, k, v, 0.125, causal))


def test_head_dim_64_reference_sample_shape_and_lse():
    """[32, 8, 128, 64] bf16 causal: the shape of the reference driver's SDPA sample command."""
    q, k, v = oracle.make_attention_inputs(32, 8, 8, 128, 128, 64, torch.bfloat16, seed=7)
    o, lse = torch.ops.b200k.attention_lse(q.to(DEV), k.to(DEV), v.to(DEV), 0.125, True)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(o, oracle.attention(q, k, v, 0.125, True))
    s = (q.float() @ k.float().transpose(-1, -2)) * 0.125
    s = s.masked_fill(torch.ones(128, 128, dtype=torch.bool).triu(1), float("-inf"))
    assert torch.allclose(lse.cpu(), torch.logsumexp(s, -1), rtol=1e-3, atol=1e-3)


def test_library_choice_and_forced_kernels_agree(forced_kernel):
    """What the library picks by itself (pair kernel for a causal problem that fills the SMs, the one-tile
    kernel for a non-causal one) agrees with the forced kernels within rounding."""
    from iree_turbine_b200 import _launcher as L

    for causal, b, h, s in [(True, 4, 37, 512), (False, 2, 8, 512)]:
        q, k, v = oracle.make_attention_inputs(b, h, h, s, s, 128, torch.bfloat16, seed=8, std=0.5)
        forced = _run(q, k, v, SCALE, causal)
        tb.ops.ATTENTION_KERNEL = L.ATTN_AUTO
        auto = _run(q, k, v, SCALE, causal)
        assert torch.allclose(auto.float(), forced.float(), rtol=1e-2, atol=1e-2)
        oracle.assert_close_half(auto[:1, :2], oracle.attention(q[:1, :2], k[:1, :2], v[:1, :2], SCALE, causal))


def test_one_tile_kernel_rejects_head_dim_64():
    import ctypes as C

    from iree_turbine_b200 import _launcher as L
    from iree_turbine_b200.ops import _fill_attention_args

    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device=DEV)
    a = _fill_attention_args(q, q, q, torch.empty_like(q), 0.125, False)
    a.kernel = L.ATTN_ONE_TILE
    assert L.lib().b200k_attention_fwd(C.byref(a), None) == L.ERR_BAD_SHAPE
    a.kernel = 7
    assert L.lib().b200k_attention_fwd(C.byref(a), None) == L.ERR_BAD_SHAPE


def _check_heads(o, q, k, v, causal, picks, group=1):
    for b, h in picks:
        ref = oracle.attention(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h // group:h // group + 1].cpu(),
                               v[b:b + 1, h // group:h // group + 1].cpu(), SCALE, causal)
        oracle.assert_close_half(o[b:b + 1, h:h + 1], ref)


def test_config_noncausal_f16_b8_h32_s1024():
    g = torch.Generator(device=DEV).manual_seed(10)
    q, k, v = (torch.randn(8, 32, 1024, 128, generator=g, device=DEV).half() for _ in range(3))
    kern = tb.get_vanilla_attention_kernel(tb.AttentionShape(32, 32, 128, 1024, 1024, 8), torch.float16)
    o = kern(q, k, v)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert o.shape == (8, 32, 1024, 128) and o.dtype == torch.float16
    _check_heads(o, q, k, v, False, [(0, 0), (3, 17), (7, 31), (5, 8)])
    # each output row is a convex combination of V rows: bounded by V's range per (b, h, d)
    assert bool((o.float() <= v.float().amax(dim=2, keepdim=True) + 1e-2).all())
    assert bool((o.float() >= v.float().amin(dim=2, keepdim=True) - 1e-2).all())


def test_config_causal_bf16_b4_h32_s4096():
    g = torch.Generator(device=DEV).manual_seed(10)
    q, k, v = ((torch.randn(4, 32, 4096, 128, generator=g, device=DEV) * 0.5).bfloat16() for _ in range(3))
    kern = tb.get_causal_attention_kernel(tb.AttentionShape(32, 32, 128, 4096, 4096, 4), torch.bfloat16)
    o = kern(q, k, v)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    _check_heads(o, q, k, v, True, [(0, 0), (3, 31), (1, 13)])
    # first query row sees only key 0: output row 0 equals V row 0 exactly (softmax of one element)
    assert torch.equal(o[:, :, 0], v[:, :, 0])
    # head sharding (what multi-GPU runs do) is bitwise the same as the full call
    o_shard = torch.ops.b200k.attention(q[:, 8:16], k[:, 8:16], v[:, 8:16], SCALE, True)
    assert torch.equal(o_shard, o[:, 8:16])


# ---- prefill over a paged K/V cache ----
def _paged_case(lens, sq, hq=8, hkv=2, page=16, dtype=torch.float16, seed=31):
    q0, k_cache, v_cache, block_table, seq_lens = oracle.make_paged_decode_inputs(
        q_heads=hq, kv_heads=hkv, page_size=page, lens=lens, dtype=dtype, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    q = (torch.randn(len(lens), hq, sq, 128, generator=g) * 0.5).to(dtype)
    return q, k_cache, v_cache, block_table, seq_lens


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("page", [16, 64, 128])
def test_paged_prefill_matches_oracle_and_dense_call(causal, page):
    lens = [300, 128, 517, 129, 40]
    sq = 40 if causal else 130
    q, kc, vc, bt, sl = _paged_case(lens, sq, page=page)
    o = torch.ops.b200k.paged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), SCALE, causal)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(o.cpu(), oracle.paged_attention(q, kc, vc, bt, sl, SCALE, causal))
    # the same kernel on the gathered, contiguous K/V of each sequence gives the same bits
    for i, n in enumerate(lens):
        kg = oracle.paged_gather(kc, bt[i:i + 1], sl[i:i + 1], n)
        vg = oracle.paged_gather(vc, bt[i:i + 1], sl[i:i + 1], n)
        od = torch.ops.b200k.attention(q[i:i + 1].to(DEV), kg.to(DEV), vg.to(DEV), SCALE, causal)
        assert torch.equal(od.cpu(), o[i:i + 1].cpu()), f"sequence {i}"


def test_paged_prefill_after_append_chunked():
    """Chunked prefill: append a chunk's K/V, attend causally over everything so far."""
    lens0, chunk = [64, 200, 0], 96
    total = [n + chunk for n in lens0]
    q, kc, vc, bt, sl = _paged_case(total, chunk, dtype=torch.bfloat16, seed=41)
    g = torch.Generator().manual_seed(5)
    k_new = torch.randn(3, chunk, 2, 128, generator=g).bfloat16()
    v_new = torch.randn(3, chunk, 2, 128, generator=g).bfloat16()
    pos = torch.tensor(lens0, dtype=torch.int32)
    k_ref, v_ref = oracle.kv_append(k_new, v_new, kc, vc, bt, pos)
    kd, vd = kc.to(DEV), vc.to(DEV)
    torch.ops.b200k.kv_append(k_new.to(DEV), v_new.to(DEV), kd, vd, bt.to(DEV), pos.to(DEV))
    o = torch.ops.b200k.paged_attention(q.to(DEV), kd, vd, bt.to(DEV), sl.to(DEV), SCALE, True)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(o.cpu(), oracle.paged_attention(q, k_ref, v_ref, bt, sl, SCALE, True))


def test_paged_prefill_zero_length_and_queries_before_first_key():
    q, kc, vc, bt, sl = _paged_case([0, 20], 64)
    o = torch.ops.b200k.paged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), SCALE, True)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert bool((o[0] == 0).all())                 # no keys at all
    assert bool((o[1, :, :44] == 0).all())         # queries 0..43 precede the first key (64 queries, 20 keys)
    oracle.assert_close_half(o.cpu(), oracle.paged_attention(q, kc, vc, bt, sl, SCALE, True))


def test_template_constructors_for_append_and_paged_prefill():
    lens0, chunk = [100, 37], 32
    total = [n + chunk for n in lens0]
    q, kc, vc, bt, sl = _paged_case(total, chunk, hq=8, hkv=2, dtype=torch.bfloat16, seed=51)
    shape = tb.AttentionShape(num_query_heads=8, num_kv_heads=2, head_size=128, query_seq_len=chunk,
                              num_seqs=2, block_size=16)
    g = torch.Generator().manual_seed(6)
    k_new = torch.randn(2, chunk, 2, 128, generator=g).bfloat16()
    v_new = torch.randn(2, chunk, 2, 128, generator=g).bfloat16()
    pos = torch.tensor(lens0, dtype=torch.int32)
    k_ref, v_ref = oracle.kv_append(k_new, v_new, kc, vc, bt, pos)
    kd, vd = kc.to(DEV), vc.to(DEV)
    tb.get_kv_append_kernel(shape, torch.bfloat16)(k_new.to(DEV), v_new.to(DEV), kd, vd, bt.to(DEV), pos.to(DEV))
    o = tb.get_paged_prefill_attention_kernel(shape, torch.bfloat16)(q.to(DEV), kd, vd, bt.to(DEV), sl.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(o.cpu(), oracle.paged_attention(q, k_ref, v_ref, bt, sl, SCALE, True))


def test_paged_prefill_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "paged_prefill_bf16.npz"))
    h = lambda n: torch.from_numpy(z[n].copy()).view(torch.bfloat16).to(DEV)  # noqa: E731
    bt, sl, pos = (torch.from_numpy(z[n]).to(DEV) for n in ("block_table", "seq_lens", "positions"))
    kc, vc = h("k_cache"), h("v_cache")
    torch.ops.b200k.kv_append(h("k_new"), h("v_new"), kc, vc, bt, pos)
    o = torch.ops.b200k.paged_attention(h("q"), kc, vc, bt, sl, float(z["scale"]), True)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert torch.equal(kc.cpu().view(torch.int16), torch.from_numpy(z["k_after"]))
    assert torch.equal(vc.cpu().view(torch.int16), torch.from_numpy(z["v_after"]))
    oracle.assert_close_half(o.cpu(), torch.from_numpy(z["o"]))
