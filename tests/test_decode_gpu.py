"""Decode / paged-decode parity on the GPU vs. the CPU oracle.  Outputs: rtol = atol = 1e-2;
block-table index math: bit-exact (gather kernel vs. host gather; paged vs. contiguous run)."""

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


def _paged(q, kc, vc, bt, sl, scale=SCALE, chunk=0):
    o = torch.ops.b200k.paged_decode_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), sl.to(DEV), scale, chunk)
    torch.cuda.synchronize()
    return o


def test_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "paged_decode_f16.npz"))
    h = lambda n: torch.from_numpy(z[n].copy()).view(torch.float16)  # noqa: E731
    bt, sl = torch.from_numpy(z["block_table"]), torch.from_numpy(z["seq_lens"])
    o = _paged(h("q"), h("k_cache"), h("v_cache"), bt, sl, float(z["scale"]))
    oracle.assert_close_half(o, torch.from_numpy(z["o"]))
    assert torch.equal(o[4].cpu(), torch.zeros(8, 128, dtype=torch.float16)), "zero-length sequence must give zeros"
    gk = torch.ops.b200k.paged_gather(h("k_cache").to(DEV), bt.to(DEV), sl.to(DEV), int(sl.max()))
    assert torch.equal(gk.cpu().view(torch.int16), torch.from_numpy(z["gathered_k"]))


@pytest.mark.parametrize("q_heads,kv_heads", [(8, 8), (8, 2), (16, 2), (32, 8), (16, 1)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_group_sizes(q_heads, kv_heads, dtype):
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=6, q_heads=q_heads, kv_heads=kv_heads, min_len=1,
                                                        max_len=700, dtype=dtype, seed=1)
    oracle.assert_close_half(_paged(q, kc, vc, bt, sl), oracle.paged_decode_attention(q, kc, vc, bt, sl, SCALE))


@pytest.mark.parametrize("chunk", [64, 128, 256, 1024])
def test_chunk_sizes_agree(chunk):
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=5, q_heads=8, kv_heads=2, min_len=1, max_len=1500,
                                                        seed=2)
    oracle.assert_close_half(_paged(q, kc, vc, bt, sl, chunk=chunk),
                             oracle.paged_decode_attention(q, kc, vc, bt, sl, SCALE))


@pytest.mark.parametrize("page_size", [16, 32, 64])
def test_page_sizes(page_size):
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=4, q_heads=8, kv_heads=2, page_size=page_size,
                                                        lens=[1, page_size, page_size + 1, 5 * page_size - 3], seed=3)
    ref_k = oracle.paged_gather(kc, bt, sl, int(sl.max()))
    got_k = torch.ops.b200k.paged_gather(kc.to(DEV), bt.to(DEV), sl.to(DEV), int(sl.max()))
    assert torch.equal(got_k.cpu().view(torch.int16), ref_k.view(torch.int16))
    ref = oracle.decode_attention(q, ref_k, oracle.paged_gather(vc, bt, sl, int(sl.max())), sl, SCALE)
    oracle.assert_close_half(_paged(q, kc, vc, bt, sl), ref)


@pytest.mark.parametrize("q_heads,kv_heads", [(8, 8), (16, 2), (32, 8)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64(q_heads, kv_heads, dtype):
    """Head dim 64: paged decode against the oracle, the gather bit for bit, paged == contiguous bitwise."""
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=6, q_heads=q_heads, kv_heads=kv_heads, head_dim=64,
                                                        min_len=1, max_len=900, dtype=dtype, seed=11)
    scale = 0.125
    qd, kcd, vcd, btd, sld = (t.to(DEV) for t in (q, kc, vc, bt, sl))
    o = torch.ops.b200k.paged_decode_attention(qd, kcd, vcd, btd, sld, scale, 128)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    oracle.assert_close_half(o, oracle.paged_decode_attention(q, kc, vc, bt, sl, scale))
    max_len = bt.shape[1] * 16
    kg = torch.ops.b200k.paged_gather(kcd, btd, sld, max_len)
    vg = torch.ops.b200k.paged_gather(vcd, btd, sld, max_len)
    assert torch.equal(kg.cpu().view(torch.int16), oracle.paged_gather(kc, bt, sl, max_len).view(torch.int16))
    assert torch.equal(torch.ops.b200k.decode_attention(qd, kg, vg, sld, scale, 128), o)


def test_paged_equals_contiguous_bitwise():
    """Same tokens, same chunking: fetching through the block table must not change a single bit."""
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=7, q_heads=16, kv_heads=4, min_len=3, max_len=2100,
                                                        seed=4)
    max_len = bt.shape[1] * 16
    qd, kcd, vcd, btd, sld = (t.to(DEV) for t in (q, kc, vc, bt, sl))
    kg = torch.ops.b200k.paged_gather(kcd, btd, sld, max_len)
    vg = torch.ops.b200k.paged_gather(vcd, btd, sld, max_len)
    assert torch.equal(kg.cpu().view(torch.int16), oracle.paged_gather(kc, bt, sl, max_len).view(torch.int16))
    for chunk in (128, 512):
        o_paged = torch.ops.b200k.paged_decode_attention(qd, kcd, vcd, btd, sld, SCALE, chunk)
        o_contig = torch.ops.b200k.decode_attention(qd, kg, vg, sld, SCALE, chunk)
        torch.cuda.synchronize()
        assert torch.equal(o_paged, o_contig)
    oracle.assert_close_half(o_contig, oracle.decode_attention(q, kg.cpu(), vg.cpu(), sl, SCALE))


def test_contiguous_decode_with_padding_rows():
    q, k, v = oracle.make_attention_inputs(5, 8, 2, 1, 333, 128, torch.float16, seed=5)
    lens = torch.tensor([333, 1, 16, 200, 0], dtype=torch.int32)
    kern = tb.get_decode_attention_kernel(tb.AttentionShape(8, 2, 128, num_seqs=5))
    o = kern(q[:, :, 0].to(DEV), k.to(DEV), v.to(DEV), lens.to(DEV))
    torch.cuda.synchronize()
    oracle.assert_close_half(o, oracle.decode_attention(q[:, :, 0], k, v, lens, SCALE))


def test_out_of_range_page_is_ignored_not_dereferenced():
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=2, q_heads=8, kv_heads=2, lens=[40, 40], seed=6)
    bt2 = bt.clone()
    bt2[1, 1] = 10 ** 6  # far outside the pool
    o = _paged(q, kc, vc, bt2, sl)
    # sequence 0 is untouched; sequence 1 sees zeros for the bad page's 16 tokens (finite result)
    ref = oracle.paged_decode_attention(q, kc, vc, bt, sl, SCALE)
    oracle.assert_close_half(o[0], ref[0])
    assert bool(torch.isfinite(o[1].float()).all())


def test_length_above_the_table_capacity_is_cut_and_reported():
    """seq_lens is device data: an entry beyond what the block table (paged) or the history buffer
    (contiguous) holds is treated as that capacity and status bit 3 is raised; nothing is read past
    the table row and the reduction stays inside the sequence's own partials."""
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=3, q_heads=8, kv_heads=2, lens=[40, 100, 7], seed=8)
    cap = bt.shape[1] * 16  # 112 tokens: the last page of sequence 1 is full of (random) rows
    too_long = sl.clone()
    too_long[1] = 5000
    cut = sl.clone()
    cut[1] = cap
    tb.reset_device_status()
    o = _paged(q, kc, vc, bt, too_long, chunk=64)
    assert tb.device_status() == 8
    tb.reset_device_status()
    oracle.assert_close_half(o, oracle.paged_decode_attention(q, kc, vc, bt, cut, SCALE))
    assert torch.equal(o, _paged(q, kc, vc, bt, cut, chunk=64)), "the cut length must behave exactly like the capacity"
    assert tb.device_status() == 0
    # contiguous form: capacity = rows of the history buffer; a negative length counts as zero
    qc, k, v = oracle.make_attention_inputs(3, 8, 2, 1, 200, 128, torch.float16, seed=9)
    lens = torch.tensor([100000, 17, -5], dtype=torch.int32)
    oc = torch.ops.b200k.decode_attention(qc[:, :, 0].to(DEV), k.to(DEV), v.to(DEV), lens.to(DEV), SCALE)
    torch.cuda.synchronize()
    assert tb.device_status() == 8
    tb.reset_device_status()
    oracle.assert_close_half(oc, oracle.decode_attention(qc[:, :, 0], k, v, torch.tensor([200, 17, 0], dtype=torch.int32), SCALE))


def test_config_paged_decode_64_seqs():
    """64 sequences, 32 q-heads / 8 kv-heads, lengths U[512, 8192], page 16, permuted pool."""
    q, kc, vc, bt, sl = oracle.make_paged_decode_inputs(seed=10)
    assert q.shape == (64, 32, 128) and kc.shape[1:] == (8, 16, 128)
    kern = tb.get_paged_decode_attention_kernel(tb.AttentionShape(32, 8, 128, num_seqs=64, block_size=16))
    qd, kcd, vcd, btd, sld = (t.to(DEV) for t in (q, kc, vc, bt, sl))
    o = kern(qd, kcd, vcd, btd, sld)
    torch.cuda.synchronize()
    picks = [0, 17, 63, int(sl.argmax()), int(sl.argmin())]
    sub = torch.tensor(picks)
    ref = oracle.paged_decode_attention(q[sub], kc, vc, bt[sub], sl[sub], SCALE)
    oracle.assert_close_half(o[sub.to(DEV)], ref)
    # the gather is bit-exact for every sequence at full size (checksum of int16 patterns per row)
    max_len = bt.shape[1] * 16
    kg = torch.ops.b200k.paged_gather(kcd, btd, sld, max_len).cpu()
    ref_g = oracle.paged_gather(kc, bt, sl, max_len)
    assert torch.equal(kg.view(torch.int16), ref_g.view(torch.int16))
    # run-to-run determinism
    assert torch.equal(kern(qd, kcd, vcd, btd, sld), o)


# ---- KV-cache append (the step before decode) ----
@pytest.mark.parametrize("new_tokens", [1, 5, 40])
def test_kv_append_bit_exact_and_decodes(new_tokens):
    lens = [17, 64, 300, 1, 129]
    q, k_cache, v_cache, block_table, seq_lens = oracle.make_paged_decode_inputs(
        lens=[n + new_tokens for n in lens], seed=21)
    g = torch.Generator().manual_seed(22)
    k_new = torch.randn(len(lens), new_tokens, 8, 128, generator=g).half()
    v_new = torch.randn(len(lens), new_tokens, 8, 128, generator=g).half()
    positions = torch.tensor(lens, dtype=torch.int32)
    k_ref, v_ref = oracle.kv_append(k_new, v_new, k_cache, v_cache, block_table, positions)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    torch.ops.b200k.kv_append(k_new.to(DEV), v_new.to(DEV), kc, vc, block_table.to(DEV), positions.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert torch.equal(kc.cpu(), k_ref) and torch.equal(vc.cpu(), v_ref)
    # the appended cache decodes like the oracle's
    o = torch.ops.b200k.paged_decode_attention(q.to(DEV), kc, vc, block_table.to(DEV), seq_lens.to(DEV), SCALE)
    torch.cuda.synchronize()
    oracle.assert_close_half(o.cpu(), oracle.paged_decode_attention(q, k_ref, v_ref, block_table, seq_lens, SCALE))


def test_kv_append_outside_pool_is_dropped_and_reported():
    q, k_cache, v_cache, block_table, seq_lens = oracle.make_paged_decode_inputs(lens=[40, 40], seed=23)
    bad = block_table.clone()
    bad[1, 2] = -1  # tokens 32..47 of sequence 1 have no page
    k_new = torch.ones(2, 4, 8, 128).half()
    positions = torch.tensor([30, 30], dtype=torch.int32)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    tb.reset_device_status()
    torch.ops.b200k.kv_append(k_new.to(DEV), k_new.to(DEV), kc, vc, bad.to(DEV), positions.to(DEV))
    torch.cuda.synchronize()
    assert tb.device_status() == 4
    tb.reset_device_status()
    # sequence 0 and tokens 30, 31 of sequence 1 were written; nothing else changed
    k_ref, _ = oracle.kv_append(k_new[:1], k_new[:1], k_cache, v_cache, block_table[:1], positions[:1])
    k_ref, _ = oracle.kv_append(k_new[1:, :2], k_new[1:, :2], k_ref, v_cache, block_table[1:], positions[1:])
    assert torch.equal(kc.cpu(), k_ref)
