"""The decode entry point that brings its own scratch (b200k_decode_attention_static).

Some users of the C ABI cannot give the library scratch memory: a host runtime that passes a
plug-in only input and output buffers and owns every device allocation itself, or a request loop
that runs inside a fixed memory plan and must not call cudaMalloc.  For them the library keeps the
split-KV partial results in an array inside its own image.  This test drives that entry point
directly through ctypes -- the output tensors are the only memory the caller provides -- and
checks it against the ordinary entry point (caller-provided workspace) on two calls in a row with
different inputs, since every call shares the one array and sees what the previous call left.
It lives in a file that sorts last so a run that stops at the first failure has already run
everything else.
"""

import ctypes as C

import pytest
import torch

from iree_turbine_b200 import _launcher as L
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCALE = 128 ** -0.5


def _args(q, kc, vc, bt, sl, o, chunk):
    a = L.DecodeArgs()
    a.q, a.k_cache, a.v_cache, a.o = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr()
    a.block_table, a.seq_lens = bt.data_ptr(), sl.data_ptr()
    a.num_seqs, a.q_heads, a.head_dim = q.size(0), q.size(1), q.size(2)
    a.kv_heads, a.page_size, a.num_pages = kc.size(1), kc.size(2), kc.size(0)
    a.block_table_stride = bt.stride(0)
    a.max_seq_len = bt.size(1) * kc.size(2)
    a.kv_page_stride, a.kv_head_stride = kc.stride(0), kc.stride(1)
    a.dtype = L.DTYPE_CODES[q.dtype]
    a.chunk_tokens = chunk
    a.scale = SCALE
    return a


def _both(lib, seed, num_seqs, max_len, chunk):
    host = oracle.make_paged_decode_inputs(num_seqs=num_seqs, q_heads=16, kv_heads=4, min_len=1, max_len=max_len,
                                           seed=seed)
    q, kc, vc, bt, sl = (t.to(DEV) for t in host)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # existing entry point: caller-provided workspace
    o_ref = torch.empty_like(q)
    a = _args(q, kc, vc, bt, sl, o_ref, chunk)
    need = lib.b200k_decode_workspace_bytes(C.byref(a))
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    L.check(lib.b200k_decode_attention(C.byref(a), stream))

    # new entry point: no workspace given at all
    o_new = torch.full_like(q, float("nan"))
    b = _args(q, kc, vc, bt, sl, o_new, chunk)
    assert need <= L.DECODE_STATIC_SCRATCH_BYTES
    L.check(lib.b200k_decode_attention_static(C.byref(b), stream))
    torch.cuda.synchronize()
    return host, o_ref, o_new


def test_static_scratch_decode_matches_the_workspace_entry_point(kernel_lib):
    lib = kernel_lib
    # two calls in a row, second one smaller and with a different chunking, so it runs on top of
    # whatever the first left in the shared array
    for seed, num_seqs, max_len, chunk in [(21, 9, 3000, 256), (22, 5, 700, 64)]:
        host, o_ref, o_new = _both(lib, seed, num_seqs, max_len, chunk)
        # same kernels, same chunking: the tolerance of the decode tests (1e-2) is far looser than
        # what is observed, which is bitwise equality
        oracle.assert_close_half(o_new, o_ref.float().cpu(), rtol=1e-2, atol=1e-2)
        assert torch.equal(o_new, o_ref)
        q, kc, vc, bt, sl = host
        oracle.assert_close_half(o_new, oracle.paged_decode_attention(q, kc, vc, bt, sl, SCALE))


def test_static_scratch_decode_cuts_a_length_beyond_the_table(kernel_lib):
    """A seq_lens entry above the block table's capacity must not make the reduction walk into the
    next head's slots of the shared array: it is cut to the capacity and reported (status bit 3)."""
    lib = kernel_lib
    host = oracle.make_paged_decode_inputs(num_seqs=3, q_heads=16, kv_heads=4, lens=[33, 90, 5], seed=23)
    q, kc, vc, bt, sl = (t.to(DEV) for t in host)
    cap = bt.size(1) * kc.size(2)
    bad = host[4].clone()
    bad[1] = 10 ** 6
    cut = host[4].clone()
    cut[1] = cap
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for lens in (bad, cut):
        o = torch.full_like(q, float("nan"))
        a = _args(q, kc, vc, bt, lens.to(DEV), o, 64)
        a.status = status.data_ptr()
        L.check(lib.b200k_decode_attention_static(C.byref(a), stream))
        torch.cuda.synchronize()
        outs.append((o, int(status.item())))
        status.zero_()
    assert outs[0][1] == 8 and outs[1][1] == 0
    assert torch.equal(outs[0][0], outs[1][0])
    oracle.assert_close_half(outs[0][0], oracle.paged_decode_attention(host[0], host[1], host[2], host[3], cut, SCALE))


def test_static_scratch_decode_rejects_oversized_problems(kernel_lib):
    lib = kernel_lib
    # 4096 sequences x 32 heads x 16 chunks of 64 tokens needs ~1 GB of partials: far over the limit.
    a = L.DecodeArgs()
    a.q = a.k_cache = a.v_cache = a.seq_lens = a.o = a.block_table = 0x1000  # never dereferenced: rejected first
    a.num_seqs, a.q_heads, a.kv_heads, a.head_dim = 4096, 32, 8, 128
    a.page_size, a.num_pages, a.block_table_stride, a.max_seq_len = 16, 1 << 20, 64, 1024
    a.kv_page_stride, a.kv_head_stride = 8 * 16 * 128, 16 * 128
    a.dtype, a.chunk_tokens, a.scale = L.F16, 64, SCALE
    assert lib.b200k_decode_workspace_bytes(C.byref(a)) > L.DECODE_STATIC_SCRATCH_BYTES
    rc = lib.b200k_decode_attention_static(C.byref(a), None)
    assert rc == L.ERR_WORKSPACE
    msg = lib.b200k_last_error().decode()
    assert "built-in array" in msg and str(L.DECODE_STATIC_SCRATCH_BYTES) in msg
