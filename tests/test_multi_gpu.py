"""Multi-GPU paths on real GPUs (needs >= 2 devices; skipped otherwise): the fused column-parallel
GEMM + all-gather through peer-mapped memory, the NCCL gather it replaces, and head-sharded
attention.  Each rank is its own process (spawned here), one GPU each, NCCL over NVLink."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import iree_turbine_b200  # noqa: F401
        from iree_turbine_b200 import dist as tdist
        from oracle import oracle

        m, n, k = 384, 512 * world, 256
        a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(m, n, k, seed=9)
        ref = oracle.gemm_fp8_nt(a8, b8, sa, sb)
        lo, hi = tdist.shard_range(n, world, rank)
        ad, bd, sad, sbd = a8.to(dev), b8[lo:hi].to(dev), sa.to(dev), sb.to(dev)

        fused = tdist.FusedColumnParallelGemm(m, n, torch.bfloat16)
        for buf in fused.bufs:
            buf.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        fused(ad, bd, sad, sbd)
        first = fused.finish()
        c_fused = first.clone()
        # a second call (other operands) goes to the other result matrix: the first result is still
        # intact after it, which is what lets a slow reader overlap a fast peer's next call
        a2, b2, sa2, sb2 = oracle.make_fp8_gemm_inputs(m, n, k, seed=19)
        fused(a2.to(dev), b2[lo:hi].to(dev), sa2.to(dev), sb2.to(dev))
        second = fused.finish()
        torch.cuda.synchronize()
        fro2, mx2 = oracle.fp8_errors(second, oracle.gemm_fp8_nt(a2, b2, sa2, sb2))
        fro, mx = oracle.fp8_errors(c_fused, ref)
        ok_fused = (fro <= 3e-2 and mx <= 3e-2 and fro2 <= 3e-2 and mx2 <= 3e-2
                    and second.data_ptr() != first.data_ptr() and torch.equal(first, c_fused))

        # the same exchange through the NVSwitch multicast address (one multimem.st per piece), where
        # the allocation has one: identical bits
        ok_mc = True
        try:
            fused_mc = tdist.FusedColumnParallelGemm(m, n, torch.bfloat16, multicast=True)
        except RuntimeError:
            fused_mc = None
        if fused_mc is not None:
            for buf in fused_mc.bufs:
                buf.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            fused_mc(ad, bd, sad, sbd)
            ok_mc = torch.equal(fused_mc.finish(), c_fused)
            torch.cuda.synchronize()

        # the same exchange with 16-byte stores from the epilogue warps instead of bulk tensor stores:
        # identical bits (ragged shard width too: 520 columns per rank is not a multiple of a 128-byte piece)
        fused_plain = tdist.FusedColumnParallelGemm(m, n, torch.bfloat16, plain_stores=True)
        for buf in fused_plain.bufs:
            buf.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        fused_plain(ad, bd, sad, sbd)
        ok_mc = ok_mc and torch.equal(fused_plain.finish(), c_fused)
        torch.cuda.synchronize()
        n3 = 520 * world
        a3, b3, sa3, sb3 = oracle.make_fp8_gemm_inputs(300, n3, k, seed=29)
        lo3, hi3 = tdist.shard_range(n3, world, rank)
        outs = []
        for plain in (False, True):
            f3 = tdist.FusedColumnParallelGemm(300, n3, torch.bfloat16, plain_stores=plain)
            for buf in f3.bufs:
                buf.fill_(-7.0)
            torch.cuda.synchronize()
            dist.barrier()
            f3(a3.to(dev), b3[lo3:hi3].to(dev), sa3.to(dev), sb3.to(dev))
            outs.append(f3.finish().clone())
            torch.cuda.synchronize()
        fro3, mx3 = oracle.fp8_errors(outs[0], oracle.gemm_fp8_nt(a3, b3, sa3, sb3))
        ok_mc = ok_mc and torch.equal(outs[0], outs[1]) and fro3 <= 3e-2 and mx3 <= 3e-2

        # the unfused baseline: local GEMM, then NCCL all-gather + de-interleave
        c_nccl = tdist.column_parallel_gemm(lambda l, h: torch.ops.b200k.gemm_fp8_nt(ad, bd, sad, sbd), n, world, rank,
                                            gather=True)
        ok_same = torch.equal(c_nccl, c_fused)

        # head-sharded attention: a rank's slice equals the same heads of the unsharded result
        q, kk, v = oracle.make_attention_inputs(1, 2 * world, world, 256, 256, 128, torch.float16, seed=3, std=0.5)
        qs, ks, vs = tdist.head_shard(q, kk, v, world, rank)
        o = torch.ops.b200k.attention(qs.to(dev), ks.to(dev), vs.to(dev), 0.1, True)
        full = oracle.attention(q, kk, v, 0.1, True)
        hl, hh = tdist.shard_range(world, world, rank)
        ok_attn = torch.allclose(o.float().cpu(), full[:, hl * 2:hh * 2], rtol=1e-2, atol=1e-2)
        torch.cuda.synchronize()
        results[rank] = (ok_fused, ok_same and ok_mc, ok_attn, float(fro))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_column_parallel_gemm_and_head_sharding():
    world = min(torch.cuda.device_count(), 4)
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for r in range(world):
            assert results[r][:3] == (True, True, True), (r, results[r])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_one_process_drives_two_devices():
    """Every kernel family on cuda:1 after cuda:0 has been used by the same process, with cuda:0
    still the current device: per-device state (the opt-in to large dynamic shared memory, the
    status word, the launch device) must follow the tensors."""
    import iree_turbine_b200 as tb
    from oracle import oracle

    scale = 128 ** -0.5
    q, k, v = oracle.make_attention_inputs(1, 4, 2, 256, 256, 128, torch.bfloat16, seed=31, std=0.5)
    d_o = torch.randn(q.shape, generator=torch.Generator().manual_seed(32)).to(q.dtype)
    a, b = oracle.make_gemm_inputs(256, 384, 192, torch.float16, seed=33)
    a8, b8, sa, sb = oracle.make_fp8_gemm_inputs(128, 256, 256, seed=34)
    qd, kc, vc, bt, sl = oracle.make_paged_decode_inputs(num_seqs=4, q_heads=8, kv_heads=2, min_len=1, max_len=300, seed=35)
    ref_o = oracle.attention(q, k, v, scale, True)
    ref_g = oracle.attention_bwd(q, k, v, d_o, scale, True)
    ref_c = oracle.gemm_nt(a, b)
    ref_c8 = oracle.gemm_fp8_nt(a8, b8, sa, sb)
    ref_d = oracle.paged_decode_attention(qd, kc, vc, bt, sl, scale)
    torch.cuda.set_device(0)
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        t = lambda x: x.to(dev)  # noqa: E731
        o, lse = torch.ops.b200k.attention_lse(t(q), t(k), t(v), scale, True)
        grads = torch.ops.b200k.attention_bwd(t(q), t(k), t(v), o, t(d_o), scale, True, lse)
        c = torch.ops.b200k.gemm_nt(t(a), t(b))
        c8 = torch.ops.b200k.gemm_fp8_nt(t(a8), t(b8), t(sa), t(sb))
        od = torch.ops.b200k.paged_decode_attention(t(qd), t(kc), t(vc), t(bt), t(sl), scale)
        torch.cuda.synchronize(dev)
        assert o.device == dev and c.device == dev
        oracle.assert_close_half(o, ref_o)
        for got, ref in zip(grads, ref_g):
            assert (got.float().cpu() - ref).abs().max().item() <= 1e-2 * max(ref.abs().max().item(), 1.0)
        oracle.assert_close_half(c, ref_c)
        fro, mx = oracle.fp8_errors(c8, ref_c8)
        assert fro <= 3e-2 and mx <= 3e-2
        oracle.assert_close_half(od, ref_d)
        assert tb.device_status(dev) == 0
    assert torch.cuda.current_device() == 0
