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
        fused.c.zero_()
        fused.finish()
        fused(ad, bd, sad, sbd)
        c_fused = fused.finish().clone()
        torch.cuda.synchronize()
        fro, mx = oracle.fp8_errors(c_fused, ref)
        ok_fused = fro <= 3e-2 and mx <= 3e-2

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
        results[rank] = (ok_fused, ok_same, ok_attn, float(fro))
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
