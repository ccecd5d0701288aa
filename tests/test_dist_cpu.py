"""Sharding helpers on CPU: index arithmetic, and a world-size-2 gloo run of the column gather
and of head-sharded attention (oracle as the per-rank compute) against the unsharded result."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from iree_turbine_b200 import dist as tdist
from oracle import oracle


def test_shard_range_covers_and_balances():
    for total in (0, 1, 7, 8, 32, 8192):
        for world in (1, 2, 3, 8):
            spans = [tdist.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        tdist.shard_range(8, 2, 2)


def test_head_shard_keeps_groups_together():
    q = torch.arange(2 * 8 * 3 * 4).reshape(2, 8, 3, 4)
    k = torch.arange(2 * 2 * 5 * 4).reshape(2, 2, 5, 4)
    qs, ks, vs = tdist.head_shard(q, k, k, 2, 1)
    assert torch.equal(qs, q[:, 4:8]) and torch.equal(ks, k[:, 1:2]) and torch.equal(vs, k[:, 1:2])
    with pytest.raises(ValueError):
        tdist.head_shard(q, k, k, 4, 0)


def test_result_buffers_alternate_and_need_the_barrier_in_between():
    turn = tdist.ResultTurn(2)
    assert turn.current == 0
    seen = []
    for _ in range(5):
        b = turn.begin()
        assert turn.current == b
        with pytest.raises(RuntimeError, match="finish"):
            turn.begin()  # the barrier of the open call has not been enqueued yet
        assert turn.end() == b and turn.current == b
        seen.append(b)
    assert seen == [0, 1, 0, 1, 0]  # a result is overwritten two calls later, never by the next one
    with pytest.raises(RuntimeError):
        turn.end()
    with pytest.raises(ValueError):
        tdist.ResultTurn(1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # column-parallel GEMM + gather == full GEMM
        a, b = oracle.make_gemm_inputs(24, 16, 32, torch.float16, seed=1)
        full = oracle.gemm_nt(a, b)
        got = tdist.column_parallel_gemm(lambda lo, hi: oracle.gemm_nt(a, b[lo:hi]), 16, world, rank, gather=True)
        ok_gemm = torch.equal(got, full)
        local = tdist.column_parallel_gemm(lambda lo, hi: oracle.gemm_nt(a, b[lo:hi]), 16, world, rank, gather=False)
        lo, hi = tdist.shard_range(16, world, rank)
        ok_local = torch.equal(local, full[:, lo:hi])
        # head-sharded attention needs no communication: each rank's slice equals the full result's slice
        q, k, v = oracle.make_attention_inputs(1, 4, 2, 40, 40, 128, torch.float16, seed=2)
        qs, ks, vs = tdist.head_shard(q, k, v, world, rank)
        o = oracle.attention(qs, ks, vs, 0.1, True)
        o_full = oracle.attention(q, k, v, 0.1, True)
        hl, hh = tdist.shard_range(2, world, rank)
        ok_attn = torch.allclose(o, o_full[:, hl * 2:hh * 2], rtol=0, atol=1e-6)
        results[rank] = (ok_gemm, ok_local, ok_attn)
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for r in range(world):
            assert results[r] == (True, True, True), (r, results[r])
