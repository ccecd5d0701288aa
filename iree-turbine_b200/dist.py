"""Partitioning of the path over the GPUs of one box (one process per GPU, ``torch.distributed``).

Attention and decode shard along batch x head: every (batch, head) is an independent unit, so a
rank runs the ordinary op on its slice and no data-path collective exists.  The fp8 GEMM is
column-parallel over N: rank r holds rows [r*N/g, (r+1)*N/g) of B and all of A and computes the
matching columns of C; an all-gather of C runs only when the caller asks for the full matrix.

The slicing helpers are pure index arithmetic and are tested on CPU with gloo; the compute
callables are the registered ops (CUDA only).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

__all__ = ["shard_range", "head_shard", "column_parallel_gemm", "gather_columns", "ResultTurn",
           "FusedColumnParallelGemm"]


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced [lo, hi) slice of `total` units for `rank` (first total % world ranks get one extra)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def head_shard(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, world: int, rank: int):
    """Slices [B, H, S, D] tensors to this rank's KV heads and the query heads that read them."""
    hq, hkv = q.shape[1], k.shape[1]
    if hq % hkv:
        raise ValueError("query heads must be a multiple of kv heads")
    if hkv % world:
        raise ValueError(f"{hkv} kv heads cannot be split evenly over {world} ranks")
    group = hq // hkv
    lo, hi = shard_range(hkv, world, rank)
    return q[:, lo * group:hi * group], k[:, lo:hi], v[:, lo:hi]


def gather_columns(c_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers equal-width column blocks [M, N/g] into the full [M, N] on every rank.

    The collective gathers into a [g, M, N/g] staging tensor (contiguous per rank, which is what
    NCCL wants); one permuting copy then places the blocks side by side."""
    world = dist.get_world_size(group)
    if world == 1:
        return c_local
    c_local = c_local.contiguous()
    m, nl = c_local.shape
    stage = torch.empty((world * m, nl), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(stage, c_local, group=group)
    return stage.view(world, m, nl).permute(1, 0, 2).reshape(m, world * nl)


def column_parallel_gemm(gemm: Callable[[int, int], torch.Tensor], b_full_rows: int, world: int, rank: int,
                         gather: bool, group: Optional[dist.ProcessGroup] = None):
    """Runs ``gemm(b_rows_slice)`` for this rank's rows of B (= columns of C).

    ``gemm`` receives the (lo, hi) row range of B and returns C[:, lo:hi]; with ``gather`` the
    full C is assembled on every rank."""
    if b_full_rows % world:
        raise ValueError(f"N = {b_full_rows} is not divisible by {world} ranks")
    lo, hi = shard_range(b_full_rows, world, rank)
    c_local = gemm(lo, hi)
    return gather_columns(c_local, group) if gather else c_local


class ResultTurn:
    """Which of `n` result buffers a call uses: ``begin()`` hands out the next one, ``end()`` closes the
    call and names the buffer that now holds a finished result.  Every ``begin()`` must be closed by
    an ``end()`` before the next one, because the barrier in between is what makes the reuse safe."""

    def __init__(self, n: int = 2):
        if n < 2:
            raise ValueError("at least two buffers are needed for a result to outlive the next call")
        self.n = n
        self.calls = 0
        self.open = False

    @property
    def current(self) -> int:
        return (self.calls - 1) % self.n if self.calls else 0

    def begin(self) -> int:
        if self.open:
            raise RuntimeError("finish() of the previous call is missing: its barrier is what lets the "
                               "buffers alternate safely")
        self.open = True
        self.calls += 1
        return (self.calls - 1) % self.n

    def end(self) -> int:
        if not self.open:
            raise RuntimeError("finish() without a call")
        self.open = False
        return (self.calls - 1) % self.n


class FusedColumnParallelGemm:
    """Column-parallel C = A @ B^T whose all-gather is done by the GEMM kernel itself.

    Each rank holds all of A and ``n / world`` rows of B.  The full C lives in symmetric
    (peer-mapped) memory; the kernel's epilogue stores every tile of the local column shard into
    every rank's copy (``b200k_gemm_nt_allgather``), so the transfer over NVLink overlaps the math
    and there is no separate collective.  ``finish()`` is the cross-rank barrier after which every
    rank may read the full matrix.

    Reuse across calls.  ``finish()`` orders writes before reads; nothing orders a rank's reads of
    result i before a faster peer's stores of result i + 1.  The class therefore owns TWO result
    matrices and alternates between them: call i + 1 stores into the other matrix, and call i + 2
    (which reuses the first) cannot start on any rank before every rank has passed the barrier of
    call i + 1, which each rank enqueues after its own reads of result i.  So a result stays valid
    until the ``finish()`` of the NEXT call, provided it is read on the stream that made the calls;
    a caller that reads it from another stream must order that stream before its next ``finish()``.
    """

    def __init__(self, m: int, n: int, out_dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None,
                 multicast: bool = False, plain_stores: bool = False):
        """``multicast``: store each piece once to the NVSwitch multicast address of the result matrix
        (``multimem.st``; the switch replicates it to every rank) instead of once per peer.  Needs
        multicast support in the symmetric-memory allocation; raises if it is missing.
        ``plain_stores``: send the pieces with 16-byte stores from the epilogue warps instead of bulk
        tensor stores (same bits; the slower of the two per-peer forms)."""
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if n % self.world:
            raise ValueError(f"N = {n} is not divisible by {self.world} ranks")
        self.m, self.n = m, n
        dev = torch.device("cuda", torch.cuda.current_device())
        self.bufs = [symm_mem.empty((m, n), dtype=out_dtype, device=dev) for _ in range(2)]
        self.handles = [symm_mem.rendezvous(c, self.group) for c in self.bufs]
        self.multicast = bool(multicast)
        self.plain_stores = bool(plain_stores)
        if self.multicast and any(int(getattr(h, "multicast_ptr", 0) or 0) == 0 for h in self.handles):
            raise RuntimeError("FusedColumnParallelGemm: this symmetric-memory allocation has no multicast address")
        self.turn = ResultTurn(2)

    @property
    def c(self) -> torch.Tensor:
        """The result matrix of the current (or, before the first call, the next) call."""
        return self.bufs[self.turn.current]

    def __call__(self, a: torch.Tensor, b_local: torch.Tensor, scale_a=None, scale_b=None) -> torch.Tensor:
        import ctypes as C

        from . import _launcher as L
        from .ops import _row_major_2d, _status_ptr

        lo, hi = shard_range(self.n, self.world, self.rank)
        if b_local.size(0) != hi - lo or a.size(0) != self.m or a.size(1) != b_local.size(1):
            raise ValueError("operand shapes do not match the sharded problem")
        a, b_local = _row_major_2d(a), _row_major_2d(b_local)
        g = L.GemmAllGatherArgs()
        g.gemm.a, g.gemm.b, g.gemm.c = a.data_ptr(), b_local.data_ptr(), None
        g.gemm.m, g.gemm.n, g.gemm.k = self.m, hi - lo, a.size(1)
        g.gemm.lda, g.gemm.ldb, g.gemm.ldc = a.stride(0), b_local.stride(0), 0
        g.gemm.in_dtype = L.DTYPE_CODES[a.dtype]
        idx = self.turn.begin()
        c = self.bufs[idx]
        g.gemm.out_dtype = L.DTYPE_CODES[c.dtype]
        g.gemm.scale_a = scale_a.data_ptr() if scale_a is not None else None
        g.gemm.scale_b = scale_b.data_ptr() if scale_b is not None else None
        g.gemm.status = _status_ptr(a.device)
        for i, ptr in enumerate(self.handles[idx].buffer_ptrs):
            g.peer_c[i] = int(ptr)
        g.num_peers = self.world
        g.self_index = self.rank
        g.multicast_c = int(self.handles[idx].multicast_ptr) if self.multicast else None
        g.plain_stores = int(self.plain_stores)
        g.peer_ldc = c.stride(0)
        g.col_offset = lo
        stream = C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)
        with torch.cuda.device(a.device):
            L.check(L.lib().b200k_gemm_nt_allgather(C.byref(g), stream))
        return c

    def finish(self) -> torch.Tensor:
        """Cross-rank barrier on the current stream; afterwards the result of the last call is complete
        on every rank and stays valid until the ``finish()`` of the next call."""
        idx = self.turn.end()
        self.handles[idx].barrier()
        return self.bufs[idx]
