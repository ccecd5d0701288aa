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

__all__ = ["shard_range", "head_shard", "column_parallel_gemm", "gather_columns"]


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


def column_parallel_gemm(gemm: Callable[[torch.Tensor], torch.Tensor], b_full_rows: int, world: int, rank: int,
                         gather: bool, group: Optional[dist.ProcessGroup] = None):
    """Runs ``gemm(b_rows_slice)`` for this rank's rows of B (= columns of C).

    ``gemm`` receives the (lo, hi) row range of B and returns C[:, lo:hi]; with ``gather`` the
    full C is assembled on every rank."""
    if b_full_rows % world:
        raise ValueError(f"N = {b_full_rows} is not divisible by {world} ranks")
    lo, hi = shard_range(b_full_rows, world, rank)
    c_local = gemm(lo, hi)
    return gather_columns(c_local, group) if gather else c_local
