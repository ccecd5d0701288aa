"""Problem-shape dataclasses consumed by the kernel template constructors.

The reference's Wave templates take a plain dataclass of problem dimensions (``AttentionShape``
and siblings) next to the tensors; that package is not part of the reference checkout this
library was built against, so the field names here are this library's own and are documented in
full.  Each field is one dimension of the problems the templates cover.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

__all__ = ["GemmShape", "AttentionShape", "DecodeShape"]


@dataclass(frozen=True)
class GemmShape:
    """C[m, n] = A[m, k] @ B[n, k]^T."""

    m: int
    n: int
    k: int

    @property
    def flops(self) -> int:
        return 2 * self.m * self.n * self.k


@dataclass(frozen=True)
class AttentionShape:
    """Dimensions of one attention problem.

    num_query_heads / num_kv_heads: heads of Q and of K/V (grouped-query when they differ);
    head_size: QK head dimension; head_size_kv: V head dimension (defaults to head_size);
    query_seq_len / kv_seq_len: rows of Q and of K/V per (batch, head); num_seqs: batch;
    block_size: tokens per KV page (paged decode only); max_seq_len: longest KV history a
    decode call may see (sizes scratch and the launch grid).
    """

    num_query_heads: int
    num_kv_heads: int
    head_size: int
    query_seq_len: int = 1
    kv_seq_len: int = 0
    num_seqs: int = 1
    head_size_kv: Optional[int] = None
    block_size: Optional[int] = None
    max_seq_len: Optional[int] = None

    def __post_init__(self):
        if self.head_size_kv is None:
            object.__setattr__(self, "head_size_kv", self.head_size)
        if self.num_query_heads % self.num_kv_heads != 0:
            raise ValueError("num_query_heads must be a multiple of num_kv_heads")

    @property
    def group_size(self) -> int:
        return self.num_query_heads // self.num_kv_heads

    def flops(self, causal: bool = False) -> int:
        """QK^T plus PV multiply-adds; a causal problem counts half (softmax is not counted)."""
        f = 4 * self.num_seqs * self.num_query_heads * self.query_seq_len * self.kv_seq_len * self.head_size
        return f // 2 if causal else f


# Decode problems are attention problems with query_seq_len == 1.
DecodeShape = AttentionShape
