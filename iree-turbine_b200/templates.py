"""Kernel template constructors: ``get_*_kernel(shape, ...) -> callable``.

In the reference a Wave template constructor takes a shape dataclass plus dtypes and returns a
launchable kernel object that is later called with torch tensors; the nearest in-tree analogue
of "kernel object exposed as a registered op" is ``tk.gen.kernel``
(iree/turbine/kernel/gen/kernel.py:44-154).  Here a constructor binds a shape and dtype, checks
them once against what the sm_100a kernels implement, and returns a small callable that
validates the tensors it is given against the bound shape and dispatches to the registered op
(``torch.ops.b200k.*``).  Nothing is compiled at construction time.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import ops as _ops  # noqa: F401  (registers torch.ops.b200k.*)
from .shapes import AttentionShape, GemmShape

__all__ = [
    "LaunchableKernel",
    "get_gemm_kernel",
    "get_fp8_gemm_kernel",
    "get_vanilla_attention_kernel",
    "get_causal_attention_kernel",
    "get_decode_attention_kernel",
    "get_paged_decode_attention_kernel",
    "get_paged_prefill_attention_kernel",
    "get_kv_append_kernel",
]

_HALF = (torch.float16, torch.bfloat16)


@dataclass(frozen=True)
class LaunchableKernel:
    """A bound kernel: ``kernel(*tensors)`` runs it on the current CUDA stream."""

    name: str
    shape: object
    dtype: torch.dtype
    _fn: Callable

    def __call__(self, *tensors):
        return self._fn(*tensors)


def _expect(t: torch.Tensor, shape: tuple, dtype: torch.dtype, what: str):
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{what}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    if t.dtype != dtype:
        raise ValueError(f"{what}: expected dtype {dtype}, got {t.dtype}")


def get_gemm_kernel(shape: GemmShape, dtype: torch.dtype = torch.float16,
                    out_dtype: Optional[torch.dtype] = None) -> LaunchableKernel:
    """C[m,n] = A[m,k] @ B[n,k]^T, f16/bf16 operands, fp32 accumulate; C fp32 unless out_dtype is given."""
    if dtype not in _HALF:
        raise ValueError(f"get_gemm_kernel: dtype must be float16 or bfloat16, got {dtype}")
    if shape.k % 8:
        raise ValueError("get_gemm_kernel: k must be a multiple of 8")

    def run(a, b):
        _expect(a, (shape.m, shape.k), dtype, "a")
        _expect(b, (shape.n, shape.k), dtype, "b")
        return torch.ops.b200k.gemm_nt(a, b, out_dtype)

    return LaunchableKernel("gemm_nt", shape, dtype, run)


def get_fp8_gemm_kernel(shape: GemmShape, out_dtype: torch.dtype = torch.bfloat16) -> LaunchableKernel:
    """C = (A8 @ B8^T) * scale_a * scale_b with float8_e4m3fn operands and per-tensor scales."""
    if shape.k % 16:
        raise ValueError("get_fp8_gemm_kernel: k must be a multiple of 16")

    def run(a, b, scale_a, scale_b):
        _expect(a, (shape.m, shape.k), torch.float8_e4m3fn, "a")
        _expect(b, (shape.n, shape.k), torch.float8_e4m3fn, "b")
        return torch.ops.b200k.gemm_fp8_nt(a, b, scale_a, scale_b, out_dtype)

    return LaunchableKernel("gemm_fp8_nt", shape, torch.float8_e4m3fn, run)


def _attention_kernel(shape: AttentionShape, dtype: torch.dtype, causal: bool, scale: Optional[float]):
    if dtype not in _HALF:
        raise ValueError(f"attention: dtype must be float16 or bfloat16, got {dtype}")
    if shape.head_size not in (64, 128) or shape.head_size_kv != shape.head_size:
        raise ValueError("attention: head_size must be 128 or 64, and head_size_kv equal to it")
    sc = shape.head_size ** -0.5 if scale is None else float(scale)
    qs = (shape.num_seqs, shape.num_query_heads, shape.query_seq_len, shape.head_size)
    ks = (shape.num_seqs, shape.num_kv_heads, shape.kv_seq_len, shape.head_size)

    def run(q, k, v):
        _expect(q, qs, dtype, "q")
        _expect(k, ks, dtype, "k")
        _expect(v, ks, dtype, "v")
        return torch.ops.b200k.attention(q, k, v, sc, causal)

    return LaunchableKernel("causal_attention" if causal else "vanilla_attention", shape, dtype, run)


def get_vanilla_attention_kernel(shape: AttentionShape, dtype: torch.dtype = torch.float16,
                                 scale: Optional[float] = None) -> LaunchableKernel:
    """softmax(scale * Q K^T) V over [num_seqs, heads, seq, head_size] tensors, head_size 128 or 64
    (scale defaults to head_size^-0.5)."""
    return _attention_kernel(shape, dtype, False, scale)


def get_causal_attention_kernel(shape: AttentionShape, dtype: torch.dtype = torch.bfloat16,
                                scale: Optional[float] = None) -> LaunchableKernel:
    """As the vanilla kernel with a lower-triangular mask (last query aligned with last key)."""
    return _attention_kernel(shape, dtype, True, scale)


def get_decode_attention_kernel(shape: AttentionShape, dtype: torch.dtype = torch.float16,
                                scale: Optional[float] = None, chunk_tokens: int = 0) -> LaunchableKernel:
    """Split-KV decode against contiguous KV: kernel(q, k, v, seq_lens)."""
    if shape.head_size not in (64, 128):
        raise ValueError("decode attention: head_size must be 128 or 64")
    sc = shape.head_size ** -0.5 if scale is None else float(scale)

    def run(q, k, v, seq_lens):
        _expect(q, (shape.num_seqs, shape.num_query_heads, shape.head_size), dtype, "q")
        if k.shape[:2] != (shape.num_seqs, shape.num_kv_heads):
            raise ValueError(f"k: expected leading dims {(shape.num_seqs, shape.num_kv_heads)}, got {tuple(k.shape[:2])}")
        return torch.ops.b200k.decode_attention(q, k, v, seq_lens, sc, chunk_tokens)

    return LaunchableKernel("decode_attention", shape, dtype, run)


def get_paged_decode_attention_kernel(shape: AttentionShape, dtype: torch.dtype = torch.float16,
                                      scale: Optional[float] = None, chunk_tokens: int = 0) -> LaunchableKernel:
    """Split-KV decode through a block table: kernel(q, k_cache, v_cache, block_table, seq_lens)."""
    if shape.head_size not in (64, 128):
        raise ValueError("paged decode attention: head_size must be 128 or 64")
    if not shape.block_size or shape.block_size % 16:
        raise ValueError("paged decode attention: block_size must be a positive multiple of 16")
    sc = shape.head_size ** -0.5 if scale is None else float(scale)

    def run(q, k_cache, v_cache, block_table, seq_lens):
        _expect(q, (shape.num_seqs, shape.num_query_heads, shape.head_size), dtype, "q")
        if tuple(k_cache.shape[1:]) != (shape.num_kv_heads, shape.block_size, shape.head_size):
            raise ValueError(
                f"k_cache: expected [pages, {shape.num_kv_heads}, {shape.block_size}, {shape.head_size}], "
                f"got {tuple(k_cache.shape)}"
            )
        return torch.ops.b200k.paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, sc, chunk_tokens)

    return LaunchableKernel("paged_decode_attention", shape, dtype, run)


def get_paged_prefill_attention_kernel(shape: AttentionShape, dtype: torch.dtype = torch.bfloat16,
                                       causal: bool = True, scale: Optional[float] = None) -> LaunchableKernel:
    """Prefill (or one chunk of it) over the paged cache: kernel(q, k_cache, v_cache, block_table, seq_lens)
    with q [num_seqs, heads, query_seq_len, head_size]; the queries of a sequence are its last query_seq_len tokens."""
    if shape.head_size not in (64, 128):
        raise ValueError("paged prefill attention: head_size must be 128 or 64")
    if shape.block_size not in (16, 32, 64, 128):
        raise ValueError("paged prefill attention: block_size must be 16, 32, 64 or 128")
    sc = shape.head_size ** -0.5 if scale is None else float(scale)

    def run(q, k_cache, v_cache, block_table, seq_lens):
        _expect(q, (shape.num_seqs, shape.num_query_heads, shape.query_seq_len, shape.head_size), dtype, "q")
        if tuple(k_cache.shape[1:]) != (shape.num_kv_heads, shape.block_size, shape.head_size):
            raise ValueError(
                f"k_cache: expected [pages, {shape.num_kv_heads}, {shape.block_size}, {shape.head_size}], "
                f"got {tuple(k_cache.shape)}"
            )
        return torch.ops.b200k.paged_attention(q, k_cache, v_cache, block_table, seq_lens, sc, causal)

    return LaunchableKernel("paged_prefill_attention", shape, dtype, run)


def get_kv_append_kernel(shape: AttentionShape, dtype: torch.dtype = torch.bfloat16) -> LaunchableKernel:
    """kernel(k_new, v_new, k_cache, v_cache, block_table, positions): writes query_seq_len new rows per
    sequence into the paged cache at token positions positions[s] + t (in place)."""
    if shape.block_size is None or shape.block_size <= 0:
        raise ValueError("kv append: block_size is required")

    def run(k_new, v_new, k_cache, v_cache, block_table, positions):
        _expect(k_new, (shape.num_seqs, shape.query_seq_len, shape.num_kv_heads, shape.head_size), dtype, "k_new")
        torch.ops.b200k.kv_append(k_new, v_new, k_cache, v_cache, block_table, positions)
        return None

    return LaunchableKernel("kv_append", shape, dtype, run)
