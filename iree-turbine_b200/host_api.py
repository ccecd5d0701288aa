"""Host-buffer entry points: the same kernels called with HOST tensors.

``AttentionHost`` / ``GemmHost`` own device staging buffers for one problem shape; a call copies
the (ideally pinned) host inputs to the device, launches, and copies the result into the host
output tensor -- all asynchronously on the current stream through one C-ABI call
(``b200k_attention_fwd_host`` / ``b200k_gemm_nt_host``).  Synchronize the stream before reading
the output.  This is the path a caller without device-resident tensors uses, and what the
benchmark's end-to-end number measures.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _launcher as L
from .ops import _fill_attention_args, _status_ptr

__all__ = ["AttentionHost", "GemmHost"]


def _check_host(t: torch.Tensor, shape, dtype, what: str):
    if t.device.type != "cpu":
        raise ValueError(f"{what}: expected a host tensor")
    if tuple(t.shape) != tuple(shape) or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{what}: expected contiguous {tuple(shape)} {dtype}, got {tuple(t.shape)} {t.dtype}")


class AttentionHost:
    def __init__(self, batch, q_heads, kv_heads, seq_q, seq_kv, dtype, device, head_dim: int = 128):
        self.device = torch.device(device)
        self.dtype = dtype
        self.qs = (batch, q_heads, seq_q, head_dim)
        self.ks = (batch, kv_heads, seq_kv, head_dim)
        self.dq = torch.empty(self.qs, dtype=dtype, device=self.device)
        self.dk = torch.empty(self.ks, dtype=dtype, device=self.device)
        self.dv = torch.empty(self.ks, dtype=dtype, device=self.device)
        self.do = torch.empty(self.qs, dtype=dtype, device=self.device)

    def __call__(self, q, k, v, out, scale: float, causal: bool):
        _check_host(q, self.qs, self.dtype, "q")
        _check_host(k, self.ks, self.dtype, "k")
        _check_host(v, self.ks, self.dtype, "v")
        _check_host(out, self.qs, self.dtype, "out")
        dev = _fill_attention_args(self.dq, self.dk, self.dv, self.do, scale, causal)
        dev.status = _status_ptr(self.device)
        host = _fill_attention_args(q, k, v, out, scale, causal)
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            L.check(L.lib().b200k_attention_fwd_host(C.byref(host), C.byref(dev), stream))
        return out


class GemmHost:
    def __init__(self, m, n, k, in_dtype, out_dtype, device):
        self.device = torch.device(device)
        self.m, self.n, self.k = m, n, k
        self.in_dtype, self.out_dtype = in_dtype, out_dtype
        self.da = torch.empty((m, k), dtype=in_dtype, device=self.device)
        self.db = torch.empty((n, k), dtype=in_dtype, device=self.device)
        self.dc = torch.empty((m, n), dtype=out_dtype, device=self.device)

    def _args(self, a, b, c, scale_a, scale_b) -> L.GemmArgs:
        g = L.GemmArgs()
        g.a, g.b, g.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
        g.m, g.n, g.k = self.m, self.n, self.k
        g.lda, g.ldb, g.ldc = self.k, self.k, self.n
        g.in_dtype = L.DTYPE_CODES[self.in_dtype]
        g.out_dtype = L.DTYPE_CODES[self.out_dtype]
        g.scale_a = scale_a.data_ptr() if scale_a is not None else None
        g.scale_b = scale_b.data_ptr() if scale_b is not None else None
        return g

    def __call__(self, a, b, out, scale_a=None, scale_b=None):
        """scale_a / scale_b (fp8 only) are one-element float32 DEVICE tensors."""
        _check_host(a, (self.m, self.k), self.in_dtype, "a")
        _check_host(b, (self.n, self.k), self.in_dtype, "b")
        _check_host(out, (self.m, self.n), self.out_dtype, "out")
        dev = self._args(self.da, self.db, self.dc, scale_a, scale_b)
        dev.status = _status_ptr(self.device)
        host = self._args(a, b, out, None, None)
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            L.check(L.lib().b200k_gemm_nt_host(C.byref(host), C.byref(dev), stream))
        return out
