"""The op library: ``torch.ops.b200k.*``.

Each op is a ``CustomOp`` registered the way the reference registers its op libraries
(iree/turbine/ops/__init__.py:7-11; e.g. iree/turbine/ops/conv_fwd.py:62-89 for a ``select``):
a schema string, a ``select`` that types every argument and declares the result meta tensors
(which also is the Meta implementation, so fake tensors and ``torch.compile`` tracing work), and
a CUDA implementation.  The CUDA implementation is ``eager_execute`` calling the C ABI on the
current stream; there is no CPU implementation, so a CPU tensor fails in the dispatcher with
torch's own "not implemented for CPU" error.

Output shape/dtype rules live in ``select`` only; ``eager_execute`` allocates outputs from the
same rules.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import Tensor

from . import _launcher as L
from .op_reg import CustomOp, KernelSelection, def_library

__all__ = [
    "LIBRARY",
    "gemm_nt",
    "gemm_fp8_nt",
    "gemm",
    "bmm",
    "linear",
    "linear_act",
    "attention",
    "attention_lse",
    "attention_bwd",
    "sdpa",
    "decode_attention",
    "paged_decode_attention",
    "quantize_e4m3",
    "paged_gather",
    "kv_append",
    "paged_attention",
    "device_status",
    "reset_device_status",
]

LIBRARY = def_library("b200k")

_HALF_TYPES = (torch.float16, torch.bfloat16)

# One int32 status word per device: kernels OR a code into it if a bounded device-side wait gave
# up (see include/b200k.h).  Reading it synchronizes, so it is only read on request.
_status_words: dict[int, Tensor] = {}


def _status_ptr(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w.data_ptr()


def device_status(device=None) -> int:
    """Returns the device status word (0 = no kernel reported a timed-out wait).  Synchronizes."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _status_ptr(dev)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return int(_status_words[idx].item())


def reset_device_status(device=None) -> None:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _status_ptr(dev)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    _status_words[idx].zero_()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: Tensor) -> C.c_void_p:
    """The current stream of the tensor's device as a raw cudaStream_t (the direct binding when torch
    has it: building a Stream object per launch costs several microseconds)."""
    if _raw_stream is not None and t.device.index is not None:
        return C.c_void_p(_raw_stream(t.device.index))
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _row_major_2d(t: Tensor) -> Tensor:
    """A 2-D view whose last dim is contiguous and whose row stride is a multiple of 16 bytes."""
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def _gemm_out_dtype(in_dtype: torch.dtype, out_dtype) -> torch.dtype:
    if in_dtype in _HALF_TYPES:
        od = torch.float32 if out_dtype is None else out_dtype
        torch._check(od in (torch.float32, in_dtype), lambda: f"gemm_nt: out_dtype must be float32 or {in_dtype}")
        return od
    od = torch.bfloat16 if out_dtype is None else out_dtype
    torch._check(od in (torch.bfloat16, torch.float32), lambda: "gemm_fp8_nt: out_dtype must be bfloat16 or float32")
    return od


def _launch_gemm(a: Tensor, b: Tensor, out: Tensor, scale_a, scale_b, tile_n: int = 0, tile_m: int = 0,
                 bias: Optional[Tensor] = None, activation: str = "none", a_km: bool = False,
                 b_kn: bool = False, split_k: int = 0) -> None:
    """a is stored [M, K] ([K, M] with a_km); b is stored [N, K] ([K, N] with b_kn).  split_k: 0 = the
    library decides, 1 = whole tiles only, 2 / 4 / 8 = CTAs per output tile."""
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    args = L.GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.k = (a.size(1), a.size(0)) if a_km else (a.size(0), a.size(1))
    args.n = b.size(1) if b_kn else b.size(0)
    args.a_km, args.b_kn = int(a_km), int(b_kn)
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.in_dtype = L.DTYPE_CODES[a.dtype]
    args.out_dtype = L.DTYPE_CODES[out.dtype]
    args.scale_a = scale_a.data_ptr() if scale_a is not None else None
    args.scale_b = scale_b.data_ptr() if scale_b is not None else None
    args.status = _status_ptr(a.device)
    args.tile_n = tile_n
    args.tile_m = tile_m
    args.split_k = split_k
    if activation not in L.ACTIVATION_CODES:
        raise ValueError(f"unknown activation {activation!r}; expected one of {sorted(L.ACTIVATION_CODES)}")
    args.activation = L.ACTIVATION_CODES[activation]
    if bias is not None:
        bias = bias.contiguous()
        args.bias = bias.data_ptr()
        args.bias_dtype = L.DTYPE_CODES[bias.dtype]
    L.check(L.lib().b200k_gemm_nt(C.byref(args), _stream(a)))


def _batched_operand(t: Tensor):
    """A [B, R, C] operand as the kernel can read it without a copy: (tensor, stored_transposed).
    Either the last dim is contiguous (rows of the matrix) or the middle one is (the matrix is stored
    transposed); row pitch and batch stride must be multiples of 16 bytes.  Otherwise a contiguous copy."""
    es = t.element_size()

    def ok(x):
        return (x.stride(2) == 1 and (x.stride(1) * es) % 16 == 0 and (x.stride(0) * es) % 16 == 0
                and x.stride(1) >= x.size(2) and x.data_ptr() % 16 == 0 and x.size(2) % 8 == 0)

    if ok(t):
        return t, False
    tt = t.transpose(1, 2)
    if ok(tt):
        return tt, True
    return t.contiguous(), False


@CustomOp.register(library=LIBRARY)
class gemm_nt(CustomOp):
    """C[M,N] = A[M,K] @ B[N,K]^T, f16 or bf16 operands, fp32 accumulation.

    Output dtype: float32 unless ``out_dtype`` names the operand dtype.
    """

    signature = "gemm_nt(Tensor a, Tensor b, ScalarType? out_dtype=None) -> Tensor"

    def select(self, sel: KernelSelection):
        a = sel.arg_tensor(0)
        b = sel.arg_tensor(1)
        od = sel.attr_optional(2)
        torch._check(a.t.dim() == 2 and b.t.dim() == 2, lambda: "gemm_nt: a and b must be 2-D")
        torch._check(a.t.dtype in _HALF_TYPES, lambda: f"gemm_nt: dtype must be float16 or bfloat16, got {a.t.dtype}")
        torch._check(a.t.dtype == b.t.dtype, lambda: "gemm_nt: a and b must have the same dtype")
        torch._check(a.t.size(1) == b.t.size(1), lambda: f"gemm_nt: K mismatch: a is {list(a.t.shape)}, b is {list(b.t.shape)}")
        torch._check(a.t.size(1) % 8 == 0, lambda: "gemm_nt: K must be a multiple of 8")
        a.specialize_dims(1)
        b.specialize_dims(1)
        sel.return_new_tensor([a.t.size(0), b.t.size(0)], _gemm_out_dtype(a.t.dtype, od.v))

    def eager_execute(self, a, b, out_dtype=None):
        out = torch.empty((a.size(0), b.size(0)), dtype=_gemm_out_dtype(a.dtype, out_dtype), device=a.device)
        _launch_gemm(a, b, out, None, None)
        return out


@CustomOp.register(library=LIBRARY)
class gemm(CustomOp):
    """C = op(a) @ op(b) with BLAS-style flags: ``a`` is [M, K] ([K, M] with ``trans_a``), ``b`` is
    [K, N] ([N, K] with ``trans_b``); f16 / bf16, fp32 accumulation.  No operand is repacked: the
    kernel reads either storage order.  ``gemm_nt(a, b)`` is ``gemm(a, b, trans_b=True)``."""

    signature = ("gemm(Tensor a, Tensor b, bool trans_a=False, bool trans_b=False, "
                 "ScalarType? out_dtype=None) -> Tensor")

    @staticmethod
    def _mnk(a, b, trans_a, trans_b):
        m, k = (a.size(1), a.size(0)) if trans_a else (a.size(0), a.size(1))
        kb, n = (b.size(1), b.size(0)) if trans_b else (b.size(0), b.size(1))
        return m, n, k, kb

    def select(self, sel: KernelSelection):
        a = sel.arg_tensor(0)
        b = sel.arg_tensor(1)
        ta = sel.attr_bool(2)
        tb_ = sel.attr_bool(3)
        od = sel.attr_optional(4)
        torch._check(a.t.dim() == 2 and b.t.dim() == 2, lambda: "gemm: a and b must be 2-D")
        torch._check(a.t.dtype in _HALF_TYPES and a.t.dtype == b.t.dtype,
                     lambda: f"gemm: a and b must both be float16 or bfloat16, got {a.t.dtype}, {b.t.dtype}")
        m, n, k, kb = self._mnk(a.t, b.t, bool(ta.v), bool(tb_.v))
        torch._check(k == kb, lambda: f"gemm: contraction sizes differ ({k} vs {kb})")
        torch._check(a.t.size(1) % 8 == 0 and b.t.size(1) % 8 == 0,
                     lambda: "gemm: the contiguous dimension of each operand must be a multiple of 8")
        sel.return_new_tensor([m, n], _gemm_out_dtype(a.t.dtype, od.v))

    def eager_execute(self, a, b, trans_a=False, trans_b=False, out_dtype=None):
        m, n, _, _ = self._mnk(a, b, trans_a, trans_b)
        out = torch.empty((m, n), dtype=_gemm_out_dtype(a.dtype, out_dtype), device=a.device)
        _launch_gemm(a, b, out, None, None, a_km=bool(trans_a), b_kn=not trans_b)
        return out


@CustomOp.register(library=LIBRARY)
class bmm(CustomOp):
    """Batched product ``a[B, M, K] @ b[B, K, N]`` (aten::bmm; the reference's BOO layer registers it
    beside mm and addmm, kernel/boo/op_exports/registry.py:99-104), f16 / bf16, fp32 accumulation, every
    problem's tiles in one persistent launch.  Either operand may be a transposed view (e.g.
    ``k.transpose(1, 2)``): the kernel reads both storage orders."""

    signature = "bmm(Tensor a, Tensor b, ScalarType? out_dtype=None) -> Tensor"

    def select(self, sel: KernelSelection):
        a = sel.arg_tensor(0)
        b = sel.arg_tensor(1)
        od = sel.attr_optional(2)
        torch._check(a.t.dim() == 3 and b.t.dim() == 3, lambda: "bmm: a and b must be 3-D")
        torch._check(a.t.dtype in _HALF_TYPES and a.t.dtype == b.t.dtype,
                     lambda: f"bmm: a and b must both be float16 or bfloat16, got {a.t.dtype}, {b.t.dtype}")
        torch._check(a.t.size(0) == b.t.size(0) and a.t.size(2) == b.t.size(1),
                     lambda: f"bmm: shapes {list(a.t.shape)} and {list(b.t.shape)} do not multiply")
        torch._check(a.t.size(1) % 8 == 0 or a.t.size(2) % 8 == 0, lambda: "bmm: M or K must be a multiple of 8")
        sel.return_new_tensor([a.t.size(0), a.t.size(1), b.t.size(2)], _gemm_out_dtype(a.t.dtype, od.v))

    def eager_execute(self, a, b, out_dtype=None):
        bsz, m, k = a.shape
        n = b.size(2)
        out = torch.empty((bsz, m, n), dtype=_gemm_out_dtype(a.dtype, out_dtype), device=a.device)
        if bsz == 0 or m == 0 or n == 0:
            return out
        a_s, a_t = _batched_operand(a)   # a_t: stored [B, K, M]
        b_s, b_t = _batched_operand(b)   # b_t: stored [B, N, K]  (the kernel's native form)
        args = L.GemmArgs()
        args.a, args.b, args.c = a_s.data_ptr(), b_s.data_ptr(), out.data_ptr()
        args.m, args.n, args.k = m, n, k
        args.a_km, args.b_kn = int(a_t), int(not b_t)
        args.lda, args.ldb, args.ldc = a_s.stride(1), b_s.stride(1), out.stride(1)
        args.batch = bsz
        args.a_batch_stride, args.b_batch_stride, args.c_batch_stride = a_s.stride(0), b_s.stride(0), out.stride(0)
        args.in_dtype = L.DTYPE_CODES[a.dtype]
        args.out_dtype = L.DTYPE_CODES[out.dtype]
        args.status = _status_ptr(a.device)
        L.check(L.lib().b200k_gemm_nt(C.byref(args), _stream(a)))
        return out


class _LinearFunction(torch.autograd.Function):
    """y = x @ w^T (+ bias) with both backward products on the same kernel (the reference wraps its
    own op the same way, kernel/boo/ops/conv.py:313-372; the products are those of
    kernel/boo/op_exports/gemm.py:233-270): dx = dy @ w, dw = dy^T @ x, db = sum(dy)."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return torch.ops.b200k.linear_act(x, w, bias, "none", x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.ops.b200k.gemm(dy, w, False, False, x.dtype)       # [M, N] @ [N, K]
        if ctx.needs_input_grad[1]:
            dw = torch.ops.b200k.gemm(dy, x, True, False, w.dtype)        # [M, N]^T @ [M, K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: Tensor, w: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """Differentiable ``x[M, K] @ w[N, K]^T + bias`` (f16 / bf16 CUDA tensors) on the b200k GEMM."""
    return _LinearFunction.apply(x, w, bias)


@CustomOp.register(library=LIBRARY)
class linear_act(CustomOp):
    """act(A[M,K] @ W[N,K]^T + bias[N]) in one kernel: the GEMM with bias and activation applied in
    its epilogue (the shape of a linear layer with trailing optional bias).  ``activation`` is
    "none", "relu", "gelu" (erf form) or "silu"; output dtype as for ``gemm_nt``."""

    signature = ("linear_act(Tensor a, Tensor w, Tensor? bias=None, str activation=\"none\", "
                 "ScalarType? out_dtype=None) -> Tensor")

    def select(self, sel: KernelSelection):
        a = sel.arg_tensor(0)
        w = sel.arg_tensor(1)
        bias = sel.arg_optional_tensor(2)
        act = sel.attr_str(3)
        od = sel.attr_optional(4)
        torch._check(a.t.dim() == 2 and w.t.dim() == 2, lambda: "linear_act: a and w must be 2-D")
        torch._check(a.t.dtype in _HALF_TYPES and a.t.dtype == w.t.dtype,
                     lambda: f"linear_act: a and w must both be float16 or bfloat16, got {a.t.dtype}, {w.t.dtype}")
        torch._check(a.t.size(1) == w.t.size(1) and a.t.size(1) % 8 == 0,
                     lambda: "linear_act: K must match and be a multiple of 8")
        torch._check(act.v in L.ACTIVATION_CODES, lambda: f"linear_act: unknown activation {act.v!r}")
        bt = bias.t if bias is not None else None
        if bt is not None:
            torch._check(bt.dim() == 1 and bt.size(0) == w.t.size(0), lambda: "linear_act: bias must be [N]")
            torch._check(bt.dtype in (torch.float32,) + _HALF_TYPES, lambda: "linear_act: bias must be float32 / float16 / bfloat16")
        sel.return_new_tensor([a.t.size(0), w.t.size(0)], _gemm_out_dtype(a.t.dtype, od.v))

    def eager_execute(self, a, w, bias=None, activation="none", out_dtype=None):
        out = torch.empty((a.size(0), w.size(0)), dtype=_gemm_out_dtype(a.dtype, out_dtype), device=a.device)
        _launch_gemm(a, w, out, None, None, bias=bias, activation=activation)
        return out


@CustomOp.register(library=LIBRARY)
class gemm_fp8_nt(CustomOp):
    """C = (A8 @ B8^T) * scale_a * scale_b with float8_e4m3fn operands and per-tensor fp32 scales.

    ``scale_a`` / ``scale_b`` are one-element float32 device tensors.  Output bfloat16 (default)
    or float32.
    """

    signature = (
        "gemm_fp8_nt(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, ScalarType? out_dtype=None) -> Tensor"
    )

    def select(self, sel: KernelSelection):
        a = sel.arg_tensor(0)
        b = sel.arg_tensor(1)
        sa = sel.arg_tensor(2)
        sb = sel.arg_tensor(3)
        od = sel.attr_optional(4)
        torch._check(a.t.dim() == 2 and b.t.dim() == 2, lambda: "gemm_fp8_nt: a and b must be 2-D")
        torch._check(
            a.t.dtype == torch.float8_e4m3fn and b.t.dtype == torch.float8_e4m3fn,
            lambda: "gemm_fp8_nt: a and b must be float8_e4m3fn",
        )
        torch._check(a.t.size(1) == b.t.size(1), lambda: "gemm_fp8_nt: K mismatch")
        torch._check(a.t.size(1) % 16 == 0, lambda: "gemm_fp8_nt: K must be a multiple of 16")
        torch._check(
            sa.t.numel() == 1 and sb.t.numel() == 1 and sa.t.dtype == torch.float32 and sb.t.dtype == torch.float32,
            lambda: "gemm_fp8_nt: scales must be one-element float32 tensors",
        )
        sel.return_new_tensor([a.t.size(0), b.t.size(0)], _gemm_out_dtype(a.t.dtype, od.v))

    def eager_execute(self, a, b, scale_a, scale_b, out_dtype=None):
        out = torch.empty((a.size(0), b.size(0)), dtype=_gemm_out_dtype(a.dtype, out_dtype), device=a.device)
        _launch_gemm(a, b, out, scale_a, scale_b)
        return out


@CustomOp.register(library=LIBRARY)
class quantize_e4m3(CustomOp):
    """Per-tensor quantisation: returns (x / s cast to float8_e4m3fn, s) with s = max|x| / 448."""

    signature = "quantize_e4m3(Tensor x) -> (Tensor, Tensor)"

    def select(self, sel: KernelSelection):
        x = sel.arg_tensor(0)
        torch._check(x.t.dtype == torch.float32, lambda: "quantize_e4m3: x must be float32")
        sel.return_new_tensor(list(x.t.shape), torch.float8_e4m3fn)
        sel.return_new_tensor([1], torch.float32)

    def eager_execute(self, x):
        x = x.contiguous()
        y = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scale = torch.empty(1, dtype=torch.float32, device=x.device)
        scratch = torch.empty(1, dtype=torch.int32, device=x.device)
        L.check(
            L.lib().b200k_quantize_e4m3(
                x.data_ptr(), y.data_ptr(), scale.data_ptr(), scratch.data_ptr(), x.numel(), _stream(x)
            )
        )
        return y, scale


# ---------------------------------------------------------------------------------------------
# attention forward
# ---------------------------------------------------------------------------------------------
def _bhsd(t: Tensor) -> Tensor:
    s0, s1, s2, s3 = t.stride()
    ok = (s3 == 1 and s0 > 0 and s1 > 0 and s2 > 0 and (s0 | s1 | s2) % 8 == 0 and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


# Which forward kernel ``attention`` / ``attention_lse`` / ``paged_attention`` ask for: 0 lets the
# library choose (one-tile or tile-pair kernel, see include/b200k.h), 1 / 2 force one of them
# (head dim 64 only exists in the pair kernel).  A tuning and testing knob, like the GEMM tile shape.
ATTENTION_KERNEL = L.ATTN_AUTO


def _fill_attention_args(q: Tensor, k: Tensor, v: Tensor, o: Tensor, scale: float, causal: bool) -> L.AttentionArgs:
    args = L.AttentionArgs()
    args.batch, args.q_heads, args.seq_q, args.head_dim = q.shape
    args.kernel = ATTENTION_KERNEL if args.head_dim == 128 else L.ATTN_AUTO
    args.q, args.k, args.v, args.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    _, args.kv_heads, args.seq_kv, _ = k.shape
    args.q_stride_b, args.q_stride_h, args.q_stride_s, _ = q.stride()
    args.k_stride_b, args.k_stride_h, args.k_stride_s, _ = k.stride()
    args.v_stride_b, args.v_stride_h, args.v_stride_s, _ = v.stride()
    args.o_stride_b, args.o_stride_h, args.o_stride_s, _ = o.stride()
    args.dtype = L.DTYPE_CODES[q.dtype]
    args.causal = 1 if causal else 0
    args.scale = float(scale)
    return args


def _attention_out_like(q: Tensor, device) -> Tensor:
    """The output takes the memory layout of q when q's rows are contiguous (as
    aten.scaled_dot_product_attention does: a [B, H, S, D] view of [B, S, H, D] memory stays one),
    so graphs traced against the ATen op keep their views valid; otherwise it is contiguous.  The
    kernel writes any layout with contiguous rows."""
    if q.dim() == 4 and q.stride(-1) == 1:
        return torch.empty_like(q, device=device)
    return torch.empty(q.shape, dtype=q.dtype, device=device)


def _attention_select(sel: KernelSelection):
    q = sel.arg_tensor(0)
    k = sel.arg_tensor(1)
    v = sel.arg_tensor(2)
    sel.attr_float(3)
    sel.attr_bool(4)
    torch._check(q.t.dim() == 4 and k.t.dim() == 4 and v.t.dim() == 4, lambda: "attention: q, k, v must be 4-D [B,H,S,D]")
    torch._check(q.t.dtype in _HALF_TYPES, lambda: f"attention: dtype must be float16 or bfloat16, got {q.t.dtype}")
    torch._check(q.t.dtype == k.t.dtype == v.t.dtype, lambda: "attention: q, k, v must share a dtype")
    torch._check(q.t.size(3) in (64, 128) and k.t.size(3) == q.t.size(3) and v.t.size(3) == q.t.size(3),
                 lambda: "attention: head dim must be 128 or 64, the same for q, k and v")
    torch._check(k.t.shape == v.t.shape, lambda: "attention: k and v must have the same shape")
    torch._check(q.t.size(0) == k.t.size(0), lambda: "attention: batch mismatch")
    torch._check(q.t.size(1) % k.t.size(1) == 0, lambda: "attention: query heads must be a multiple of kv heads")
    q.specialize_dims(3)
    sel.return_tensor(_attention_out_like(q.t, "meta"))
    return q


@CustomOp.register(library=LIBRARY)
class attention(CustomOp):
    """O = softmax(scale * Q K^T [causal]) V.  q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] -> [B,Hq,Sq,D], D = 128 or 64."""

    signature = "attention(Tensor q, Tensor k, Tensor v, float scale, bool is_causal) -> Tensor"

    def select(self, sel: KernelSelection):
        _attention_select(sel)

    def eager_execute(self, q, k, v, scale, is_causal):
        o = _attention_out_like(q, q.device)
        q, k, v = _bhsd(q), _bhsd(k), _bhsd(v)
        args = _fill_attention_args(q, k, v, o, scale, is_causal)
        args.status = _status_ptr(q.device)
        L.check(L.lib().b200k_attention_fwd(C.byref(args), _stream(q)))
        return o


@CustomOp.register(library=LIBRARY)
class attention_lse(CustomOp):
    """``attention`` that also returns the row statistic the backward needs:
    lse[b, h, i] = ln sum_j exp(scale * q_i . k_j) over the visible keys (float32, -inf for a row
    that sees none)."""

    signature = "attention_lse(Tensor q, Tensor k, Tensor v, float scale, bool is_causal) -> (Tensor, Tensor)"

    def select(self, sel: KernelSelection):
        q = _attention_select(sel)
        sel.return_new_tensor(list(q.t.shape[:3]), torch.float32)

    def eager_execute(self, q, k, v, scale, is_causal):
        o = _attention_out_like(q, q.device)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
        q, k, v = _bhsd(q), _bhsd(k), _bhsd(v)
        args = _fill_attention_args(q, k, v, o, scale, is_causal)
        args.status = _status_ptr(q.device)
        args.lse = lse.data_ptr()
        L.check(L.lib().b200k_attention_fwd(C.byref(args), _stream(q)))
        return o, lse


def _attention_bwd_checks(q: Tensor, k: Tensor, v: Tensor, o: Tensor, d_o: Tensor, lse: Optional[Tensor] = None) -> None:
    if lse is not None:
        torch._check(lse.dtype == torch.float32 and tuple(lse.shape) == tuple(q.shape[:3]),
                     lambda: "attention_bwd: lse must be float32 [B, Hq, Sq]")
    for t in (q, k, v, o, d_o):
        torch._check(t.dim() == 4 and t.size(3) in (64, 128) and t.size(3) == q.size(3),
                     lambda: "attention_bwd: tensors must be [B,H,S,D] with D = 128 or 64, the same for all")
        torch._check(t.dtype == q.dtype, lambda: "attention_bwd: all tensors must share a dtype")
    torch._check(q.dtype in _HALF_TYPES, lambda: f"attention_bwd: dtype must be float16 or bfloat16, got {q.dtype}")
    torch._check(k.shape == v.shape, lambda: "attention_bwd: k and v must have the same shape")
    torch._check(o.shape == q.shape and d_o.shape == q.shape, lambda: "attention_bwd: o and d_o must have q's shape")
    torch._check(q.size(0) == k.size(0), lambda: "attention_bwd: batch mismatch")
    torch._check(k.size(1) > 0 and q.size(1) % k.size(1) == 0,
                 lambda: "attention_bwd: query heads must be a multiple of kv heads")


@CustomOp.register(library=LIBRARY)
class attention_bwd(CustomOp):
    """Gradients of ``attention``: (q, k, v, o, d_o) -> (d_q, d_k, d_v).  d_k / d_v are summed over
    the query heads of a group.  Only the forward OUTPUT is needed; row statistics are recomputed."""

    signature = ("attention_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor d_o, float scale, bool is_causal, "
                 "Tensor? lse=None) -> (Tensor, Tensor, Tensor)")

    def select(self, sel: KernelSelection):
        q, k, v, o, d_o = (sel.arg_tensor(i) for i in range(5))
        sel.attr_float(5)
        sel.attr_bool(6)
        lse = sel.arg_optional_tensor(7)
        _attention_bwd_checks(q.t, k.t, v.t, o.t, d_o.t, lse.t if lse is not None else None)
        sel.return_new_tensor(list(q.t.shape), q.t.dtype)
        sel.return_new_tensor(list(k.t.shape), q.t.dtype)
        sel.return_new_tensor(list(k.t.shape), q.t.dtype)

    def eager_execute(self, q, k, v, o, d_o, scale, is_causal, lse=None):
        _attention_bwd_checks(q, k, v, o, d_o, lse)
        if lse is not None:
            lse = lse.contiguous()
        q, k, v, o, d_o = (_bhsd(t) for t in (q, k, v, o, d_o))
        d_q, d_k, d_v = torch.empty_like(q, memory_format=torch.contiguous_format), \
            torch.empty_like(k, memory_format=torch.contiguous_format), \
            torch.empty_like(v, memory_format=torch.contiguous_format)
        a = L.AttentionBwdArgs()
        for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", d_o), ("dq", d_q), ("dk", d_k), ("dv", d_v)):
            setattr(a, {"do": "d_o", "dq": "d_q", "dk": "d_k", "dv": "d_v"}.get(name, name), t.data_ptr())
            for d, i in (("b", 0), ("h", 1), ("s", 2)):
                setattr(a, f"{name}_stride_{d}", t.stride(i))
        a.batch, a.q_heads, a.seq_q, a.head_dim = q.shape
        a.kv_heads, a.seq_kv = k.size(1), k.size(2)
        a.dtype = L.DTYPE_CODES[q.dtype]
        a.causal = 1 if is_causal else 0
        a.scale = float(scale)
        a.status = _status_ptr(q.device)
        a.lse = lse.data_ptr() if lse is not None else None
        lib = L.lib()
        need = lib.b200k_attention_bwd_workspace_bytes(C.byref(a))
        ws = torch.empty(max(int(need), 16), dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        L.check(lib.b200k_attention_bwd(C.byref(a), _stream(q)))
        return d_q, d_k, d_v


class _AttentionFunction(torch.autograd.Function):
    """``attention`` with its gradient on the backward kernels (wrapped the way the reference wraps
    its own forward / backward ops, kernel/boo/ops/conv.py:313-372)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, is_causal):
        o, lse = torch.ops.b200k.attention_lse(q, k, v, scale, is_causal)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.is_causal = scale, is_causal
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        d_q, d_k, d_v = torch.ops.b200k.attention_bwd(q, k, v, o, d_o, ctx.scale, ctx.is_causal, lse)
        return d_q, d_k, d_v, None, None


def sdpa(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None, is_causal: bool = False) -> Tensor:
    """Differentiable scaled-dot-product attention on the b200k kernels ([B, H, S, D] f16 / bf16
    CUDA tensors, D = 128 or 64; grouped-query heads; causal mask aligned to the bottom-right corner)."""
    if q.size(-1) not in (64, 128):
        raise ValueError("sdpa: head dim must be 128 or 64")
    if scale is None:
        scale = 1.0 / (q.size(-1) ** 0.5)
    return _AttentionFunction.apply(q, k, v, float(scale), bool(is_causal))


# ---------------------------------------------------------------------------------------------
# decode / paged decode
# ---------------------------------------------------------------------------------------------
def _decode_common_checks(name: str, q: Tensor, kc: Tensor, vc: Tensor, lens: Tensor):
    torch._check(q.dim() == 3, lambda: f"{name}: q must be [num_seqs, q_heads, head_dim]")
    torch._check(q.dtype in _HALF_TYPES, lambda: f"{name}: dtype must be float16 or bfloat16, got {q.dtype}")
    torch._check(q.dtype == kc.dtype == vc.dtype, lambda: f"{name}: q and the KV cache must share a dtype")
    torch._check(q.size(2) in (64, 128), lambda: f"{name}: head dim must be 128 or 64")
    torch._check(kc.dim() == 4 and kc.shape == vc.shape, lambda: f"{name}: k and v caches must be 4-D and equal in shape")
    torch._check(kc.size(3) == q.size(2), lambda: f"{name}: cache head dim must equal q's")
    torch._check(lens.dtype == torch.int32 and lens.dim() == 1 and lens.size(0) == q.size(0),
                 lambda: f"{name}: seq_lens must be int32 [num_seqs]")
    torch._check(q.size(1) % kc.size(1) == 0 and q.size(1) // kc.size(1) <= 16,
                 lambda: f"{name}: query heads must be a multiple (at most 16x) of kv heads")


def _launch_decode(args: L.DecodeArgs, q: Tensor) -> None:
    lib = L.lib()
    need = lib.b200k_decode_workspace_bytes(C.byref(args))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    args.workspace = ws.data_ptr()
    args.workspace_bytes = need
    args.status = _status_ptr(q.device)
    L.check(lib.b200k_decode_attention(C.byref(args), _stream(q)))


@CustomOp.register(library=LIBRARY)
class decode_attention(CustomOp):
    """One query token per sequence against a contiguous KV history.

    q [num_seqs, Hq, D]; k, v [num_seqs, Hkv, max_len, D]; seq_lens int32 [num_seqs]
    (tokens t >= seq_lens[s] are ignored; D = 128 or 64).  Returns [num_seqs, Hq, D].
    """

    signature = (
        "decode_attention(Tensor q, Tensor k, Tensor v, Tensor seq_lens, float scale, int chunk_tokens=0) -> Tensor"
    )

    def select(self, sel: KernelSelection):
        q = sel.arg_tensor(0)
        k = sel.arg_tensor(1)
        v = sel.arg_tensor(2)
        lens = sel.arg_tensor(3)
        sel.attr_float(4)
        sel.attr_int(5)
        _decode_common_checks("decode_attention", q.t, k.t, v.t, lens.t)
        torch._check(k.t.size(0) == q.t.size(0), lambda: "decode_attention: k must have one history per sequence")
        sel.return_new_tensor(list(q.t.shape), q.t.dtype)

    def eager_execute(self, q, k, v, seq_lens, scale, chunk_tokens=0):
        q, k, v, seq_lens = q.contiguous(), k.contiguous(), v.contiguous(), seq_lens.contiguous()
        o = torch.empty_like(q)
        args = L.DecodeArgs()
        args.q, args.k_cache, args.v_cache, args.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
        args.block_table = None
        args.seq_lens = seq_lens.data_ptr()
        args.num_seqs, args.q_heads, args.head_dim = q.size(0), q.size(1), q.size(2)
        args.kv_heads = k.size(1)
        args.max_seq_len = k.size(2)
        args.kv_batch_stride, args.kv_head_stride = k.stride(0), k.stride(1)
        args.dtype = L.DTYPE_CODES[q.dtype]
        args.chunk_tokens = int(chunk_tokens)
        args.scale = float(scale)
        _launch_decode(args, q)
        return o


@CustomOp.register(library=LIBRARY)
class paged_decode_attention(CustomOp):
    """One query token per sequence against a paged KV cache.

    q [num_seqs, Hq, D]; k_cache, v_cache [num_pages, Hkv, page_size, D], D = 128 or 64;
    block_table int32 [num_seqs, max_pages]: physical page of logical page p of sequence s;
    seq_lens int32 [num_seqs].  Returns [num_seqs, Hq, D].
    """

    signature = (
        "paged_decode_attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, "
        "float scale, int chunk_tokens=0) -> Tensor"
    )

    def select(self, sel: KernelSelection):
        q = sel.arg_tensor(0)
        kc = sel.arg_tensor(1)
        vc = sel.arg_tensor(2)
        bt = sel.arg_tensor(3)
        lens = sel.arg_tensor(4)
        sel.attr_float(5)
        sel.attr_int(6)
        _decode_common_checks("paged_decode_attention", q.t, kc.t, vc.t, lens.t)
        torch._check(bt.t.dtype == torch.int32 and bt.t.dim() == 2 and bt.t.size(0) == q.t.size(0),
                     lambda: "paged_decode_attention: block_table must be int32 [num_seqs, max_pages]")
        torch._check(kc.t.size(2) % 16 == 0, lambda: "paged_decode_attention: page size must be a multiple of 16")
        sel.return_new_tensor(list(q.t.shape), q.t.dtype)

    def eager_execute(self, q, k_cache, v_cache, block_table, seq_lens, scale, chunk_tokens=0):
        q, k_cache, v_cache = q.contiguous(), k_cache.contiguous(), v_cache.contiguous()
        block_table, seq_lens = block_table.contiguous(), seq_lens.contiguous()
        o = torch.empty_like(q)
        args = L.DecodeArgs()
        args.q, args.k_cache, args.v_cache, args.o = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), o.data_ptr()
        args.block_table = block_table.data_ptr()
        args.seq_lens = seq_lens.data_ptr()
        args.num_seqs, args.q_heads, args.head_dim = q.size(0), q.size(1), q.size(2)
        args.kv_heads = k_cache.size(1)
        args.page_size = k_cache.size(2)
        args.num_pages = k_cache.size(0)
        args.block_table_stride = block_table.stride(0)
        args.max_seq_len = block_table.size(1) * k_cache.size(2)
        args.kv_page_stride, args.kv_head_stride = k_cache.stride(0), k_cache.stride(1)
        args.dtype = L.DTYPE_CODES[q.dtype]
        args.chunk_tokens = int(chunk_tokens)
        args.scale = float(scale)
        _launch_decode(args, q)
        return o


@CustomOp.register(library=LIBRARY)
class paged_gather(CustomOp):
    """out[s, h, t, :] = cache[block_table[s, t // page], h, t % page, :] for t < seq_lens[s].

    Uses the paged decode kernel's address function; rows beyond seq_lens[s] are zero.
    """

    signature = "paged_gather(Tensor cache, Tensor block_table, Tensor seq_lens, int max_seq_len) -> Tensor"

    def select(self, sel: KernelSelection):
        c = sel.arg_tensor(0)
        bt = sel.arg_tensor(1)
        lens = sel.arg_tensor(2)
        n = sel.attr_int(3)
        torch._check(c.t.dim() == 4, lambda: "paged_gather: cache must be [num_pages, heads, page_size, head_dim]")
        torch._check(bt.t.dtype == torch.int32 and bt.t.dim() == 2, lambda: "paged_gather: block_table must be int32 2-D")
        torch._check(lens.t.dtype == torch.int32 and lens.t.dim() == 1, lambda: "paged_gather: seq_lens must be int32 1-D")
        sel.return_new_tensor([bt.t.size(0), c.t.size(1), n.v, c.t.size(3)], c.t.dtype)

    def eager_execute(self, cache, block_table, seq_lens, max_seq_len):
        cache = cache.contiguous()
        block_table, seq_lens = block_table.contiguous(), seq_lens.contiguous()
        out = torch.zeros((block_table.size(0), cache.size(1), max_seq_len, cache.size(3)), dtype=cache.dtype,
                          device=cache.device)
        L.check(
            L.lib().b200k_paged_gather(
                cache.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), block_table.size(0),
                cache.size(1), cache.size(3), cache.size(2), cache.size(0), block_table.stride(0), max_seq_len,
                cache.stride(0), cache.stride(1), cache.element_size(), _stream(cache),
            )
        )
        return out


@CustomOp.register(library=LIBRARY)
class kv_append(CustomOp):
    """Writes new K/V rows into the paged cache through the block table (in place).

    ``k_new`` / ``v_new``: [num_seqs, new_tokens, kv_heads, head_dim]; row ``t`` of sequence ``s``
    goes to token position ``positions[s] + t``, i.e. to
    ``cache[block_table[s, p // page], h, p % page, :]``.  The pages must already be in the table.
    Same address function as the paged decode kernel.
    """

    signature = ("kv_append(Tensor k_new, Tensor v_new, Tensor(a!) k_cache, Tensor(b!) v_cache, "
                 "Tensor block_table, Tensor positions) -> ()")

    def select(self, sel: KernelSelection):
        kn = sel.arg_tensor(0)
        vn = sel.arg_tensor(1)
        kc = sel.arg_tensor(2)
        vc = sel.arg_tensor(3)
        bt = sel.arg_tensor(4)
        pos = sel.arg_tensor(5)
        torch._check(kn.t.dim() == 4 and vn.t.shape == kn.t.shape,
                     lambda: "kv_append: k_new and v_new must be [num_seqs, new_tokens, kv_heads, head_dim]")
        torch._check(kc.t.dim() == 4 and vc.t.shape == kc.t.shape,
                     lambda: "kv_append: caches must be [num_pages, kv_heads, page_size, head_dim]")
        torch._check(kc.t.dtype == kn.t.dtype and vc.t.dtype == kn.t.dtype and vn.t.dtype == kn.t.dtype,
                     lambda: "kv_append: dtypes of new rows and caches must match")
        torch._check(kn.t.size(2) == kc.t.size(1) and kn.t.size(3) == kc.t.size(3),
                     lambda: "kv_append: heads / head_dim of new rows and caches must match")
        torch._check(bt.t.dtype == torch.int32 and bt.t.dim() == 2 and bt.t.size(0) == kn.t.size(0),
                     lambda: "kv_append: block_table must be int32 [num_seqs, max_pages]")
        torch._check(pos.t.dtype == torch.int32 and pos.t.dim() == 1 and pos.t.size(0) == kn.t.size(0),
                     lambda: "kv_append: positions must be int32 [num_seqs]")

    def eager_execute(self, k_new, v_new, k_cache, v_cache, block_table, positions):
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError("kv_append: the caches are written in place and must be contiguous")
        k_new, v_new = k_new.contiguous(), v_new.contiguous()
        block_table, positions = block_table.contiguous(), positions.contiguous()
        L.check(
            L.lib().b200k_kv_append(
                k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
                positions.data_ptr(), k_new.size(0), k_new.size(1), k_new.size(2), k_new.size(3), k_cache.size(2),
                k_cache.size(0), block_table.stride(0), k_cache.stride(0), k_cache.stride(1), k_cache.element_size(),
                _status_ptr(k_cache.device), _stream(k_cache),
            )
        )
        return None


@CustomOp.register(library=LIBRARY)
class paged_attention(CustomOp):
    """Attention forward (prefill) over a paged K/V cache.

    q [B, Hq, Sq, 128]; caches [num_pages, Hkv, page_size, 128]; block_table int32 [B, max_pages];
    seq_lens int32 [B] = number of keys of each sequence.  The Sq queries of a sequence are its last
    Sq tokens (append their K/V first, see ``kv_append``); with ``is_causal`` query i sees keys
    j <= i + seq_lens[b] - Sq.  Rows of a sequence's last page past its length must be finite.
    """

    signature = ("paged_attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, "
                 "float scale, bool is_causal) -> Tensor")

    def select(self, sel: KernelSelection):
        q = sel.arg_tensor(0)
        kc = sel.arg_tensor(1)
        vc = sel.arg_tensor(2)
        bt = sel.arg_tensor(3)
        lens = sel.arg_tensor(4)
        sel.attr_float(5)
        sel.attr_bool(6)
        torch._check(q.t.dim() == 4 and q.t.size(3) in (64, 128), lambda: "paged_attention: q must be [B, Hq, Sq, 128 or 64]")
        torch._check(q.t.dtype in _HALF_TYPES, lambda: f"paged_attention: dtype must be float16 or bfloat16, got {q.t.dtype}")
        torch._check(kc.t.dim() == 4 and kc.t.shape == vc.t.shape and kc.t.size(3) == q.t.size(3),
                     lambda: "paged_attention: caches must be [num_pages, Hkv, page_size, head dim of q] and equal in shape")
        torch._check(kc.t.dtype == q.t.dtype and vc.t.dtype == q.t.dtype, lambda: "paged_attention: dtypes must match")
        torch._check(kc.t.size(2) in (16, 32, 64, 128), lambda: "paged_attention: page_size must be 16, 32, 64 or 128")
        torch._check(q.t.size(1) % kc.t.size(1) == 0, lambda: "paged_attention: query heads must be a multiple of kv heads")
        torch._check(bt.t.dtype == torch.int32 and bt.t.dim() == 2 and bt.t.size(0) == q.t.size(0),
                     lambda: "paged_attention: block_table must be int32 [B, max_pages]")
        torch._check(lens.t.dtype == torch.int32 and lens.t.dim() == 1 and lens.t.size(0) == q.t.size(0),
                     lambda: "paged_attention: seq_lens must be int32 [B]")
        sel.return_tensor(_attention_out_like(q.t, "meta"))

    def eager_execute(self, q, k_cache, v_cache, block_table, seq_lens, scale, is_causal):
        o = _attention_out_like(q, q.device)
        q = _bhsd(q)
        k_cache, v_cache = k_cache.contiguous(), v_cache.contiguous()
        block_table, seq_lens = block_table.contiguous(), seq_lens.contiguous()
        a = L.PagedAttentionArgs()
        a.q, a.k_cache, a.v_cache, a.o = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), o.data_ptr()
        a.block_table, a.seq_lens = block_table.data_ptr(), seq_lens.data_ptr()
        a.batch, a.q_heads, a.kv_heads, a.seq_q = q.size(0), q.size(1), k_cache.size(1), q.size(2)
        a.page_size, a.num_pages, a.block_table_stride = k_cache.size(2), k_cache.size(0), block_table.stride(0)
        a.max_seq_kv = block_table.size(1) * k_cache.size(2)
        a.head_dim = q.size(3)
        a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(0), q.stride(1), q.stride(2)
        a.o_stride_b, a.o_stride_h, a.o_stride_s = o.stride(0), o.stride(1), o.stride(2)
        a.kv_page_stride, a.kv_head_stride = k_cache.stride(0), k_cache.stride(1)
        a.dtype = L.DTYPE_CODES[q.dtype]
        a.causal = 1 if is_causal else 0
        a.scale = float(scale)
        a.status = _status_ptr(q.device)
        a.kernel = ATTENTION_KERNEL if q.size(3) == 128 else L.ATTN_AUTO
        L.check(L.lib().b200k_paged_attention_fwd(C.byref(a), _stream(q)))
        return o
