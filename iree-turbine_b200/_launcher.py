"""ctypes binding of ``libb200kern.so`` (the C ABI declared in ``include/b200k.h``).

This module plays the role that ``eager_dispatch`` + ``invoke_vm_function`` play in the reference
(iree/turbine/runtime/op_reg/eager.py:58-206, runtime/invoke.py:28-75): it turns torch tensors
into raw pointers, sizes and strides and hands them, with the caller's current CUDA stream, to
native code.  Unlike the reference it never synchronizes the host
(cf. runtime/device.py:158-162) and there is no compilation step at call time.

There is no fallback of any kind: if the shared library has not been built, or a call returns a
non-zero status, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

__all__ = [
    "B200kError",
    "DTYPE_CODES",
    "GemmArgs",
    "GemmAllGatherArgs",
    "AttentionArgs",
    "AttentionBwdArgs",
    "DecodeArgs",
    "lib",
    "lib_path",
    "check",
    "EXPORTED_SYMBOLS",
]

_PKG_DIR = Path(__file__).resolve().parent
_LIB_NAME = "libb200kern.so"

ABI_VERSION = 3  # B200K_ABI_VERSION this binding was written against

# Status codes (b200k_status).
OK = 0
ERR_BAD_SHAPE = -1
ERR_BAD_ALIGN = -2
ERR_BAD_DTYPE = -3
ERR_UNSUPPORTED_ARCH = -4
ERR_CUDA = -5
ERR_NULL = -6
ERR_TIMEOUT = -7
ERR_WORKSPACE = -8

# Capacity of the library-owned decode scratch (B200K_DECODE_STATIC_SCRATCH_BYTES).
DECODE_STATIC_SCRATCH_BYTES = 32 << 20

# b200k_dtype
F16, BF16, F32, E4M3 = 0, 1, 2, 3

# attention forward kernel choice (B200K_ATTN_*)
ATTN_AUTO, ATTN_ONE_TILE, ATTN_TILE_PAIR = 0, 1, 2


class B200kError(RuntimeError):
    """A C-ABI call returned a non-OK status (CUDA failure, unsupported device, ...)."""

    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"b200k call failed: {name} ({status}): {message}")
        self.status = status
        self.status_name = name


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("c", C.c_void_p),
        ("m", C.c_int64),
        ("n", C.c_int64),
        ("k", C.c_int64),
        ("lda", C.c_int64),
        ("ldb", C.c_int64),
        ("ldc", C.c_int64),
        ("in_dtype", C.c_int32),
        ("out_dtype", C.c_int32),
        ("scale_a", C.c_void_p),
        ("scale_b", C.c_void_p),
        ("status", C.c_void_p),
        ("tile_n", C.c_int32),
        ("tile_m", C.c_int32),
        ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32),
        ("activation", C.c_int32),
        ("a_km", C.c_int32),
        ("b_kn", C.c_int32),
        ("batch", C.c_int64),
        ("a_batch_stride", C.c_int64),
        ("b_batch_stride", C.c_int64),
        ("c_batch_stride", C.c_int64),
        ("split_k", C.c_int32),
        ("reserved", C.c_int32),
    ]


class GemmAllGatherArgs(C.Structure):
    _fields_ = [
        ("gemm", GemmArgs),
        ("peer_c", C.c_void_p * 8),
        ("num_peers", C.c_int32),
        ("self_index", C.c_int32),
        ("peer_ldc", C.c_int64),
        ("col_offset", C.c_int64),
        ("multicast_c", C.c_void_p),
        ("plain_stores", C.c_int32),
        ("reserved", C.c_int32),
    ]


class AttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("o", C.c_void_p),
        ("batch", C.c_int32),
        ("q_heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("seq_q", C.c_int32),
        ("seq_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_stride_b", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("q_stride_s", C.c_int64),
        ("k_stride_b", C.c_int64),
        ("k_stride_h", C.c_int64),
        ("k_stride_s", C.c_int64),
        ("v_stride_b", C.c_int64),
        ("v_stride_h", C.c_int64),
        ("v_stride_s", C.c_int64),
        ("o_stride_b", C.c_int64),
        ("o_stride_h", C.c_int64),
        ("o_stride_s", C.c_int64),
        ("dtype", C.c_int32),
        ("causal", C.c_int32),
        ("scale", C.c_float),
        ("status", C.c_void_p),
        ("lse", C.c_void_p),
        ("kernel", C.c_int32),
        ("reserved", C.c_int32),
    ]


class AttentionBwdArgs(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("q", "k", "v", "o", "d_o", "d_q", "d_k", "d_v", "workspace")]
        + [("workspace_bytes", C.c_uint64)]
        + [(n, C.c_int32) for n in ("batch", "q_heads", "kv_heads", "seq_q", "seq_kv", "head_dim")]
        + [(f"{t}_stride_{d}", C.c_int64) for t in ("q", "k", "v", "o", "do", "dq", "dk", "dv") for d in "bhs"]
        + [("dtype", C.c_int32), ("causal", C.c_int32), ("scale", C.c_float), ("reserved", C.c_int32),
           ("status", C.c_void_p), ("lse", C.c_void_p)]
    )


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("block_table", C.c_void_p),
        ("seq_lens", C.c_void_p),
        ("o", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
        ("num_seqs", C.c_int32),
        ("q_heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_size", C.c_int32),
        ("num_pages", C.c_int32),
        ("block_table_stride", C.c_int32),
        ("max_seq_len", C.c_int32),
        ("kv_batch_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("kv_page_stride", C.c_int64),
        ("dtype", C.c_int32),
        ("chunk_tokens", C.c_int32),
        ("scale", C.c_float),
        ("reserved", C.c_int32),
        ("status", C.c_void_p),
    ]


class PagedAttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("o", C.c_void_p),
        ("block_table", C.c_void_p), ("seq_lens", C.c_void_p),
        ("batch", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32), ("seq_q", C.c_int32),
        ("max_seq_kv", C.c_int32), ("head_dim", C.c_int32),
        ("page_size", C.c_int32), ("num_pages", C.c_int32), ("block_table_stride", C.c_int32), ("reserved", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_s", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_s", C.c_int64),
        ("kv_page_stride", C.c_int64), ("kv_head_stride", C.c_int64),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("scale", C.c_float), ("kernel", C.c_int32),
        ("status", C.c_void_p),
    ]


ACTIVATION_CODES = {"none": 0, "relu": 1, "gelu": 2, "silu": 3}

# name -> (restype, argtypes); this table is also what the symbol-export test walks.
EXPORTED_SYMBOLS = {
    "b200k_abi_version": (C.c_int, []),
    "b200k_last_error": (C.c_char_p, []),
    "b200k_status_string": (C.c_char_p, [C.c_int]),
    "b200k_gemm_nt": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "b200k_gemm_nt_allgather": (C.c_int, [C.POINTER(GemmAllGatherArgs), C.c_void_p]),
    "b200k_attention_fwd": (C.c_int, [C.POINTER(AttentionArgs), C.c_void_p]),
    "b200k_attention_bwd_workspace_bytes": (C.c_uint64, [C.POINTER(AttentionBwdArgs)]),
    "b200k_attention_bwd": (C.c_int, [C.POINTER(AttentionBwdArgs), C.c_void_p]),
    "b200k_decode_workspace_bytes": (C.c_uint64, [C.POINTER(DecodeArgs)]),
    "b200k_decode_default_chunk": (C.c_int32, [C.POINTER(DecodeArgs)]),
    "b200k_decode_attention": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "b200k_decode_attention_static": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "b200k_paged_gather": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
         C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p],
    ),
    "b200k_paged_attention_fwd": (C.c_int, [C.POINTER(PagedAttentionArgs), C.c_void_p]),
    "b200k_kv_append": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
         C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p],
    ),
    "b200k_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p]),
    "b200k_quantize_e4m3": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "b200k_gemm_nt_host": (C.c_int, [C.POINTER(GemmArgs), C.POINTER(GemmArgs), C.c_void_p]),
    "b200k_attention_fwd_host": (C.c_int, [C.POINTER(AttentionArgs), C.POINTER(AttentionArgs), C.c_void_p]),
}

_lib = None
_lib_lock = threading.Lock()


def lib_path() -> Path:
    """Location of the shared library: ``$B200K_LIB`` if set, else next to this file."""
    env = os.environ.get("B200K_LIB")
    return Path(env) if env else _PKG_DIR / _LIB_NAME


def lib() -> C.CDLL:
    """Loads (once) and returns the kernel library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} does not exist: the CUDA kernel library has not been built. "
                f"Run `python {_PKG_DIR / 'csrc' / 'build.py'}` (needs nvcc). There is no CPU fallback."
            )
        handle = C.CDLL(str(path))
        for name, (restype, argtypes) in EXPORTED_SYMBOLS.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        version = handle.b200k_abi_version()
        if version != ABI_VERSION:
            raise RuntimeError(f"{path}: ABI version {version}, this binding expects {ABI_VERSION}")
        _lib = handle
    return _lib


def check(status: int) -> None:
    """Raises for a non-OK status: ValueError for argument errors, B200kError otherwise."""
    if status == OK:
        return
    handle = lib()
    name = handle.b200k_status_string(status).decode()
    msg = handle.b200k_last_error().decode()
    if status in (ERR_BAD_SHAPE, ERR_BAD_ALIGN, ERR_BAD_DTYPE, ERR_NULL, ERR_WORKSPACE):
        raise ValueError(f"b200k: {name}: {msg}")
    raise B200kError(status, name, msg)


def _torch_dtype_codes():
    import torch

    return {
        torch.float16: F16,
        torch.bfloat16: BF16,
        torch.float32: F32,
        torch.float8_e4m3fn: E4M3,
    }


class _LazyCodes(dict):
    def __missing__(self, key):
        self.update(_torch_dtype_codes())
        if key in self:
            return self[key]
        raise ValueError(f"b200k: dtype {key} is not supported")


DTYPE_CODES = _LazyCodes()
