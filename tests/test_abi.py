"""The C-ABI library: loads without a GPU, exports every function the header declares, its
structs have the layout the ctypes binding assumes, and argument errors are reported as status
codes before anything is launched."""

import ctypes as C
import os
import re
import subprocess
import tempfile

import pytest

from iree_turbine_b200 import _launcher as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200k.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200k_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(kernel_lib):
    declared = _declared_functions()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(kernel_lib, name), f"{name} is declared in include/b200k.h but not exported"
        assert name in L.EXPORTED_SYMBOLS, f"{name} has no ctypes prototype"
    assert sorted(L.EXPORTED_SYMBOLS) == declared
    assert kernel_lib.b200k_abi_version() == L.ABI_VERSION == 3


def test_struct_layouts_match_the_header():
    """Compiles a C probe against the header and compares sizeof / offsetof with ctypes."""
    fields = {
        "b200k_gemm_args": (L.GemmArgs, ["a", "ldc", "in_dtype", "scale_a", "status", "tile_n", "c_batch_stride", "split_k"]),
        "b200k_attention_args": (L.AttentionArgs, ["q", "batch", "head_dim", "q_stride_b", "o_stride_s", "dtype",
                                                   "scale", "status", "lse", "kernel"]),
        "b200k_decode_args": (L.DecodeArgs, ["q", "workspace_bytes", "num_seqs", "max_seq_len", "kv_batch_stride",
                                             "kv_page_stride", "dtype", "scale", "status"]),
        "b200k_paged_attention_args": (L.PagedAttentionArgs, ["q", "seq_lens", "batch", "head_dim", "page_size",
                                                              "block_table_stride", "q_stride_b", "o_stride_s",
                                                              "kv_page_stride", "kv_head_stride", "dtype", "scale",
                                                              "kernel", "status"]),
        "b200k_attention_bwd_args": (L.AttentionBwdArgs, ["q", "d_o", "d_v", "workspace", "workspace_bytes", "batch",
                                                          "head_dim", "q_stride_b", "do_stride_h", "dv_stride_s",
                                                          "dtype", "scale", "status", "lse"]),
        "b200k_gemm_allgather_args": (L.GemmAllGatherArgs, ["gemm", "peer_c", "num_peers", "self_index", "peer_ldc", "col_offset",
                                                             "multicast_c", "plain_stores"]),
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for cname, (_, fs) in fields.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f in fs:
            lines.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    lines.append("return 0; }")
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "p.c"), os.path.join(d, "p")
        open(src, "w").write("\n".join(lines))
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", src, "-o", exe], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    got = dict(line.split() for line in out.strip().splitlines())
    for cname, (ctype, fs) in fields.items():
        assert int(got[cname]) == C.sizeof(ctype), cname
        for f in fs:
            assert int(got[f"{cname}.{f}"]) == getattr(ctype, f).offset, f"{cname}.{f}"


def test_argument_errors_are_status_codes(kernel_lib):
    lib = kernel_lib
    assert lib.b200k_gemm_nt(None, None) == L.ERR_NULL
    g = L.GemmArgs()
    assert lib.b200k_gemm_nt(C.byref(g), None) == L.ERR_NULL
    assert b"non-NULL" in lib.b200k_last_error()
    g.a = g.b = g.c = 0x1000
    g.m, g.n, g.k = 128, 128, 0
    assert lib.b200k_gemm_nt(C.byref(g), None) == L.ERR_BAD_SHAPE
    g.k = 64
    g.lda = g.ldb = 64
    g.ldc = 128
    g.in_dtype, g.out_dtype = L.F32, L.F32
    assert lib.b200k_gemm_nt(C.byref(g), None) == L.ERR_BAD_DTYPE
    g.in_dtype = L.F16
    g.a = 0x1008
    assert lib.b200k_gemm_nt(C.byref(g), None) == L.ERR_BAD_ALIGN
    g.a = 0x1000
    g.lda = 68  # 136-byte rows
    assert lib.b200k_gemm_nt(C.byref(g), None) == L.ERR_BAD_ALIGN
    assert lib.b200k_status_string(L.ERR_BAD_ALIGN) == b"BAD_ALIGN"

    a = L.AttentionArgs()
    assert lib.b200k_attention_fwd(C.byref(a), None) == L.ERR_NULL
    a.q = a.k = a.v = a.o = 0x1000
    a.batch = a.q_heads = a.kv_heads = 1
    a.seq_q = a.seq_kv = 128
    a.head_dim = 96
    assert lib.b200k_attention_fwd(C.byref(a), None) == L.ERR_BAD_SHAPE
    assert b"head_dim" in lib.b200k_last_error()

    w = L.AttentionBwdArgs()
    assert lib.b200k_attention_bwd(None, None) == L.ERR_NULL
    assert lib.b200k_attention_bwd(C.byref(w), None) == L.ERR_NULL
    w.q = w.k = w.v = w.o = w.d_o = w.d_q = w.d_k = w.d_v = 0x1000
    w.batch, w.q_heads, w.kv_heads, w.seq_q, w.seq_kv, w.head_dim = 2, 6, 4, 100, 128, 128
    assert lib.b200k_attention_bwd(C.byref(w), None) == L.ERR_BAD_SHAPE  # 6 % 4 != 0
    w.q_heads = 8
    w.dtype = L.F32
    assert lib.b200k_attention_bwd(C.byref(w), None) == L.ERR_BAD_DTYPE
    w.dtype = L.BF16
    assert lib.b200k_attention_bwd(C.byref(w), None) == L.ERR_BAD_ALIGN  # strides are still zero
    for t in ("q", "k", "v", "o", "do", "dq", "dk", "dv"):
        setattr(w, f"{t}_stride_s", 128), setattr(w, f"{t}_stride_h", 128 * 128), setattr(w, f"{t}_stride_b", 8 * 128 * 128)
    w.scale = 0.1
    assert lib.b200k_attention_bwd_workspace_bytes(C.byref(w)) == 2 * 4 * 2 * 8 * 100
    assert lib.b200k_attention_bwd(C.byref(w), None) == L.ERR_WORKSPACE

    d = L.DecodeArgs()
    assert lib.b200k_decode_attention(C.byref(d), None) == L.ERR_NULL
    d.q = d.k_cache = d.v_cache = d.seq_lens = d.o = 0x1000
    d.num_seqs, d.q_heads, d.kv_heads, d.head_dim, d.max_seq_len = 4, 6, 4, 128, 512
    assert lib.b200k_decode_attention(C.byref(d), None) == L.ERR_BAD_SHAPE  # 6 % 4 != 0
    d.q_heads = 8
    d.dtype = L.F16
    d.kv_batch_stride, d.kv_head_stride = 8 * 512 * 128, 512 * 128
    need = lib.b200k_decode_workspace_bytes(C.byref(d))
    chunk = lib.b200k_decode_default_chunk(C.byref(d))
    assert chunk % 64 == 0 and chunk >= 64
    n_chunks = (512 + chunk - 1) // chunk
    assert need == 4 * 8 * n_chunks * (128 * 4 + 8)
    assert lib.b200k_decode_attention(C.byref(d), None) == L.ERR_WORKSPACE
    d.chunk_tokens = 100
    assert lib.b200k_decode_attention(C.byref(d), None) == L.ERR_BAD_SHAPE


def test_check_maps_statuses_to_exceptions(kernel_lib):
    L.check(0)
    kernel_lib.b200k_gemm_nt(None, None)
    with pytest.raises(ValueError, match="NULL"):
        L.check(L.ERR_NULL)
    with pytest.raises(L.B200kError):
        L.check(L.ERR_CUDA)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("B200K_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(L, "_lib", None)
    with pytest.raises(RuntimeError, match="has not been built"):
        L.lib()
