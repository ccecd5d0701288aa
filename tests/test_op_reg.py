"""Registration semantics of the CustomOp surface (mirrors the reference's
tests/runtime/op_reg/kernel_reg_test.py and tests/transforms/general/custom_op_expansion_test.py,
which register throw-away ops into a private library) and the Meta implementations of the
shipped ops."""

import pytest
import torch

import iree_turbine_b200 as tb
from iree_turbine_b200.op_reg import ALL_CUSTOM_OP_REGS, CustomOp, EagerKernelSelection, def_library

LIB = def_library("b200k_test")


def test_register_defines_schema_meta_and_registry_entry():
    @CustomOp.register(library=LIB)
    class twice(CustomOp):
        signature = "twice(Tensor t, int n) -> Tensor"

        def select(self, sel):
            t = sel.arg_tensor(0)
            n = sel.arg_int(1)
            sel.return_new_tensor([t.t.size(0) * n.v], t.t.dtype)

        def eager_execute(self, t, n):
            return t.repeat(n)

    assert "b200k_test.twice" in ALL_CUSTOM_OP_REGS
    assert twice is torch.ops.b200k_test.twice
    meta = twice(torch.empty(3, device="meta"), 4)
    assert meta.device.type == "meta" and meta.shape == (4 * 3,)

    with pytest.raises(RuntimeError, match="Duplicate"):
        @CustomOp.register(library=LIB)
        class twice_again(CustomOp):
            signature = "twice(Tensor t, int n) -> Tensor"

            def select(self, sel):
                pass


def test_unique_names_and_missing_eager_execute():
    def make():
        @CustomOp.register(library=LIB, dispatch_key="CPU")
        class anon(CustomOp):
            signature = "anon_@UNIQUE@(Tensor t) -> Tensor"

            def select(self, sel):
                sel.return_tensor(sel.arg_tensor(0).t)

        return anon

    a, b = make(), make()
    assert a is not b
    assert str(a).endswith("anon_1") and str(b).endswith("anon_2")
    # no eager_execute: nothing is compiled at call time, so the call must fail loudly
    with pytest.raises(NotImplementedError, match="no device implementation"):
        a(torch.zeros(2))


def test_selection_type_checks_and_spec_key():
    op = ALL_CUSTOM_OP_REGS["b200k.gemm_nt"]
    a = torch.empty(64, 32, dtype=torch.float16, device="meta")
    b = torch.empty(48, 32, dtype=torch.float16, device="meta")
    sel = EagerKernelSelection(op, [a, b, None])
    op.select(sel)
    assert "gemm_nt" in sel.spec_key and "32" in sel.spec_key and "float16" in sel.spec_key
    bad = EagerKernelSelection(op, [a, 3, None])
    with pytest.raises(AssertionError, match="Expected tensor"):
        op.select(bad)


def test_shipped_ops_meta_shapes_and_dtypes():
    f16, bf16 = torch.float16, torch.bfloat16
    m = lambda *s, dtype=f16: torch.empty(*s, dtype=dtype, device="meta")  # noqa: E731
    assert torch.ops.b200k.gemm_nt(m(256, 64), m(100, 64)).dtype == torch.float32
    assert torch.ops.b200k.gemm_nt(m(256, 64, dtype=bf16), m(100, 64, dtype=bf16), bf16).shape == (256, 100)
    a8 = m(128, 64, dtype=torch.float8_e4m3fn)
    s = m(1, dtype=torch.float32)
    assert torch.ops.b200k.gemm_fp8_nt(a8, a8, s, s).dtype == bf16
    q = m(2, 8, 300, 128)
    kv = m(2, 2, 500, 128)
    o = torch.ops.b200k.attention(q, kv, kv, 0.1, True)
    assert o.shape == q.shape and o.dtype == f16
    qd = m(5, 8, 128)
    lens = m(5, dtype=torch.int32)
    assert torch.ops.b200k.decode_attention(qd, m(5, 2, 64, 128), m(5, 2, 64, 128), lens, 0.1).shape == (5, 8, 128)
    bt = m(5, 7, dtype=torch.int32)
    pool = m(40, 2, 16, 128)
    assert torch.ops.b200k.paged_decode_attention(qd, pool, pool, bt, lens, 0.1).shape == (5, 8, 128)
    y, sc = torch.ops.b200k.quantize_e4m3(m(10, 10, dtype=torch.float32))
    assert y.dtype == torch.float8_e4m3fn and sc.shape == (1,)
    assert torch.ops.b200k.paged_gather(pool, bt, lens, 112).shape == (5, 2, 112, 128)


def test_shipped_ops_reject_bad_arguments():
    m = lambda *s, dtype=torch.float16: torch.empty(*s, dtype=dtype, device="meta")  # noqa: E731
    with pytest.raises(RuntimeError, match="K mismatch"):
        torch.ops.b200k.gemm_nt(m(8, 64), m(8, 32))
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        torch.ops.b200k.gemm_nt(m(8, 64, dtype=torch.float32), m(8, 64, dtype=torch.float32))
    with pytest.raises(RuntimeError, match="head dim must be 128 or 64"):
        torch.ops.b200k.attention(m(1, 1, 8, 96), m(1, 1, 8, 96), m(1, 1, 8, 96), 1.0, False)
    with pytest.raises(RuntimeError, match="head dim must be 128 or 64"):
        torch.ops.b200k.attention(m(1, 1, 8, 64), m(1, 1, 8, 128), m(1, 1, 8, 128), 1.0, False)
    assert torch.ops.b200k.attention(m(1, 2, 8, 64), m(1, 1, 9, 64), m(1, 1, 9, 64), 1.0, True).shape == (1, 2, 8, 64)
    with pytest.raises(RuntimeError, match="multiple of kv heads"):
        torch.ops.b200k.attention(m(1, 3, 8, 128), m(1, 2, 8, 128), m(1, 2, 8, 128), 1.0, False)


def test_tensor_arguments_on_different_devices_are_rejected_before_any_launch():
    """A host-resident seq_lens / scale next to device tensors would hand a host pointer to a kernel:
    both the Meta path and the device trampoline refuse it."""
    from iree_turbine_b200.op_reg import _impl_trampoline

    m = lambda *s, dtype=torch.float16: torch.empty(*s, dtype=dtype, device="meta")  # noqa: E731
    qd, kv = m(5, 8, 128), m(5, 2, 64, 128)
    with pytest.raises(RuntimeError, match="one device"):
        torch.ops.b200k.decode_attention(qd, kv, kv, torch.zeros(5, dtype=torch.int32), 0.1)
    a8 = m(128, 64, dtype=torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="one device"):
        torch.ops.b200k.gemm_fp8_nt(a8, a8, torch.ones(1), m(1, dtype=torch.float32))
    # the device implementation's trampoline, called directly: rejected before eager_execute runs
    op = ALL_CUSTOM_OP_REGS["b200k.paged_decode_attention"]
    pool, bt = m(40, 2, 16, 128), m(5, 7, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="one device"):
        _impl_trampoline(op)(qd, pool, pool, bt, torch.zeros(5, dtype=torch.int32), 0.1, 0)


def test_cpu_tensors_have_no_implementation():
    a = torch.zeros(8, 8, dtype=torch.float16)
    with pytest.raises(NotImplementedError, match="CPU"):
        torch.ops.b200k.gemm_nt(a, a)


def test_template_constructors_validate_shapes():
    k = tb.get_gemm_kernel(tb.GemmShape(128, 64, 32), torch.float16)
    assert k.name == "gemm_nt" and k.shape.flops == 2 * 128 * 64 * 32
    with pytest.raises(ValueError, match="expected shape"):
        k(torch.empty(128, 16, dtype=torch.float16, device="meta"), torch.empty(64, 32, dtype=torch.float16, device="meta"))
    out = k(torch.empty(128, 32, dtype=torch.float16, device="meta"), torch.empty(64, 32, dtype=torch.float16, device="meta"))
    assert out.shape == (128, 64)
    shape = tb.AttentionShape(num_query_heads=32, num_kv_heads=8, head_size=128, query_seq_len=1024, kv_seq_len=1024, num_seqs=8)
    assert shape.group_size == 4
    assert shape.flops() == 4 * 8 * 32 * 1024 * 1024 * 128
    assert shape.flops(causal=True) == shape.flops() // 2
    with pytest.raises(ValueError):
        tb.AttentionShape(num_query_heads=6, num_kv_heads=4, head_size=128)
    with pytest.raises(ValueError, match="head_size"):
        tb.get_vanilla_attention_kernel(tb.AttentionShape(4, 4, 96, 16, 16))
    assert tb.get_vanilla_attention_kernel(tb.AttentionShape(4, 4, 64, 16, 16)).name == "vanilla_attention"
    with pytest.raises(ValueError, match="block_size"):
        tb.get_paged_decode_attention_kernel(tb.AttentionShape(32, 8, 128, num_seqs=4))
