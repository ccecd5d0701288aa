"""Host-buffer entry points on the GPU (b200k_attention_fwd_host / b200k_gemm_nt_host through
AttentionHost / GemmHost): the sliced upload / compute / copy-back pipeline must give exactly what
the device-resident call gives on the same data, and stay within the path's tolerance of the oracle."""

import pytest
import torch

import iree_turbine_b200 as tb
from iree_turbine_b200.host_api import AttentionHost, GemmHost
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCALE = 128 ** -0.5


@pytest.mark.parametrize("causal", [False, True])
def test_attention_host_equals_device_call(causal):
    g = torch.Generator().manual_seed(3)
    b, hq, hkv, s = 3, 8, 4, 384
    q = (torch.randn(b, hq, s, 128, generator=g) * 0.5).half().pin_memory()
    k = (torch.randn(b, hkv, s, 128, generator=g) * 0.5).half().pin_memory()
    v = (torch.randn(b, hkv, s, 128, generator=g) * 0.5).half().pin_memory()
    out = torch.empty_like(q).pin_memory()
    host = AttentionHost(b, hq, hkv, s, s, torch.float16, DEV)
    for _ in range(2):  # twice in a row: the copy-back stream is reused
        out.zero_()
        host(q, k, v, out, SCALE, causal)
        torch.cuda.synchronize()
        assert tb.device_status() == 0
        ref = torch.ops.b200k.attention(q.to(DEV), k.to(DEV), v.to(DEV), SCALE, causal)
        torch.cuda.synchronize()
        assert torch.equal(out, ref.cpu())
    oracle.assert_close_half(out, oracle.attention(q, k, v, SCALE, causal))


def test_gemm_host_row_blocks_equal_device_call():
    # 16384 x 512 f16 = 16 MB of A: the host entry point splits it into two row blocks
    m, n, k = 16384, 256, 512
    a, b = oracle.make_gemm_inputs(m, n, k, torch.float16, seed=5)
    a, b = a.pin_memory(), b.pin_memory()
    out = torch.empty(m, n, dtype=torch.float32).pin_memory()
    host = GemmHost(m, n, k, torch.float16, torch.float32, DEV)
    for _ in range(2):
        out.zero_()
        host(a, b, out)
        torch.cuda.synchronize()
        assert tb.device_status() == 0
        ref = torch.ops.b200k.gemm_nt(a.to(DEV), b.to(DEV), torch.float32)
        torch.cuda.synchronize()
        assert torch.equal(out, ref.cpu())
    rows = torch.arange(0, m, 97)
    oracle.assert_close_half(out[rows], oracle.gemm_nt(a[rows], b))


def test_gemm_host_single_block_ragged():
    m, n, k = 300, 200, 136
    a, b = oracle.make_gemm_inputs(m, n, k, torch.float16, seed=6)
    out = torch.empty(m, n, dtype=torch.float32)
    GemmHost(m, n, k, torch.float16, torch.float32, DEV)(a, b, out)
    torch.cuda.synchronize()
    oracle.assert_close_half(out, oracle.gemm_nt(a, b))


def test_bounded_wait_runs_out_and_reports():
    """A device-side wait that nothing will ever satisfy gives up after its limit: the kernel returns,
    the status word carries the code, and the context keeps working (the next kernel runs)."""
    import ctypes as C
    import time

    import iree_turbine_b200 as tb
    from iree_turbine_b200 import _launcher as L

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    L.check(L.lib().b200k_selftest_bounded_wait(status.data_ptr(), 3000, stream))  # 3 ms
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert int(status.item()) == 16
    assert 0.002 < dt < 1.0, dt
    # the context is intact: an ordinary kernel still runs and no status bit leaks into the library's own word
    a, b = oracle.make_gemm_inputs(128, 128, 64, torch.float16, seed=1)
    oracle.assert_close_half(torch.ops.b200k.gemm_nt(a.to(DEV), b.to(DEV)), oracle.gemm_nt(a, b))
    assert tb.device_status() == 0
    assert L.lib().b200k_selftest_bounded_wait(None, 3000, stream) == L.ERR_NULL
    assert L.lib().b200k_selftest_bounded_wait(status.data_ptr(), 0, stream) == L.ERR_BAD_SHAPE
