"""The numerics report: criteria and the block-of-ones pattern on CPU (host logic), the report itself
and the structured tests of attention and of the paged gather on the GPU.  Mirrors the reference's
numerics driver (kernel/boo/driver/numerics.py:29-35, 266-316, 319-411) and its smoke test
(tests/kernel/boo/driver/numerics_smoke_test.py)."""

import pytest
import torch

from iree_turbine_b200 import numerics

DEV = "cuda"


def test_error_statistics_and_criteria():
    ref = torch.zeros(4000, dtype=torch.float64)
    g = torch.Generator().manual_seed(0)
    ours = torch.randn(4000, generator=g, dtype=torch.float64) * 1e-3
    vendor = torch.randn(4000, generator=g, dtype=torch.float64) * 1e-3
    e_o, e_v = numerics.error_statistics(ours, ref), numerics.error_statistics(vendor, ref)
    assert e_o.num_samples == 4000 and abs(e_o.stddev - 1e-3) < 1e-4 and abs(e_o.mean) < 1e-4
    assert numerics.evaluate(e_o, e_v)[:2] == (True, True)
    # a bias of one standard deviation is detected, so is twice the vendor's spread
    mean_ok, std_ok, why = numerics.evaluate(numerics.error_statistics(ours + 1e-3, ref), e_v)
    assert (mean_ok, std_ok) == (False, True) and "mean error" in why[0]
    mean_ok, std_ok, why = numerics.evaluate(numerics.error_statistics(ours * 2, ref), e_v)
    assert (mean_ok, std_ok) == (True, False) and "stddev" in why[0]
    # tiny absolute errors pass whatever the ratio is; non-finite reference entries are left out
    assert numerics.evaluate(numerics.ErrorStatistics(1e-7, 5e-6, 1e-5, 1000), numerics.ErrorStatistics(0, 1e-9, 0, 1000))[:2] == (True, True)
    ref2 = ref.clone()
    ref2[:10] = float("-inf")
    assert numerics.error_statistics(ours, ref2).num_samples == 3990


def test_block_of_ones_pattern():
    t = torch.full((7, 9, 11), 3.0)
    numerics.apply_block_of_ones(t, seed=4)
    flat = t.flatten()
    assert int(flat.sum()) == 128 and set(flat.unique().tolist()) == {0.0, 1.0}
    on = flat.nonzero().flatten()
    assert int(on[-1] - on[0]) == 127  # one contiguous run
    small = numerics.apply_block_of_ones(torch.empty(10), seed=1)
    assert int(small.sum()) == 2  # at most a quarter of the tensor
    # through strides: a transposed view gets the run in ITS logical order
    base = torch.zeros(6, 8)
    numerics.apply_block_of_ones(base.t(), seed=2)
    assert torch.equal(base.t().flatten().nonzero().flatten(), numerics.apply_block_of_ones(torch.zeros(8, 6), seed=2).flatten().nonzero().flatten())
    assert numerics.apply_block_of_ones(torch.zeros(8, 6), seed=2).sum() == numerics.apply_block_of_ones(torch.zeros(8, 6), seed=3).sum()


@pytest.mark.gpu
@pytest.mark.parametrize("argv", [
    ["gemmfp16", "--a_w", "256", "--a_h", "512", "--b_w", "384", "--transB", "1"],
    ["aten::mm", "[[384, 256], [256, 192]]", "['c10::BFloat16', 'c10::BFloat16']", "[[256, 1], [192, 1]]", "['', '']"],
    ["aten::bmm", "[[4, 128, 64], [4, 64, 256]]", "['c10::Half', 'c10::Half']", "[[8192, 64, 1], [16384, 256, 1]]", "['', '']"],
    ["aten::scaled_dot_product_attention",
     "[[2, 8, 256, 128], [2, 8, 256, 128], [2, 8, 256, 128], [], [], [], [], []]",
     "['c10::Half', 'c10::Half', 'c10::Half', '', 'Scalar', 'Scalar', 'Scalar', 'Scalar']",
     "[[262144, 32768, 128, 1], [262144, 32768, 128, 1], [262144, 32768, 128, 1], [], [], [], [], []]",
     "['', '', '', 'None', '0.0', 'True', 'None', 'False']"],
    ["aten::scaled_dot_product_attention",
     "[[4, 8, 128, 64], [4, 8, 128, 64], [4, 8, 128, 64], [], [], [], [], []]",
     "['c10::BFloat16', 'c10::BFloat16', 'c10::BFloat16', '', 'Scalar', 'Scalar', 'Scalar', 'Scalar']",
     "[[65536, 8192, 64, 1], [65536, 8192, 64, 1], [65536, 8192, 64, 1], [], [], [], [], []]",
     "['', '', '', 'None', '0.0', 'True', 'None', 'False']"],
])
def test_numerics_report_passes_on_the_gpu(argv):
    from iree_turbine_b200 import driver

    cmd = driver.parse_command(argv)
    v = numerics.verify_command(cmd, torch.device(DEV, 0), command_text=" ".join(argv))
    text = numerics.format_verdict(v)
    assert v.structured_test_passed, text
    assert v.mean_near_zero and v.stddev_ratio_ok and v.passed, text
    assert v.b200k_err.num_samples >= numerics.MIN_SAMPLES


@pytest.mark.gpu
def test_driver_flag_prints_the_report(capsys):
    from iree_turbine_b200 import driver

    rc = driver.main(["gemmfp16", "--a_w", "128", "--a_h", "256", "--b_w", "128", "--transB", "1", "--iter", "2",
                      "--verify-numerics"])
    out = capsys.readouterr().out
    assert rc == 0 and "numerics: PASS" in out and "block-of-ones test: True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_attention_block_of_ones(causal):
    """Structured indexing test for attention: V is zero except one block of ones, Q = K = 0 (uniform
    softmax over the visible keys), so O[b, h, i, d] = (ones among the visible keys of column d) / visible."""
    import iree_turbine_b200 as tb

    b, h, s, d = 2, 3, 384, 128
    q = torch.zeros(b, h, s, d, dtype=torch.float16)
    v = numerics.apply_block_of_ones(torch.zeros(b, h, s, d, dtype=torch.float16), seed=9)
    o = torch.ops.b200k.attention(q.to(DEV), q.to(DEV), v.to(DEV), 1.0, causal).float().cpu()
    assert tb.device_status() == 0
    vis = torch.arange(1, s + 1).float() if causal else torch.full((s,), float(s))
    csum = v.float().cumsum(2) if causal else v.float().sum(2, keepdim=True).expand(b, h, s, d)
    assert torch.allclose(o, csum / vis.view(1, 1, s, 1), rtol=0, atol=2e-3)
    assert int((o != 0).any(-1).any(-1).sum()) == 1  # only the (batch, head) that holds the block


@pytest.mark.gpu
def test_paged_gather_block_of_ones():
    """Structured indexing test for the block-table gather: a pool of zeros with one block of ones."""
    from oracle import oracle

    _, kc, _, bt, sl = oracle.make_paged_decode_inputs(num_seqs=5, q_heads=8, kv_heads=2, min_len=1, max_len=600, seed=3)
    pool = numerics.apply_block_of_ones(torch.zeros_like(kc), seed=5)
    max_len = bt.shape[1] * 16
    got = torch.ops.b200k.paged_gather(pool.to(DEV), bt.to(DEV), sl.to(DEV), max_len).cpu()
    ref = oracle.paged_gather(pool, bt, sl, max_len)
    assert torch.equal(got, ref)
    assert float(got.sum()) == float(ref.sum())
