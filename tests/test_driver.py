"""The bench driver's command-line contract (no GPU): flag meanings, the reference's naming, the
CSV header, and that it refuses to run without a device instead of falling back to the CPU."""

import pytest
import torch

from iree_turbine_b200 import driver


def test_gemm_flags_follow_the_reference_parser_not_its_help_text():
    # --a_w is M, --a_h is K, --b_w is N (kernel/boo/op_exports/gemm.py:104-107,173-175)
    c = driver.parse_command(["gemmfp16", "--a_w", "32", "--a_h", "64", "--b_w", "128"])
    assert (c.m, c.k, c.n) == (32, 64, 128) and c.dtype == torch.float16
    assert not c.transpose_a and not c.transpose_b and c.mode == 1
    assert c.func_name == "gemm_float16_forward_32x64x128"
    # the short flags are the reference's too: -k sets a_w (= M), -m sets a_h (= K)
    c = driver.parse_command(["gemm", "-k", "8", "-m", "16", "-n", "24", "-v", "1", "-u", "1"])
    assert (c.m, c.k, c.n) == (8, 16, 24) and c.dtype == torch.float32
    assert c.func_name == "gemm_float32_forward_8x16x24_transA_transB"
    c = driver.parse_command(["gemmfp16"])
    assert (c.m, c.k, c.n) == (256, 256, 256)


@pytest.mark.parametrize("argv", [["gemmfp16", "--a_w", "0"], ["gemmfp16", "-F", "7"], ["conv"], []])
def test_bad_commands_raise(argv):
    with pytest.raises((ValueError, SystemExit)):
        driver.parse_command(argv)


def test_aten_commands_parse_like_the_sample_file():
    # the shapes of driver/sample_commands.txt:22 and :26, not their contents
    c = driver.parse_command(["aten::mm", "[[3840, 4352], [4352, 3840]]", "['c10::BFloat16', 'c10::BFloat16']",
                              "[[1, 3840], [3840, 1]]", "['', '']"])
    assert c.name == "aten::mm" and c.input_dims[0] == [3840, 4352] and c.input_strides[0] == [1, 3840]
    c = driver.parse_command([
        "aten::scaled_dot_product_attention",
        "[[2, 8, 256, 128], [2, 8, 256, 128], [2, 8, 256, 128], [], [], [], [], []]",
        "['c10::Half', 'c10::Half', 'c10::Half', '', 'Scalar', 'Scalar', 'Scalar', 'Scalar']",
        "[[262144, 32768, 128, 1], [262144, 32768, 128, 1], [262144, 32768, 128, 1], [], [], [], [], []]",
        "['', '', '', 'None', '0.0', 'True', 'None', 'False']"])
    assert c.concrete_inputs[5] == "True" and len(c.input_dims) == 8


def test_timing_flags_are_split_off():
    t, rest = driver.timing_parser().parse_known_args(["gemmfp16", "--a_w", "32", "--iter", "7", "-t", "1"])
    assert t.iter == 7 and rest == ["gemmfp16", "--a_w", "32"]


def test_csv_header_contract():
    assert driver.csv_headers(["b200k", "torch"]) == ["arguments"] + [
        f"{b} {s}" for b in ("b200k", "torch") for s in ("min", "max", "mean", "stddev", "num_dispatches")]


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_cpu_fallback(tmp_path):
    with pytest.raises(RuntimeError, match="no CPU path"):
        driver.main([f"--csv={tmp_path / 'x.csv'}", "gemmfp16", "--a_w", "32"])
    # the header is still written first, as in the reference
    assert (tmp_path / "x.csv").read_text().splitlines()[0].startswith("arguments,b200k min")


def test_aten_bmm_command_parses():
    c = driver.parse_command(["aten::bmm", "[[8, 128, 64], [8, 64, 256]]", "['c10::Half', 'c10::Half']",
                              "[[8192, 64, 1], [16384, 256, 1]]", "['', '']"])
    assert c.name == "aten::bmm" and c.input_dims == [[8, 128, 64], [8, 64, 256]]
