"""Numerics report for a bench-driver command: the statistical criteria and the structured
indexing test of the reference's numerics driver (kernel/boo/driver/numerics.py:29-35, 266-316,
319-411), stated for this library's backends.

For one command (same seeded operands for every backend):

* the CPU result of the torch operator in float64 is the reference value;
* ``b200k`` and ``torch`` (the vendor's GPU kernel) each give a signed element-wise error against
  it; the b200k error must have no detectable bias -- |mean| <= 1e-5 + 0.2 * its own standard
  deviation -- and no more spread than the vendor kernel's -- stddev <= 1e-5 + 1.2 * torch's;
* the structured test feeds operands that are zero except for one block of ones at a seeded
  offset (at most a quarter of the tensor, at most 128 elements): an indexing mistake moves or
  loses the block, so the two GPU results must agree to 1e-7 absolute.

The tolerance tests of ``tests/`` stay the gate for parity; this is the secondary report the
reference prints beside its timings (``--verify-numerics``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

MIN_SAMPLES = 1000
MEAN_CHECK_ATOL = 1e-5
MEAN_CHECK_RTOL = 0.2
STDDEV_CHECK_ATOL = 1e-5
STDDEV_CHECK_RTOL = 1.2
STRUCTURED_ATOL = 1e-7
STRUCTURED_BLOCK_LIMIT = 128

__all__ = ["ErrorStatistics", "Verdict", "error_statistics", "evaluate", "apply_block_of_ones", "verify_command"]


@dataclass
class ErrorStatistics:
    mean: float
    stddev: float
    max_abs_err: float
    num_samples: int


@dataclass
class Verdict:
    command: str
    passed: bool
    b200k_err: Optional[ErrorStatistics] = None
    torch_err: Optional[ErrorStatistics] = None
    mean_near_zero: bool = True
    stddev_ratio_ok: bool = True
    structured_test_passed: Optional[bool] = None
    reasons: List[str] = field(default_factory=list)


def error_statistics(result: torch.Tensor, reference: torch.Tensor) -> ErrorStatistics:
    """Signed element-wise error ``result - reference`` in float64 (non-finite reference entries,
    e.g. attention rows without a visible key, are left out)."""
    r, ref = result.detach().double().cpu().flatten(), reference.detach().double().cpu().flatten()
    keep = torch.isfinite(ref)
    e = (r - ref)[keep]
    if e.numel() == 0:
        return ErrorStatistics(0.0, 0.0, 0.0, 0)
    return ErrorStatistics(float(e.mean()), float(e.std(unbiased=False)), float(e.abs().max()), int(e.numel()))


def _negligible(value: float, reference: float, atol: float, rtol: float) -> bool:
    return abs(value) <= atol + rtol * abs(reference)


def evaluate(ours: ErrorStatistics, vendor: ErrorStatistics, mean_atol: float = MEAN_CHECK_ATOL,
             mean_rtol: float = MEAN_CHECK_RTOL, stddev_atol: float = STDDEV_CHECK_ATOL,
             stddev_rtol: float = STDDEV_CHECK_RTOL):
    """(mean_near_zero, stddev_ok, reasons)."""
    reasons = []
    mean_ok = _negligible(ours.mean, ours.stddev, mean_atol, mean_rtol)
    if not mean_ok:
        reasons.append(f"mean error |{ours.mean:.3e}| > {mean_atol:.1e} + {mean_rtol} * own stddev {ours.stddev:.3e}")
    std_ok = _negligible(ours.stddev, vendor.stddev, stddev_atol, stddev_rtol)
    if not std_ok:
        reasons.append(f"error stddev {ours.stddev:.3e} > {stddev_atol:.1e} + {stddev_rtol} * torch stddev {vendor.stddev:.3e}")
    return mean_ok, std_ok, reasons


def apply_block_of_ones(t: torch.Tensor, seed: int = 0, block_limit: int = STRUCTURED_BLOCK_LIMIT) -> torch.Tensor:
    """Zeroes ``t`` (through its strides) and writes one run of ones into its elements, in logical
    row-major order: at most a quarter of the tensor and ``block_limit`` elements, at an offset drawn
    from ``seed``."""
    t.zero_()
    n = t.numel()
    if n == 0:
        return t
    block = max(1, min(n // 4, block_limit))
    gen = torch.Generator(device="cpu").manual_seed(seed)
    offset = int(torch.randint(0, max(1, n - block), (1,), generator=gen))
    idx = torch.arange(offset, offset + block, device=t.device)
    coords = torch.unravel_index(idx, t.shape)
    t[coords] = 1
    return t


def verify_command(cmd, device, min_samples: int = MIN_SAMPLES, command_text: str = "") -> Verdict:
    """Runs one parsed driver command on b200k, torch-GPU and torch-CPU-float64 and applies the criteria."""
    from . import driver

    notes: List[str] = []
    with torch.no_grad():
        ours = driver.build_callable(cmd, "b200k", device, notes)()
        vendor = driver.build_callable(cmd, "torch", device, notes)()
        ref = driver.build_callable(cmd, "cpu_fp64", device, notes)()
        torch.cuda.synchronize(device)
        e_ours, e_vendor = error_statistics(ours, ref), error_statistics(vendor, ref)
        mean_ok, std_ok, reasons = evaluate(e_ours, e_vendor)
        if e_ours.num_samples < min_samples:
            reasons.append(f"only {e_ours.num_samples} samples (< {min_samples}): statistics are indicative")
        s_ours = driver.build_callable(cmd, "b200k", device, notes, fill="structured")()
        s_vendor = driver.build_callable(cmd, "torch", device, notes, fill="structured")()
        torch.cuda.synchronize(device)
        structured = bool(torch.allclose(s_ours.double(), s_vendor.double(), atol=STRUCTURED_ATOL, rtol=0))
        if not structured:
            reasons.append(f"structured test: max difference {float((s_ours.double() - s_vendor.double()).abs().max()):.3e}")
    return Verdict(command_text, mean_ok and std_ok and structured, e_ours, e_vendor, mean_ok, std_ok, structured, reasons)


def format_verdict(v: Verdict) -> str:
    def st(e):
        return f"mean {e.mean:+.3e} stddev {e.stddev:.3e} max {e.max_abs_err:.3e} (n={e.num_samples})"

    lines = [f"numerics: {'PASS' if v.passed else 'FAIL'}",
             f"  b200k vs fp64 CPU: {st(v.b200k_err)}",
             f"  torch vs fp64 CPU: {st(v.torch_err)}",
             f"  mean near zero: {v.mean_near_zero}; stddev within {STDDEV_CHECK_RTOL} x torch: {v.stddev_ratio_ok}; "
             f"block-of-ones test: {v.structured_test_passed}"]
    lines += [f"  note: {r}" for r in v.reasons]
    return "\n".join(lines)
